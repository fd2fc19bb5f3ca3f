"""The drop-in claim, tested: the reference's own callers of the operator path — autograd.cpp,
layer.cpp, loss.cpp, batchnorm.cpp, Relu.cpp of both generations and, in the second, dropout.cpp,
norm.cpp and metrics.h behind the umbrella headers, UNCHANGED — compile and link against the B200 host
layers (CPU test, where the reference sources exist), and the program they form
(tests/cpp/callers_program.cpp: Linear -> losses -> backward, broadcast chains) gives on the GPU
what the same program gives when it is linked against the reference itself (GPU test; golden lines
in tests/golden/callers_*_ref.txt, made by tests/golden/make_callers_golden.py).

Which reference build a line is compared with:
  first generation   every line against callers_gen1_ref (the reference's root tree).
  second generation  against callers_gen2_ref_scalar: the reference with its CPU feature probes
                     answering "no", i.e. its scalar+OpenMP back-end, the only one that honours
                     strides and dim-wise reductions.  As shipped on an AVX-512 host
                     (callers_gen2_ref) the dispatcher multiplies the permuted weight matrix as if
                     it were contiguous and throws "sum_avx512: only dim=-1" inside every backward
                     pass that folds a broadcast dim.  Two lines depend on what dim = -1 means
                     (everything on the SIMD back-ends and in the API documentation, the last dim
                     on the scalar back-end): the loss values of Loss::MSE and Loss::CrossEntropy;
                     they are checked against their definition, computed here with numpy.
Tolerance 1e-5 relative (the operator path's fp32 tolerance; exp/ln/tanh are the reference's SIMD
polynomial flavours on the GPU and libm on its scalar back-end, a difference of ~1e-7)."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILT = os.path.join(ROOT, "tests", "cpp", "_built")
GOLDEN = os.path.join(ROOT, "tests", "golden")
from ctensor_b200.build import reference_root      # noqa: E402

REFERENCE = reference_root()
RTOL, ATOL = 1e-5, 2e-7


def parse(text):
    """-> dict name -> np.ndarray | str (the reason of an 'unavailable' line)"""
    out = {}
    for line in text.splitlines():
        w = line.split()
        if len(w) >= 2 and w[1] == "unavailable":
            out[w[0]] = " ".join(w[2:])
        elif len(w) >= 2:
            vals = np.array([float(x) for x in w[2:]], np.float64)
            assert vals.size == int(w[1]), line[:80]
            out[w[0]] = vals
    return out


def golden(name):
    return parse(open(os.path.join(GOLDEN, name + ".txt")).read())


def run_built(name):
    exe = os.path.join(BUILT, name)
    if not os.path.exists(exe):
        pytest.skip(f"{exe} was not built (tests/cpp/build_callers.sh needs the reference sources)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return parse(r.stdout)


def assert_lines_match(got, want, names, what):
    for n in names:
        assert n in got, f"{what}: line {n} missing"
        assert isinstance(got[n], np.ndarray), f"{what}: {n} unavailable on the GPU build: {got[n]}"
        assert isinstance(want[n], np.ndarray), f"{what}: {n} unavailable in the reference build: {want[n]}"
        np.testing.assert_allclose(got[n], want[n], rtol=RTOL, atol=ATOL, err_msg=f"{what}: {n}")


# ---- CPU: the unchanged callers compile and link ----------------------------------------------------
@pytest.mark.skipif(not REFERENCE, reason="no reference sources here (CTENSOR_REFERENCE, or a checkout beside the repository)")
def test_unchanged_reference_callers_compile_and_link_against_the_host_layers():
    from ctensor_b200 import build as b
    b.build()
    b.build_host()
    b.build_gen1()
    subprocess.check_call([os.path.join(ROOT, "tests", "cpp", "build_callers.sh"), REFERENCE])
    for name in ("callers_gen2_b200", "callers_gen1_b200"):
        assert os.path.exists(os.path.join(BUILT, name))


def test_built_programs_refuse_to_run_without_a_gpu():
    import ctensor_b200
    if ctensor_b200.lib().ctb_device_count() > 0:
        pytest.skip("a CUDA device is present")
    for name in ("callers_gen2_b200", "callers_gen1_b200"):
        exe = os.path.join(BUILT, name)
        if not os.path.exists(exe):
            pytest.skip("not built")
        r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
        assert "no CUDA device" in r.stdout + r.stderr          # every section reports it; nothing is computed


def test_reference_twins_still_give_the_golden_lines():
    """Where the reference twins were built (oracle/build_callers_ref.sh) they reproduce the committed lines."""
    ran = 0
    for name in ("callers_gen1_ref", "callers_gen2_ref", "callers_gen2_ref_scalar"):
        exe = os.path.join(ROOT, "oracle", "_ref", name)
        if not os.path.exists(exe):
            continue
        r = subprocess.run([exe], capture_output=True, text=True, timeout=120, cwd="/tmp")
        assert r.returncode == 0
        got, want = parse(r.stdout), golden(name)
        assert got.keys() == want.keys()
        for k, v in want.items():
            if isinstance(v, np.ndarray):
                np.testing.assert_allclose(got[k], v, rtol=1e-6, atol=1e-9, err_msg=f"{name}: {k}")
        ran += 1
    if not ran:
        pytest.skip("oracle/_ref twins not built on this machine")


# ---- known answers for the two lines whose meaning depends on dim = -1 -------------------------------------
def _lcg(seed, n, scale, shift=0.0):
    mask = (1 << 64) - 1
    s = (seed * 6364136223846793005 + 1442695040888963407) & mask
    out = np.empty(n)
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & mask
        out[i] = ((s >> 11) & ((1 << 53) - 1)) / float(1 << 52) - 1.0
    return (out * scale + shift).astype(np.float32).astype(np.float64)


def _known_losses():
    batch, in_f, out_f = 12, 16, 10
    y = _lcg(3, batch * in_f, 1.0).reshape(batch, in_f) @ _lcg(1, out_f * in_f, 0.5).reshape(out_f, in_f).T + _lcg(2, out_f, 0.1)
    mse = np.mean((y - _lcg(4, batch * out_f, 1.0).reshape(batch, out_f)) ** 2)
    logits = _lcg(7, batch * in_f, 1.0).reshape(batch, in_f) @ _lcg(5, out_f * in_f, 0.5).reshape(out_f, in_f).T + _lcg(6, out_f, 0.1)
    logp = logits - logits.max(1, keepdims=True)
    logp = logp - np.log(np.exp(logp).sum(1, keepdims=True))
    labels = (np.arange(batch) * 7 + 3) % out_f
    ce = -logp[np.arange(batch), labels].mean()
    return mse, ce


# ---- GPU: the programs run and agree with the reference builds -----------------------------------------------
@pytest.mark.gpu
def test_first_generation_callers_run_on_the_gpu_like_the_reference():
    got, want = run_built("callers_gen1_b200"), golden("callers_gen1_ref")
    names = [k for k, v in want.items() if isinstance(v, np.ndarray)]
    assert sum(k.startswith("optim_") for k in names) == 27          # loss, weight, bias of nine optimizers
    assert sum(k.startswith("dropout.") for k in names) == 4         # root dropout.cpp ran in the reference build
    assert_lines_match(got, want, names, "gen 1")


@pytest.mark.gpu
def test_second_generation_callers_run_on_the_gpu_like_the_reference():
    got, want = run_built("callers_gen2_b200"), golden("callers_gen2_ref_scalar")
    # (the loss lines of the optimizer sections are CrossEntropy values too: same dim = -1 question)
    dim_minus_one = {"mse.loss", "ce.loss"} | {k for k in want if k.startswith("optim_") and k.endswith(".loss")}
    names = [k for k, v in want.items() if isinstance(v, np.ndarray) and k not in dim_minus_one]
    assert len(names) >= 15 + 18                            # + weight and bias after three steps of nine optimizers
    for line in ("dropout.forward", "dropout.grad_x", "dropout.eval_forward", "norm.l2_cols", "norm.l3_rows_keepdim",
                 "norm.l2_global", "norm.zero_cols", "metrics.accuracy", "metrics.f1", "metrics.r2"):
        assert line in names, line                          # dropout.cpp, norm.cpp, metrics.h ran in the reference build
    assert_lines_match(got, want, names, "gen 2")
    mse, ce = _known_losses()
    np.testing.assert_allclose(got["mse.loss"], [mse], rtol=RTOL, err_msg="Loss::MSE")
    np.testing.assert_allclose(got["ce.loss"], [ce], rtol=RTOL, err_msg="Loss::CrossEntropy")
    np.testing.assert_allclose(got["mse.loss_from_operators"], [mse], rtol=RTOL)
    for k in sorted(dim_minus_one):
        assert isinstance(got[k], np.ndarray) and got[k].size == 1 and np.isfinite(got[k][0]) and 0.0 < got[k][0] < 5.0, k


# ---- the timed training step: same numbers with and without the integration edits ----------------------------
def _train_step_known_losses(batch, features, hidden, classes, steps, lr=0.05):
    """tests/cpp/train_step_program.cpp in numpy (fp64): two warm-up steps + `steps` steps of plain SGD on
    Linear -> relu -> Linear -> mean cross entropy; -> (loss of the first step, loss of the last step)."""
    w1, b1 = _lcg(1, hidden * features, 0.05).reshape(hidden, features), _lcg(2, hidden, 0.01)
    w2, b2 = _lcg(3, classes * hidden, 0.05).reshape(classes, hidden), _lcg(4, classes, 0.01)
    x = _lcg(5, batch * features, 1.0).reshape(batch, features)
    labels, rows = (np.arange(batch) * 5 + 1) % classes, np.arange(batch)
    losses = []
    for _ in range(steps + 2):
        h = x @ w1.T + b1
        a = np.maximum(h, 0)
        z = a @ w2.T + b2
        logp = z - z.max(1, keepdims=True)
        logp = logp - np.log(np.exp(logp).sum(1, keepdims=True))
        losses.append(-logp[rows, labels].mean())
        g = np.exp(logp)
        g[rows, labels] -= 1
        g /= batch
        gh = (g @ w2) * (h > 0)
        w2, b2 = w2 - lr * (g.T @ a), b2 - lr * g.sum(0)
        w1, b1 = w1 - lr * (gh.T @ x), b1 - lr * gh.sum(0)
    return losses[0], losses[-1]


@pytest.mark.gpu
@pytest.mark.parametrize("exe,env,rtol", [
    ("train_step_gen2_b200", {}, 2e-5),                       # the reference's callers unchanged
    ("train_step_gen2_b200_edited", {}, 2e-5),                # the three bodies replaced by host-layer calls
    ("train_step_gen2_b200_edited", {"CTB_HOST_MATMUL_TENSOR_CORES": "1"}, 5e-3),      # TF32 products
    ("train_step_gen2_b200_edited4", {}, 2e-5),               # + Loss::CrossEntropy's body as one host-layer call
])
def test_training_step_follows_the_definition(exe, env, rtol):
    import json
    path = os.path.join(BUILT, exe)
    if not os.path.exists(path):
        pytest.skip(f"{path} was not built (tests/cpp/build_callers.sh needs the reference sources)")
    shape = (64, 128, 128, 16, 5)
    r = subprocess.run([path] + [str(v) for v in shape], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, **env))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    got = json.loads(r.stdout.strip().splitlines()[-1])
    first, last = _train_step_known_losses(*shape)
    np.testing.assert_allclose([got["loss_first"], got["loss_last"]], [first, last], rtol=rtol)
    assert last < first


# ---- the reference's own unit tests, unchanged, over the host layer ----------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("exe,last_line", [
    ("reference_test_tensor_b200", "All Tests Passed!"),                       # test/test.cpp
    ("reference_test_ops_b200", "All tests completed successfully."),          # test/test_ops.cpp
])
def test_reference_unit_tests_pass_over_the_host_layer(exe, last_line):
    path = os.path.join(BUILT, exe)
    if not os.path.exists(path):
        pytest.skip(f"{path} was not built (tests/cpp/build_callers.sh needs the reference sources)")
    r = subprocess.run([path], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.strip().splitlines()[-1] == last_line
    assert "Skipped" not in r.stdout and "Skipping" not in r.stdout           # broadcasting and the gradient check ran


_NUMBER = r"[-+]?(?:\d+\.?\d*|\.\d+)(?:[eE][-+]?\d+)?"


def _text_and_numbers(text):
    """-> (the text with every number replaced by '#', the numbers)"""
    import re
    return re.sub(_NUMBER, "#", text), [float(x) for x in re.findall(_NUMBER, text)]


@pytest.mark.gpu
def test_first_generation_gradient_checks_print_what_the_reference_prints():
    """The reference's root verify.cpp (Huber / MAE / CrossEntropy / MSE losses and one backward pass per
    operator through ops1.h, printed), unchanged over the first-generation host layer, against the same
    file linked with the reference (tests/golden/verify_gen1_ref.txt): same text, numbers equal to the
    printed precision."""
    path = os.path.join(BUILT, "reference_verify_gen1_b200")
    if not os.path.exists(path):
        pytest.skip(f"{path} was not built (tests/cpp/build_callers.sh needs the reference sources)")
    r = subprocess.run([path], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    got_text, got = _text_and_numbers(r.stdout)
    want_text, want = _text_and_numbers(open(os.path.join(GOLDEN, "verify_gen1_ref.txt")).read())
    assert got_text == want_text
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
