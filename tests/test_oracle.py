"""CPU tests of the checker itself: the plain-C oracle against (a) the golden vectors the real
reference produced, (b) the real reference run live where it is built, (c) the known answers
of the reference's own unit tests (test/test_ops.cpp)."""
import numpy as np
import pytest

import cases as C
import oracle_lib as ol
from oracle_lib import HostView

CASES = C.all_cases()
GOLDEN = C.load_golden()


def _check(case, got, gold_digest, gold_out):
    if case["exact"]:
        assert C.digest(got) == gold_digest, f"{case['name']}: differs from the reference's output"
    else:
        np.testing.assert_allclose(got, gold_out, rtol=1e-6, atol=0, equal_nan=True, err_msg=case["name"])


def test_golden_file_matches_catalogue():
    assert sorted(GOLDEN) == sorted(c["name"] for c in CASES)
    for c in CASES:                      # stored inputs are the inputs the catalogue generates
        for v, g in zip(c["views"], GOLDEN[c["name"]]["views"]):
            assert v.shape == g.shape and v.strides == g.strides and v.offset == g.offset
            assert C.digest(v.buf) == C.digest(g.buf), c["name"]


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_vs_golden(oracle, case):
    g = GOLDEN[case["name"]]
    stored = dict(case, views=g["views"])
    _check(case, C.run_case(oracle, stored), g["digest"], g["out"])


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_vs_live_reference(oracle, reference, case):
    ref = C.run_case(reference, case)
    got = C.run_case(oracle, case)
    _check(case, got, C.digest(ref), ref)


def test_causal_flag_equals_mask_tensor(oracle):
    case = next(c for c in CASES if c["name"] == "softmax_causal_as_mask")
    with_mask = oracle.softmax(case["views"][0], case["views"][1])
    with_flag = oracle.softmax(case["views"][0], None, causal=True)
    assert C.digest(with_mask) == C.digest(with_flag)


@pytest.mark.parametrize("op,path", [(ol.EXP, ol.PATH_AVX512), (ol.EXP, ol.PATH_AVX2), (ol.TANH, ol.PATH_AVX512),
                                     (ol.TANH, ol.PATH_AVX2), (ol.SIGMOID, ol.PATH_AVX512), (ol.LOG, ol.PATH_AVX2),
                                     (ol.GELU_TANH, ol.PATH_AVX512), (ol.SQRT, ol.PATH_AVX512), (ol.RELU, ol.PATH_MP)])
def test_sampled_bit_pattern_sweep(oracle, reference, op, path):
    """Every 2053rd fp32 bit pattern (2.09 M inputs incl. NaN/inf/denormals), bit for bit."""
    count = (1 << 32) // 2053
    xin, got = oracle.sweep(op, 12345, 2053, count)
    ref = reference.unary(op, HostView.contig(xin), 0.0, path)
    assert C.digest(got) == C.digest(ref)


# ---- the reference's own known-answer tests (test/test_ops.cpp) -------------------------------------
def _full(shape, v):
    return HostView.contig(np.full(shape, v, np.float32))


def test_known_answers_arithmetic(oracle):          # test/test_ops.cpp:63-85
    a, b = _full((2, 2), 2.0), _full((2, 2), 3.0)
    assert np.all(oracle.binary(ol.ADD, a, b) == 5.0)
    assert np.all(oracle.binary(ol.SUB, b, a) == 1.0)
    assert np.all(oracle.binary(ol.MUL, a, b) == 6.0)
    np.testing.assert_allclose(oracle.binary(ol.DIV, a, b), 2.0 / 3.0, atol=1e-5)


def test_known_answers_reductions(oracle):           # test/test_ops.cpp:113-128
    t = HostView.contig(np.array([[1, 2], [3, 4]], np.float32))
    assert oracle.reduce(ol.SUM, t, -1)[0] == 10.0
    assert oracle.reduce(ol.MEAN, t, -1)[0] == 2.5
    assert oracle.reduce(ol.MAX, t, -1)[0] == 4.0


def test_known_answers_broadcast(oracle):            # test/test_ops.cpp:130-149
    out = oracle.binary(ol.ADD, _full((2, 2), 1.0), _full((1, 2), 2.0))
    assert out.shape == (2, 2) and np.all(out == 3.0)


def test_known_answers_int_truncation(oracle):       # test/test_ops.cpp:203-213 (1.5 -> 1, 2.5 -> 2)
    t = HostView.contig(np.array([3, 5], np.int32))
    assert list(oracle.unary(ol.DIV_S, t, 2.0)) == [1, 2]


def test_argmax_first_maximum(oracle):               # src/core/ops_dispatch.cpp:468 strict '>'
    t = HostView.contig(np.array([[5, 7, 7, 1]], np.float32))
    assert list(oracle.reduce(ol.ARGMAX, t, 1)) == [1]


def test_edge_semantics(oracle):
    x = HostView.contig(np.array([-100.0, 100.0, np.nan, np.inf], np.float32))
    e = oracle.unary(ol.EXP, x)
    assert e[0] == 0.0 and e[1] == e[2] == e[3] and 2.4e38 < e[1] < 2.41e38      # clamp, NaN -> HI
    assert oracle.unary(ol.TANH, HostView.contig(np.array([np.nan], np.float32)))[0] == 1.0
    r = oracle.unary(ol.RELU, HostView.contig(np.array([np.nan, -0.0], np.float32)))
    assert r.view(np.uint32).tolist() == [0, 0]                                   # NaN -> 0, -0 -> +0
    lg = oracle.unary(ol.LOG, HostView.contig(np.array([0.0, -1.0, 1.5], np.float32)))
    assert lg.view(np.uint32)[0] == 0xFFFFFFFF and lg.view(np.uint32)[1] == 0xFFFFFFFF
    assert abs(lg[2] - 0.405465) < 1e-6
    d = oracle.binary(ol.ADD, HostView.contig(np.array([1e-40], np.float32)), HostView.contig(np.array([1e-40], np.float32)))
    assert d[0] != 0.0                                                            # denormals are kept
