"""GPU test of ctb_reduce_dim_noalloc, the dim-wise reduction for callers that cannot allocate
device memory (allocator callbacks, processes whose device memory is fully budgeted up front).
Its scratch is a fixed array inside the library instead of the cudaMalloc'ed workspace, so its
results must equal ctb_reduce's bit for bit — on the first call and on the next one, which
finds the previous call's leftovers in that array.  Collected last on purpose: a failure here
cannot hide the rest of the suite behind `pytest -x`."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.cpu().numpy().view(np.uint32)


def test_noalloc_reduction_matches_regular_entry_point(ct):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    x = torch.randn(4096, 2048, device="cuda", generator=gen)       # dim 0: split column kernel (uses scratch)
    y = torch.randn(3000, 1000, device="cuda", generator=gen) * 3 + 1
    assert ct.reduce_workspace_bytes(x, 0) > 0                      # the case really exercises the scratch
    for t in (x, y):
        for op in (ct.SUM, ct.MEAN, ct.MAX, ct.MIN, ct.VAR, ct.ARGMAX):
            want = ct.reduce(op, t, 0)
            for call in range(2):                                   # second call reuses the dirty array
                got = torch.empty_like(want)
                ct.reduce_dim_noalloc(op, t, 0, got)
                assert np.array_equal(_bits(got), _bits(want)), (op, tuple(t.shape), call)
    # shapes that need no scratch go through the same entry point
    want = ct.reduce(ct.SUM, x, 1)
    got = torch.empty_like(want)
    ct.reduce_dim_noalloc(ct.SUM, x, 1, got)
    assert np.array_equal(_bits(got), _bits(want))


def test_noalloc_reduction_matches_the_cpu_oracle(ct, oracle):
    """The entry point against the CPU restatement of the reference directly (not only against the
    regular entry point): exact for max/min/argmax, 1e-5 relative for the sums; signed zeros included."""
    import oracle_lib as ol
    from oracle_lib import HostView
    from gpu_util import to_device, assert_bits_equal, assert_close
    rng = np.random.default_rng(12)
    x = rng.standard_normal((4096, 640)).astype(np.float32)
    x[rng.integers(0, 4096, 500), rng.integers(0, 640, 500)] = 0.0
    x[rng.integers(0, 4096, 500), rng.integers(0, 640, 500)] = -0.0
    z = np.minimum(x, 0.0).astype(np.float32)                      # column maxima are zeros of either sign
    for arr in (x, z):
        h = HostView.contig(arr)
        d = to_device(h)
        assert ct.reduce_workspace_bytes(d, 0) > 0
        for op in (ol.SUM, ol.MEAN, ol.MAX, ol.MIN, ol.VAR, ol.ARGMAX):
            ref = oracle.reduce(op, h, 0)
            for call in range(2):
                got = torch.empty(ref.shape, dtype=torch.int32 if op == ol.ARGMAX else torch.float32, device="cuda")
                ct.reduce_dim_noalloc(op, d, 0, got)
                if op in (ol.MAX, ol.MIN, ol.ARGMAX):
                    assert_bits_equal(got, ref, f"op {op} call {call}")
                else:
                    assert_close(got, ref, 1e-5, f"op {op} call {call}")


def test_noalloc_reduction_rejects_what_does_not_fit(ct):
    wide = torch.zeros(256, 131072, device="cuda")                  # needs ~6 MiB of partials
    assert ct.reduce_workspace_bytes(wide, 0) > ct.NOALLOC_SCRATCH_BYTES
    out = torch.empty(131072, device="cuda")
    with pytest.raises(ct.CtbError) as e:
        ct.reduce_dim_noalloc(ct.SUM, wide, 0, out)
    assert e.value.code == 8 and "fixed buffer holds" in e.value.message
    with pytest.raises(ct.CtbError) as e:
        ct.reduce_dim_noalloc(ct.SUM, wide, -1, torch.empty(1, device="cuda"))
    assert e.value.code == 4
