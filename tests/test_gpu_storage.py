"""GPU tests of the device allocators behind Storage::allocate: the stream-ordered ctb_alloc /
ctb_free pair and the pool of managed (host-dereferenceable) blocks the C++ host layers use."""
import ctypes

import numpy as np
import pytest
import torch

import oracle_lib as ol
from oracle_lib import HostView

pytestmark = pytest.mark.gpu


def test_stream_ordered_alloc_feeds_the_kernels(ct, oracle):
    """ctb_alloc'ed buffers as operands: upload, add on the stream, download; zero = 1 clears."""
    L = ct.lib()
    n = 1 << 20
    rng = np.random.default_rng(5)
    a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    ptrs = [ctypes.c_void_p() for _ in range(4)]
    stream = torch.cuda.current_stream().cuda_stream
    for p, zero in zip(ptrs, (0, 0, 0, 1)):
        ct.check(L.ctb_alloc(ctypes.byref(p), n * 4, zero, stream))
    # data moves between torch-held memory and the allocated buffers through the library's own copy
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    va, vb, vo, vz = (ct.make_view(p.value, ct.F32, (n,), (1,)) for p in ptrs)
    ct.check(L.ctb_copy_strided(ct.DView.of(da).cview(), va, stream))
    ct.check(L.ctb_copy_strided(ct.DView.of(db).cview(), vb, stream))
    ct.check(L.ctb_binary(ct.ADD, va, vb, vo, stream))
    res, zer = torch.empty(n, device="cuda"), torch.ones(n, device="cuda")
    ct.check(L.ctb_copy_strided(vo, ct.DView.of(res).cview(), stream))
    ct.check(L.ctb_copy_strided(vz, ct.DView.of(zer).cview(), stream))
    ct.check(L.ctb_sync(stream))
    out, zeros = res.cpu().numpy(), zer.cpu().numpy()
    assert np.array_equal(out.view(np.uint32), oracle.binary(ol.ADD, HostView.contig(a), HostView.contig(b)).view(np.uint32))
    assert not zeros.any()
    for p in ptrs:
        ct.check(L.ctb_free(p, stream))
    ct.check(L.ctb_sync(stream))


def test_managed_pool_reuses_blocks_and_is_host_dereferenceable(ct):
    L = ct.lib()
    dev = torch.cuda.current_device()
    ct.check(L.ctb_pool_trim(dev))
    info = ct.PoolInfo()
    ct.check(L.ctb_pool_stats(dev, ctypes.byref(info)))
    base_hits, base_misses, base_live = info.hits, info.misses, info.live_bytes

    p = ctypes.c_void_p()
    ct.check(L.ctb_pool_alloc_managed(ctypes.byref(p), 1000, 1, dev, None))
    ct.check(L.ctb_sync(None))
    host_view = (ctypes.c_float * 250).from_address(p.value)                     # the host reads managed memory
    assert all(v == 0.0 for v in host_view)
    host_view[3] = 7.5                                                           # and writes it
    x = ct.make_view(p.value, ct.F32, (250,), (1,))
    q = ctypes.c_void_p()
    ct.check(L.ctb_pool_alloc_managed(ctypes.byref(q), 1000, 0, dev, None))
    assert q.value != p.value
    ct.check(L.ctb_unary(ct.MUL_S, x, 2.0, ct.make_view(q.value, ct.F32, (250,), (1,)), None))
    ct.check(L.ctb_sync(None))
    assert (ctypes.c_float * 250).from_address(q.value)[3] == 15.0               # the kernel saw the host's write

    first = p.value
    ct.check(L.ctb_pool_free_managed(p))
    ct.check(L.ctb_pool_stats(dev, ctypes.byref(info)))
    assert info.cached_blocks >= 1 and info.cached_bytes >= 1024                 # rounded to 512-byte units
    r = ctypes.c_void_p()
    ct.check(L.ctb_pool_alloc_managed(ctypes.byref(r), 900, 0, dev, None))       # same 1024-byte class: reused
    assert r.value == first
    ct.check(L.ctb_pool_stats(dev, ctypes.byref(info)))
    assert info.hits == base_hits + 1 and info.misses == base_misses + 2
    ct.check(L.ctb_pool_free_managed(q))
    ct.check(L.ctb_pool_free_managed(r))
    assert L.ctb_pool_free_managed(ctypes.c_void_p(12345)) == 5                   # not a block of the pool
    ct.check(L.ctb_pool_set_limit(dev, 0))                                       # nothing may stay cached
    ct.check(L.ctb_pool_stats(dev, ctypes.byref(info)))
    assert info.cached_bytes == 0 and info.live_bytes == base_live
    ct.check(L.ctb_pool_set_limit(dev, 64 << 30))


def test_large_managed_blocks_run_at_device_speed_once_resident(ct):
    """A 1 GiB managed tensor from the pool, prefetched: the add kernel reads and writes it in HBM."""
    L = ct.lib()
    dev = torch.cuda.current_device()
    n = 1 << 28
    ptrs = [ctypes.c_void_p() for _ in range(3)]
    for p in ptrs:
        ct.check(L.ctb_pool_alloc_managed(ctypes.byref(p), n * 4, 1, dev, None))
        ct.check(L.ctb_prefetch_managed(p, n * 4, dev, None))
    va, vb, vo = (ct.make_view(p.value, ct.F32, (n,), (1,)) for p in ptrs)
    for _ in range(3):
        ct.check(L.ctb_binary(ct.ADD, va, vb, vo, None))
    ct.check(L.ctb_sync(None))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    legacy = torch.cuda.ExternalStream(0)
    e0.record(legacy)
    for _ in range(5):
        ct.check(L.ctb_binary(ct.ADD, va, vb, vo, None))
    e1.record(legacy)
    torch.cuda.synchronize()
    gbs = 12 * n * 5 / e0.elapsed_time(e1) / 1e6
    for p in ptrs:
        ct.check(L.ctb_pool_free_managed(p))
    ct.check(L.ctb_pool_trim(dev))
    assert gbs > 3000, f"managed operands ran at {gbs:.0f} GB/s"
