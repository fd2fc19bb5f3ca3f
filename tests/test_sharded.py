"""Host-side logic of the multi-GPU path, run as two gloo ranks on the CPU: shard bookkeeping
and the partial -> all-reduce -> finalise sequence (the per-shard arithmetic is replaced by
numpy stand-ins; the GPU arithmetic itself is covered by the -m gpu tests)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import ctensor_b200 as ct                      # noqa: E402
from ctensor_b200 import sharded               # noqa: E402


def test_shard_ranges_partition_the_dim():
    for n in (0, 1, 7, 8, 1000, 2 ** 31):
        for world in (1, 2, 3, 8):
            ranges = [sharded.shard_range(n, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            for (a, b), (c, d) in zip(ranges, ranges[1:]):
                assert b == c and b - a >= d - c >= b - a - 1
    with pytest.raises(ValueError):
        sharded.shard_range(10, 2, 2)


def _host_partial(op, x):
    x64 = x.double()
    v = {ct.SUM: x64.sum(), ct.MEAN: x64.sum(), ct.MAX: x64.max(), ct.MIN: x64.min()}[op]
    return v.reshape(1)


def _host_finalize(op, partial, total):
    s = partial.float()
    if op == ct.MEAN:
        s = (s.double() * (1.0 / total)).float()
    return s


def _worker(rank, world, port, n, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.from_numpy(np.random.default_rng(3).standard_normal(n).astype(np.float32))
        local = sharded.shard_of(full, world, rank)
        out = {}
        for op in (ct.SUM, ct.MEAN, ct.MAX, ct.MIN):
            r = sharded.full_reduce(op, local, n, partial_fn=_host_partial, finalize_fn=_host_finalize)
            out[op] = float(r.item())
        m = full.view(-1, 8)
        part = sharded.dim0_reduce(ct.SUM, sharded.shard_of(m, world, rank), m.shape[0],
                                   partial_fn=lambda o, x: x.double().sum(0))
        out["dim0"] = part.tolist()
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("n", [4096, 8])
def test_full_reduce_two_ranks_gloo(n):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    full = np.random.default_rng(3).standard_normal(n).astype(np.float32)
    s32 = np.float32(full.astype(np.float64).sum())
    want = {ct.SUM: float(s32), ct.MEAN: float(np.float32(np.float64(s32) * (1.0 / n))),
            ct.MAX: float(full.max()), ct.MIN: float(full.min())}
    for r in range(world):
        for op, v in want.items():
            assert results[r][op] == pytest.approx(v, rel=1e-6), (r, op)
        np.testing.assert_allclose(results[r]["dim0"], full.reshape(-1, 8).astype(np.float64).sum(0), rtol=1e-12)
    assert results[0] == results[1]              # every rank holds the same values


def test_empty_shard_contributes_identity():
    t = torch.zeros(0)
    assert sharded.full_reduce(ct.MAX, t, 0, partial_fn=_host_partial,
                               finalize_fn=lambda op, p, n: p).item() == float("-inf")


# ---- the C ABI's own multi-GPU entry points (single process) --------------------------------------------
def test_c_abi_shard_ranges_match_the_python_ones():
    import ctypes
    L = ct.lib()
    lo, hi = ctypes.c_int64(), ctypes.c_int64()
    for n in (0, 1, 7, 8, 1000, 2 ** 31 + 5):
        for parts in (1, 2, 3, 8):
            for r in range(parts):
                assert L.ctb_shard_range(n, parts, r, ctypes.byref(lo), ctypes.byref(hi)) == 0
                assert (lo.value, hi.value) == sharded.shard_range(n, parts, r)
    assert L.ctb_shard_range(10, 2, 2, ctypes.byref(lo), ctypes.byref(hi)) == 5
    assert L.ctb_shard_range(10, 0, 0, ctypes.byref(lo), ctypes.byref(hi)) == 5
    assert L.ctb_shard_range(10, 2, 0, None, ctypes.byref(hi)) == 1


def test_c_abi_collectives_need_a_communicator_and_a_gpu():
    import ctypes
    L = ct.lib()
    assert L.ctb_comm_size() == 0
    bufs = (ctypes.c_void_p * 1)(None)
    assert L.ctb_allreduce(bufs, 4, ct.F64, ct.SUM) == 5
    assert b"no communicator" in L.ctb_last_error()
    assert L.ctb_comm_sync() == 5
    assert L.ctb_comm_destroy() == 0                       # nothing to destroy is not an error
    if L.ctb_device_count() == 0:
        assert L.ctb_comm_init_all(2, None) == 6           # CTB_ERR_CUDA: no CPU fallback
        assert b"no CUDA device" in L.ctb_last_error()


def _c_abi_sharded_reduce(ndev, oracle):
    """ctb_comm_init_all over `ndev` GPUs; a tensor sharded along dim 0 across them."""
    import ctypes
    import oracle_lib as ol
    from oracle_lib import HostView
    L = ct.lib()
    ct.check(L.ctb_comm_init_all(ndev, None))
    try:
        assert L.ctb_comm_size() == ndev
        n = (1 << 22) + 11
        x = (np.random.default_rng(8).standard_normal(n) * 2 + 0.1).astype(np.float32)
        shards, outs = [], []
        for r in range(ndev):
            lo, hi = sharded.shard_range(n, ndev, r)
            dev = L.ctb_comm_device(r)
            shards.append(torch.from_numpy(x[lo:hi]).to(f"cuda:{dev}"))
            outs.append(torch.empty(1, device=f"cuda:{dev}"))
        torch.cuda.synchronize()
        vp = ctypes.POINTER(ct.View)
        for op in (ct.SUM, ct.MEAN, ct.MAX, ct.MIN):
            sv = [ct.DView.of(s).cview() for s in shards]
            ov = [ct.DView.of(o).cview() for o in outs]
            ct.check(L.ctb_full_reduce_sharded(op, (vp * ndev)(*[ctypes.pointer(v) for v in sv]), n,
                                               (vp * ndev)(*[ctypes.pointer(v) for v in ov])))
            ref = oracle.reduce(op, HostView.contig(x), -1)
            for o in outs:                                   # every GPU holds the same, correct value
                if op in (ct.MAX, ct.MIN):
                    assert o.cpu().numpy().view(np.uint32)[0] == ref.view(np.uint32)[0]
                else:
                    np.testing.assert_allclose(o.cpu().numpy(), ref, rtol=1e-5)
            assert all(torch.equal(outs[0].cpu(), o.cpu()) for o in outs)
        # a dim-0 reduction of row shards: fp64 partial rows, one all-reduce of 4096 doubles
        m = x[: 1 << 22].reshape(-1, 4096)
        parts = []
        for r in range(ndev):
            lo, hi = sharded.shard_range(m.shape[0], ndev, r)
            dev = L.ctb_comm_device(r)
            parts.append(torch.from_numpy(m[lo:hi].astype(np.float64).sum(0)).to(f"cuda:{dev}"))
        torch.cuda.synchronize()
        ptrs = (ctypes.c_void_p * ndev)(*[p.data_ptr() for p in parts])
        ct.check(L.ctb_allreduce(ptrs, 4096, ct.F64, ct.SUM))
        ct.check(L.ctb_comm_sync())
        for p in parts:
            np.testing.assert_allclose(p.cpu().numpy(), m.astype(np.float64).sum(0), rtol=1e-12)
    finally:
        ct.check(L.ctb_comm_destroy())
    assert L.ctb_comm_size() == 0


@pytest.mark.gpu
def test_c_abi_sharded_full_reduce_on_one_gpu(oracle):
    _c_abi_sharded_reduce(1, oracle)


@pytest.mark.gpu
def test_c_abi_sharded_full_reduce_on_all_gpus(oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    _c_abi_sharded_reduce(torch.cuda.device_count(), oracle)
