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
