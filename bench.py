#!/usr/bin/env python
"""Benchmark of the elementwise operator path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (the "large contiguous fp32 bandwidth sweep" configuration): 1-d fp32 tensors x, y of
n = 2^30 elements per GPU drawn N(0,1) from a seed; one step = add(x,y), mul(x,y), exp(x),
relu(x), gelu(x) through the C ABI, i.e. 2 x 12n + 3 x 8n = 48n algorithmic bytes per GPU per
step.  Every rank owns one shard of a leading-dim split (no data-path collective), so the
per-GPU work is fixed as N grows ("weak"); `--scaling strong` keeps the total at 2^30 instead.

Keys beyond the base contract:
  roofline      the kernel with the largest share of the step, timed per launch with CUDA events
                inside the timed region, against the measured HBM copy bandwidth
  cpu_baseline  the reference's own CPU code (oracle/_ref) timed on this box's host cores on a
                bounded sample (N=1, rank 0 only)
  e2e           the same step through the host-buffer entry points (pinned host memory in,
                pinned host memory out, copies inside the timed region)
  per_op        GB/s of every op of the step
  sweep         GB/s at the other sizes of the configuration (2^20, 2^24, 2^28), N=1 only
  other_configs GB/s (algorithmic bytes / CUDA-event time, 20 back-to-back launches) of the
                reduction, permuted-softmax-chain and GPT-2 non-GEMM configurations, N=1 only
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

OPS = [("add", "binary", 12), ("mul", "binary", 12), ("exp", "unary", 8), ("relu", "unary", 8),
       ("gelu", "unary", 8)]
BYTES_PER_ELEM_STEP = sum(b for _, _, b in OPS)          # 48
DRAM_BYTES_PER_ELEMENT = {"add": 11.35, "mul": 11.35, "exp": 7.20, "relu": 7.20, "gelu": 7.29}   # ncu, small case
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def wait_first_sample(self, timeout=5.0):
        """nvidia-smi needs a moment to start on a fresh box: do not enter the timed region blind."""
        t_end = time.monotonic() + timeout
        while self.proc is not None and not self.rows and time.monotonic() < t_end:
            time.sleep(0.01)

    def samples_between(self, t0, t1):
        return sum(1 for t, _ in self.rows if t0 <= t <= t1)

    def stop(self, t0=None, t1=None):
        """Statistics over the samples that arrived in [t0, t1] (host clock; every sample when
        no window is given)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [r for t, r in self.rows if (t0 is None or t >= t0) and (t1 is None or t <= t1)]
        for r in rows:
            try:
                sm.append(float(r[0]))
                smax = float(r[1])
                for nme, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(nme)
            except Exception:
                pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "samples": len(sm),
                "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------
def run_step(ct, x, y, out, events=None):
    """The five ops of one step; `events` (list of (start, end) pairs) times each launch."""
    import torch
    calls = [lambda: ct.binary(ct.ADD, x, y, out=out), lambda: ct.binary(ct.MUL, x, y, out=out),
             lambda: ct.unary(ct.EXP, x, out=out), lambda: ct.unary(ct.RELU, x, out=out),
             lambda: ct.unary(ct.GELU_TANH, x, out=out)]
    for i, c in enumerate(calls):
        if events is not None:
            events[i][0].record()
        c()
        if events is not None:
            events[i][1].record()


def run_step_host(ct, hx, hy, hout, device):
    ct.binary_host(ct.ADD, hx, hy, hout, device)
    ct.binary_host(ct.MUL, hx, hy, hout, device)
    ct.unary_host(ct.EXP, hx, hout, 0.0, device)
    ct.unary_host(ct.RELU, hx, hout, 0.0, device)
    ct.unary_host(ct.GELU_TANH, hx, hout, 0.0, device)


def mem_available_bytes():
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemAvailable"):
                return int(line.split()[1]) * 1024
    except Exception:
        pass
    return 0


def bench_ours(args):
    import torch
    import torch.distributed as dist
    import ctensor_b200 as ct

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ct.lib()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    n_total = args.n * world if args.scaling == "weak" else args.n
    n = n_total // world                                  # this rank's shard of the leading dim
    gen = torch.Generator(device=dev)
    gen.manual_seed(1 + rank)                             # shard i of the seeded tensor
    x = torch.randn(n, device=dev, generator=gen)
    y = torch.randn(n, device=dev, generator=gen)
    out = torch.empty(n, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        run_step(ct, x, y, out)
    barrier()
    if rank == 0:
        sampler.wait_first_sample()
    barrier()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in OPS]
          for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_host0 = time.monotonic()
    e0.record()
    for k in range(args.steps):
        run_step(ct, x, y, out, ev[k])
    e1.record()
    barrier()
    t_host1 = time.monotonic()
    clocks = None
    if rank == 0:
        window = "timed region"
        if sampler.samples_between(t_host0, t_host1) < 3:
            # a short timed region (few steps) gives the 20 ms sampler too little: keep the same
            # kernels running, untimed, until there are samples under load
            t_more = time.monotonic() + 0.6
            while time.monotonic() < t_more:
                run_step(ct, x, y, out)
                torch.cuda.synchronize()
            t_host1 = time.monotonic()
            window = "timed region + 0.6 s of the same step, untimed"
        clocks = sampler.stop(t_host0, t_host1)
        clocks["window"] = window
    barrier()
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / args.steps

    # per-op launch durations (max over ranks of the mean over steps)
    per_op_ms = torch.tensor([sum(ev[k][i][0].elapsed_time(ev[k][i][1]) for k in range(args.steps)) / args.steps
                              for i in range(len(OPS))], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(per_op_ms, op=dist.ReduceOp.MAX)
    per_op_ms = per_op_ms.tolist()

    # ---- end to end through the host-buffer entry points --------------------------------------------
    e2e = None
    try:
        if args.kernel_only:
            raise RuntimeError("skipped (--kernel-only)")
        n_e2e = n
        need = 3 * 4 * n_e2e * max(world, 1)
        avail = mem_available_bytes()
        while n_e2e > (1 << 24) and avail and need * 3 > avail:
            n_e2e //= 2
            need //= 2
        n_e2e = min(n_e2e, args.e2e_n) if args.e2e_n else n_e2e
        hx = torch.empty(n_e2e, dtype=torch.float32).pin_memory()
        hy = torch.empty(n_e2e, dtype=torch.float32).pin_memory()
        hout = torch.empty(n_e2e, dtype=torch.float32).pin_memory()
        hx.copy_(x[:n_e2e])
        hy.copy_(y[:n_e2e])
        run_step_host(ct, hx, hy, hout, local)            # warm-up (allocates the staging buffers)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            run_step_host(ct, hx, hy, hout, local)
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        sec = float(dt.item()) / args.e2e_steps
        e2e = {"value": round(BYTES_PER_ELEM_STEP * n_e2e * world / sec / 1e9, 2), "unit": "GB/s",
               "h2d_bytes_per_step": 28 * n_e2e, "d2h_bytes_per_step": 20 * n_e2e,
               "elements_per_gpu": n_e2e, "ms_per_step": round(sec * 1e3, 3),
               "note": "ctb_binary_host/ctb_unary_host on pinned host buffers; every op uploads its "
                       "inputs and downloads its result (chunked, copies overlap the kernels)"}
        del hx, hy, hout
    except Exception as exc:                               # report, do not hide
        e2e = {"value": None, "unit": "GB/s", "error": repr(exc)}

    # ---- the one op with an exchange step: full-tensor sum of a sharded tensor ----------------------
    # (2^28 elements per GPU; local fp64 partial on the GPU, one NCCL all-reduce of a double, finalise)
    sharded_sum = None
    try:
        if args.kernel_only:
            raise RuntimeError("skipped (--kernel-only)")
        from ctensor_b200 import sharded
        m = min(n, 1 << 28)
        xs = x[:m]
        for _ in range(3):
            sharded.full_reduce(ct.SUM, xs, m * world)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 20
        s0.record()
        for _ in range(reps):
            res = sharded.full_reduce(ct.SUM, xs, m * world)
        s1.record()
        barrier()
        tt = torch.tensor([s0.elapsed_time(s1) / reps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        # the value, checked: an fp64 sum of the same shard computed independently (torch), all-reduced
        chk = xs.double().sum().reshape(1)
        if world > 1:
            dist.all_reduce(chk)
        want = float(chk.item())
        got = float(res.item())
        checked = abs(got - want) <= 1e-5 * max(abs(want), (m * world) ** 0.5)
        # eight such sums whose partials share ONE all-reduce (the ~20 us collective amortised)
        parts = torch.empty(8, dtype=torch.float64, device=dev)
        chunks = xs.view(8, -1)

        def batched():
            for i in range(8):
                ct.reduce_full_partial(ct.SUM, chunks[i], partial=parts[i:i + 1])
            if world > 1:
                dist.all_reduce(parts)
            return parts

        for _ in range(3):
            batched()
        barrier()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(reps):
            batched()
        b1.record()
        barrier()
        bt = torch.tensor([b0.elapsed_time(b1) / reps], device=dev, dtype=torch.float64)
        # the collective alone
        one = torch.zeros(1, dtype=torch.float64, device=dev)
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            for _ in range(3):
                dist.all_reduce(one)
        barrier()
        c0.record()
        if world > 1:
            for _ in range(reps):
                dist.all_reduce(one)
        c1.record()
        barrier()
        ctm = torch.tensor([c0.elapsed_time(c1) / reps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(bt, op=dist.ReduceOp.MAX)
            dist.all_reduce(ctm, op=dist.ReduceOp.MAX)
        sharded_sum = {"elements_per_gpu": m, "ms": round(float(tt.item()), 4),
                       "GB/s": round(4.0 * m * world / float(tt.item()) / 1e6, 1), "value": got,
                       "checked": bool(checked), "check": "fp64 sum of the same shards computed by torch, all-reduced; 1e-5 relative",
                       "allreduce_one_fp64_ms": round(float(ctm.item()), 4),
                       "eight_sums_one_allreduce": {"ms": round(float(bt.item()), 4),
                                                    "GB/s": round(4.0 * m * world / float(bt.item()) / 1e6, 1)},
                       "collective": "none (1 rank)" if world == 1 else "1 all-reduce of one fp64 (NCCL)"}
    except Exception as exc:
        sharded_sum = {"error": repr(exc)}

    # ---- the other configurations on row shards, every N (strong scaling: the config's size is fixed) ----
    sharded_cfgs = None
    if not args.kernel_only:
        try:
            sharded_cfgs = sharded_configs(ct, torch, dist, dev, rank, world, x, y, out)
        except Exception as exc:
            sharded_cfgs = {"error": repr(exc)}

    # ---- extras on rank 0 ------------------------------------------------------------------------------
    sweep, cpu, other = None, None, None
    if world == 1 and not args.kernel_only:
        sweep = {}
        for lg in (20, 24, 28):
            m = 1 << lg
            if m >= n:
                continue
            reps = 8 if lg >= 28 else 50
            res = {}
            # rotate over distinct slices so the small sizes are not served from L2
            nslices = max(1, min(n // m, (1 << 30) // (4 * m) * 3))
            # ready-made views of the slices: at these sizes the launches are host-bound
            sl = [tuple(ct.DView.of(t[i * m:(i + 1) * m]) for t in (x, y, out)) for i in range(nslices)]
            for (name, kind, bpe), fn in zip(OPS, (
                    lambda a, b, o: ct.binary(ct.ADD, a, b, out=o), lambda a, b, o: ct.binary(ct.MUL, a, b, out=o),
                    lambda a, b, o: ct.unary(ct.EXP, a, out=o), lambda a, b, o: ct.unary(ct.RELU, a, out=o),
                    lambda a, b, o: ct.unary(ct.GELU_TANH, a, out=o))):
                for r in range(3):
                    fn(*sl[r % nslices])
                torch.cuda.synchronize()
                windows = []                 # median of three windows: one host hiccup in a
                for _ in range(3):           # 1 ms window otherwise halves the figure
                    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a0.record()
                    for r in range(reps):
                        fn(*sl[r % nslices])
                    a1.record()
                    torch.cuda.synchronize()
                    windows.append(a0.elapsed_time(a1))
                res[name] = round(bpe * m * reps / sorted(windows)[1] / 1e6, 1)
            sweep[f"2^{lg}"] = res
        del x, y, out
        try:
            other = other_configs(ct, torch, dev)
        except Exception as exc:                      # never lose the headline line to an extra
            other = {"error": repr(exc)}
        if not args.no_cpu_baseline:
            cpu = cpu_baseline(sample_log2=args.cpu_log2)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peak()
    top = max(range(len(OPS)), key=lambda i: per_op_ms[i])
    ach = OPS[top][2] * n / per_op_ms[top] / 1e6
    value = BYTES_PER_ELEM_STEP * n * world / ms_per_step / 1e6
    line = {
        "metric": "op GB/s and % of 8 TB/s HBM peak at 1/2/4/8 B200 vs host-CPU reference",
        "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"contiguous fp32 sweep, n=2^{n.bit_length() - 1} elements per GPU: add, mul, exp, relu, "
                               "gelu(tanh) of N(0,1) tensors, sharded along dim 0",
                   "elements_per_gpu": n, "elements_total": n * world, "parallelism": f"dp{world}",
                   "algorithmic_bytes_per_step_per_gpu": BYTES_PER_ELEM_STEP * n,
                   "l2": "inputs (4 GiB per tensor and GPU) exceed the 126 MB L2; no flush needed"},
        "elements_per_s": round(5 * n * world / (ms_per_step * 1e-3), 1),
        "pct_of_8TBs_per_gpu": round(100 * value / world / NOMINAL_HBM_GBS, 2),
        "per_op": {OPS[i][0]: {"ms": round(per_op_ms[i], 4), "GB/s": round(OPS[i][2] * n / per_op_ms[i] / 1e6, 1)}
                   for i in range(len(OPS))},
        "roofline": {"bound": "hbm", "kernel": f"ew_flat_kernel<{OPS[top][0]}>", "achieved": round(ach, 1),
                     "peak": peak, "peak_kind": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650",
                     "unit": "GB/s", "frac": round(ach / peak, 4), "frac_of_8TBs": round(ach / NOMINAL_HBM_GBS, 4),
                     "traffic": None},
        "clocks": clocks, "e2e": e2e, "gpu_launches": 5 * args.steps * world,
    }
    line["sharded_full_sum"] = sharded_sum
    if sharded_cfgs is not None:
        line["sharded_configs"] = sharded_cfgs
    if world == 1 and not args.kernel_only:
        line["host_layer"] = host_layer_bench()
    if sweep is not None:
        line["sweep"] = sweep
    if other is not None:
        line["other_configs"] = other
    if cpu is not None:
        line["cpu_baseline"] = cpu
    # DRAM bytes per element from the ncu capture of the small case (n = 2^26), see
    # profiles/ew_flat_small_case_full_set.md; traffic grows in proportion to n.
    line["roofline"]["traffic"] = round(DRAM_BYTES_PER_ELEMENT[OPS[top][0]] * n)
    line["roofline"]["traffic_source"] = "ncu capture of the n=2^26 case (DRAM read+write bytes per element) x n, not a counter read in this run"
    _emit(line)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------
def host_layer_bench():
    """The C++ host layer (the drop-in path of a caller of the reference) timed by its own program:
    `a + b`, relu(a), sum(a, 1) on pooled managed tensors, output allocation and the wait for the
    kernel inside every call.  us per call and GB/s at 2^20 / 2^24 / 2^28 elements."""
    exe = os.path.join(ROOT, "ctensor_b200", "host", "bench_host_layer.bin")
    if not os.path.exists(exe):
        return {"error": "ctensor_b200/host/bench_host_layer.bin not built"}
    try:
        r = subprocess.run([exe, "20", "24", "28"], capture_output=True, text=True, timeout=300)
        res = json.loads(r.stdout.strip().splitlines()[-1])
    except Exception as exc:
        return {"error": repr(exc)}
    res["train_step"] = train_step_bench()
    res["reference_time_avx"] = reference_timing_program()
    return res


def reference_timing_program():
    """The reference's own timing program (test/time_avx.cpp: 100 x add_mp, then 100 x add, of two
    1000 x 1000 tensors), built unchanged over the host layer and against the reference itself; seconds
    for the 100 calls as the program prints them."""
    import re
    out = {}
    for name, exe in (("b200", os.path.join(ROOT, "tests", "cpp", "_built", "reference_time_avx_b200")),
                      ("reference_cpu", os.path.join(ROOT, "oracle", "_ref", "time_avx_gen2_ref"))):
        if not os.path.exists(exe):
            out[name] = "not built"
            continue
        try:
            subprocess.run([exe], capture_output=True, text=True, timeout=120)          # first run: page faults, pool
            r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
            t = re.findall(r"100 (\w+) additions of 1000x1000 tensors: ([-+.eE0-9]+) seconds", r.stdout)
            out[name] = ({("add_mp_100_calls_s" if k == "Scalar" else "add_100_calls_s"): float(v) for k, v in t}
                         or {"error": (r.stdout + r.stderr)[-200:]})
        except Exception as exc:
            out[name] = {"error": repr(exc)}
    out["note"] = ("the program times its first loop (add_mp) from a cold start: on the GPU build that loop contains the "
                   "one-time load of the elementwise kernel module (about 0.1 s, measured: first call 100 ms, later calls "
                   "13 us); the second loop (add) is the steady state")
    return out


def train_step_bench():
    """A training step as a user of the reference writes it (two Linear layers, relu, CrossEntropy,
    backward, SGD from train_utils.h; tests/cpp/train_step_program.cpp), ms per step:
      drop_in       the reference's autograd.cpp / layer.cpp / loss.cpp unchanged over the host layer —
                    their host loops (accumulate_grad, the memset of ensure_grad_buffer, the loop of
                    GradCrossEntropy) pull every gradient buffer across PCIe and back
      three_edits   the three bodies replaced by calls of the host layer, as the integration notes describe
      three_edits_tensor_cores   the same with matmul on the tensor cores (TF32 products)
      four_edits_tensor_cores    the same with the body of Loss::CrossEntropy replaced by one host-layer call as well
      reference_cpu the same program linked with the reference itself (scalar back-end, host cores)
    The programs are built where the reference's sources are; absent binaries are reported as such."""
    built = os.path.join(ROOT, "tests", "cpp", "_built")
    runs = {"drop_in": (os.path.join(built, "train_step_gen2_b200"), {}),
            "three_edits": (os.path.join(built, "train_step_gen2_b200_edited"), {}),
            "three_edits_tensor_cores": (os.path.join(built, "train_step_gen2_b200_edited"), {"CTB_HOST_MATMUL_TENSOR_CORES": "1"}),
            "four_edits_tensor_cores": (os.path.join(built, "train_step_gen2_b200_edited4"), {"CTB_HOST_MATMUL_TENSOR_CORES": "1"}),
            "reference_cpu": (os.path.join(ROOT, "oracle", "_ref", "train_step_gen2_ref_scalar"), {})}
    out = {}
    for shape_name, argv in (("batch512_1024x1024x16", ["512", "1024", "1024", "16"]),
                             ("batch4096_4096x4096x1000", ["4096", "4096", "4096", "1000"])):
        row = {}
        for name, (exe, env) in runs.items():
            if name == "reference_cpu" and shape_name != "batch512_1024x1024x16":
                continue                                    # minutes per step on the host cores
            if not os.path.exists(exe):
                row[name] = "not built"
                continue
            try:
                steps = "3" if name == "reference_cpu" else "10"
                r = subprocess.run([exe] + argv + [steps], capture_output=True, text=True, timeout=300,
                                   env=dict(os.environ, **env))
                d = json.loads(r.stdout.strip().splitlines()[-1])
                row[name] = {k: d[k] for k in ("ms_per_step", "forward_ms", "loss_ms", "backward_ms", "optimizer_ms") if k in d}
            except Exception as exc:
                row[name] = {"error": repr(exc)}
        out[shape_name] = row
    return out


def sharded_configs(ct, torch, dist, dev, rank, world, x, y, out):
    """The reduction, permuted-softmax and GPT-2 configurations with their leading dim cut into
    `world` row shards (strong scaling: the configuration's size is fixed, each GPU owns 1/world of
    the rows), and the 2^30-element step cut the same way.  Row-wise work needs no communication;
    the dim-0 sum of the reduction matrix combines fp64 partial rows with one all-reduce of 16384
    doubles, timed on its own as well.  ms = max over ranks of the CUDA-event time per call."""
    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(reps):
            fn()
        a1.record()
        torch.cuda.synchronize()
        t = torch.tensor([a0.elapsed_time(a1) / reps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def entry(total_bytes, ms):
        return {"ms": round(ms, 4), "GB/s": round(total_bytes / ms / 1e6, 1)}

    res = {"scaling": "strong", "ranks": world}
    g = torch.Generator(device=dev)
    # the step itself on shards of ONE 2^30-element tensor pair
    n = x.numel() // world
    xs, ys, os_ = x[:n], y[:n], out[:n]
    res["step_2^30_total"] = entry(BYTES_PER_ELEM_STEP * n * world, timed(lambda: run_step(ct, xs, ys, os_), reps=5))
    # reductions: X[8192,16384], rows sharded
    rows = 8192 // world
    g.manual_seed(2 + 100 * rank)
    X = torch.randn(rows, 16384, device=dev, generator=g)
    r_rows = torch.empty(rows, device=dev)
    part = torch.empty(16384, dtype=torch.float64, device=dev)
    fin = torch.empty(16384, device=dev)

    def dim0_sum():
        # per-GPU fp64 partial rows -> one all-reduce -> rounding to fp32 (sum's finaliser)
        ct.reduce(ct.SUM, X, 0, out=fin)
        part.copy_(fin)                                  # stands for the fp64 partial rows of the shard
        if world > 1:
            dist.all_reduce(part)
        fin.copy_(part)

    nbX = 8192 * 16384 * 4
    V = ct.DView.of                 # ready-made views: the shards shrink with N and the launches become host-bound
    vX, vrows = V(X), V(r_rows)
    res["reductions_8192x16384"] = {
        "sum_dim1_row_shards": entry(nbX, timed(lambda: ct.reduce(ct.SUM, vX, 1, out=vrows))),
        "max_dim1_row_shards": entry(nbX, timed(lambda: ct.reduce(ct.MAX, vX, 1, out=vrows))),
        "var_dim1_row_shards": entry(nbX, timed(lambda: ct.reduce(ct.VAR, vX, 1, out=vrows))),
        "sum_dim0_row_shards_plus_allreduce": entry(nbX, timed(dim0_sum)),
        "allreduce_16384_fp64_ms": round(timed(lambda: dist.all_reduce(part) if world > 1 else None), 4),
    }
    del X, vX
    # permuted softmax chain: batch 32 sharded
    bsz = 32 // world
    g.manual_seed(4 + 100 * rank)
    buf = torch.randn(bsz, 1024, 12, 1024, device=dev, generator=g)
    S = buf.permute(0, 2, 1, 3)
    M = -torch.rand(1, 12, 1, 1024, device=dev, generator=g)
    O = torch.empty(bsz, 12, 1024, 1024, device=dev)
    nb = 32 * 1024 * 12 * 1024 * 4
    res["permuted_softmax_chain"] = {
        "S_plus_M": entry(2 * nb, timed(lambda: ct.binary(ct.ADD, S, M, out=O), reps=10)),
        "fused_chain_softmax_S_plus_M": entry(2 * nb, timed(lambda: ct.softmax(S, M, out=O), reps=10)),
    }
    del buf, S, O
    # GPT-2 small non-GEMM ops: batch 8 sharded
    b5 = max(8 // world, 1)
    g.manual_seed(6 + 100 * rank)
    hx = torch.randn(b5, 1024, 768, device=dev, generator=g)
    hr = torch.randn(b5, 1024, 768, device=dev, generator=g)
    gam, bet = torch.ones(768, device=dev), torch.zeros(768, device=dev)
    hh = torch.randn(b5, 1024, 3072, device=dev, generator=g)
    ha = torch.randn(b5, 12, 1024, 1024, device=dev, generator=g)
    ox, oh, oa = torch.empty_like(hx), torch.empty_like(hh), torch.empty_like(ha)
    tot = b5 * world
    hx, hr, gam, bet, hh, ha, ox, oh, oa = (V(t) for t in (hx, hr, gam, bet, hh, ha, ox, oh, oa))
    res["gpt2_small_non_gemm"] = {
        "residual_add": entry(3 * tot * 1024 * 768 * 4, timed(lambda: ct.binary(ct.ADD, hx, hr, out=ox))),
        "layernorm": entry(2 * tot * 1024 * 768 * 4, timed(lambda: ct.layernorm(hx, gam, bet, out=ox))),
        "gelu": entry(2 * tot * 1024 * 3072 * 4, timed(lambda: ct.unary(ct.GELU_TANH, hh, out=oh))),
        "causal_softmax": entry(2 * tot * 12 * 1024 * 1024 * 4, timed(lambda: ct.softmax(ha, None, True, out=oa))),
        "note": "per-GPU tensors shrink with N (3-48 MiB at N=8): launch-bound and L2-resident, reported not gated",
    }
    return res


def other_configs(ct, torch, dev):
    """GB/s of the other benchmark configurations on one GPU.  Bytes are the algorithmic bytes
    (each distinct input element read once, each output element written once); every kernel is
    timed over 20 back-to-back launches with CUDA events on tensors larger than L2 (the GPT-2
    layer-norm / residual tensors are 24 MiB and L2-resident: reported, not a bandwidth figure)."""
    def gbs(nbytes, fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(reps):
            fn()
        a1.record()
        torch.cuda.synchronize()
        return round(nbytes * reps / a0.elapsed_time(a1) / 1e6, 1)

    g = torch.Generator(device=dev)
    res = {}
    # every named op that is not in the timed step, on 2^28-element tensors (1 GiB each)
    n28 = 1 << 28
    g.manual_seed(1)
    xa = torch.randn(n28, device=dev, generator=g)
    xb = torch.randn(n28, device=dev, generator=g)
    xp = xa.abs() + 0.5                               # positive arguments for log
    o28 = torch.empty(n28, device=dev)
    o1 = torch.empty(1, device=dev)
    res["named_ops_2^28"] = {
        "sub": gbs(12 * n28, lambda: ct.binary(ct.SUB, xa, xb, out=o28)),
        "div": gbs(12 * n28, lambda: ct.binary(ct.DIV, xa, xb, out=o28)),
        "log": gbs(8 * n28, lambda: ct.unary(ct.LOG, xp, out=o28)),
        "tanh": gbs(8 * n28, lambda: ct.unary(ct.TANH, xa, out=o28)),
        "sum_full": gbs(4 * n28, lambda: ct.reduce(ct.SUM, xa, -1, out=o1)),
        "mean_full": gbs(4 * n28, lambda: ct.reduce(ct.MEAN, xa, -1, out=o1)),
        "max_full": gbs(4 * n28, lambda: ct.reduce(ct.MAX, xa, -1, out=o1)),
        "min_full": gbs(4 * n28, lambda: ct.reduce(ct.MIN, xa, -1, out=o1)),
        "var_full": gbs(4 * n28, lambda: ct.reduce(ct.VAR, xa, -1, out=o1)),
    }
    del xa, xb, xp, o28
    # the CPU-runnable configuration: A[1024,1024], B[1,1024] ~ U(-1,1), seed 0 (4 MiB: L2-resident and
    # launch-bound from Python; reported, not a bandwidth figure)
    g.manual_seed(0)
    A = torch.rand(1024, 1024, device=dev, generator=g) * 2 - 1
    B = torch.rand(1, 1024, device=dev, generator=g) * 2 - 1
    OA, r1k = torch.empty_like(A), torch.empty(1024, device=dev)
    den = ct.unary(ct.ADD_S, ct.unary(ct.ABS, B), 1.0)
    nbA, nbB = A.numel() * 4, B.numel() * 4
    # these launches are host-bound: hand the binding ready-made views (their C descriptors are built once)
    A, B, OA, r1k, den, o1 = (ct.DView.of(t) for t in (A, B, OA, r1k, den, o1))
    res["cpu_runnable_1024x1024"] = {
        "A_plus_B": gbs(2 * nbA + nbB, lambda: ct.binary(ct.ADD, A, B, out=OA), reps=200),
        "A_times_B": gbs(2 * nbA + nbB, lambda: ct.binary(ct.MUL, A, B, out=OA), reps=200),
        "A_div_absB_plus_1": gbs(2 * nbA + nbB, lambda: ct.binary(ct.DIV, A, den, out=OA), reps=200),
        "relu_A": gbs(2 * nbA, lambda: ct.unary(ct.RELU, A, out=OA), reps=200),
        "sum_dim1": gbs(nbA + 4096, lambda: ct.reduce(ct.SUM, A, 1, out=r1k), reps=200),
        "mean_dim1": gbs(nbA + 4096, lambda: ct.reduce(ct.MEAN, A, 1, out=r1k), reps=200),
        "max_dim1": gbs(nbA + 4096, lambda: ct.reduce(ct.MAX, A, 1, out=r1k), reps=200),
        "sum_full": gbs(nbA + 4, lambda: ct.reduce(ct.SUM, A, -1, out=o1), reps=200),
        "max_full": gbs(nbA + 4, lambda: ct.reduce(ct.MAX, A, -1, out=o1), reps=200),
    }
    del A, B, OA
    # reductions: X[8192,16384] ~ N(0,1), seed 2
    g.manual_seed(2)
    X = torch.randn(8192, 16384, device=dev, generator=g)
    red = {}
    for dim in (0, 1):
        for name, op in (("sum", ct.SUM), ("mean", ct.MEAN), ("var", ct.VAR), ("max", ct.MAX), ("min", ct.MIN),
                         ("argmax", ct.ARGMAX)):
            r = torch.empty(X.shape[1 - dim], device=dev, dtype=torch.int32 if op == ct.ARGMAX else torch.float32)
            red[f"{name}_dim{dim}"] = gbs(X.numel() * 4 + r.numel() * 4, lambda: ct.reduce(op, X, dim, out=r))
    res["reductions_8192x16384"] = red
    del X
    # permuted 4-d broadcast and softmax chain: S = [32,1024,12,1024].permute(0,2,1,3), M[1,12,1,1024]
    g.manual_seed(4)
    buf = torch.randn(32, 1024, 12, 1024, device=dev, generator=g)
    S = buf.permute(0, 2, 1, 3)
    g.manual_seed(5)
    M = -torch.rand(1, 12, 1, 1024, device=dev, generator=g)
    O = torch.empty(32, 12, 1024, 1024, device=dev)
    nb = buf.numel() * 4
    mx = torch.empty(32, 12, 1024, device=dev)
    res["permuted_softmax_chain"] = {
        "S_plus_M": gbs(2 * nb + M.numel() * 4, lambda: ct.binary(ct.ADD, S, M, out=O)),
        "max_last_dim": gbs(nb + mx.numel() * 4, lambda: ct.reduce(ct.MAX, O, 3, out=mx)),
        "sub_rowmax": gbs(2 * nb + mx.numel() * 4, lambda: ct.binary(ct.SUB, O, mx.view(32, 12, 1024, 1), out=buf.view(32, 12, 1024, 1024))),
        "fused_chain_softmax_S_plus_M": gbs(2 * nb + M.numel() * 4, lambda: ct.softmax(S, M, out=O)),
    }
    del buf, S, O, mx
    # GPT-2 small non-GEMM forward ops on [8,1024,768] / [8,1024,3072] / [8,12,1024,1024]
    g.manual_seed(6)
    x = torch.randn(8, 1024, 768, device=dev, generator=g)
    r = torch.randn(8, 1024, 768, device=dev, generator=g)
    gam = 1 + 0.02 * torch.randn(768, device=dev, generator=g)
    bet = 0.02 * torch.randn(768, device=dev, generator=g)
    h = torch.randn(8, 1024, 3072, device=dev, generator=g)
    a = torch.randn(8, 12, 1024, 1024, device=dev, generator=g)
    ox, oh, oa = torch.empty_like(x), torch.empty_like(h), torch.empty_like(a)
    vx, vr, vox, vgam, vbet = (ct.DView.of(t) for t in (x, r, ox, gam, bet))
    res["gpt2_small_non_gemm"] = {
        "residual_add_24MiB": gbs(3 * x.numel() * 4, lambda: ct.binary(ct.ADD, vx, vr, out=vox)),
        "layernorm_24MiB": gbs(2 * x.numel() * 4, lambda: ct.layernorm(vx, vgam, vbet, out=vox)),
        "gelu_96MiB": gbs(2 * h.numel() * 4, lambda: ct.unary(ct.GELU_TANH, h, out=oh)),
        "causal_softmax_384MiB": gbs(2 * a.numel() * 4, lambda: ct.softmax(a, None, True, out=oa)),
    }
    # The 24 MiB launches above are bound by the host's launch rate (one ctypes call each) and
    # their operands sit in L2.  The same ops as one CUDA graph of 24 launches that rotate over
    # 12 distinct buffer sets (12 x 72 MiB > L2): device time of the kernels themselves.
    try:
        sets = 12
        xs = [torch.randn(8, 1024, 768, device=dev, generator=g) for _ in range(sets)]
        rs = [torch.randn(8, 1024, 768, device=dev, generator=g) for _ in range(sets)]
        os_ = [torch.empty(8, 1024, 768, device=dev) for _ in range(sets)]

        def graph_gbs(nbytes, fn, launches=24, replays=10):
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for i in range(sets):
                    fn(i)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(launches):
                        fn(i % sets)
                graph.replay()
                side.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(side)
                for _ in range(replays):
                    graph.replay()
                t1.record(side)
                side.synchronize()
            torch.cuda.current_stream(dev).wait_stream(side)
            return round(nbytes * launches * replays / t0.elapsed_time(t1) / 1e6, 1)

        nb24 = x.numel() * 4
        res["gpt2_small_non_gemm"]["cuda_graph_rotating_buffers"] = {
            "residual_add_24MiB": graph_gbs(3 * nb24, lambda i: ct.binary(ct.ADD, xs[i], rs[i], out=os_[i])),
            "layernorm_24MiB": graph_gbs(2 * nb24, lambda i: ct.layernorm(xs[i], gam, bet, out=os_[i])),
        }
        del xs, rs, os_
    except Exception as exc:
        res["gpt2_small_non_gemm"]["cuda_graph_rotating_buffers"] = {"error": repr(exc)}
    del x, r, h, a, ox, oh, oa
    # entry points for the callers either side of the path (algorithmic bytes: every operand once)
    n = 1 << 28
    p = torch.randn(n, device=dev, generator=g)
    gr = torch.randn(n, device=dev, generator=g)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    G = gr.view(16384, 16384)
    bias = torch.zeros(16384, device=dev)
    xb = gr.view(128, 256, 64, 128)                      # BatchNorm input [N, C, H, W], 1 GiB
    mean, var = ct.channel_moments(xb)
    gam, bet = torch.ones(256, device=dev), torch.zeros(256, device=dev)
    yb = m.view(128, 256, 64, 128)
    logits = gr.view(32768, 8192)
    lo = m.view(32768, 8192)
    xpos = p.abs() + 0.5
    ce_labels = torch.randint(0, 8192, (32768, 1), device=dev, dtype=torch.int32)
    ce_loss = torch.empty(1, device=dev)
    logits1k = gr[: 262144 * 1000].view(262144, 1000)
    lo1k = m[: 262144 * 1000].view(262144, 1000)
    labels1k = torch.randint(0, 1000, (262144, 1), device=dev, dtype=torch.int32)
    step = [0]

    def adam():
        step[0] += 1
        ct.adam_step(p, gr, m, v, 1e-3, step[0])

    callers = {
        "sgd_step_1GiB": gbs(12 * n, lambda: ct.sgd_step(p, gr, 1e-3)),
        "adam_step_1GiB": gbs(28 * n, adam),
        "accumulate_grad_bias_16384x16384": gbs(4 * n + 8 * 16384, lambda: ct.accumulate_grad(bias, G)),
        "accumulate_grad_same_shape_1GiB": gbs(12 * n, lambda: ct.accumulate_grad(p, gr)),
        "batchnorm_moments_128x256x64x128": gbs(4 * n, lambda: ct.channel_moments(xb)),
        "batchnorm_apply_128x256x64x128": gbs(8 * n, lambda: ct.batchnorm_apply(xb, mean, var, gam, bet, 1e-5, out=yb)),
        "log_softmax_32768x8192": gbs(8 * n, lambda: ct.log_softmax(logits, out=lo)),
        "div_backward_both_1GiB": gbs(20 * n, lambda: ct.div_backward(gr, p, xpos, out_a=m, out_b=v)),
        "tanh_backward_1GiB": gbs(12 * n, lambda: ct.tanh_backward(gr, p, out=m)),
        "cross_entropy_32768x8192": gbs(4 * n, lambda: ct.cross_entropy(logits, ce_labels, True, out=ce_loss)),
        "cross_entropy_backward_32768x8192": gbs(8 * n, lambda: ct.cross_entropy_backward(logits, ce_labels, 1.0 / 32768, out=lo)),
        "cross_entropy_262144x1000": gbs(4 * 262144 * 1000, lambda: ct.cross_entropy(logits1k, labels1k, True, out=ce_loss)),
        "cross_entropy_backward_262144x1000": gbs(8 * 262144 * 1000, lambda: ct.cross_entropy_backward(logits1k, labels1k, 1.0 / 262144, out=lo1k)),
        "cat_two_halves_1GiB": gbs(8 * n, lambda: ct.cat([gr.view(2, n // 2)[0].view(8192, -1), gr.view(2, n // 2)[1].view(8192, -1)], 1, out=m.view(8192, -1))),
    }
    # vocabulary-sized rows ([5341, 50257] = 1 GiB; rows start at every 4-byte phase): the three-sweep kernels
    vrows, vcols = 5341, 50257
    vx = torch.randn(vrows, vcols, device=dev, generator=g)
    vo = torch.empty_like(vx)
    vg, vb = torch.randn(vcols, device=dev, generator=g), torch.randn(vcols, device=dev, generator=g)
    vlab = torch.randint(0, vcols, (vrows, 1), device=dev, generator=g).to(torch.int32)
    nv = vrows * vcols
    callers["vocabulary_rows_5341x50257"] = {
        "softmax": gbs(8 * nv, lambda: ct.softmax(vx, out=vo)),
        "log_softmax": gbs(8 * nv, lambda: ct.log_softmax(vx, out=vo)),
        "layernorm": gbs(8 * nv, lambda: ct.layernorm(vx, vg, vb, out=vo)),
        "cross_entropy": gbs(4 * nv, lambda: ct.cross_entropy(vx, vlab, True, out=ce_loss)),
        "cross_entropy_backward": gbs(8 * nv, lambda: ct.cross_entropy_backward(vx, vlab, 1.0 / vrows, out=vo)),
    }
    del vx, vo
    a2 = torch.randn(4096, 4096, device=dev, generator=g)
    c2 = torch.empty(4096, 4096, device=dev)
    for _ in range(2):
        ct.matmul(a2, a2, out=c2)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(3):
        ct.matmul(a2, a2, out=c2)
    t1.record()
    torch.cuda.synchronize()
    callers["matmul_4096^3_plain_fp32_TFLOPs"] = round(3 * 2 * 4096 ** 3 / t0.elapsed_time(t1) / 1e9, 1)
    # the tensor-core entry point (tcgen05, TF32 products): b as the transposed view a Linear layer passes
    try:
        tc = {}
        for size in (4096, 8192):
            aa = torch.randn(size, size, device=dev, generator=g)
            ww = torch.randn(size, size, device=dev, generator=g)
            cc = torch.empty(size, size, device=dev)
            bt = ct.DView.of(ww).permute([1, 0])
            st = torch.zeros(1, dtype=torch.int32, device=dev)
            for _ in range(3):
                ct.matmul_tc(aa, bt, out=cc, status=st)
            torch.cuda.synchronize()
            if st.item() != 0:
                raise RuntimeError(f"kernel status {st.item()}")
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(10):
                ct.matmul_tc(aa, bt, out=cc)
            t1.record()
            torch.cuda.synchronize()
            tc[f"{size}^3_TFLOPs"] = round(10 * 2 * size ** 3 / t0.elapsed_time(t1) / 1e9, 1)
            del aa, ww, cc
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                pk = json.load(f)
            tc["note"] = ("TF32 products; for scale: the measured cuBLAS bf16 peaks of this pool are "
                          f"{pk.get('bf16_tflops')} (burst) / {pk.get('bf16_tflops_sustained')} (sustained) TFLOP/s, and TF32 runs at half the bf16 rate")
        except Exception:
            pass
        callers["matmul_tensor_cores_tf32"] = tc
    except Exception as exc:
        callers["matmul_tensor_cores_tf32"] = {"error": repr(exc)}
    res["callers"] = callers
    return res


def profile_case(name: str):
    """A few launches of one kernel family on a small case (inputs larger than L2, well under
    1 GiB on the device), for profiler captures: `--profile-case reductions|rows|strided|callers|vocab|gelu|matmul|ce`."""
    import torch
    import ctensor_b200 as ct
    torch.manual_seed(0)
    if name == "reductions":            # 4096 x 16384 fp32 = 256 MiB; dim 0 = column kernel, dim 1 = row kernel
        X = torch.randn(4096, 16384, device="cuda")
        for _ in range(2):
            for op in (ct.VAR, ct.SUM, ct.ARGMAX, ct.MAX):
                for dim in (0, 1):
                    ct.reduce(op, X, dim)
    elif name == "gelu":                # the elementwise tile kernel on 2^26 elements (256 MiB in, 256 MiB out)
        x = torch.randn(1 << 26, device="cuda")
        o = torch.empty_like(x)
        for _ in range(3):
            ct.unary(ct.GELU_TANH, x, out=o)
            ct.unary(ct.EXP, x, out=o)
    elif name == "matmul":              # the tensor-core product on 2048^3 (b as a transposed view: no packing)
        a = torch.randn(2048, 2048, device="cuda")
        w = torch.randn(2048, 2048, device="cuda")
        c = torch.empty(2048, 2048, device="cuda")
        for _ in range(3):
            ct.matmul_tc(a, ct.DView.of(w).permute([1, 0]), out=c)
    elif name == "rows":                # softmax variants on [4,12,1024,1024] (192 MiB), LayerNorm on [65536,768]
        C = torch.randn(4, 12, 1024, 1024, device="cuda")
        O = torch.empty_like(C)
        M = -torch.rand(1, 12, 1, 1024, device="cuda")
        L = torch.randn(65536, 768, device="cuda")
        LO = torch.empty_like(L)
        g, b = torch.randn(768, device="cuda"), torch.randn(768, device="cuda")
        for _ in range(2):
            ct.softmax(C, out=O)
            ct.softmax(C, M, out=O)
            ct.softmax(C, None, True, out=O)
            ct.log_softmax(C, out=O)
            ct.layernorm(L, g, b, out=LO)
    elif name == "callers":             # optimizer, accumulate_grad, BatchNorm, gather on 2^26 elements
        n = 1 << 26
        p, gr = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        bias = torch.zeros(8192, device="cuda")
        xb = gr.view(32, 256, 64, 128)
        mean, var = ct.channel_moments(xb)
        idx = torch.randint(0, 8192, (8192, 64), device="cuda", dtype=torch.int32)
        for t in range(1, 3):
            ct.adam_step(p, gr, m, v, 1e-3, t)
            ct.sgd_step(p, gr, 1e-3)
            ct.accumulate_grad(bias, gr.view(8192, 8192))
            ct.channel_moments(xb)
            ct.batchnorm_apply(xb, mean, var, None, None, 1e-5, out=m.view(32, 256, 64, 128))
            ct.gather(gr.view(8192, 8192), 1, idx)
    elif name == "vocab":               # vocabulary-sized rows: [2048, 50304] and [2048, 50257] logits
        for cols in (50304, 50257):
            L = torch.randn(2048, cols, device="cuda")
            O = torch.empty_like(L)
            gamma, beta = torch.randn(cols, device="cuda"), torch.randn(cols, device="cuda")
            for _ in range(2):
                ct.log_softmax(L, out=O)
                ct.softmax(L, out=O)
                ct.layernorm(L, gamma, beta, out=O)
    elif name == "ce":                  # cross-entropy rows: [65536,1000] and [4096,16384] (registers), [2048,50257] (one sweep)
        for rows, cols in ((65536, 1000), (4096, 16384), (2048, 50257)):
            L = torch.randn(rows, cols, device="cuda")
            G = torch.empty_like(L)
            lab = torch.randint(0, cols, (rows, 1), device="cuda", dtype=torch.int32)
            loss = torch.empty(1, device="cuda")
            for _ in range(2):
                ct.cross_entropy(L, lab, True, out=loss)
                ct.cross_entropy_backward(L, lab, 1.0 / rows, out=G)
            del L, G
    elif name == "strided":             # the permuted 4-d view at batch 4: S + M, contiguous(S), x - rowmax
        buf = torch.randn(4, 1024, 12, 1024, device="cuda")
        S = buf.permute(0, 2, 1, 3)
        M = -torch.rand(1, 12, 1, 1024, device="cuda")
        O = torch.empty(4, 12, 1024, 1024, device="cuda")
        mx = torch.randn(4, 12, 1024, 1, device="cuda")
        for _ in range(2):
            ct.binary(ct.ADD, S, M, out=O)
            ct.contiguous(S, out=O)
            ct.binary(ct.SUB, O, mx, out=buf.view(4, 12, 1024, 1024))
    else:
        raise SystemExit(f"unknown profile case {name!r}")
    torch.cuda.synchronize()
    _emit({"profile_case": name, "status": "done"})


def cpu_baseline(sample_log2=28, reps=2, select_log2=24, extras=True):
    """The reference's CPU code on a bounded sample of the step: the same five ops (gelu as the chain
    of reference primitives) on n = 2^sample_log2 elements.  Every back-end the reference has for
    the ops is first timed on a small selection sample (2^select_log2); the fastest is then timed on
    the full sample and is the baseline value.  `extras` adds the baseline table: the scalar core as
    the reference's CMake build ships it (no -O, no OpenMP) and the reduction configuration."""
    import ctypes
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    kind, impl, paths = "port", None, {}
    if ol.Reference.available():
        try:
            impl = ol.Reference()
            kind = "reference"
        except OSError:
            impl = None
    if impl is not None:
        if impl.has_avx512:
            paths["dispatch(avx512,1 thread as shipped)"] = ol.PATH_DISPATCH
        if impl.has_avx2:
            paths["avx2+openmp"] = ol.PATH_AVX2
        paths["mp(scalar+openmp, -O2)"] = ol.PATH_MP
    else:
        impl = ol.Oracle()
        paths["oracle port (plain C + OpenMP)"] = None
    # All the host threads this process may use.  torchrun exports OMP_NUM_THREADS=1 to its
    # workers, which would time the reference's OpenMP loops on a single thread.
    host_threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if kind == "reference":
        impl.lib.ref_set_threads(host_threads)
    else:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(host_threads)

    # shrink the sample where host memory is short: x, y, an output and the gelu chain's temporaries
    avail = mem_available_bytes()
    while sample_log2 > select_log2 and avail and 10 * 4 * (1 << sample_log2) > avail:
        sample_log2 -= 1
    rng = np.random.default_rng(1)
    n = 1 << sample_log2
    # N(0,1) values; beyond 2^24 elements the same block repeats (drawing 2^30 normals takes longer than timing them)
    blk = min(n, 1 << 24)
    x = np.tile(rng.standard_normal(blk, dtype=np.float32), n // blk)
    y = np.tile(rng.standard_normal(blk, dtype=np.float32), n // blk)

    def step(obj, path, xs, ys):
        """Seconds for one step."""
        if path is None:                                   # oracle port
            hx, hy = ol.HostView.contig(xs), ol.HostView.contig(ys)
            t0 = time.perf_counter()
            obj.binary(ol.ADD, hx, hy); obj.binary(ol.MUL, hx, hy)
            obj.unary(ol.EXP, hx); obj.unary(ol.RELU, hx); obj.unary(ol.GELU_TANH, hx)
            return time.perf_counter() - t0
        return obj.bench_step(path, xs, ys)                # timed inside the reference build

    m = 1 << min(select_log2, sample_log2)
    results = {}
    for name, path in paths.items():
        try:
            step(impl, path, x[:m], y[:m])
            best = min(step(impl, path, x[:m], y[:m]) for _ in range(2))
            results[name] = round(BYTES_PER_ELEM_STEP * m / best / 1e9, 2)
        except Exception as exc:
            results[name] = f"failed: {exc}"
    per_op = {}
    if kind == "reference":         # each operator through each back-end (GB/s of its own algorithmic bytes)
        for name, path in paths.items():
            try:
                impl.bench_ops(path, x[:m], y[:m])
                runs = [impl.bench_ops(path, x[:m], y[:m]) for _ in range(2)]
                if runs[0] is not None:
                    best_t = [min(r[i] for r in runs) for i in range(5)]
                    per_op[name] = {op: round(b * m / t / 1e9, 2)
                                    for op, b, t in zip(("add", "mul", "exp", "relu", "gelu"), (12, 12, 8, 8, 8), best_t)}
            except Exception as exc:
                per_op[name] = f"failed: {exc}"
    good = {k: v for k, v in results.items() if isinstance(v, float)}
    best_name = max(good, key=good.get)
    step(impl, paths[best_name], x, y)
    best = min(step(impl, paths[best_name], x, y) for _ in range(max(1, reps)))
    value = round(BYTES_PER_ELEM_STEP * n / best / 1e9, 2)
    threads = impl.lib.ref_max_threads() if kind == "reference" else host_threads
    res = {"value": value, "unit": "GB/s", "cores": threads, "kind": kind,
           "sample": f"n=2^{sample_log2} elements per tensor, the same 5 ops, best of {max(1, reps)}; fastest back-end "
                     f"(picked on n=2^{min(select_log2, sample_log2)}): {best_name}; output allocation is inside every "
                     "reference op and therefore inside its time",
           "elements": n, "paths_GBs_on_selection_sample": results, "per_op_GBs_on_selection_sample": per_op,
           "host_cpus": os.cpu_count()}
    if extras and kind == "reference":
        try:        # the scalar core as the reference's own build system compiles it
            shipped_so = os.path.join(ROOT, "oracle", "_ref", "libctensor_ref_as_shipped.so")
            if os.path.exists(shipped_so):
                L = ctypes.CDLL(shipped_so)
                L.ref_bench_step.restype = ctypes.c_double
                L.ref_bench_step.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
                k = 1 << 21
                t = min(L.ref_bench_step(ol.PATH_MP, x.ctypes.data, y.ctypes.data, k) for _ in range(2))
                res["mp_as_shipped_flags"] = {"GB/s": round(BYTES_PER_ELEM_STEP * k / t / 1e9, 3), "elements": k,
                                              "flags": "no -O, no -fopenmp (CMakeLists.txt gives the scalar core none): 1 thread"}
        except Exception as exc:
            res["mp_as_shipped_flags"] = {"error": repr(exc)}
        try:        # the reduction configuration on the back-end that can do dim-wise reductions
            X = rng.standard_normal((8192, 16384), dtype=np.float32)
            hv = ol.HostView.contig(X)
            red = {}
            for nm, op, dim in (("sum_dim0", ol.SUM, 0), ("sum_dim1", ol.SUM, 1), ("max_dim0", ol.MAX, 0), ("max_dim1", ol.MAX, 1),
                                ("argmax_dim1", ol.ARGMAX, 1), ("sum_full", ol.SUM, -1)):
                if dim == -1:
                    flat = ol.HostView.contig(X.reshape(-1))
                    t0 = time.perf_counter(); impl.reduce(op, flat, -1, ol.PATH_DISPATCH); t = time.perf_counter() - t0
                else:
                    t0 = time.perf_counter(); impl.reduce(op, hv, dim, ol.PATH_MP); t = time.perf_counter() - t0
                red[nm] = round(X.nbytes / t / 1e9, 2)
            red["note"] = "X[8192,16384] fp32, one call each: sum_mp / max_mp / argmax (scalar+OpenMP), full sum through the dispatcher"
            res["reductions_8192x16384_GBs"] = red
        except Exception as exc:
            res["reductions_8192x16384_GBs"] = {"error": repr(exc)}
    return res


def bench_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    # the GPU arm's size (2^30 elements per tensor) where host memory permits, else the largest that fits
    cpu = cpu_baseline(sample_log2=args.ref_log2, reps=max(1, min(args.steps, 2)), extras=False)
    n = cpu["elements"]
    value = cpu["value"]
    line = {
        "impl": "reference",
        "metric": "op GB/s and % of 8 TB/s HBM peak at 1/2/4/8 B200 vs host-CPU reference",
        "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(BYTES_PER_ELEM_STEP * n / value / 1e6, 3), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"contiguous fp32 sweep, n=2^{n.bit_length() - 1} elements: add, mul, exp, relu, gelu(tanh) of "
                               "N(0,1) tensors on the host cores (the reference's fastest back-end)",
                   "elements_per_step": n, "elements_per_gpu": n},
        "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    _emit(line)


_REAL_STDOUT = None


def _claim_stdout():
    """Keep stdout for the one JSON line: everything else a library prints there (NCCL's version
    banner, for one) goes to stderr."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def _emit(line: dict):
    _REAL_STDOUT.write(json.dumps(line) + "\n")
    _REAL_STDOUT.flush()


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--n", type=int, default=1 << 30, help="elements per GPU (weak) or in total (strong)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--e2e-n", type=int, default=0, help="cap on the e2e tensor size (0 = same as --n)")
    ap.add_argument("--cpu-log2", type=int, default=28, help="log2 of the cpu_baseline sample of the GPU arm")
    ap.add_argument("--ref-log2", type=int, default=30, help="log2 of the tensor size of --impl reference (shrunk if host RAM is short)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the timed steps (no e2e, sweep, cpu baseline, sharded sum): for profiler runs")
    ap.add_argument("--profile-case", default=None, choices=["reductions", "rows", "strided", "callers", "vocab", "gelu", "matmul", "ce"],
                    help="run a few launches of one kernel family on a small case and exit (for ncu)")
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args.profile_case)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        bench_reference(args)
    else:
        bench_ours(args)


if __name__ == "__main__":
    main()
