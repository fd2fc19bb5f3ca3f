"""The reference arm of bench.py runs without a GPU: its JSON line carries the contract's keys and
it uses every host thread the process may use, also when the launcher exports OMP_NUM_THREADS=1
(as torchrun does for its workers)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_reference_arm(extra_env):
    env = dict(os.environ)
    env.update(extra_env)
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1",
         "--ref-log2", "20"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, proc.stdout
    return json.loads(lines[0])


def test_reference_arm_line_and_threads():
    line = _run_reference_arm({"OMP_NUM_THREADS": "1"})
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["unit"] == "GB/s" and line["value"] > 0
    assert line["vs_baseline"] is None
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cpu = line["cpu_baseline"]
    assert cpu["kind"] in ("reference", "port")
    assert cpu["value"] == line["value"]
    assert cpu["cores"] == len(os.sched_getaffinity(0))
