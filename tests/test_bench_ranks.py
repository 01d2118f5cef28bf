"""The N > 1 path of bench.py on CPU: two gloo ranks launched the way the driver launches the
benchmark (torch.distributed.run, 127.0.0.1).  The hot path has no cross-GPU exchange, so the
only multi-rank logic is the barrier, the max over ranks of the timed duration, the sum of
the work, and "rank 0 alone prints" - including for the CPU reference arm."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def launch(extra, nproc=2, port=29611, timeout=300):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "bench.py"),
           "--gpus", str(nproc)] + extra
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)


def json_lines(text):
    out = []
    for line in text.splitlines():
        line = line.strip()
        if line.startswith("{") and line.endswith("}"):
            out.append(json.loads(line))
    return out


def test_two_ranks_aggregate_max_and_sum():
    r = launch(["--check-ranks"])
    assert r.returncode == 0, r.stderr[-3000:]
    lines = json_lines(r.stdout)
    assert len(lines) == 1, "exactly one JSON line, printed by rank 0"
    assert lines[0]["world"] == 2 and lines[0]["max_ms"] == 2.0 and lines[0]["sum_gb"] == 3.0
    assert abs(lines[0]["value"] - 1500.0) < 1e-9


def test_reference_arm_runs_on_rank_zero_only():
    r = launch(["--impl", "reference", "--steps", "3", "--warmup", "3"], port=29612, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = json_lines(r.stdout)
    assert len(lines) == 1 and lines[0]["impl"] == "reference"
    assert lines[0]["unit"] == "GB/s" and lines[0]["value"] > 0 and lines[0]["n_gpus"] == 2
    assert lines[0]["e2e"]["h2d_bytes_per_step"] == 0 and lines[0]["cpu_baseline"]["cores"] >= 1


def test_single_process_refuses_multi_gpu_without_launcher():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2", "--check-ranks"],
                       capture_output=True, text=True, timeout=120, cwd=ROOT, env={k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")})
    assert r.returncode != 0 and "torch.distributed.run" in (r.stderr + r.stdout)
