"""torch integration on a B200: CUDAPluggableAllocator entry points and torch.ops.sideaware.*
(the usage of test.py:14-15, :147-184), each in a fresh process."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_script(args, timeout=900):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, *args], capture_output=True, text=True, timeout=timeout, cwd=ROOT, env=env)
    return r


def test_pluggable_allocator_flow():
    r = run_script([os.path.join(ROOT, "tests", "pluggable_allocator_script.py"), "400"])
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert lines, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads(lines[-1][7:])
    print(json.dumps(res, indent=1)[:3000])
    assert r.returncode == 0 and res["ok"], res
    assert res["stats_mid"]["large_allocs"] >= 1 and res["stats_mid"]["small_allocs"] >= 1
    assert res["stats_end"]["cross_side_pages"] == 0


def test_custom_op_under_torch_compile():
    code = """
import torch, l2_torch_alloc_b200 as pkg
sa = pkg.sideaware_init()
@torch.compile(fullgraph=True)
def f(dst, src):
    torch.ops.sideaware.memcpy(dst, src)
    return dst
src = torch.ones((8, 8), device="cuda") * 2.0
dst = torch.zeros((8, 8), device="cuda")
out = f(dst, src)
torch.cuda.synchronize()
assert torch.equal(out, src) and torch.equal(dst, src)
print("COMPILED-OK")
"""
    r = run_script(["-c", code])
    assert "COMPILED-OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_rope_ops_under_torch_compile():
    """Table made on the GPU and rotation, both as custom ops inside one compiled graph, against the oracle
    (tolerance: 1e-6 of the pair's magnitude, the fp32 tolerance of the task; the table differs from libm's by <= 1 ulp)."""
    code = """
import numpy as np, torch, l2_torch_alloc_b200 as pkg
from oracle import oracle
sa = pkg.sideaware_init()
B, T, Nq, Nkv, HS = 2, 128, 4, 2, 64
@torch.compile(fullgraph=True)
def f(qkv, table):
    torch.ops.sideaware.rope_freqs(table, 10000.0, False)
    torch.ops.sideaware.rope_forward(qkv, table, Nq, Nkv)
    return qkv
x = np.random.default_rng(5).uniform(-1, 1, size=(B, T, Nq + 2 * Nkv, HS)).astype(np.float32)
qkv = torch.from_numpy(x).cuda()
table = torch.empty((T, HS // 2, 2), device="cuda")
out = f(qkv, table).cpu().numpy()
want = oracle.rope_forward_f32(x, oracle.freqs_cis(HS, T, 10000.0, 0), B, T, Nq, Nkv, HS)
pairs = x.reshape(B, T, -1, HS // 2, 2).astype(np.float64)
mag = np.sqrt((pairs ** 2).sum(-1, keepdims=True)).repeat(2, -1).reshape(x.shape)
assert (np.abs(out.astype(np.float64) - want) <= 1e-6 * mag + 1e-12).all()
print("COMPILED-ROPE-OK")
"""
    r = run_script(["-c", code])
    assert "COMPILED-ROPE-OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_training_steps_match_torchs_own_allocator():
    """Six optimizer steps of a small MLP under the pluggable allocator give the losses torch's own allocator gives."""
    out = {}
    for mode in ("native", "sideaware"):
        r = run_script([os.path.join(ROOT, "tests", "training_equivalence_script.py"), mode])
        lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
        assert lines, r.stdout[-3000:] + r.stderr[-3000:]
        out[mode] = json.loads(lines[-1][7:])
    a = [float.fromhex(v) for v in out["native"]["losses"]]
    b = [float.fromhex(v) for v in out["sideaware"]["losses"]]
    print("ms per step: native", out["native"]["ms_per_step"], "sideaware", out["sideaware"]["ms_per_step"])
    print("losses native   ", a)
    print("losses sideaware", b)
    assert len(a) == len(b) == 6
    for u, v in zip(a, b):
        assert abs(u - v) <= 1e-6 * abs(u), (a, b)  # same kernels on the same data: equal up to cuBLAS's choice of algorithm
    st = out["sideaware"]["stats"]
    assert out["sideaware"]["errors"] == 0 and st["large_allocs"] >= 10 and st["cross_side_pages"] == 0
    assert st["reuse_hits"] >= st["large_allocs"] // 2, "after the first step most blocks come from mapped runs"
    assert out["sideaware"]["ms_per_step"] <= 1.25 * out["native"]["ms_per_step"] + 1.0, "the allocator must not slow the steady state down"
