"""The user-functor (NVRTC) path on a B200: the reference's own functor check restated
(test.py:191-237, exact equality on small integers, mixed element sizes, reverse order),
plus the benchmark functors compiled from header text."""
import numpy as np
import pytest

from oracle import oracle
from tests import cuda_helpers as ch
from tests.test_abi import MIXED_HEADER

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sa():
    import torch
    assert torch.cuda.is_available()
    import l2_torch_alloc_b200 as pkg
    return pkg.SideAware()


def test_mixed_size_functor_exact(sa):
    import torch
    for shape in [(8, 8), (1000, 520), (4096, 4096 + 8)]:
        n = shape[0] * shape[1]
        in0 = (torch.arange(n, device="cuda", dtype=torch.float32) % 64).reshape(shape).to(torch.bfloat16)
        in1 = torch.ones(shape, device="cuda", dtype=torch.float32) * 2
        out0 = torch.zeros(shape, device="cuda", dtype=torch.float32)
        out1 = torch.zeros(shape, device="cuda", dtype=torch.float16)
        kid = sa.create_kernel(MIXED_HEADER)
        assert kid >= 1
        sa.elementwise(kid, out0, out1, None, None, in0, in1, None, None)
        torch.cuda.synchronize()
        assert torch.equal(out0, in0.float() + in1)
        assert torch.equal(out1, (in1 * 10.0).half())
    assert sa.stats()["jit_compiles"] >= 1


def test_memcpy_functor_and_one_to_one(sa):
    import torch
    from l2_torch_alloc_b200 import functors
    kid = sa.create_kernel(functors.MEMCPY)
    src = torch.randint(0, 2**31 - 1, (3 * 1000 * 1000 + 4,), dtype=torch.int32, device="cuda")
    dst = torch.zeros_like(src)
    sa.one_to_one(kid, dst, src)
    torch.cuda.synchronize()
    assert torch.equal(dst, src)
    dst.zero_()
    sa.one_to_one(0, dst, src)  # id 0 is the built-in memcpy
    torch.cuda.synchronize()
    assert torch.equal(dst, src)


def test_silu_mul_functor_matches_oracle_and_aot_kernel(sa):
    import torch
    from l2_torch_alloc_b200 import functors
    n = (1 << 22) + 4096
    rng = np.random.default_rng(0xB200 + 4)
    a = oracle.f32_to_bf16(rng.standard_normal(n).astype(np.float32))
    b = oracle.f32_to_bf16(rng.standard_normal(n).astype(np.float32))
    want = oracle.silu_mul_bf16(a, b, 0.5)
    ta = torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    tb = torch.from_numpy(b.view(np.int16)).cuda().view(torch.bfloat16)
    out = torch.zeros_like(ta)
    kid = sa.create_kernel(functors.silu_mul_bf16())
    scale_bits = int(np.float32(0.5).view(np.int32))
    sa.elementwise(kid, out, None, None, None, ta, tb, None, None, None, scale_bits)
    torch.cuda.synchronize()
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.ulp_diff_bf16(got, want).max() <= 1
    out2 = torch.zeros_like(ta)
    sa.silu_mul(out2, ta, tb, 0.5)
    torch.cuda.synchronize()
    got2 = out2.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.ulp_diff_bf16(got2, want).max() <= 1


@pytest.mark.parametrize("bf16", [False, True])
def test_rope_functor_header_matches_oracle(sa, bf16):
    import torch
    from l2_torch_alloc_b200 import functors
    B, T, Nq, Nkv, HS = 2, 128, 8, 2, 64
    H = Nq + 2 * Nkv
    rng = np.random.default_rng(9)
    table = oracle.freqs_cis(HS, T, 500000.0, 0)
    tt = torch.from_numpy(table).cuda()
    kid = sa.create_kernel(functors.rope_forward(T, Nq, Nkv, HS, bf16))
    if bf16:
        x = oracle.f32_to_bf16(rng.standard_normal((B, T, H, HS)).astype(np.float32))
        want = oracle.rope_forward_bf16(x, table, B, T, Nq, Nkv, HS)
        tx = torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16)
    else:
        x = rng.uniform(-1, 1, (B, T, H, HS)).astype(np.float32)
        want = oracle.rope_forward_f32(x, table, B, T, Nq, Nkv, HS)
        tx = torch.from_numpy(x).cuda()
    sa.elementwise(kid, tx, None, None, None, tx, tt, None, None)
    torch.cuda.synchronize()
    if bf16:
        got = tx.view(torch.int16).cpu().numpy().view(np.uint16)
    else:
        got = tx.cpu().numpy()
    assert got.tobytes() == want.tobytes()


def test_bad_functor_is_an_error_not_a_crash(sa):
    import torch
    kid = sa.create_kernel(b"typedef int o0; typedef int i0; broken")
    t = torch.zeros(1024, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="NVRTC|compil"):
        sa.one_to_one(kid, t, t)
    with pytest.raises(RuntimeError, match="unknown kernel id"):
        sa.one_to_one(10_000, t, t)
