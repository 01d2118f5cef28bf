"""The oracle is pinned before anything trusts it: C restatement == numpy
restatement == golden vectors produced by the compiled reference
(example_llmc_rope.cu:19-86), and == the compiled reference itself where
oracle/_ref exists."""
import hashlib
import json
import os

import numpy as np
import pytest

from oracle import oracle


def test_small_f32_matches_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "rope_small_f32.npz"))
    B, T, NH, HS = (int(v) for v in g["shape"])
    for scaled in (0, 1):
        tab = oracle.freqs_cis(HS, T, 10000.0, scaled)
        assert tab.tobytes() == g[f"table_s{scaled}"].tobytes()
        out = oracle.rope_forward_f32(g["inp"], tab, B, T, NH, NH, HS)
        assert out.tobytes() == g[f"out_s{scaled}"].tobytes()
        out_np = oracle.np_rope_forward_f32(g["inp"], tab, B, T, NH, NH, HS)
        assert out_np.tobytes() == g[f"out_s{scaled}"].tobytes()
        # backward pass of the reference (example_llmc_rope.cu:166-195) on the forward output
        dinp = oracle.rope_backward_f32(out, tab, B, T, NH, NH, HS)
        assert dinp.tobytes() == g[f"dinp_s{scaled}"].tobytes()
        # rotating back recovers the input up to rounding
        assert np.allclose(dinp, g["inp"], rtol=0, atol=1e-6)


def test_gqa_bf16_matches_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "rope_gqa_bf16.npz"))
    B, T, Nq, Nkv, HS = (int(v) for v in g["shape"])
    tab = oracle.freqs_cis(HS, T, 500000.0, 0)
    assert tab.tobytes() == g["table"].tobytes()
    out = oracle.rope_forward_bf16(g["inp_bf16"], tab, B, T, Nq, Nkv, HS)
    assert out.tobytes() == g["out_bf16"].tobytes()
    # value heads are passed through untouched
    assert np.array_equal(out[:, :, Nq + Nkv:], g["inp_bf16"][:, :, Nq + Nkv:])
    # threaded variant (used by the timed CPU baseline) is the same function
    out_mt = oracle.rope_forward_bf16(g["inp_bf16"], tab, B, T, Nq, Nkv, HS, threads=2)
    assert out_mt.tobytes() == out.tobytes()


def test_c1_shape_hashes(golden_dir):
    """B=4 T=1024 NH=12 HS=64 fp32, U[-1,1) from seed: the CPU-runnable benchmark config."""
    rec = json.load(open(os.path.join(golden_dir, "rope_c1.json")))
    B, T, NH, HS = rec["shape"]
    rng = np.random.default_rng(rec["seed"])
    inp = rng.uniform(-1.0, 1.0, size=(B, T, 3 * NH, HS)).astype(np.float32)
    assert hashlib.sha256(inp.tobytes()).hexdigest() == rec["input_sha256"]
    for scaled in (0, 1):
        tab = oracle.freqs_cis(HS, T, rec["theta"], scaled)
        assert hashlib.sha256(tab.tobytes()).hexdigest() == rec[f"table_sha256_s{scaled}"]
        out = oracle.rope_forward_f32(inp, tab, B, T, NH, NH, HS)
        assert hashlib.sha256(out.tobytes()).hexdigest() == rec[f"out_sha256_s{scaled}"]


@pytest.mark.skipif(not oracle.ref_available(), reason="compiled reference not present")
def test_restatement_equals_compiled_reference():
    from tests.golden.make_golden import ref_forward, ref_table
    rng = np.random.default_rng(7)
    for (B, T, NH, HS, theta, scaled) in [(1, 3, 1, 2, 10000.0, 0), (3, 17, 5, 32, 500000.0, 1), (2, 64, 4, 128, 10000.0, 1)]:
        inp = rng.uniform(-4, 4, size=(B, T, 3 * NH, HS)).astype(np.float32)
        tab = ref_table(HS, T, theta, scaled)
        assert oracle.freqs_cis(HS, T, theta, scaled).tobytes() == tab.tobytes()
        want = ref_forward(inp, tab, B, T, NH, HS)
        assert oracle.rope_forward_f32(inp, tab, B, T, NH, NH, HS).tobytes() == want.tobytes()


def test_bf16_conversions_round_to_nearest_even():
    f = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.3895313892515355e38, np.inf, 0.0, -0.0], dtype=np.float32)
    got = oracle.f32_to_bf16(f)
    # 1.00390625 = 0x3F808000 is a tie -> even (0x3F80); 1.01171875 = 0x3F818000 tie -> 0x3F82
    assert list(got[:4]) == [0x3F80, 0x3F80, 0x3F82, 0xBF80]
    assert got[5] == 0x7F80 and got[6] == 0 and got[7] == 0x8000
    back = oracle.bf16_to_f32(got)
    assert back[0] == 1.0
    buf = np.empty(f.size, dtype=np.uint16)
    oracle.lib().oracle_f32_to_bf16(oracle._ptr(buf, oracle._u16p), oracle._ptr(f, oracle._f32p), f.size)
    assert np.array_equal(buf, got)


def test_silu_mul_restatement():
    rng = np.random.default_rng(0xB200 + 4)
    a = oracle.f32_to_bf16(rng.standard_normal(4096).astype(np.float32))
    b = oracle.f32_to_bf16(rng.standard_normal(4096).astype(np.float32))
    got = oracle.silu_mul_bf16(a, b, 0.5)
    af, bf = oracle.bf16_to_f32(a).astype(np.float64), oracle.bf16_to_f32(b).astype(np.float64)
    want = oracle.f32_to_bf16((af / (1 + np.exp(-af)) * bf * 0.5).astype(np.float32))
    assert oracle.ulp_diff_bf16(got, want).max() <= 1


def test_memcpy_mt_is_exact():
    rng = np.random.default_rng(1)
    src = rng.integers(0, 256, size=(3 << 20) + 77, dtype=np.uint8)
    for threads in (1, 3, 8):
        dst = np.zeros_like(src)
        oracle.lib().oracle_memcpy_mt(dst.ctypes.data, src.ctypes.data, src.size, threads)
        assert np.array_equal(dst, src)


def test_e4m3_restatement_known_values():
    """Known encodings of FP8 E4M3 (bias 7, largest finite 448, smallest subnormal 2^-9)."""
    vals = [0.0, -0.0, 1.0, -1.0, 448.0, 1e9, -1e9, 2.0 ** -9, 2.0 ** -10, 2.0 ** -10 * 1.0001, 2.0 ** -6, 1.0625, 1.1875, 464.0, 17.0, 0.875]
    want = [0x00, 0x80, 0x38, 0xB8, 0x7E, 0x7E, 0xFE, 0x01, 0x00, 0x01, 0x08, 0x38, 0x3A, 0x7E, 0x58, 0x36]
    got = oracle.f64_to_e4m3_bytes(np.array(vals))
    assert [int(g) for g in got] == want
    # 1.0625 is halfway between 1.0 and 1.125: ties go to the even mantissa (1.0); 1.1875 between 1.125 and 1.25 -> 1.25
    x = np.zeros(64, dtype=np.float32)
    x[:32] = 3.0      # amax 3 -> floor(log2) = 1 -> shared exponent -7 -> elements 3 * 2^7 = 384 = 1.5 * 2^8
    x[32:] = 0.0
    el, sc = oracle.mxfp8_quantize_bf16(oracle.f32_to_bf16(x))
    assert sc.tolist() == [120, 0] and set(el[:32].tolist()) == {0x7C} and set(el[32:].tolist()) == {0}
