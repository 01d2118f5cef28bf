"""Regenerates the golden vectors in this directory from the COMPILED REFERENCE.

Run where the reference tree is available (it is compiled in place by
``make -C oracle ref`` into oracle/_ref/libref_rope.so):

    python tests/golden/make_golden.py

Outputs (all small, committed):
  rope_small_f32.npz   input/table/output of the reference's CPU RoPE on a tiny
                       packed-QKV tensor, llama-3 scaling off and on, plus the
                       reference's backward pass applied to that output
  rope_gqa_bf16.npz    grouped-query bf16 case obtained from the unmodified
                       reference function through the padded-head construction
                       (rotation depends on (t, d) only)
  rope_c1.json         SHA-256 of the reference's table and output at the
                       CPU-runnable benchmark shape B=4 T=1024 NH=12 HS=64
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import oracle  # noqa: E402

_f32p = oracle._f32p


def ref_table(dim, end, theta, scaled):
    t = np.empty((end, dim // 2, 2), dtype=np.float32)
    oracle.ref().ref_precompute_freqs_cis(oracle._ptr(t, _f32p), dim, end, theta, scaled)
    return t


def ref_forward(inp, table, B, T, NH, HS):
    inp = np.ascontiguousarray(inp, dtype=np.float32)
    out = np.empty_like(inp)
    oracle.ref().ref_apply_rotary_emb_forward(oracle._ptr(out, _f32p), oracle._ptr(inp, _f32p),
                                              oracle._ptr(table, _f32p), B, T, NH, HS)
    return out


def ref_backward(dout, table, B, T, NH, HS):
    dout = np.ascontiguousarray(dout, dtype=np.float32)
    dinp = np.zeros_like(dout)  # the reference accumulates into a zeroed buffer (example_llmc_rope.cu:301-303)
    oracle.ref().ref_apply_rotary_emb_backward(oracle._ptr(dinp, _f32p), oracle._ptr(dout, _f32p), oracle._ptr(dout, _f32p),
                                               oracle._ptr(table, _f32p), B, T, NH, HS)
    return dinp


def main():
    assert oracle.ref_available(), "build oracle/_ref first (make -C oracle ref)"

    # -- tiny fp32 MHA case, both table flavours --------------------------------
    B, T, NH, HS = 2, 5, 3, 8
    rng = np.random.default_rng(0xB200)
    inp = rng.uniform(-1.0, 1.0, size=(B, T, 3 * NH, HS)).astype(np.float32)
    out = {}
    for scaled in (0, 1):
        tab = ref_table(HS, T, 10000.0, scaled)
        out[f"table_s{scaled}"] = tab
        out[f"out_s{scaled}"] = ref_forward(inp, tab, B, T, NH, HS)
        out[f"dinp_s{scaled}"] = ref_backward(out[f"out_s{scaled}"], tab, B, T, NH, HS)  # gradient = forward output
    np.savez_compressed(os.path.join(HERE, "rope_small_f32.npz"), inp=inp,
                        shape=np.array([B, T, NH, HS]), **out)

    # -- grouped-query bf16 through the padded-head construction ------------------
    B, T, Nq, Nkv, HS = 2, 9, 4, 1, 16
    heads = Nq + 2 * Nkv
    rng = np.random.default_rng(0xB200 + 3)
    x = rng.standard_normal(size=(B, T, heads, HS)).astype(np.float32)
    x_bf = oracle.f32_to_bf16(x)
    xf = oracle.bf16_to_f32(x_bf)
    tab = ref_table(HS, T, 500000.0, 0)
    rot = Nq + Nkv
    npad = (rot + 1) // 2
    padded = np.zeros((B, T, 3 * npad, HS), dtype=np.float32)
    padded[:, :, :rot] = xf[:, :, :rot]
    pout = ref_forward(padded, tab, B, T, npad, HS)
    want = xf.copy()
    want[:, :, :rot] = pout[:, :, :rot]
    np.savez_compressed(os.path.join(HERE, "rope_gqa_bf16.npz"), inp_bf16=x_bf, table=tab,
                        out_bf16=oracle.f32_to_bf16(want), shape=np.array([B, T, Nq, Nkv, HS]))

    # -- hash of the reference at the CPU benchmark shape -------------------------
    B, T, NH, HS = 4, 1024, 12, 64
    rng = np.random.default_rng(0xB200 + 1)
    inp = rng.uniform(-1.0, 1.0, size=(B, T, 3 * NH, HS)).astype(np.float32)
    rec = {"shape": [B, T, NH, HS], "seed": 0xB200 + 1, "theta": 10000.0,
           "input_sha256": hashlib.sha256(inp.tobytes()).hexdigest()}
    for scaled in (0, 1):
        tab = ref_table(HS, T, 10000.0, scaled)
        o = ref_forward(inp, tab, B, T, NH, HS)
        rec[f"table_sha256_s{scaled}"] = hashlib.sha256(tab.tobytes()).hexdigest()
        rec[f"out_sha256_s{scaled}"] = hashlib.sha256(o.tobytes()).hexdigest()
    with open(os.path.join(HERE, "rope_c1.json"), "w") as f:
        json.dump(rec, f, indent=1)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
