"""CPU oracle for the side-aware elementwise path.  TEST INFRASTRUCTURE ONLY.

Three layers, each checked against the next one down:

* numpy restatements (this file) - small, readable, vectorised;
* ``liboracle.so`` - the C restatement in ``rope_oracle.c`` (fast enough for the
  full benchmark shapes, also the timed CPU baseline);
* ``_ref/libref_rope.so`` - the reference's own CPU code compiled in place
  (``ref_shim.cu``); present wherever the reference tree was available at
  build time.

Parity status: PINNED (restatements == compiled reference == committed golden
vectors under ``tests/golden``).

Nothing in the shipped package imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_f32p = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def _ptr(a, ty):
    return a.ctypes.data_as(ty)


STAGED_TEXTS = ("test.py", "example_wrapper.py", "kernel_rope.cuh")


def reference_tree():
    """Where the reference's sources lie: SIDEAWARE_REFERENCE_TREE, else a checkout named
    ``reference`` beside this repository; None when neither exists."""
    cands = [os.environ.get("SIDEAWARE_REFERENCE_TREE"), os.path.join(_HERE, "..", "..", "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "example_llmc_rope.cu")):
            return os.path.abspath(c)
    return None


def build(force: bool = False) -> None:
    """Compile liboracle.so and, where the reference tree is present, everything under _ref/:
    the reference compiled in place and its harness texts staged unmodified."""
    if force or not os.path.exists(os.path.join(_HERE, "liboracle.so")) or (
        os.path.getmtime(os.path.join(_HERE, "liboracle.so")) < os.path.getmtime(os.path.join(_HERE, "rope_oracle.c"))
    ):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    ref_src = reference_tree()
    wanted = ("libref_rope.so", "sideaware_reference.so", os.path.join("cxx_example_reference", "rope_example")) + STAGED_TEXTS
    product = os.path.join(_HERE, "..", "l2_torch_alloc_b200", "sideaware.so")
    example = os.path.join(_HERE, "_ref", "cxx_example", "rope_example")
    if os.path.exists(product):  # the reference's C++ example linked against this project's library (make decides if it is stale)
        wanted += (os.path.join("cxx_example", "rope_example"),)
    stale = os.path.exists(example) and os.path.exists(product) and any(
        os.path.getmtime(f) > os.path.getmtime(example)
        for f in (os.path.join(_HERE, "..", "include", "sideaware.h"), os.path.join(_HERE, "..", "include", "sideaware.hpp"),
                  os.path.join(_HERE, "sideaware_cu_stand_in.cu")))
    if ref_src and (force or stale or not all(os.path.exists(os.path.join(_HERE, "_ref", f)) for f in wanted)):
        subprocess.check_call(["make", "-C", _HERE, "ref", f"REF={ref_src}"], stdout=subprocess.DEVNULL)


def lib() -> ctypes.CDLL:
    """The C restatement."""
    global _LIB
    if _LIB is None:
        build()
        L = ctypes.CDLL(os.path.join(_HERE, "liboracle.so"))
        L.oracle_precompute_freqs_cis.argtypes = [_f32p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int]
        L.oracle_rope_forward_f32.argtypes = [_f32p, _f32p, _f32p] + [ctypes.c_int] * 5
        L.oracle_rope_forward_bf16.argtypes = [_u16p, _u16p, _f32p] + [ctypes.c_int] * 5
        L.oracle_rope_backward_f32.argtypes = [_f32p, _f32p, _f32p] + [ctypes.c_int] * 5
        L.oracle_rope_backward_bf16.argtypes = [_u16p, _u16p, _f32p] + [ctypes.c_int] * 5
        L.oracle_silu_mul_bf16.argtypes = [_u16p, _u16p, _u16p, ctypes.c_float, ctypes.c_size_t]
        L.oracle_memcpy_mt.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        L.oracle_rope_forward_mt.argtypes = [ctypes.c_void_p, ctypes.c_void_p, _f32p] + [ctypes.c_int] * 7
        L.oracle_bf16_to_f32.argtypes = [_f32p, _u16p, ctypes.c_size_t]
        L.oracle_f32_to_bf16.argtypes = [_u16p, _f32p, ctypes.c_size_t]
        for f in ("oracle_precompute_freqs_cis", "oracle_rope_forward_f32", "oracle_rope_forward_bf16",
                  "oracle_rope_backward_f32", "oracle_rope_backward_bf16",
                  "oracle_silu_mul_bf16", "oracle_memcpy_mt", "oracle_rope_forward_mt",
                  "oracle_bf16_to_f32", "oracle_f32_to_bf16"):
            getattr(L, f).restype = None
        _LIB = L
    return _LIB


def ref_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libref_rope.so"))


def ref() -> ctypes.CDLL:
    """The compiled reference (its CPU functions only are ever called)."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libref_rope.so")
        try:
            R = ctypes.CDLL(path)
        except OSError:
            # No GPU driver on this machine: satisfy the libcuda.so.1 dependency with
            # the toolkit's link stub (none of its entry points are called).
            stub = "/usr/local/cuda/lib64/stubs/libcuda.so"
            ctypes.CDLL(stub, mode=ctypes.RTLD_GLOBAL)
            R = ctypes.CDLL(path)
        R.ref_precompute_freqs_cis.argtypes = [_f32p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int]
        R.ref_precompute_freqs_cis.restype = None
        R.ref_apply_rotary_emb_forward.argtypes = [_f32p, _f32p, _f32p] + [ctypes.c_int] * 4
        R.ref_apply_rotary_emb_forward.restype = None
        if hasattr(R, "ref_apply_rotary_emb_backward"):
            R.ref_apply_rotary_emb_backward.argtypes = [_f32p, _f32p, _f32p, _f32p] + [ctypes.c_int] * 4
            R.ref_apply_rotary_emb_backward.restype = None
        _REF = R
    return _REF


# ---------------------------------------------------------------------------
# C restatement wrappers
# ---------------------------------------------------------------------------
def freqs_cis(dim: int, end: int, theta: float, use_scaled: int = 0) -> np.ndarray:
    """[end, dim/2, 2] fp32 cos/sin table (example_llmc_rope.cu:19-52)."""
    t = np.empty((end, dim // 2, 2), dtype=np.float32)
    lib().oracle_precompute_freqs_cis(_ptr(t, _f32p), dim, end, theta, use_scaled)
    return t


def rope_forward_f32(inp: np.ndarray, table: np.ndarray, B, T, Nq, Nkv, HS) -> np.ndarray:
    inp = np.ascontiguousarray(inp, dtype=np.float32)
    table = np.ascontiguousarray(table, dtype=np.float32)
    out = np.empty_like(inp)
    lib().oracle_rope_forward_f32(_ptr(out, _f32p), _ptr(inp, _f32p), _ptr(table, _f32p), B, T, Nq, Nkv, HS)
    return out


def rope_forward_bf16(inp_u16: np.ndarray, table: np.ndarray, B, T, Nq, Nkv, HS, threads: int = 1) -> np.ndarray:
    """bf16 bit patterns in and out (uint16 arrays)."""
    inp_u16 = np.ascontiguousarray(inp_u16, dtype=np.uint16)
    table = np.ascontiguousarray(table, dtype=np.float32)
    out = np.empty_like(inp_u16)
    if threads > 1:
        lib().oracle_rope_forward_mt(out.ctypes.data, inp_u16.ctypes.data, _ptr(table, _f32p), B, T, Nq, Nkv, HS, 1, threads)
    else:
        lib().oracle_rope_forward_bf16(_ptr(out, _u16p), _ptr(inp_u16, _u16p), _ptr(table, _f32p), B, T, Nq, Nkv, HS)
    return out


def rope_backward_f32(dout: np.ndarray, table: np.ndarray, B, T, Nq, Nkv, HS) -> np.ndarray:
    """Gradient w.r.t. the input, accumulated into zeros as the reference does (example_llmc_rope.cu:166-195)."""
    dout = np.ascontiguousarray(dout, dtype=np.float32)
    table = np.ascontiguousarray(table, dtype=np.float32)
    dinp = np.zeros_like(dout)
    lib().oracle_rope_backward_f32(_ptr(dinp, _f32p), _ptr(dout, _f32p), _ptr(table, _f32p), B, T, Nq, Nkv, HS)
    return dinp


def rope_backward_bf16(dout_u16: np.ndarray, table: np.ndarray, B, T, Nq, Nkv, HS) -> np.ndarray:
    dout_u16 = np.ascontiguousarray(dout_u16, dtype=np.uint16)
    table = np.ascontiguousarray(table, dtype=np.float32)
    dinp = np.empty_like(dout_u16)
    lib().oracle_rope_backward_bf16(_ptr(dinp, _u16p), _ptr(dout_u16, _u16p), _ptr(table, _f32p), B, T, Nq, Nkv, HS)
    return dinp


def silu_mul_bf16(a_u16: np.ndarray, b_u16: np.ndarray, scale: float) -> np.ndarray:
    a_u16 = np.ascontiguousarray(a_u16, dtype=np.uint16)
    b_u16 = np.ascontiguousarray(b_u16, dtype=np.uint16)
    out = np.empty_like(a_u16)
    lib().oracle_silu_mul_bf16(_ptr(out, _u16p), _ptr(a_u16, _u16p), _ptr(b_u16, _u16p), scale, a_u16.size)
    return out


def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(u16, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(f: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(f, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7FFF
    return r


# ---------------------------------------------------------------------------
# numpy restatements (independent of the C code; used to cross-check it)
# ---------------------------------------------------------------------------
def np_rope_forward_f32(inp: np.ndarray, table: np.ndarray, B, T, Nq, Nkv, HS) -> np.ndarray:
    """Same arithmetic as example_llmc_rope.cu:54-86 with separate fp32 roundings."""
    heads = Nq + 2 * Nkv
    x = np.ascontiguousarray(inp, dtype=np.float32).reshape(B, T, heads, HS // 2, 2)
    tab = np.ascontiguousarray(table, dtype=np.float32).reshape(T, HS // 2, 2)
    c = tab[None, :, None, :, 0]
    s = tab[None, :, None, :, 1]
    out = x.copy()
    r = Nq + Nkv
    xr, xi = x[:, :, :r, :, 0], x[:, :, :r, :, 1]
    out[:, :, :r, :, 0] = (xr * c).astype(np.float32) - (xi * s).astype(np.float32)
    out[:, :, :r, :, 1] = (xr * s).astype(np.float32) + (xi * c).astype(np.float32)
    return out.reshape(inp.shape)


def ulp_diff_bf16(a_u16: np.ndarray, b_u16: np.ndarray) -> np.ndarray:
    """Distance in bf16 units of last place between two bit-pattern arrays."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)
    return np.abs(key(a_u16) - key(b_u16))


def f64_to_e4m3_bytes(x: np.ndarray) -> np.ndarray:
    """FP8 E4M3 (the "fn" flavour of the OCP 8-bit floating point specification: bias 7, no infinities, largest
    finite value 448) from exact values, round to nearest even, saturating: what a conversion with the
    saturate-to-finite option produces for finite inputs."""
    x = np.asarray(x, dtype=np.float64)
    sign = np.signbit(x).astype(np.uint8) << 7
    a = np.abs(x)
    out = np.zeros(a.shape, dtype=np.uint8)
    normal = a >= 2.0 ** -6
    # subnormals and zero: multiples of 2^-9; rounding up to 8 gives the smallest normal, whose bit pattern is 8 as well
    out[~normal] = np.rint(a[~normal] * 2.0 ** 9).astype(np.uint8)
    an = a[normal]
    e = np.floor(np.log2(an)).astype(np.int64)
    e = np.where(an < 2.0 ** e, e - 1, e)          # guard against log2 rounding up at powers of two
    e = np.where(an >= 2.0 ** (e + 1), e + 1, e)
    r = np.rint(an / 2.0 ** (e - 3)).astype(np.int64)  # 8..16
    carry = r == 16
    e = np.where(carry, e + 1, e)
    r = np.where(carry, 8, r)
    too_big = (e > 8) | ((e == 8) & (r > 14))
    e = np.where(too_big, 8, e)
    r = np.where(too_big, 14, r)
    out[normal] = (((e + 7) << 3) | (r - 8)).astype(np.uint8)
    return out | sign


def mxfp8_quantize_bf16(x_u16: np.ndarray):
    """bf16 -> MXFP8 restated from the OCP Microscaling Formats specification v1.0: blocks of 32 elements, one
    shared scale 2^(floor(log2(max |v|)) - 8) per block stored as E8M0 (exponent + 127; 8 is the largest E4M3
    exponent), elements v / scale in E4M3.  The block maximum's exponent is read from its float exponent field,
    so an all-zero block gives the smallest scale (2^-127, byte 0).  Returns (element bytes, scale bytes).
    The reference only names this use (sideaware.cu:81-83); there is no reference implementation to compare with."""
    v = bf16_to_f32(np.asarray(x_u16).reshape(-1)).reshape(-1, 32).copy()
    # functor kernels are built with flush-to-zero (-use_fast_math, as in the reference, sideaware.cu:535):
    # bf16 subnormals, which are float subnormals too, count as zero
    v[((v.view(np.uint32) >> 23) & 0xFF) == 0] = 0.0
    amax = np.abs(v).max(axis=1)
    field = (amax.astype(np.float32).view(np.uint32) >> 23) & 0xFF
    shared = np.maximum(field.astype(np.int64) - 127 - 8, -127)
    scaled = np.ldexp(v.astype(np.float64), (-shared)[:, None])
    return f64_to_e4m3_bytes(scaled).reshape(-1), (shared + 127).astype(np.uint8)
