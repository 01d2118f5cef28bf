"""Host-side mirror of the reference's Python interface (example_wrapper.py:1-187,
test.py:41-157), rewritten around a small class so several users can share one
loaded library.  Argument names, meanings and assertion behaviour follow the
reference; the known slip there (``src_bytes`` computed from ``dst``,
example_wrapper.py:131) is not repeated.
"""
from __future__ import annotations

import ctypes
from typing import Optional

from . import _binding

_state = {"sa": None}


def _stream_ptr(stream) -> int:
    if stream is None:
        return 0
    if isinstance(stream, int):
        return stream
    if isinstance(stream, ctypes.c_void_p):
        return stream.value or 0
    return int(stream.cuda_stream)


class SideAware:
    """One loaded sideaware.so plus thin, checked wrappers around its launchers."""

    def __init__(self, path: Optional[str] = None):
        self.lib = _binding.load(path)
        self.path = self.lib._path

    # -- errors ---------------------------------------------------------------
    def last_error(self) -> str:
        return (self.lib.sideaware_last_error() or b"").decode()

    def error_count(self) -> int:
        return int(self.lib.sideaware_error_count())

    def _checked(self, before: int, what: str) -> None:
        if self.error_count() != before:
            raise RuntimeError(f"{what}: {self.last_error()}")

    # -- metadata ---------------------------------------------------------------
    def summary(self):
        """(num_sms, num_side0, num_side1, min_sm_per_side, hash_mask)"""
        before = self.error_count()
        out = tuple(self.lib.sideaware_sm_side_summary().contents)
        self._checked(before, "sideaware_sm_side_summary")
        return out

    def summary_dict(self):
        n, s0, s1, m, h = self.summary()
        return {"num_sms": n, "side0": s0, "side1": s1, "min": m, "hash": h}

    def cpu_side_index(self) -> bytes:
        n = self.summary()[0]
        ptr = self.lib.sideaware_cpu_side_index()
        return ctypes.string_at(ptr, n)

    def stats(self) -> dict:
        st = _binding.Stats()
        self.lib.sideaware_get_stats(ctypes.byref(st))
        return st.as_dict()

    def driver_call_times(self) -> dict:
        """Host milliseconds and call counts the allocator spent in driver calls, by kind."""
        ns = (ctypes.c_ulonglong * 8)()
        calls = (ctypes.c_ulonglong * 8)()
        self.lib.sideaware_driver_call_times(ctypes.byref(ns), ctypes.byref(calls))
        names = ["create", "release", "reserve", "map", "unmap", "set_access", "probe", "sync"]
        return {n: {"ms": ns[i] / 1e6, "calls": int(calls[i])} for i, n in enumerate(names)}

    def topology_json(self) -> str:
        return (self.lib.sideaware_topology_json() or b"{}").decode()

    def set_placement(self, mode) -> None:
        modes = {"aware": 0, "unaware": 1, "wrong": 2}
        self.lib.sideaware_set_placement(modes.get(mode, mode))

    # -- raw allocation (no torch) --------------------------------------------
    def malloc(self, size: int, stream=None) -> int:
        p = ctypes.c_void_p()
        rc = self.lib.sideaware_malloc_async(ctypes.byref(p), size, _stream_ptr(stream))
        if rc != 0 or not p.value:
            raise MemoryError(f"sideaware_malloc_async({size}) failed with CUDA error {rc}: {self.last_error()}")
        return int(p.value)

    def free(self, ptr: int, stream=None) -> None:
        rc = self.lib.sideaware_free_async(ptr, _stream_ptr(stream))
        if rc != 0:
            raise RuntimeError(f"sideaware_free_async failed with CUDA error {rc}: {self.last_error()}")

    # -- kernels on raw pointers --------------------------------------------------
    def memcpy_ptr(self, dst: int, src: int, num_bytes: int, device: int = 0, stream=None) -> None:
        before = self.error_count()
        self.lib.sideaware_memcpy(dst, src, num_bytes, device, _stream_ptr(stream))
        self._checked(before, "sideaware_memcpy")

    def rope_backward_ptr(self, dqkv: int, freqs: int, B, T, Nq, Nkv, HS, bf16: bool, device: int = 0, stream=None) -> None:
        rc = self.lib.sideaware_rope_backward(dqkv, freqs, B, T, Nq, Nkv, HS, 1 if bf16 else 0, device, _stream_ptr(stream))
        if rc != 0:
            raise RuntimeError(f"sideaware_rope_backward failed with CUDA error {rc}: {self.last_error()}")

    def rope_forward_ptr(self, qkv: int, freqs: int, B, T, Nq, Nkv, HS, bf16: bool, device: int = 0, stream=None) -> None:
        rc = self.lib.sideaware_rope_forward(qkv, freqs, B, T, Nq, Nkv, HS, 1 if bf16 else 0, device, _stream_ptr(stream))
        if rc != 0:
            raise RuntimeError(f"sideaware_rope_forward failed with CUDA error {rc}: {self.last_error()}")

    def rope_precompute_freqs_ptr(self, table: int, dim: int, end: int, theta: float, use_scaled: bool,
                                  device: int = 0, stream=None) -> None:
        rc = self.lib.sideaware_rope_precompute_freqs(table, dim, end, theta, 1 if use_scaled else 0, device, _stream_ptr(stream))
        if rc != 0:
            raise RuntimeError(f"sideaware_rope_precompute_freqs failed with CUDA error {rc}: {self.last_error()}")

    def silu_mul_ptr(self, out: int, a: int, b: int, scale: float, n: int, device: int = 0, stream=None) -> None:
        rc = self.lib.sideaware_silu_mul_bf16(out, a, b, scale, n, device, _stream_ptr(stream))
        if rc != 0:
            raise RuntimeError(f"sideaware_silu_mul_bf16 failed with CUDA error {rc}: {self.last_error()}")

    def create_kernel(self, header_code: bytes) -> int:
        if isinstance(header_code, str):
            header_code = header_code.encode()
        return int(self.lib.sideaware_create_kernel(header_code))

    def compile_check(self, header_code: bytes, wide: bool = False) -> str:
        """Compiles a functor header for sm_100a without a GPU; returns "" or the compiler log."""
        if isinstance(header_code, str):
            header_code = header_code.encode()
        buf = ctypes.create_string_buffer(1 << 16)
        rc = self.lib.sideaware_compile_check(header_code, 1 if wide else 0, buf, len(buf))
        log = buf.value.decode()
        if rc == 0:
            if log:  # compiles, but uses something that does not carry over from the reference's launch shape
                import warnings
                warnings.warn(log)
            return ""
        return log or "compile failed"

    def chunk_sides(self, ptr: int, num_bytes: int) -> bytes:
        n = (num_bytes + (ptr & 4095) + 4095) // 4096
        buf = ctypes.create_string_buffer(n)
        got = self.lib.sideaware_chunk_sides(ptr, num_bytes, buf)
        return buf.raw[:got]

    def verify_chunk_sides(self, ptr: int, num_bytes: int, samples: int = 256, seed: int = 0) -> int:
        return int(self.lib.sideaware_verify_chunk_sides(ptr, num_bytes, samples, seed))

    # -- torch tensors --------------------------------------------------------------
    def memcpy(self, dst, src) -> None:
        import torch
        assert dst.device.type == "cuda" and src.device.type == "cuda", "Both tensors must be on CUDA"
        assert dst.dtype == src.dtype, "Source and destination must have the same dtype"
        assert dst.numel() >= src.numel(), "Destination tensor must be at least as large as source"
        assert src.is_contiguous(), "src must be contiguous"
        assert dst.is_contiguous(), "dst must be contiguous"
        assert dst.data_ptr() % 16 == 0 and src.data_ptr() % 16 == 0, "dst and src must be 16-byte aligned"
        self.memcpy_ptr(dst.data_ptr(), src.data_ptr(), src.numel() * src.element_size(),
                        src.device.index, torch.cuda.current_stream(src.device))

    def one_to_one(self, kernel_id: int, dst, src) -> None:
        import torch
        dst_bytes = dst.numel() * dst.element_size() if dst is not None else 0
        src_bytes = src.numel() * src.element_size() if src is not None else 0
        num_bytes = max(src_bytes, dst_bytes)
        assert num_bytes > 0
        for t, name in ((dst, "dst"), (src, "src")):
            assert t is None or (t.is_contiguous() and t.device.type == "cuda"), f"{name} must be contiguous"
        dst_ptr = dst.data_ptr() if dst is not None else 0
        src_ptr = src.data_ptr() if src is not None else 0
        assert dst_ptr % 16 == 0 and src_ptr % 16 == 0, "dst and src must be 16-byte aligned"
        ref = dst if dst is not None else src
        before = self.error_count()
        self.lib.sideaware_one_to_one(kernel_id, num_bytes, dst_ptr, src_ptr, ref.device.index,
                                      _stream_ptr(torch.cuda.current_stream(ref.device)))
        self._checked(before, "sideaware_one_to_one")

    def elementwise(self, kernel_id: int, out0, out1, out2, out3, in0, in1, in2, in3,
                    sideband_tensor=None, sideband_value: int = 0, parallel_chunks: int = 0,
                    forced_sm_per_side: int = 0) -> None:
        import torch
        tensors = [out0, out1, out2, out3, in0, in1, in2, in3]
        names = ["out0", "out1", "out2", "out3", "in0", "in1", "in2", "in3"]
        # num_bytes is the byte size of the one array the kernel moves as 16-byte vectors: in0, or out0 if its
        # element is wider (sideaware.cu:127-129, :1378).  The other arrays may be any size the functor's
        # index function asks for (a short broadcast table, a wider auxiliary array): they do not count.
        num_bytes = max((t.numel() * t.element_size() for t in (in0, out0) if t is not None), default=0)
        assert num_bytes > 0, "in0 or out0 must be given"
        ptrs = []
        for t, name in zip(tensors, names):
            assert t is None or (t.is_contiguous() and t.device.type == "cuda"), f"{name} must be contiguous"
            ptrs.append(t.data_ptr() if t is not None else 0)
            assert ptrs[-1] % 16 == 0, "16B alignment"
        sideband_ptr = sideband_tensor.data_ptr() if sideband_tensor is not None else 0
        ref = next(t for t in tensors if t is not None)
        before = self.error_count()
        self.lib.sideaware_elementwise(kernel_id, num_bytes, *ptrs, sideband_ptr, sideband_value, parallel_chunks,
                                       forced_sm_per_side, ref.device.index,
                                       _stream_ptr(torch.cuda.current_stream(ref.device)))
        self._checked(before, "sideaware_elementwise")

    def rope_forward(self, qkv, freqs_cis, n_q_heads: int, n_kv_heads: int) -> None:
        """In place on packed [B, T, Nq + 2 Nkv, HS] (fp32 or bf16); freqs_cis fp32 [T, HS/2, 2]."""
        import torch
        assert qkv.is_cuda and freqs_cis.is_cuda and qkv.is_contiguous() and freqs_cis.is_contiguous()
        assert qkv.dtype in (torch.float32, torch.bfloat16) and freqs_cis.dtype == torch.float32
        B, T, H, HS = qkv.shape
        assert H == n_q_heads + 2 * n_kv_heads, "head dimension must hold q, k and v heads"
        assert tuple(freqs_cis.shape) == (T, HS // 2, 2), "freqs_cis must be [T, HS/2, 2]"
        self.rope_forward_ptr(qkv.data_ptr(), freqs_cis.data_ptr(), B, T, n_q_heads, n_kv_heads, HS,
                              qkv.dtype == torch.bfloat16, qkv.device.index, torch.cuda.current_stream(qkv.device))

    def rope_backward(self, dqkv, freqs_cis, n_q_heads: int, n_kv_heads: int) -> None:
        """In place on the gradient of a packed [B, T, Nq + 2 Nkv, HS] tensor."""
        import torch
        assert dqkv.is_cuda and freqs_cis.is_cuda and dqkv.is_contiguous() and freqs_cis.is_contiguous()
        assert dqkv.dtype in (torch.float32, torch.bfloat16) and freqs_cis.dtype == torch.float32
        B, T, H, HS = dqkv.shape
        assert H == n_q_heads + 2 * n_kv_heads and tuple(freqs_cis.shape) == (T, HS // 2, 2)
        self.rope_backward_ptr(dqkv.data_ptr(), freqs_cis.data_ptr(), B, T, n_q_heads, n_kv_heads, HS,
                               dqkv.dtype == torch.bfloat16, dqkv.device.index, torch.cuda.current_stream(dqkv.device))

    def rope_precompute_freqs_into(self, freqs_cis, theta: float = 10000.0, use_scaled: bool = False) -> None:
        """Fills an existing fp32 CUDA tensor [end, dim/2, 2] with (cos, sin)."""
        import torch
        assert freqs_cis.is_cuda and freqs_cis.is_contiguous() and freqs_cis.dtype == torch.float32
        assert freqs_cis.dim() == 3 and freqs_cis.shape[2] == 2, "freqs_cis must be [end, dim/2, 2]"
        end, half, _ = freqs_cis.shape
        self.rope_precompute_freqs_ptr(freqs_cis.data_ptr(), 2 * half, end, float(theta), use_scaled,
                                       freqs_cis.device.index, torch.cuda.current_stream(freqs_cis.device))

    def rope_precompute_freqs(self, dim: int, end: int, theta: float = 10000.0, use_scaled: bool = False, device=None):
        """The fp32 table [end, dim/2, 2] of (cos, sin) that rope_forward / rope_backward read, made on the GPU."""
        import torch
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        table = torch.empty((end, dim // 2, 2), dtype=torch.float32, device=device)
        self.rope_precompute_freqs_ptr(table.data_ptr(), dim, end, float(theta), use_scaled, device.index,
                                       torch.cuda.current_stream(device))
        return table

    def silu_mul(self, out, a, b, scale: float) -> None:
        import torch
        for t in (out, a, b):
            assert t.is_cuda and t.is_contiguous() and t.dtype == torch.bfloat16
        assert out.numel() == a.numel() == b.numel()
        self.silu_mul_ptr(out.data_ptr(), a.data_ptr(), b.data_ptr(), float(scale), a.numel(), a.device.index,
                          torch.cuda.current_stream(a.device))

    def mxfp8_quantize(self, out, scales, x) -> None:
        """bf16 -> MXFP8 with functors.mxfp8_quantize_bf16: `out` uint8 (E4M3 bytes, one per element), `scales`
        uint8 (E8M0 bytes, one per block of 32 elements; its size must be a multiple of 4), `x` bfloat16.
        A block is reduced inside one warp instruction, which needs x to start on a 64-byte boundary; the
        element count must be a multiple of 8 (whole 16-byte vectors), a last block of fewer than 32
        elements is scaled by the elements it has."""
        import torch
        from . import functors
        assert x.dtype == torch.bfloat16 and out.dtype == torch.uint8 and scales.dtype == torch.uint8
        n = x.numel()
        assert n % 8 == 0, "the element count must be a multiple of 8"
        assert x.data_ptr() % 64 == 0, "x must start on a 64-byte boundary (a block of 32 elements may not straddle two warp instructions)"
        assert out.numel() >= n and scales.numel() >= (n + 31) // 32 and scales.numel() % 4 == 0
        assert n // 8 < 2 ** 31
        kid = self.create_kernel(functors.mxfp8_quantize_bf16())
        # the vector count tells the functor where the last, partial block ends; 0 = there is none (the common case,
        # in which the functor skips that bookkeeping)
        self.elementwise(kid, out[:n], None, None, None, x, None, None, None, scales.view(torch.int32),
                         n // 8 if n % 32 else 0)

    def side_index_tensor(self):
        import torch
        n = self.summary()[0]
        t = torch.zeros(n, dtype=torch.uint8, device="cuda")
        self.lib.sideaware_fill_side_index(t.data_ptr())
        return t

    # -- torch integration -----------------------------------------------------------
    def install_allocator(self) -> None:
        """Routes torch's CUDA allocations through sideaware_malloc_auto / sideaware_free_auto
        (test.py:14-15).  Must run before the first CUDA allocation of the process."""
        import torch
        alloc = torch.cuda.memory.CUDAPluggableAllocator(self.path, "sideaware_malloc_auto", "sideaware_free_auto")
        torch.cuda.memory.change_current_allocator(alloc)

    def register_ops(self) -> None:
        """torch.ops.sideaware.{memcpy, one_to_one, elementwise, rope_forward, silu_mul}"""
        from . import torch_ops
        torch_ops.register(self)


# ---------------------------------------------------------------------------
# module-level functions with the reference wrapper's names (example_wrapper.py:21-43)
# ---------------------------------------------------------------------------
def sideaware_init(path: Optional[str] = None, install_allocator: bool = True) -> SideAware:
    sa = SideAware(path)
    if install_allocator:
        sa.install_allocator()
    sa.register_ops()
    _state["sa"] = sa
    _state["info"] = sa.summary()
    _state["torch_side_index"] = sa.side_index_tensor()
    print(f"L2 Side Aware metadata: {sa.summary_dict()}")
    return sa


def sideaware_enabled() -> int:
    return 1 if _state["sa"] is not None else 0


def _sa() -> SideAware:
    if _state["sa"] is None:
        raise RuntimeError("call sideaware_init() first")
    return _state["sa"]


def sideaware_create_kernel(header_code: bytes) -> int:
    return _sa().create_kernel(header_code)


def sideaware_torch_side_index():
    return _state.get("torch_side_index")


def sideaware_gpu_side_index():
    return _sa().lib.sideaware_gpu_side_index()


def sideaware_cpu_side_index():
    return _sa().lib.sideaware_cpu_side_index()


def sideaware_info():
    n, s0, s1, m, h = _state.get("info", (0, 0, 0, 0, 0))
    return {"num_sms": n, "side0": s0, "side1": s1, "min": m, "hash": h}


def sideaware_info_raw():
    return _state.get("info", (0, 0, 0, 0, 0))
