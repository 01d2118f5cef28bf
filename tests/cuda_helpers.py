"""Small helpers for the GPU tests: raw device buffers through the C ABI, host<->device
copies through the CUDA runtime (independent of the kernels under test), canaries."""
from __future__ import annotations

import ctypes
import glob
import os

import numpy as np

_rt = None


def cudart():
    global _rt
    if _rt is None:
        import torch  # noqa: F401  (loads the CUDA runtime torch ships with)
        cands = glob.glob(os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "cuda_runtime", "lib", "libcudart.so*"))
        cands += ["libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so.12"]
        for c in cands:
            try:
                _rt = ctypes.CDLL(c)
                break
            except OSError:
                continue
        assert _rt is not None, "CUDA runtime not found"
        _rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        _rt.cudaMemset.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t]
        _rt.cudaMalloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t]
        _rt.cudaFree.argtypes = [ctypes.c_void_p]
    return _rt


def check(rc, what):
    assert rc == 0, f"{what} failed with CUDA error {rc}"


def h2d(dev_ptr: int, arr: np.ndarray) -> None:
    arr = np.ascontiguousarray(arr)
    check(cudart().cudaMemcpy(dev_ptr, arr.ctypes.data, arr.nbytes, 1), "cudaMemcpy H2D")


def d2h(dev_ptr: int, nbytes: int, dtype=np.uint8) -> np.ndarray:
    out = np.empty(nbytes // np.dtype(dtype).itemsize, dtype=dtype)
    check(cudart().cudaMemcpy(out.ctypes.data, dev_ptr, nbytes, 2), "cudaMemcpy D2H")
    return out


def memset(dev_ptr: int, value: int, nbytes: int) -> None:
    check(cudart().cudaMemset(dev_ptr, value, nbytes), "cudaMemset")


def sync() -> None:
    check(cudart().cudaDeviceSynchronize(), "cudaDeviceSynchronize")


def cuda_malloc(nbytes: int) -> int:
    p = ctypes.c_void_p()
    check(cudart().cudaMalloc(ctypes.byref(p), nbytes), "cudaMalloc")
    return int(p.value)


def cuda_free(ptr: int) -> None:
    check(cudart().cudaFree(ptr), "cudaFree")


class Guarded:
    """A side-aware buffer with one 2 MiB canary page on each side of the payload."""
    PAGE = 2 << 20
    CANARY = 0xA5

    def __init__(self, sa, nbytes: int):
        self.sa = sa
        self.nbytes = nbytes
        self.payload_bytes = (nbytes + self.PAGE - 1) // self.PAGE * self.PAGE
        self.total = self.payload_bytes + 2 * self.PAGE
        self.base = sa.malloc(self.total)
        self.ptr = self.base + self.PAGE
        memset(self.base, self.CANARY, self.PAGE)
        memset(self.ptr + self.payload_bytes, self.CANARY, self.PAGE)

    def canaries_intact(self) -> bool:
        lo = d2h(self.base, self.PAGE)
        hi = d2h(self.ptr + self.payload_bytes, self.PAGE)
        return bool((lo == self.CANARY).all() and (hi == self.CANARY).all())

    def free(self):
        self.sa.free(self.base)
