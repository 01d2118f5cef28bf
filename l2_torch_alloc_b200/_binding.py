"""ctypes binding of sideaware.so - one declaration per symbol of include/sideaware.h.

The argument types are those the reference's Python harness declares for the
same symbols (test.py:18-39, example_wrapper.py:52-80); streams travel as
void pointers.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_PATH = os.path.join(HERE, "sideaware.so")

c = ctypes
_vp, _sz, _i = c.c_void_p, c.c_size_t, c.c_int


class Stats(ctypes.Structure):
    _fields_ = [(n, c.c_ulonglong) for n in (
        "bytes_mapped_live", "bytes_mapped_cached", "pages_pool_side0", "pages_pool_side1", "pages_created",
        "cross_side_pages", "reuse_hits", "large_allocs", "small_allocs", "trims", "jit_compiles",
        "kernel_launches", "probe_confidence_ppm", "hash_validation_errors", "kernel_wait_timeouts",
        "handles_created", "handles_discarded", "extensions", "hole_refills", "headroom_pages", "top_ups")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


# name -> (restype, argtypes); the complete exported surface
SIGNATURES = {
    # reference-compatible entry points
    "sideaware_malloc_async": (_i, [c.POINTER(_vp), _sz, _vp]),
    "sideaware_free_async": (_i, [_vp, _vp]),
    "sideaware_malloc": (_i, [c.POINTER(_vp), _sz]),
    "sideaware_free": (_i, [_vp]),
    "sideaware_release_unused": (_sz, []),
    "sideaware_malloc_auto": (_vp, [_sz, _i, _vp]),
    "sideaware_free_auto": (None, [_vp, _sz, _i, _vp]),
    "sideaware_elementwise": (None, [_i, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "sideaware_one_to_one": (None, [_i, _sz, _vp, _vp, _i, _vp]),
    "sideaware_memcpy": (None, [_vp, _vp, _sz, _i, _vp]),
    "sideaware_create_kernel_advanced": (_i, [c.c_char_p, c.c_bool, _i]),
    "sideaware_create_kernel": (_i, [c.c_char_p]),
    "sideaware_compression": (None, [c.c_bool]),
    "sideaware_alloc_threshold": (None, [_sz]),
    "sideaware_prealloc_config": (None, [_i, _i]),
    "sideaware_prealloc": (_i, [_sz, _i]),
    "sideaware_free_mapped_thresholds": (None, [_sz, _sz]),
    "sideaware_write_sass": (None, [c.c_char_p]),
    "sideaware_fill_side_index": (None, [_vp]),
    "sideaware_gpu_side_index": (_vp, []),
    "sideaware_cpu_side_index": (_vp, []),
    "sideaware_sm_side_summary": (c.POINTER(_i * 5), []),
    "sideaware_num_sms": (_i, []),
    "sideaware_num_sm_side0": (_i, []),
    "sideaware_num_sm_side1": (_i, []),
    "sideaware_min_sm_per_side": (_i, []),
    "sideaware_hash_mask": (_i, []),
    # additions
    "sideaware_last_error": (c.c_char_p, []),
    "sideaware_error_count": (c.c_ulonglong, []),
    "sideaware_rope_forward": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "sideaware_rope_backward": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "sideaware_rope_precompute_freqs": (_i, [_vp, _i, _i, c.c_float, _i, _i, _vp]),
    "sideaware_silu_mul_bf16": (_i, [_vp, _vp, _vp, c.c_float, _sz, _i, _vp]),
    "sideaware_compile_check": (_i, [c.c_char_p, _i, c.c_char_p, _sz]),
    "sideaware_set_placement": (None, [_i]),
    "sideaware_get_placement": (_i, []),
    "sideaware_set_memcpy_engine": (None, [_i]),
    "sideaware_get_memcpy_engine": (_i, []),
    "sideaware_set_rope_engine": (None, [_i]),
    "sideaware_get_rope_engine": (_i, []),
    "sideaware_chunk_sides": (_sz, [_vp, _sz, _vp]),
    "sideaware_verify_chunk_sides": (_i, [_vp, _sz, _i, c.c_uint]),
    "sideaware_get_stats": (None, [c.POINTER(Stats)]),
    "sideaware_topology_json": (c.c_char_p, []),
    "sideaware_driver_call_times": (None, [c.POINTER(c.c_ulonglong * 8), c.POINTER(c.c_ulonglong * 8)]),
    "sideaware_memcpy_noalloc": (_i, [_vp, _vp, _sz, _i, _vp]),
}


def load(path: str | None = None) -> ctypes.CDLL:
    """Opens the library and declares every signature.  Raises if it is missing:
    there is no Python or CPU stand-in for the kernels."""
    path = path or os.environ.get("SIDEAWARE_SO") or DEFAULT_PATH
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"{path} not found: build it with `python -m l2_torch_alloc_b200.build` (needs nvcc, no GPU)")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    lib._path = path
    return lib
