"""B200 (sm_100a) side-aware allocator and elementwise kernels, host side.

This package is the Python face of ``sideaware.so`` and mirrors the reference's
Python harness (example_wrapper.py): ``sideaware_init`` installs the pluggable
allocator and registers ``torch.ops.sideaware.{memcpy,one_to_one,elementwise}``;
the ``sideaware_*`` helpers return the SM side metadata.  New here:
``torch.ops.sideaware.rope_forward`` / ``silu_mul`` for the ahead-of-time
kernels, placement control for A/B runs, and the chunk-side queries.

Everything computes on the GPU through the C ABI; there is no CPU fallback and
importing torch is deferred until a function that needs it is called.
"""
from __future__ import annotations

from . import _binding
from ._binding import Stats, load  # noqa: F401
from .api import (  # noqa: F401
    SideAware,
    sideaware_cpu_side_index,
    sideaware_create_kernel,
    sideaware_enabled,
    sideaware_gpu_side_index,
    sideaware_info,
    sideaware_info_raw,
    sideaware_init,
    sideaware_torch_side_index,
)

__all__ = [
    "SideAware", "Stats", "load", "sideaware_init", "sideaware_enabled", "sideaware_create_kernel",
    "sideaware_torch_side_index", "sideaware_gpu_side_index", "sideaware_cpu_side_index",
    "sideaware_info", "sideaware_info_raw",
]
