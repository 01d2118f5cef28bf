"""torch.ops.sideaware.* registration (the custom ops of test.py:147-157, plus rope_forward,
rope_backward, rope_freqs and silu_mul).  Kept in a module of its own WITHOUT postponed annotation evaluation:
torch.library.infer_schema reads the real annotation objects."""
from typing import Optional

import torch
from torch import Tensor

_registered = {}


def register(sa) -> None:
    """Registers the ops once per process, bound to the loaded library `sa`."""
    if _registered:
        return

    def memcpy(dst: Tensor, src: Tensor) -> None:
        sa.memcpy(dst, src)

    def one_to_one(kernel_id: int, dst: Tensor, src: Tensor) -> None:
        sa.one_to_one(kernel_id, dst, src)

    def elementwise(kernel_id: int, out0: Tensor, out1: Optional[Tensor], out2: Optional[Tensor],
                    out3: Optional[Tensor], in0: Optional[Tensor], in1: Optional[Tensor], in2: Optional[Tensor],
                    in3: Optional[Tensor], sideband_tensor: Optional[Tensor] = None, sideband_value: int = 0,
                    parallel_chunks: int = 0, forced_sm_per_side: int = 0) -> None:
        sa.elementwise(kernel_id, out0, out1, out2, out3, in0, in1, in2, in3, sideband_tensor, sideband_value,
                       parallel_chunks, forced_sm_per_side)

    def rope_forward(qkv: Tensor, freqs_cis: Tensor, n_q_heads: int, n_kv_heads: int) -> None:
        sa.rope_forward(qkv, freqs_cis, n_q_heads, n_kv_heads)

    def rope_backward(dqkv: Tensor, freqs_cis: Tensor, n_q_heads: int, n_kv_heads: int) -> None:
        sa.rope_backward(dqkv, freqs_cis, n_q_heads, n_kv_heads)

    def rope_freqs(freqs_cis: Tensor, theta: float, use_scaled: bool) -> None:
        sa.rope_precompute_freqs_into(freqs_cis, theta, use_scaled)

    def silu_mul(out: Tensor, a: Tensor, b: Tensor, scale: float) -> None:
        sa.silu_mul(out, a, b, scale)

    lib = torch.library.Library("sideaware", "FRAGMENT")

    def reg(name, fn, mutates):
        schema = torch.library.infer_schema(fn, mutates_args=mutates)
        lib.define(name + schema)
        lib.impl(name, fn, "CUDA")

    reg("memcpy", memcpy, ["dst"])
    reg("one_to_one", one_to_one, ["dst"])
    reg("elementwise", elementwise, ["out0", "out1", "out2", "out3", "sideband_tensor"])
    reg("rope_forward", rope_forward, ["qkv"])
    reg("rope_backward", rope_backward, ["dqkv"])
    reg("rope_freqs", rope_freqs, ["freqs_cis"])
    reg("silu_mul", silu_mul, ["out"])
    _registered["lib"] = lib
