"""Dense gated feed-forward (SwiGLU): d = (silu(x Wg^T) * (x Wu^T)) Wd^T, no biases,
silu(g) = g / (1 + exp(-g)) in float32 (reference: model/src/qwen3_paged_batch.cpp:281-295,
kernels/src/swiglu_kernel_cpu.cpp:20-24).  Gate and up projections are one product with
one weight of 2 I rows, fused at load time: eight rows of Wg, the eight rows of Wu that belong
to them, and so on (``ops.interleave_gate_up``), so that a gate and its up meet in one
accumulator of the products' kernels; [Wg; Wu] if I is no multiple of eight.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .registry import register
from .spec import ParamSpec


@register("feed_forward", "swiglu")
class SwiGLUFeedForward:
    def __init__(self, hidden_size: int, intermediate_size: int, dtype: torch.dtype, device):
        self.hidden, self.inter, self.dtype, self.device = hidden_size, intermediate_size, dtype, device
        self.w_gate_up = self.w_down = None

    @classmethod
    def param_specs(cls, hidden_size, intermediate_size) -> Dict[str, ParamSpec]:
        return {
            "gate_proj.weight": ParamSpec((intermediate_size, hidden_size)),
            "up_proj.weight": ParamSpec((intermediate_size, hidden_size)),
            "down_proj.weight": ParamSpec((hidden_size, intermediate_size)),
        }

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        parts = [t["gate_proj.weight"], t["up_proj.weight"]]
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.interleaved = self.inter % 8 == 0
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(*[p.to(common) for p in parts]).contiguous()
        else:
            self.w_gate_up = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_down = t["down_proj.weight"].contiguous()

    def workspace_floats(self, tokens: int) -> int:
        return 3 * tokens * self.inter          # the product of gate and up, and the activation

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        act = ops.linear_swiglu(x, self.w_gate_up, out_dtype=self.dtype, interleaved=self.interleaved)
        return ops.linear(act, self.w_down, out_dtype=self.dtype)
