"""Rotary position encoding with the rotate-half pairing.

Pair (i, i + d/2), i < d/2, of the first ``rotary_dim`` = d elements of a head:
f_i = theta^(-2i/d), a = pos * f_i in float32,
x'_i = x_i cos a - x_{i+d/2} sin a,  x'_{i+d/2} = x_i sin a + x_{i+d/2} cos a
(reference: kernels/src/rope_kernel_cpu.cpp:127-141 for the table,
kernels/src/rope_kernel_cuda.cu:228-261 for the rotation; it always rotates the whole
head).  The frequencies are computed once on the host in float64 and rounded to
float32; the angle, sine and cosine are computed per token of the step, once per step for
all layers with the same frequencies (``step_table``), so there is no table whose length
bounds the context.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import ops
from .registry import register
from .spec import ParamSpec


@register("position", "rotary_half")
class RotaryHalf:
    def __init__(self, head_dim: int, theta: float, dtype: torch.dtype, device,
                 rotary_dim: Optional[int] = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {head_dim}")
        self.theta = float(theta)
        half = self.rotary_dim // 2
        idx = torch.arange(half, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-2.0 * idx / self.rotary_dim)).to(torch.float32).to(device)

    @classmethod
    def param_specs(cls, **params) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors) -> None:
        pass

    def fused_rotary(self) -> Tuple[torch.Tensor, int]:
        return self.inv_freq, self.rotary_dim

    def step_table(self, ctx) -> Optional[torch.Tensor]:
        """Cosines and sines of this step's positions, [tokens, 2, rotary_dim / 2] float32, made by the
        first layer of the step that asks and kept in the step's context for the others."""
        memo = getattr(ctx, "memo", None)
        if memo is None or not self.inv_freq.is_cuda:
            return None
        key = ("rotary_half", self.theta, self.rotary_dim)
        table = memo.get(key)
        if table is None:
            table = memo[key] = ops.rope_table(ctx.positions, self.inv_freq)
        return table
