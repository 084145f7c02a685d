"""RMSNorm, fused with the residual sum that precedes it.

x = gain * v / sqrt(mean(v^2) + eps) with eps inside the root and the gain multiplying
directly, no "1 + gain" (reference: kernels/src/rmsnorm_kernel_cuda.cu:17-38).  The
reference adds the residual in a separate half-precision kernel
(model/src/qwen3_paged_batch.cpp:273-279); here the sum is float32 and happens in the
same pass that computes the norm.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .registry import register
from .spec import ParamSpec


@register("norm", "rmsnorm")
class RMSNorm:
    def __init__(self, width: int, eps: float, dtype: torch.dtype, device):
        self.width, self.eps, self.dtype, self.device = int(width), float(eps), dtype, device
        self.gain: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, width: int, eps: float) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((int(width),), "norm")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gain = tensors["weight"].contiguous()

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.dtype, device=h.device)
        return ops.add_rmsnorm(h, delta, self.gain, self.eps, out, rows)
