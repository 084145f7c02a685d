"""Arrangements of parts in a layer.

``prenorm``: h += pending; a = mixer(norm1(h)); h += a; m = ffn(norm2(h)); pending = m.
This is the reference's decoder layer (model/src/qwen3_paged_batch.cpp:146-301) with the
two residual sums moved into the norm that follows them; the sum left over after the
last layer is taken by the model's final norm.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .registry import register


@register("block", "prenorm")
class PreNormBlock:
    roles = ("norm1", "mixer", "norm2", "ffn")

    def __init__(self, parts: Dict[str, object]):
        self.norm1, self.mixer = parts["norm1"], parts["mixer"]
        self.norm2, self.ffn = parts["norm2"], parts["ffn"]

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        x = self.norm1.forward(h, pending)
        a = self.mixer.forward(x, ctx, cache)
        x = self.norm2.forward(h, a)
        return self.ffn.forward(x, ctx)
