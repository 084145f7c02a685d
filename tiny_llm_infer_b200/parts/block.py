"""Arrangements of parts in a layer.

``prenorm``: h += pending; a = mixer(norm1(h)); h += a; m = ffn(norm2(h)); pending = m.
This is the reference's decoder layer (model/src/qwen3_paged_batch.cpp:146-301) with the
two residual sums moved into the norm that follows them; the sum left over after the
last layer is taken by the model's final norm.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .registry import register


class Block:
    """Base of the arrangements.  A block class declares ``roles``: the names of the parts it
    arranges and, for each, the registry it is chosen from (``norm``, ``mixer``,
    ``feed_forward``); any number of each.  The model builds the parts a layer's description
    gives for these names and hands them over; they become attributes under their role names.
    ``forward(h, pending, ctx, cache)``: ``cache`` is the ``LayerCacheView`` of the block's mixer,
    or, for a block with several mixers, the list of their views in the order of ``roles``."""
    roles: Dict[str, str] = {}

    def __init__(self, parts: Dict[str, object]):
        self.parts = {role: parts[role] for role in self.roles}
        for role, part in self.parts.items():
            setattr(self, role, part)

    def mixers(self) -> List[object]:
        """The block's mixers in the order of ``roles`` (the cache manager and the run order give
        each a cache of its own)."""
        return [self.parts[role] for role, category in self.roles.items() if category == "mixer"]


@register("block", "prenorm")
class PreNormBlock(Block):
    roles = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "feed_forward"}

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        x = self.norm1.forward(h, pending)
        a = self.mixer.forward(x, ctx, cache)
        x = self.norm2.forward(h, a)
        return self.ffn.forward(x, ctx)
