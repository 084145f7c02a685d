"""A model assembled from a description: embedding, the layers' parts, the run order,
final norm and head.  It owns the weights and knows nothing of requests, pages or
scheduling; ``forward`` runs exactly the rows it is given against the caches it is
handed (the reference's counterpart is the body of ``forward_paged_batch``,
model/src/qwen3_paged_batch.cpp:81-346).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts import registry
from ..parts.spec import CacheSpec, ModelDescription, ParamSpec, PartSpec, StateSpec


def _make(category: str, spec: PartSpec, dtype, device):
    return registry.lookup(category, spec.kind)(dtype=dtype, device=device, **spec.params)


def _specs(category: str, spec: PartSpec) -> Dict[str, ParamSpec]:
    return {spec.prefix + k: v for k, v in
            registry.lookup(category, spec.kind).param_specs(**spec.params).items()}


_ROLE_CATEGORY = {"norm1": "norm", "norm2": "norm", "norm": "norm", "mixer": "mixer",
                  "ffn": "feed_forward", "feed_forward": "feed_forward"}


def role_category(role: str) -> str:
    try:
        return _ROLE_CATEGORY[role]
    except KeyError:
        raise KeyError(f"a block role must be one of {sorted(_ROLE_CATEGORY)}, got {role!r}") from None


def expected_tensors(desc: ModelDescription) -> Tuple[Dict[str, ParamSpec], List[str]]:
    """(name -> ParamSpec for every tensor the model reads, names that may be present
    without being read)."""
    out: Dict[str, ParamSpec] = {}
    out.update(_specs("embedding", desc.embedding))
    for layer in desc.layers:
        for role, spec in layer.parts.items():
            out.update(_specs(role_category(role), spec))
    out.update(_specs("norm", desc.final_norm))
    head = _specs("head", desc.head)
    out.update(head)
    ignorable = [] if head else [desc.head.prefix + "weight"]
    return out, ignorable


class Model:
    def __init__(self, desc: ModelDescription, dtype: torch.dtype, device):
        self.desc, self.dtype, self.device = desc, dtype, device
        self.embedding = _make("embedding", desc.embedding, dtype, device)
        self.blocks = []
        self._parts: List[Tuple[PartSpec, object]] = [(desc.embedding, self.embedding)]
        for layer in desc.layers:
            parts = {}
            for role, spec in layer.parts.items():
                parts[role] = _make(role_category(role), spec, dtype, device)
                self._parts.append((spec, parts[role]))
            block_cls = registry.lookup("block", layer.block)
            missing = [r for r in block_cls.roles if r not in parts]
            if missing:
                raise ValueError(f"block {layer.block!r} needs parts {missing}")
            self.blocks.append(block_cls(parts))
        self.final_norm = _make("norm", desc.final_norm, dtype, device)
        self.head = _make("head", desc.head, dtype, device)
        self._parts += [(desc.final_norm, self.final_norm), (desc.head, self.head)]
        self.order = desc.resolved_order()          # (layer, cache id, writes)
        self.loaded = False

    # ---- weights
    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand every part its tensors (names without the part's prefix).  Entries are
        removed from ``tensors`` as they are consumed so that fused copies do not double
        the memory for long."""
        for spec, part in self._parts:
            names = type(part).param_specs(**spec.params)
            part.load({k: tensors.pop(spec.prefix + k) for k in names})
        if hasattr(self.head, "tie"):
            self.head.tie(self.embedding)
        self.loaded = True

    # ---- what the cache manager must provide, per cache id
    def cache_needs(self) -> Dict[int, Tuple[Optional[CacheSpec], Optional[StateSpec]]]:
        needs: Dict[int, Tuple[Optional[CacheSpec], Optional[StateSpec]]] = {}
        for layer, cache_id, _ in self.order:
            mixer = self.blocks[layer].mixer
            need = (mixer.cache_spec(), mixer.state_spec())
            if cache_id in needs and needs[cache_id] != need:
                raise ValueError(f"cache {cache_id} is shared by mixers with different needs")
            needs[cache_id] = need
        return needs

    # ---- one step
    def forward(self, ctx, caches) -> torch.Tensor:
        """Logits [len(ctx.want_rows), vocab] float32.  ``caches.view(cache_id, writes)``
        gives the ``LayerCacheView`` of a visit."""
        h = self.embedding.forward(ctx.token_ids)
        pending = None
        for layer, cache_id, writes in self.order:
            pending = self.blocks[layer].forward(h, pending, ctx, caches.view(cache_id, writes))
        x = self.final_norm.forward(h, pending, rows=ctx.want_rows)
        return self.head.forward(x)
