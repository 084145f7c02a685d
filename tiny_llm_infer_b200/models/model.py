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


def role_categories(block: str) -> Dict[str, str]:
    """role -> registry of its part, as the block class declares them."""
    roles = registry.lookup("block", block).roles
    if not isinstance(roles, dict):
        raise TypeError(f"block {block!r} must declare roles as {{role: registry}}, got {roles!r}")
    return roles


def expected_tensors(desc: ModelDescription) -> Tuple[Dict[str, ParamSpec], List[str]]:
    """(name -> ParamSpec for every tensor the model reads, names that may be present
    without being read)."""
    out: Dict[str, ParamSpec] = {}
    out.update(_specs("embedding", desc.embedding))
    for layer in desc.layers:
        roles = role_categories(layer.block)
        for role, spec in layer.parts.items():
            if role not in roles:
                raise KeyError(f"block {layer.block!r} has roles {sorted(roles)}, the layer names {role!r}")
            out.update(_specs(roles[role], spec))
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
            roles = role_categories(layer.block)
            missing = [r for r in roles if r not in layer.parts]
            unknown = [r for r in layer.parts if r not in roles]
            if missing or unknown:
                raise ValueError(f"block {layer.block!r} has roles {sorted(roles)}: missing {missing}, unknown {unknown}")
            parts = {}
            for role, spec in layer.parts.items():
                parts[role] = _make(roles[role], spec, dtype, device)
                self._parts.append((spec, parts[role]))
            self.blocks.append(registry.lookup("block", layer.block)(parts))
        self.final_norm = _make("norm", desc.final_norm, dtype, device)
        self.head = _make("head", desc.head, dtype, device)
        self._parts += [(desc.final_norm, self.final_norm), (desc.head, self.head)]
        # (layer, one cache id per mixer of its block, writes)
        self.order = desc.resolved_order([len(b.mixers()) for b in self.blocks])
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
        for layer, cache_ids, _ in self.order:
            for mixer, cache_id in zip(self.blocks[layer].mixers(), cache_ids):
                need = (mixer.cache_spec(), mixer.state_spec())
                if cache_id in needs and needs[cache_id] != need:
                    raise ValueError(f"cache {cache_id} is shared by mixers with different needs")
                needs[cache_id] = need
        return needs

    def parts(self) -> List[object]:
        """Every part of the model (embedding, the layers' parts, final norm, head)."""
        return [part for _, part in self._parts]

    def workspace_floats(self, tokens: int, wanted: int) -> int:
        """Float32 words (an upper estimate) of the activations alive at once in a step of ``tokens``
        rows of which ``wanted`` get logits: the residual stream and a handful of rows of the model's
        width, plus the widest thing any one part makes.  A part says what it makes with
        ``workspace_floats(tokens)``; one that does not is taken to stay within the model's width."""
        widest = max([0] + [int(part.workspace_floats(tokens)) for part in self.parts()
                            if part is not self.head and hasattr(part, "workspace_floats")])
        head = int(self.head.workspace_floats(wanted)) if hasattr(self.head, "workspace_floats") else wanted * self.desc.vocab_size
        return 6 * tokens * self.desc.hidden_size + widest + head

    # ---- one step
    def forward(self, ctx, caches) -> torch.Tensor:
        """Logits [len(ctx.want_rows), vocab] float32.  ``caches.view(cache_id, writes)``
        gives the ``LayerCacheView`` of a visit's mixer (a list of them for a block with several)."""
        if hasattr(ctx, "memo"):
            ctx.memo.clear()
        h = self.embedding.forward(ctx.token_ids)
        pending = None
        for layer, cache_ids, writes in self.order:
            views = [caches.view(cache_id, writes) for cache_id in cache_ids]
            pending = self.blocks[layer].forward(h, pending, ctx, views[0] if len(views) == 1 else views)
        x = self.final_norm.forward(h, pending, rows=ctx.want_rows)
        return self.head.forward(x)
