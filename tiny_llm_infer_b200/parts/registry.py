"""Registries of the kinds of parts a layer can be made of.

A part is registered under a name in exactly one of five registries (mixer,
feed-forward, norm, position encoding, block arrangement) and is then available to
every architecture's description; tests register toy parts the same way.  Interfaces
(all tensors are CUDA tensors, T = rows of the step, H = model width):

* every part: ``__init__(**params, dtype, device)``; classmethod
  ``param_specs(**params) -> {local name: ParamSpec}``; ``load({local name: tensor})``.
* norm: ``forward(h, delta, rows=None) -> x``.  ``h`` [T, H] float32 is the residual
  stream; ``delta`` (storage dtype, or None) is added to it in float32 first and, without
  ``rows``, written back; the result is the normed rows in storage dtype.
* mixer: ``cache_spec() -> CacheSpec | None``, ``state_spec() -> StateSpec | None``,
  ``forward(x, ctx, cache) -> delta`` with ``x`` [T, H] storage dtype, ``ctx`` the
  ``StepContext`` and ``cache`` the ``LayerCacheView`` of this visit.
* feed-forward: ``forward(x, ctx) -> delta``.
* position encoding: ``apply(q, k, positions)`` rotating views [T, heads, hd] in place;
  optionally ``fused_rotary() -> (inv_freq, rotary_dim)`` when the attention kernel can
  apply it itself.
* block: ``__init__(parts: {role: part})``, ``roles`` (tuple of role names it needs),
  ``forward(h, pending, ctx, cache) -> pending`` where ``pending`` is the delta not yet
  added to ``h``.
"""
from __future__ import annotations

from typing import Callable, Dict

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}

_ALL = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITIONS,
        "block": BLOCKS, "embedding": EMBEDDINGS, "head": HEADS}


def register(category: str, name: str) -> Callable[[type], type]:
    table = _ALL[category]

    def deco(cls: type) -> type:
        table[name] = cls
        cls.kind = name
        return cls
    return deco


def lookup(category: str, name: str) -> type:
    table = _ALL[category]
    if name not in table:
        raise KeyError(f"no {category} part named {name!r}; registered: {sorted(table)}")
    return table[name]


def unregister(category: str, name: str) -> None:
    _ALL[category].pop(name, None)
