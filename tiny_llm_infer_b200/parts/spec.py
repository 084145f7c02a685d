"""Data that describes a model: which parts each layer is made of and in which order
the layers run.  An architecture's ``describe(config)`` returns a ``ModelDescription``;
everything below it (weights, cache groups, the step function) is derived from this
data, so no part knows which model it is in.

The reference wires its one decoder layer by hand as a struct of layer pointers
(model/include/qwen3.h:17-45) and loops ``for layer in 0..L`` in its step function
(model/src/qwen3_paged_batch.cpp:144-302).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part owns.  ``init`` is what random-weights mode fills it with:
    ``normal`` (matrices, embeddings), ``norm`` (norm gains, uniform in a range) or
    ``index`` (integer tables, kept as int32)."""
    shape: Tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class PartSpec:
    """A part chosen from a registry (``kind``) with its sizes and constants (``params``)
    and the prefix its tensors carry in the checkpoint."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it arranges."""
    block: str
    parts: Dict[str, PartSpec]


@dataclass(frozen=True)
class ExecEntry:
    """One visit of the run order.  ``layer`` names the layer whose weights run.
    ``cache`` names the cache instance the visit's mixer works on (``None``: an instance
    of its own); for a block with several mixers it is a tuple, one id per mixer in the
    order of the block's roles.  Two visits that name the same ``cache`` share keys and
    values; the one with ``writes_cache=False`` only reads what the other has written in
    this step."""
    layer: int
    cache: Union[None, int, Tuple[int, ...]] = None
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelDescription:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[ExecEntry, ...]
    final_norm: PartSpec
    head: PartSpec

    def resolved_order(self, mixers_per_layer: Optional[Sequence[int]] = None) -> List[Tuple[int, Tuple[int, ...], bool]]:
        """(layer, cache ids, writes) for every visit, one cache id per mixer of the layer's
        block (``mixers_per_layer``; one each if not given), with default ids filled in.
        Cache ids given explicitly keep their value; mixers without one get fresh ids above
        every explicit id."""
        def ids_of(entry) -> Tuple[int, ...]:
            if entry.cache is None:
                return ()
            return (entry.cache,) if isinstance(entry.cache, int) else tuple(entry.cache)

        explicit = [c for e in self.order for c in ids_of(e)]
        next_id = (max(explicit) + 1) if explicit else 0
        out = []
        for e in self.order:
            if e.layer < 0 or e.layer >= len(self.layers):
                raise ValueError(f"run order names layer {e.layer}, model has {len(self.layers)}")
            count = 1 if mixers_per_layer is None else mixers_per_layer[e.layer]
            ids = ids_of(e)
            if not ids:
                ids = tuple(range(next_id, next_id + count))
                next_id += count
            elif len(ids) != count:
                raise ValueError(f"visit of layer {e.layer} names {len(ids)} caches, its block has {count} mixers")
            out.append((e.layer, ids, e.writes_cache))
        written = {c for _, ids, w in out if w for c in ids}
        for layer, ids, writes in out:
            if not writes and any(c not in written for c in ids):
                raise ValueError(f"visit of layer {layer} reads a cache among {ids} that no visit writes")
        return out


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps per token in the paged cache: one or more *planes*, each ``heads``
    vectors of ``width`` elements per token (keys and values of grouped-query attention are
    two planes of equal shape; a mixer that caches one compressed vector per token has one
    plane of one head; keys and values of different widths are two planes of different
    shape).  ``window=None`` keeps every token, a number keeps the last ``window``."""
    planes: Tuple[Tuple[int, int], ...]
    window: Optional[int] = None

    @classmethod
    def keys_and_values(cls, kv_heads: int, head_dim: int, window: Optional[int] = None) -> "CacheSpec":
        return cls(((kv_heads, head_dim), (kv_heads, head_dim)), window)

    def __post_init__(self):
        if not self.planes or any(h <= 0 or w <= 0 for h, w in self.planes):
            raise ValueError(f"a cache needs at least one plane of positive size, got {self.planes}")

    @property
    def uniform(self) -> bool:
        """All planes have one shape: the cache is one tensor [pages, planes, heads, page, width]."""
        return all(p == self.planes[0] for p in self.planes)

    @property
    def elements_per_token(self) -> int:
        return sum(h * w for h, w in self.planes)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state a mixer keeps per request (zeroed at admission)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
