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
from typing import Any, Dict, List, Optional, Tuple


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
    of its own).  Two visits that name the same ``cache`` share keys and values; the one
    with ``writes_cache=False`` only reads what the other has written in this step."""
    layer: int
    cache: Optional[int] = None
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

    def resolved_order(self) -> List[Tuple[int, int, bool]]:
        """(layer, cache id, writes) for every visit, with default cache ids filled in.
        Cache ids given explicitly keep their value; visits without one get fresh ids
        above every explicit id."""
        explicit = [e.cache for e in self.order if e.cache is not None]
        next_id = (max(explicit) + 1) if explicit else 0
        out = []
        for e in self.order:
            if e.layer < 0 or e.layer >= len(self.layers):
                raise ValueError(f"run order names layer {e.layer}, model has {len(self.layers)}")
            if e.cache is None:
                out.append((e.layer, next_id, e.writes_cache))
                next_id += 1
            else:
                out.append((e.layer, e.cache, e.writes_cache))
        written = {c for _, c, w in out if w}
        for layer, cache, writes in out:
            if not writes and cache not in written:
                raise ValueError(f"visit of layer {layer} reads cache {cache} that no visit writes")
        return out


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer needs from the paged cache: keys and values of ``kv_heads`` heads of
    width ``head_dim`` per token; ``window=None`` keeps every key, a number keeps the
    last ``window`` keys."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state a mixer keeps per request (zeroed at admission)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
