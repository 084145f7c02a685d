"""Typed configuration of the Qwen3 dense architecture, read from its own config.json keys.

The reference reads ``model_type``, the six sizes, ``max_position_embeddings``,
``head_dim`` (0 or absent means hidden/heads), ``rms_norm_eps`` (default 1e-6) and
``rope_theta`` (default 1e6) (model/src/qwen3_checkpoint.cpp:29-46) and derives
``kv_dim``, ``kv_mul`` and the query width (model/src/qwen3_checkpoint.cpp:175-190).
It never reads ``tie_word_embeddings``, the sliding-window keys, ``attention_bias``
or ``rope_scaling``; this class reads them so that a checkpoint that needs them is
either run as it asks or refused, never run wrongly.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, coerce, optional, require

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    # A query at position p in a sliding layer sees the keys p-sliding_window+1 .. p.
    sliding_window: Optional[int] = None
    layer_types: Tuple[str, ...] = ()
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = field(default="Qwen3ForCausalLM")

    # ---- derived sizes (reference: model/src/qwen3_checkpoint.cpp:175-190) ----
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        """Query heads per key/value head (the reference's ``kv_mul``)."""
        return self.num_attention_heads // self.num_key_value_heads

    def window_of_layer(self, layer: int) -> Optional[int]:
        return self.sliding_window if self.layer_types[layer] == SLIDING_ATTENTION else None

    # ---- reading ----
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        model_type = raw.get("model_type", "qwen3")
        if model_type != "qwen3":
            raise ConfigError(f"config.json: model_type {model_type!r} is not 'qwen3'")
        hidden = require(raw, "hidden_size")
        heads = require(raw, "num_attention_heads")
        layers = require(raw, "num_hidden_layers")
        head_dim = optional(raw, "head_dim", 0)
        if head_dim == 0:
            if heads <= 0 or hidden % heads:
                raise ConfigError("config.json: head_dim is absent and hidden_size is not a "
                                  "multiple of num_attention_heads")
            head_dim = hidden // heads
        if raw.get("rope_scaling") not in (None, {}):
            rs = raw["rope_scaling"]
            kind = rs.get("rope_type", rs.get("type")) if isinstance(rs, dict) else rs
            if kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling {rs!r} is not supported")
        if optional(raw, "attention_bias", False, bool):
            raise ConfigError("config.json: attention_bias=true is not part of Qwen3 dense")
        act = optional(raw, "hidden_act", "silu", str)

        window = None
        layer_types: Tuple[str, ...]
        use_window = optional(raw, "use_sliding_window", False, bool)
        if raw.get("layer_types") is not None:
            lt = raw["layer_types"]
            if not isinstance(lt, (list, tuple)) or len(lt) != layers:
                raise ConfigError("config.json: layer_types must list one entry per layer")
            layer_types = tuple(coerce(x, "layer_types[]", str) for x in lt)
        elif use_window:
            first_sliding = optional(raw, "max_window_layers", layers)
            layer_types = tuple(SLIDING_ATTENTION if i >= first_sliding else FULL_ATTENTION
                                for i in range(layers))
        else:
            layer_types = tuple(FULL_ATTENTION for _ in range(layers))
        if SLIDING_ATTENTION in layer_types:
            window = require(raw, "sliding_window")

        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(coerce(x, "eos_token_id[]", int) for x in eos)
        else:
            eos_ids = (coerce(eos, "eos_token_id", int),)
        bos = raw.get("bos_token_id")
        return cls(
            hidden_size=hidden,
            intermediate_size=require(raw, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=optional(raw, "num_key_value_heads", heads),
            head_dim=head_dim,
            vocab_size=require(raw, "vocab_size"),
            max_position_embeddings=require(raw, "max_position_embeddings"),
            rms_norm_eps=optional(raw, "rms_norm_eps", 1e-6, float),
            rope_theta=optional(raw, "rope_theta", 1e6, float),
            tie_word_embeddings=optional(raw, "tie_word_embeddings", False, bool),
            hidden_act=act,
            sliding_window=window,
            layer_types=layer_types,
            eos_token_ids=eos_ids,
            bos_token_id=None if bos is None else coerce(bos, "bos_token_id", int),
        )

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "rope_scaling": None,
        }
        if SLIDING_ATTENTION in self.layer_types:
            out["use_sliding_window"] = True
            out["sliding_window"] = self.sliding_window
            out["layer_types"] = list(self.layer_types)
        else:
            out["use_sliding_window"] = False
        if self.eos_token_ids:
            out["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                   else list(self.eos_token_ids))
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out

    def validate(self) -> None:
        """Positive sizes and a whole number of query heads per key/value head, as the
        reference checks (model/src/qwen3_checkpoint.cpp:175-190); its extra demand that
        hidden_size be a multiple of the head count (model/src/model.cpp:57-59) is not
        needed by Qwen3 (the head width is its own key) and is dropped."""
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be positive, got {getattr(self, name)}")
        if self.num_key_value_heads > self.num_attention_heads \
                or self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("config.json: num_attention_heads must be a multiple of "
                              "num_key_value_heads")
        if self.head_dim % 2:
            raise ConfigError("config.json: head_dim must be even (rotary pairs)")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if not (self.rope_theta > 0):
            raise ConfigError("config.json: rope_theta must be positive")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act {self.hidden_act!r} is not 'silu'")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError("config.json: layer_types must list one entry per layer")
        for t in self.layer_types:
            if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                raise ConfigError(f"config.json: unknown layer type {t!r}")
        if SLIDING_ATTENTION in self.layer_types and not (self.sliding_window and self.sliding_window > 0):
            raise ConfigError("config.json: sliding layers need a positive sliding_window")
        for tok in self.eos_token_ids:
            if not 0 <= tok < self.vocab_size:
                raise ConfigError(f"config.json: eos_token_id {tok} is outside the vocabulary")
