"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed, or the same tensors made directly on a device.

The reference has no such mode.  The generator is counter-based: element ``e`` of the tensor
``name`` under ``seed`` is a function of (seed, name, e) alone, a splitmix64 hash turned into a
uniform number in float64 and, for matrices, into a normal one by Box and Muller's
transformation (elements 2p and 2p + 1 are the cosine and the sine branch of pair p).  So a
tensor does not depend on the order or the sharding in which tensors are made, nor on the slabs a
large one is made in, and, being plain integer and float64 torch operations, it is the same on
the CPU and on a GPU: a folder written here and a model filled on the device from the same seed
hold the same weights, and a slow implementation on the host can be given the numbers the engine
runs with.  (The float64 logarithm and cosine of the two may differ in the last bit; after
rounding to float32 and to the storage type that shows in about one element of 2^29.)
Matrices and embeddings are N(0, std), norm gains uniform in ``norm_range``, integer tables zero;
values are rounded to float32 and then to the storage type.
"""
from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path
from typing import Dict, Tuple

import torch

from ..config.base import ModelConfig, describe_model
from ..parts.spec import ParamSpec
from .safetensors_io import save_file, save_sharded

_M64 = (1 << 64) - 1


def _i64(value: int) -> int:
    """An unsigned 64-bit number as the int64 with the same bits."""
    value &= _M64
    return value - (1 << 64) if value >= (1 << 63) else value


_GOLDEN, _C1, _C2 = _i64(0x9E3779B97F4A7C15), _i64(0xBF58476D1CE4E5B9), _i64(0x94D049BB133111EB)
_SECOND = 0x5DEECE66D1CE4E5B          # makes the key of a pair's second uniform number


def _tensor_key(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little")


def _lsr(z: torch.Tensor, k: int) -> torch.Tensor:
    return (z >> k) & ((1 << (64 - k)) - 1)            # logical shift of an int64


def _uniform(key: int, start: int, n: int, device) -> torch.Tensor:
    """float64 in (0, 1) for the counters start .. start + n - 1: splitmix64 of key + counter * golden
    ratio (int64 arithmetic wraps), its top 53 bits, centred in their cell."""
    z = torch.arange(start, start + n, dtype=torch.int64, device=device) * _GOLDEN + _i64(key)
    z = (z ^ _lsr(z, 30)) * _C1
    z = (z ^ _lsr(z, 27)) * _C2
    z = z ^ _lsr(z, 31)
    return (_lsr(z, 11).to(torch.float64) + 0.5) * (1.0 / (1 << 53))


def _normal(key: int, start: int, n: int, device) -> torch.Tensor:
    """float64 N(0, 1) for the elements start .. start + n - 1."""
    first = start // 2
    pairs = (start + n + 1) // 2 - first
    radius = torch.sqrt(-2.0 * torch.log(_uniform(key, first, pairs, device)))
    angle = (2.0 * math.pi) * _uniform(key ^ _SECOND, first, pairs, device)
    both = torch.stack([radius * torch.cos(angle), radius * torch.sin(angle)], dim=1).reshape(-1)
    return both[start - 2 * first:start - 2 * first + n]


def random_tensor(name: str, spec: ParamSpec, seed: int, std: float, norm_range: Tuple[float, float],
                  dtype: torch.dtype, device) -> torch.Tensor:
    key = _tensor_key(seed, name)
    count = math.prod(spec.shape) if spec.shape else 1
    if spec.init == "index":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init not in ("norm", "normal"):
        raise ValueError(f"{name}: unknown init {spec.init!r}")
    out = torch.empty(count, dtype=dtype, device=device)
    slab = 1 << 24                                       # elements made at a time (float64 and int64 temporaries)
    for start in range(0, count, slab):
        n = min(slab, count - start)
        if spec.init == "norm":
            lo, hi = norm_range
            values = _uniform(key, start, n, device) * (hi - lo) + lo
        else:
            values = _normal(key, start, n, device) * std
        out[start:start + n] = values.to(torch.float32).to(dtype)
    return out.view(spec.shape)


def random_tensors(expected: Dict[str, ParamSpec], seed: int, std: float = 0.02,
                   norm_range: Tuple[float, float] = (0.8, 1.2), dtype: torch.dtype = torch.bfloat16,
                   device="cpu") -> Dict[str, torch.Tensor]:
    return {name: random_tensor(name, spec, seed, std, norm_range, dtype, device)
            for name, spec in expected.items()}


def write_random_model(folder, config: ModelConfig, seed: int, std: float = 0.02,
                       norm_range: Tuple[float, float] = (0.8, 1.2),
                       dtype: torch.dtype = torch.bfloat16, shards: int = 1) -> Path:
    """Write ``config.json`` and the weights of ``config`` into ``folder``."""
    from ..models.model import expected_tensors
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    config.validate()
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    expected, _ = expected_tensors(describe_model(config))
    tensors = random_tensors(expected, seed, std, norm_range, dtype, "cpu")
    if shards > 1:
        save_sharded(tensors, folder, shards)
    else:
        save_file(tensors, folder / "model.safetensors",
                  metadata={"format": "pt", "seed": str(seed), "std": str(std)})
    return folder
