"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed, or the same tensors made directly on a device.

The reference has no such mode.  Every tensor has its own generator, keyed by
(seed, tensor name), so its values do not depend on the order or the sharding in which
tensors are made.  Matrices and embeddings are N(0, std), norm gains uniform in
``norm_range``, integer tables zero; values are drawn in float32 and rounded to the
storage type.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Tuple

import torch

from ..config.base import ModelConfig, describe_model
from ..parts.spec import ParamSpec
from .safetensors_io import save_file, save_sharded


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec: ParamSpec, seed: int, std: float, norm_range: Tuple[float, float],
                  dtype: torch.dtype, device) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    if spec.init == "index":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "norm":
        lo, hi = norm_range
        t = torch.rand(spec.shape, generator=gen, dtype=torch.float32, device=device) * (hi - lo) + lo
        return t.to(dtype)
    if spec.init == "normal":
        rows = spec.shape[0] if spec.shape else 1
        if len(spec.shape) == 2 and rows * spec.shape[1] > (1 << 26):
            # large matrices in slabs, so that the float32 draw never doubles the footprint
            out = torch.empty(spec.shape, dtype=dtype, device=device)
            step = max(1, (1 << 26) // spec.shape[1])
            for r0 in range(0, rows, step):
                r1 = min(rows, r0 + step)
                out[r0:r1] = (torch.randn((r1 - r0, spec.shape[1]), generator=gen, dtype=torch.float32,
                                          device=device) * std).to(dtype)
            return out
        return (torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * std).to(dtype)
    raise ValueError(f"{name}: unknown init {spec.init!r}")


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
