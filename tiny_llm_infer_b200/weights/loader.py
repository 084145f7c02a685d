"""Weights by tensor name.

``load_weights`` is given the tensors a model expects (name -> shape, from the parts'
own declarations) and a model folder.  It compares the two completely before it reads
a byte of data and raises one ``WeightsError`` that lists every missing tensor, every
unexpected tensor and every wrong shape.  The reference stops at the first missing
tensor or shape mismatch (model/src/qwen3_layers.cpp:79-108) and never notices
tensors it does not use.

Storage rule: floating tensors are kept in the mode's storage type (bfloat16, or
float32 in float32 mode) except that a tensor the file stores in 32-bit stays 32-bit;
integer tables become int32.  Nothing is renamed here; fusing of projections is the
business of the part that owns them.
"""
from __future__ import annotations

from typing import Dict, Iterable, Optional

import torch

from ..parts.spec import ParamSpec
from .safetensors_io import SafetensorsError, SafetensorsFile, checkpoint_files


class WeightsError(ValueError):
    def __init__(self, where, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)      # (name, expected, found)
        self.wrong_dtype = list(wrong_dtype)      # (name, found)
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unsupported dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOATS = ("F32", "BF16", "F16", "F64")
_INTS = ("I64", "I32", "I16", "I8", "U8")


def stored_dtype(file_dtype: str, mode: torch.dtype, integer: bool) -> Optional[torch.dtype]:
    """The dtype a tensor is kept in, or None if its file dtype cannot serve."""
    if integer:
        return torch.int32 if file_dtype in _INTS else None
    if file_dtype not in _FLOATS:
        return None
    if mode == torch.float32 or file_dtype in ("F32", "F64"):
        return torch.float32
    return mode


def load_weights(model_path, expected: Dict[str, ParamSpec], mode: torch.dtype, device,
                 ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """All expected tensors, on ``device``.  ``ignorable`` names may be present in the
    files without being expected (a tied head's duplicate, for instance)."""
    try:
        files = [SafetensorsFile(p) for p in checkpoint_files(model_path)]
    except SafetensorsError as exc:
        raise WeightsError(model_path, wrong_dtype=[("(container)", str(exc))]) from None
    try:
        found = {}
        for f in files:
            for name, info in f.tensors.items():
                found[name] = (f, info)
        ignorable = set(ignorable)
        missing = sorted(n for n in expected if n not in found)
        unexpected = sorted(n for n in found if n not in expected and n not in ignorable)
        wrong_shape, wrong_dtype = [], []
        for name, spec in expected.items():
            if name not in found:
                continue
            info = found[name][1]
            if tuple(info.shape) != tuple(spec.shape):
                wrong_shape.append((name, spec.shape, info.shape))
            if stored_dtype(info.dtype, mode, spec.init == "index") is None:
                wrong_dtype.append((name, info.dtype))
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightsError(model_path, missing, unexpected, wrong_shape, wrong_dtype)
        out = {}
        for name, spec in expected.items():
            f, info = found[name]
            keep = stored_dtype(info.dtype, mode, spec.init == "index")
            out[name] = f.read(name).to(device=device, dtype=keep, copy=True)
        return out
    finally:
        for f in files:
            f.close()
