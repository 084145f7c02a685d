"""Reading and writing of the safetensors container, by hand.

Layout, as the reference reads it (model/src/qwen3_checkpoint.cpp:93-150): eight bytes
of little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}}``
(``__metadata__`` skipped), then the tensor bytes; offsets are relative to the end of the
header and are bounds-checked.  A folder may hold one ``model.safetensors`` or shards
listed by ``model.safetensors.index.json`` (``weight_map``: tensor name -> file,
model/src/qwen3_checkpoint.cpp:61-83).
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: Path


class SafetensorsFile:
    """One mapped .safetensors file."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as exc:
            raise SafetensorsError(f"cannot open {self.path}: {exc}") from None
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._fh.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as exc:
            raise SafetensorsError(f"{self.path}: header is not JSON ({exc})") from None
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.tensors: Dict[str, TensorInfo] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape = meta["dtype"], tuple(int(x) for x in meta["shape"])
                begin, end = (int(x) for x in meta["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: malformed entry for {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{self.path}: {name!r} has unsupported dtype {dtype}")
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if begin < 0 or end < begin or end > data_len or end - begin != count * _DTYPES[dtype][1]:
                raise SafetensorsError(
                    f"{self.path}: {name!r} offsets [{begin}, {end}) do not match shape {shape} "
                    f"of {dtype} inside {data_len} data bytes")
            self.tensors[name] = TensorInfo(name, dtype, shape, begin, end, self.path)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored (a view into the mapping; copy or move it before close)."""
        info = self.tensors[name]
        dtype, _ = _DTYPES[info.dtype]
        nbytes = info.end - info.begin
        if nbytes == 0:
            return torch.empty(info.shape, dtype=dtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=nbytes,
                            offset=self._data_start + info.begin)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # read-only buffer: we never write through it
            t = torch.from_numpy(raw)
        return t.view(dtype).reshape(info.shape)

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass                            # views still alive; the OS unmaps at exit
            self._map = None
        self._fh.close()


def checkpoint_files(model_path) -> List[Path]:
    """The .safetensors files of a model folder (or the one file given)."""
    path = Path(model_path)
    if path.is_file():
        return [path]
    index = path / "model.safetensors.index.json"
    single = path / "model.safetensors"
    if index.is_file():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError):
            raise SafetensorsError(f"{index}: no weight_map") from None
        files = sorted({str(v) for v in weight_map.values()})
        missing = [f for f in files if not (path / f).is_file()]
        if missing:
            raise SafetensorsError(f"{index} names shards that are absent: {missing}")
        return [path / f for f in files]
    if single.is_file():
        return [single]
    raise SafetensorsError(f"{path}: neither model.safetensors nor model.safetensors.index.json")


def save_file(tensors: Dict[str, torch.Tensor], path, metadata: Dict[str, str] = None) -> None:
    """Write tensors (CPU) to one .safetensors file, in name order, 8-byte aligned header."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"{name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def save_sharded(tensors: Dict[str, torch.Tensor], folder, shards: int) -> None:
    """Write ``shards`` files plus the index that maps names to them."""
    folder = Path(folder)
    names = sorted(tensors)
    weight_map = {}
    for s in range(shards):
        part = {n: tensors[n] for n in names[s::shards]}
        fname = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        save_file(part, folder / fname)
        weight_map.update({n: fname for n in part})
    (folder / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {}, "weight_map": weight_map}, indent=1))
