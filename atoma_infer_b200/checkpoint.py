"""Checkpoint reading: a model folder holds `config.json` and one or more `*.safetensors` files.

A safetensors file is an 8-byte little-endian header length, that many bytes of JSON (tensor name ->
dtype, shape, data_offsets) and the raw little-endian data.  The reference loads the same format through
candle's `VarBuilder::from_mmaped_safetensors` (backends/vllm/src/model_executor.rs: model loading);
here the file is memory-mapped and tensors are handed out as torch CPU tensors that view the mapping
(no copy until a loader moves them to the device).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterator, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (np.float64, torch.float64), "F32": (np.float32, torch.float32), "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16), "I64": (np.int64, torch.int64), "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16), "I8": (np.int8, torch.int8), "U8": (np.uint8, torch.uint8), "BOOL": (np.bool_, torch.bool),
}


class SafetensorsFile:
    """Lazy view of one file; `file[name]` returns a CPU tensor backed by the mapping."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: not a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if n > size - 8:
            raise ValueError(f"{self.path}: header length {n} exceeds the file")
        self.header = json.loads(self._f.read(n).decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + n
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        for name, e in self.header.items():
            lo, hi = e["data_offsets"]
            if e["dtype"] not in _DTYPES:
                raise ValueError(f"{self.path}: tensor {name} has unsupported dtype {e['dtype']}")
            count = int(np.prod(e["shape"], dtype=np.int64)) if e["shape"] else 1
            if hi - lo != count * np.dtype(_DTYPES[e["dtype"]][0]).itemsize or self._base + hi > size:
                raise ValueError(f"{self.path}: tensor {name} has inconsistent offsets")

    def keys(self):
        return self.header.keys()

    def __contains__(self, name) -> bool:
        return name in self.header

    def shape(self, name) -> Tuple[int, ...]:
        return tuple(self.header[name]["shape"])

    def __getitem__(self, name) -> torch.Tensor:
        e = self.header[name]
        npdt, tdt = _DTYPES[e["dtype"]]
        lo, hi = e["data_offsets"]
        count = (hi - lo) // np.dtype(npdt).itemsize
        arr = np.frombuffer(self._map, dtype=npdt, count=count, offset=self._base + lo)
        t = torch.from_numpy(arr.copy())      # the mapping is read-only; tensors own their bytes
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(e["shape"])

    def items(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for k in self.header:
            yield k, self[k]


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    """Writes `tensors` in the same format (used by tests and by tools that make random checkpoints)."""
    rev = {v[1]: k for k, v in _DTYPES.items()}
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": rev[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = metadata
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def read_config(model_dir) -> dict:
    with open(Path(model_dir) / "config.json") as f:
        return json.load(f)


def open_checkpoint(model_dir) -> Dict[str, torch.Tensor]:
    """Every tensor of every `*.safetensors` file in the folder, name -> CPU tensor."""
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors file in {model_dir}")
    out: Dict[str, torch.Tensor] = {}
    for p in files:
        f = SafetensorsFile(p)
        for k, t in f.items():
            if k in out:
                raise ValueError(f"tensor {k} appears in more than one file of {model_dir}")
            out[k] = t
    return out
