"""Minimal safetensors reader/writer (8-byte little-endian header length, JSON header, raw data).

Writer: tensors sorted by (-element size, name) and a header padded to 8 bytes, like the writer of
the reference (atorch/utils/fsdp_save_util.py:139-174). Reader: lazy, returns arbitrary element
ranges of a stored tensor by seeking, so a rank only touches the bytes it needs when a checkpoint is
loaded at a different world size.
"""
from __future__ import annotations

import json
import struct
from typing import Dict, Optional, Tuple

import torch

_DT = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64",
       torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
       torch.bool: "BOOL"}
_RDT = {v: k for k, v in _DT.items()}


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    items = sorted(tensors.items(), key=lambda kv: (-kv[1].element_size(), kv[0]))
    header, off = {}, 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in items:
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for _, t in items:
            c = t.detach().contiguous().cpu()
            f.write(c.reshape(-1).view(torch.uint8).numpy().tobytes() if c.numel() else b"")


class SafeFile:
    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            self.header = json.loads(f.read(n))
        self.data_start = 8 + n
        self.metadata = self.header.pop("__metadata__", {})

    def keys(self):
        return list(self.header.keys())

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        h = self.header[name]
        return _RDT[h["dtype"]], tuple(h["shape"])

    def get_slice(self, name: str, start: int, end: int) -> torch.Tensor:
        """Elements [start, end) of the flattened tensor ``name``."""
        h = self.header[name]
        dt = _RDT[h["dtype"]]
        es = torch.empty((), dtype=dt).element_size()
        b0 = self.data_start + h["data_offsets"][0] + start * es
        with open(self.path, "rb") as f:
            f.seek(b0)
            raw = f.read((end - start) * es)
        return torch.frombuffer(bytearray(raw), dtype=dt) if end > start else torch.empty(0, dtype=dt)

    def get_tensor(self, name: str) -> torch.Tensor:
        dt, shape = self.info(name)
        n = 1
        for s in shape:
            n *= s
        return self.get_slice(name, 0, n).view(shape)


def load_file(path: str) -> Dict[str, torch.Tensor]:
    f = SafeFile(path)
    return {k: f.get_tensor(k) for k in f.keys()}
