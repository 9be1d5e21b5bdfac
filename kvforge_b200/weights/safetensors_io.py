"""Reading and writing the safetensors container without a model library.

Layout: 8 bytes little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets"}``, then the raw little-endian tensor bytes.  Reading
maps the file and hands out tensors that view it (no copy until they are moved).
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

_TO_TORCH = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


class SafetensorsFile:
    """An open safetensors file: ``keys()``, ``info(name)`` and ``tensor(name)``."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self._f = open(self.path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: not a safetensors file (too short)")
        (hlen,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if hlen <= 0 or 8 + hlen > size:
            raise ValueError(f"{self.path}: not a safetensors file (bad header length)")
        self.header = json.loads(self._f.read(hlen))
        self.header.pop("__metadata__", None)
        self._base = 8 + hlen
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def keys(self) -> list[str]:
        return list(self.header)

    def info(self, name: str) -> tuple[torch.dtype, tuple[int, ...]]:
        meta = self.header[name]
        if meta["dtype"] not in _TO_TORCH:
            raise ValueError(f"{self.path}: tensor {name} has unsupported dtype {meta['dtype']}")
        return _TO_TORCH[meta["dtype"]], tuple(meta["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape = self.info(name)
        lo, hi = self.header[name]["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        t = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._base + lo)
        return t.reshape(shape)

    def close(self) -> None:
        # tensors handed out may still view the map; it is released with them
        self._f.close()


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor]) -> None:
    header: dict[str, dict] = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _FROM_TORCH:
            raise ValueError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _FROM_TORCH[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def open_model_files(model_dir: str | Path) -> list[SafetensorsFile]:
    """``model.safetensors``, or the shards an index names, or every ``*.safetensors`` there."""
    d = Path(model_dir)
    single = d / "model.safetensors"
    index = d / "model.safetensors.index.json"
    if single.is_file():
        return [SafetensorsFile(single)]
    if index.is_file():
        names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        return [SafetensorsFile(d / n) for n in names]
    files = sorted(d.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors file in {d}")
    return [SafetensorsFile(p) for p in files]
