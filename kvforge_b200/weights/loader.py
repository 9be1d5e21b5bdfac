"""Weights by tensor name, with one error that says everything that is wrong.

The names a model needs come from its parts (``DecoderModel.expected_weights``); for the
Llama decoder they are umarhassan-cloud/kvforge's parameter names under the ``model.`` prefix
that its importer strips (src/tokenvault/model_loader.py:104), with ``lm_head.weight``
optional (model_loader.py:105-106).  kvforge reports missing tensors only and lets torch
report shapes (model_loader.py:108-111); here missing, unexpected and wrongly shaped
tensors are gathered into a single ``WeightsError``.

Storage: matrices go to the engine's storage type (bfloat16 stays bfloat16; float32 is
chosen by ``dtype=float32``); vectors are held in float32, so a tensor stored in 32-bit
keeps every bit and a 16-bit one is widened exactly; integer tables are held as int32.
"""

from __future__ import annotations

from pathlib import Path

import torch

from ..parts.base import WeightDecl
from .safetensors_io import open_model_files


class WeightsError(RuntimeError):
    """Lists ``missing``, ``unexpected`` and ``wrong_shape`` tensors of a checkpoint."""

    def __init__(self, missing: list[str], unexpected: list[str], wrong_shape: list[str], where: str = "") -> None:
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"checkpoint {where} does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape or type ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        super().__init__("\n".join(lines))


def _is_float(dt: torch.dtype) -> bool:
    return dt in (torch.float32, torch.bfloat16, torch.float16, torch.float64)


def place(t: torch.Tensor, decl: WeightDecl, dtype: torch.dtype, device: torch.device | str) -> torch.Tensor:
    """Move one checkpoint tensor to the device in the type its kind is held in."""
    if decl.kind == "matrix":
        return t.to(device=device, dtype=dtype).contiguous()
    if decl.kind == "vector":
        return t.to(device=device, dtype=torch.float32).contiguous()
    if decl.kind == "table":
        return t.to(device=device, dtype=torch.int32).contiguous()
    raise ValueError(f"unknown weight kind {decl.kind!r}")


def load_weights(
    model_dir: str | Path,
    expected: dict[str, WeightDecl],
    dtype: torch.dtype,
    device: torch.device | str,
    ignore_suffixes: tuple[str, ...] = (),
) -> dict[str, torch.Tensor]:
    files = open_model_files(model_dir)
    found: dict[str, tuple] = {}
    for f in files:
        for name in f.keys():
            found[name] = (f, *f.info(name))
    missing = [n for n, d in expected.items() if n not in found and not d.optional]
    unexpected = [n for n in found if n not in expected and not any(n.endswith(s) for s in ignore_suffixes)]
    wrong = []
    for name, decl in expected.items():
        if name not in found:
            continue
        _, dt, shape = found[name]
        if tuple(shape) != tuple(decl.shape):
            wrong.append(f"{name}: expected {list(decl.shape)}, found {list(shape)}")
        elif decl.kind == "table" and _is_float(dt):
            wrong.append(f"{name}: expected an integer table, found {dt}")
        elif decl.kind != "table" and not _is_float(dt):
            wrong.append(f"{name}: expected floating point, found {dt}")
    if missing or unexpected or wrong:
        raise WeightsError(sorted(missing), sorted(unexpected), wrong, str(model_dir))
    out = {}
    for name, decl in expected.items():
        if name in found:
            out[name] = place(found[name][0].tensor(name), decl, dtype, device)
    for f in files:
        f.close()
    return out
