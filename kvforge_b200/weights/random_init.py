"""Random weights from a configuration and a seed.

Distribution as umarhassan-cloud/kvforge's ``build_model`` (src/tokenvault/model_loader.py:42-61):
matrices ~ N(0, ``init_std``) with ``init_std = 0.02``, norm weights 1.  Each tensor is drawn
from a generator seeded with the seed and the tensor's name, so a tensor's values do not
depend on which other tensors exist or where they are made.  (The values are not those of
kvforge's generator; nothing depends on that.)

``write_model_dir`` writes a model folder (``config.json`` + ``model.safetensors``) that the
loader, or any other program, can read.  ``random_weights`` makes the same tensors straight
on a device, for shapes too large to pass through a file.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from ..parts.base import WeightDecl
from .loader import place
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device: torch.device | str) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(h[:8], "little") & ((1 << 63) - 1))
    return g


def draw(name: str, decl: WeightDecl, seed: int, device: torch.device | str = "cpu", init_std: float = 0.02, norm_std: float = 0.0) -> torch.Tensor:
    """One tensor in float32 on ``device``."""
    g = _generator(seed, name, device)
    if decl.kind == "table":
        return torch.zeros(decl.shape, dtype=torch.int32, device=device)
    if decl.init == "ones":
        t = torch.ones(decl.shape, dtype=torch.float32, device=device)
        if norm_std:
            t += norm_std * torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device)
        return t
    return init_std * torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device)


def random_weights(
    expected: dict[str, WeightDecl],
    seed: int,
    dtype: torch.dtype,
    device: torch.device | str,
    init_std: float = 0.02,
    norm_std: float = 0.0,
    skip: tuple[str, ...] = (),
) -> dict[str, torch.Tensor]:
    """The model's tensors made on ``device`` in the types the loader would hold them in."""
    out = {}
    for name, decl in expected.items():
        if name in skip:
            continue
        out[name] = place(draw(name, decl, seed, device, init_std, norm_std), decl, dtype, device)
    return out


def write_model_dir(
    model_dir: str | Path,
    config_json: dict,
    expected: dict[str, WeightDecl],
    seed: int,
    store_dtype: torch.dtype = torch.bfloat16,
    init_std: float = 0.02,
    norm_std: float = 0.0,
    skip: tuple[str, ...] = (),
    device: torch.device | str = "cpu",
) -> Path:
    """Write ``config.json`` and ``model.safetensors``.  Floating tensors are stored in
    ``store_dtype``; ``skip`` names tensors to leave out (a tied output head).  ``device``:
    where the values are drawn (a device's generator draws other values than the host's; the
    folder is the record either way)."""
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    tensors = {}
    for name, decl in expected.items():
        if name in skip:
            continue
        t = draw(name, decl, seed, device, init_std, norm_std)
        tensors[name] = (t if decl.kind == "table" else t.to(store_dtype)).cpu()
    write_safetensors(d / "model.safetensors", tensors)
    (d / "config.json").write_text(json.dumps(config_json, indent=2))
    return d
