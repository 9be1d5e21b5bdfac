"""Rotary position encoding: the frequency table, with optional llama3 scaling.

Frequencies as umarhassan-cloud/kvforge builds them (src/tokenvault/model.py:44):
``inv_freq[j] = 1 / theta^(2j/d)`` in 32-bit.  The angle ``float(pos) * inv_freq[j]`` and the
rotation of pair ``(j, j + d/2)`` (model.py:47-61) are computed in the kernel
(``csrc/elementwise.cu``), in 32-bit, from this table.

llama3 scaling is not in kvforge; Llama 3.1/3.2 checkpoints need it.  For wavelength
``lam = 2*pi/f`` and original context ``P``: ``lam < P/high`` keeps ``f``; ``lam > P/low`` gives
``f/factor``; between, ``s = (P/lam - low)/(high - low)`` blends ``(1-s)*f/factor + s*f``.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position_encoding


def rotary_inv_freq(rotary_dim: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))


def llama3_scale(inv_freq: torch.Tensor, factor: float, low_freq_factor: float, high_freq_factor: float, original_max_position: int) -> torch.Tensor:
    f = inv_freq.to(torch.float64)
    lam = 2.0 * math.pi / f
    smooth = (original_max_position / lam - low_freq_factor) / (high_freq_factor - low_freq_factor)
    blended = (1.0 - smooth) * f / factor + smooth * f
    out = torch.where(lam < original_max_position / high_freq_factor, f, blended)
    out = torch.where(lam > original_max_position / low_freq_factor, f / factor, out)
    return out.to(torch.float32)


@register_position_encoding("rotary")
class RotaryEmbedding(PositionEncoding):
    """params: ``head_dim``, ``theta``, optional ``rotary_dim`` (leading dims that turn;
    default all) and ``scaling`` (``None`` or the llama3 dict: ``factor``,
    ``low_freq_factor``, ``high_freq_factor``, ``original_max_position_embeddings``)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(params["theta"])
        self.scaling = params.get("scaling")

    def inv_freq_host(self) -> torch.Tensor:
        inv = rotary_inv_freq(self.rotary_dim, self.theta)
        s = self.scaling
        if s:
            inv = llama3_scale(
                inv,
                float(s["factor"]),
                float(s["low_freq_factor"]),
                float(s["high_freq_factor"]),
                int(s["original_max_position_embeddings"]),
            )
        return inv

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.inv_freq = self.inv_freq_host().to(rt.device).contiguous()

    def table(self) -> torch.Tensor:
        return self.inv_freq
