"""RMSNorm fused with the residual sum.

Formula of umarhassan-cloud/kvforge's ``RMSNorm`` (src/tokenvault/model.py:35-38):
``y = (x * rsqrt(mean(x^2) + eps)) * w`` in 32-bit, rounded once.  The residual stream
itself is float here, so ``resid + delta`` is a 32-bit sum as well.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, WeightDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: ``dim``, ``eps``."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])

    @classmethod
    def weight_decls(cls, params):
        return {"weight": WeightDecl((int(params["dim"]),), kind="vector", init="ones")}

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.weight = weights["weight"]

    def forward(self, ctx, resid: torch.Tensor, delta, rows: torch.Tensor | None = None, num_rows: int | None = None):
        """``delta``: ``None``, a tensor in the storage type, or ``ops.Partials``."""
        n = num_rows if rows is not None else resid.shape[0]
        out = self.rt.buf("norm.out" if rows is None else "norm.rows", n, self.dim)
        ops.add_rmsnorm(resid, delta, self.weight, out, self.eps, rows)
        return out
