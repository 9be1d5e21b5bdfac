"""Gated feed-forward (SwiGLU): ``down(silu(gate(x)) * up(x))``, bias-free
(umarhassan-cloud/kvforge ``MLP``, src/tokenvault/model.py:118-132).  The gate and up
projections are one product (weights stacked at load); the gate is applied in 32-bit."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, WeightDecl, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``, ``activation`` (only ``"silu"``)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        act = params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"activation {act!r} is not supported (only 'silu')")

    @classmethod
    def weight_decls(cls, params):
        h, i = int(params["hidden_size"]), int(params["intermediate_size"])
        return {
            "gate_proj.weight": WeightDecl((i, h)),
            "up_proj.weight": WeightDecl((i, h)),
            "down_proj.weight": WeightDecl((h, i)),
        }

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.w_gate_up = torch.cat([weights["gate_proj.weight"], weights["up_proj.weight"]], dim=0).contiguous()
        self.w_down = weights["down_proj.weight"].contiguous()

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        n = x.shape[0]
        gu = rt.buf("mlp.gate_up", n, 2 * self.inter)
        ops.linear(x, self.w_gate_up, gu)
        act = rt.buf("mlp.act", n, self.inter)
        ops.silu_mul(gu, act)
        y = rt.buf("mlp.out", n, self.hidden)
        ops.linear(act, self.w_down, y)
        return y
