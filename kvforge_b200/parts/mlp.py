"""Gated feed-forward (SwiGLU): ``down(silu(gate(x)) * up(x))``, bias-free
(umarhassan-cloud/kvforge ``MLP``, src/tokenvault/model.py:118-132).  The gate and up
projections are one product (weights stacked at load); the gate is applied in 32-bit."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, WeightDecl, register_feed_forward
from .projection import project


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
        gate, up = weights["gate_proj.weight"], weights["up_proj.weight"]
        # bfloat16: gate and up rows alternate in blocks of 8, the order in which the decode
        # product finds gate_i and up_i in one thread; float32: all gates, then all ups
        self.interleaved = gate.dtype == torch.bfloat16 and self.inter % ops.GATE_UP_BLOCK == 0 and self.inter % 8 == 0
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = weights["down_proj.weight"].contiguous()

    def forward(self, ctx, x: torch.Tensor):
        rt = self.rt
        n = x.shape[0]
        act = rt.buf("mlp.act", n, self.inter)
        if self.interleaved and ops.skinny_ok(x, self.w_gate_up):
            ops.gemm_skinny(x, self.w_gate_up, act, mode="silu")  # a few tokens: stream the weights once
        elif self.interleaved and ops.tcgen05_ok(x, self.w_gate_up):
            # many tokens: tcgen05 tensor cores, the gate applied as the accumulator leaves tensor memory
            ops.gemm_tcgen05(x, self.w_gate_up, act, mode="silu", err=rt.err)
        else:
            gu = rt.buf("mlp.gate_up", n, 2 * self.inter)
            ops.linear(x, self.w_gate_up, gu)
            ops.silu_mul(gu, act, interleaved=self.interleaved)
        return project(rt, "mlp.out", act, self.w_down, ctx)
