"""Output head: float logits of the wanted rows, ``x @ W^T`` with ``W [vocab, hidden]``
(umarhassan-cloud/kvforge ``lm_head``, src/tokenvault/model.py:156-158,190-191), the embedding's
tensor when the model ties the two."""

from __future__ import annotations

import torch

from .. import ops
from .base import Head, WeightDecl, register_head


@register_head("linear_head")
class LinearHead(Head):
    """params: ``vocab_size``, ``hidden_size``.  Its tensor is optional in a checkpoint."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.weight = None

    @classmethod
    def weight_decls(cls, params):
        return {"weight": WeightDecl((int(params["vocab_size"]), int(params["hidden_size"])), optional=True)}

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.weight = weights.get("weight")

    def tie(self, table):
        self.weight = table

    def forward(self, ctx, x):
        rt = self.rt
        r = x.shape[0]
        logits = rt.buf("model.logits", r, self.vocab, torch.float32, cap=rt.max_seqs)
        if ops.skinny_ok(x, self.weight):
            ops.gemm_skinny(x, self.weight, logits)
        else:
            ops.linear(x, self.weight, logits)
        return logits
