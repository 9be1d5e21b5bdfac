"""Token embedding: the row of a ``[vocab, hidden]`` table per token, widened into the float
residual stream (umarhassan-cloud/kvforge ``embed_tokens``, src/tokenvault/model.py:170,183; no
scaling for the Llama decoder)."""

from __future__ import annotations

from .. import ops
from .base import Embedding, WeightDecl, register_embedding


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size``, ``hidden_size``.  A token id outside the table raises the device
    error flag (bit 0) and reads row 0."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])

    @classmethod
    def weight_decls(cls, params):
        return {"weight": WeightDecl((int(params["vocab_size"]), int(params["hidden_size"])))}

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.weight = weights["weight"]

    def table(self):
        return self.weight

    def forward(self, ctx, resid):
        ops.embed(self.weight, ctx.token_ids, resid, self.rt.err, ctx.feedback_rows, ctx.token_feedback)
