"""Arrangements of parts in a layer.

``prenorm`` is the Llama arrangement (umarhassan-cloud/kvforge, src/tokenvault/model.py:185-187):
``h = h + mixer(norm1(h)); h = h + ffn(norm2(h))``.  Each sum is folded into the norm that
follows it, so a block takes the sum still pending from the block before (``delta``) and
hands back its own.
"""

from __future__ import annotations

from .base import Block, PartSpec, build_part, register_block


def _spec(v) -> PartSpec:
    if isinstance(v, PartSpec):
        return v
    return PartSpec(v["kind"], v.get("params", {}))


@register_block("prenorm")
class PreNormBlock(Block):
    """params: ``norm1``, ``mixer``, ``norm2``, ``ffn`` (``PartSpec`` each) and the weight-name
    stems ``norm1_name``, ``mixer_name``, ``norm2_name``, ``ffn_name`` under the layer's prefix."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        names = {
            "norm1": params.get("norm1_name", "input_layernorm"),
            "mixer": params.get("mixer_name", "self_attn"),
            "norm2": params.get("norm2_name", "post_attention_layernorm"),
            "ffn": params.get("ffn_name", "mlp"),
        }
        self.norm1 = build_part("norm", _spec(params["norm1"]), f"{prefix}{names['norm1']}.")
        self.mixer = build_part("mixer", _spec(params["mixer"]), f"{prefix}{names['mixer']}.")
        self.norm2 = build_part("norm", _spec(params["norm2"]), f"{prefix}{names['norm2']}.")
        self.ffn = build_part("ffn", _spec(params["ffn"]), f"{prefix}{names['ffn']}.")

    def sub_parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def mixer_part(self):
        return self.mixer

    def forward(self, ctx, resid, delta, cache):
        x = self.norm1.forward(ctx, resid, delta)
        a = self.mixer.forward(ctx, x, cache)
        x = self.norm2.forward(ctx, resid, a)
        return self.ffn.forward(ctx, x)
