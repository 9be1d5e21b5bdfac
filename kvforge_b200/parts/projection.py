"""The product that brings a part's inner width back to the model's width (an attention layer's
output projection, a feed-forward's down projection): which matrix product runs for how many
tokens, and in what form the result is handed on.  Shared by mixers and feed-forwards; it knows
neither."""

from __future__ import annotations

import torch

from .. import ops

PART_ROWS = ops.SKINNY_MAX_M * ops.SKINNY_MAX_SPLIT  # rows of the largest set of split-K slices


def project(rt, name: str, x: torch.Tensor, w: torch.Tensor, ctx=None):
    """``x @ w^T`` back to the model width: the decode product (slices of K, summed by the norm
    that follows) for a few tokens, the library product otherwise.  Given the step's context, the
    library product of many bfloat16 tokens adds its result straight into the float residual
    stream (``ctx.residual``) and ``ops.ADDED`` is returned."""
    n, width = x.shape[0], w.shape[0]
    if ops.skinny_ok(x, w):
        splits = ops.skinny_splits(width, w.shape[1], n)
        if splits > 1:
            part = ops.Partials(rt.buf(name + "_part", splits * n, width, torch.float32, cap=PART_ROWS).view(splits, n, width))
            ops.gemm_skinny(x, w, part)
            return part
        y = rt.buf(name, n, width)
        ops.gemm_skinny(x, w, y)
        return y
    splits = ops.library_splits(n, width, w.shape[1]) if x.dtype == torch.bfloat16 else 1
    if splits > 1:
        # a few dozen tokens: the library product over slices of K, summed by the same norm
        part = ops.Partials(rt.buf(name + "_part", splits * n, width, torch.float32, cap=PART_ROWS).view(splits, n, width))
        ops.linear_split_k(x, w, part)
        return part
    resid = getattr(ctx, "residual", None)
    if resid is not None and x.dtype == torch.bfloat16 and resid.shape[0] >= n and resid.shape[1] == width:
        ops.linear_add(x, w, resid[:n])
        return ops.ADDED
    y = rt.buf(name, n, width)
    ops.linear(x, w, y)
    return y
