"""Batched sampling on the device with per-request options.

The options mean what they mean in umarhassan-cloud/kvforge (src/tokenvault/sampling.py:40-88):
temperature 0 is greedy, top-k and top-p cut the distribution before the draw.  kvforge
draws every row from one generator, so a request's tokens depend on its neighbours in the
batch; here each request has a random stream of its own: the key of its ``i``-th output
token is ``base(seed, request) + i``, and the draw depends on the key alone.
"""

from __future__ import annotations

import hashlib
from collections.abc import Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams

_MASK63 = (1 << 63) - 1


def request_stream_base(engine_seed: int, request_id: str, params: SamplingParams) -> int:
    """First key of a request's random stream."""
    if params.seed is not None:
        src = f"seed:{params.seed}"
    else:
        src = f"engine:{engine_seed}:{request_id}"
    return int.from_bytes(hashlib.sha256(src.encode()).digest()[:8], "little") & _MASK63


class Sampler:
    """``sample(logits, params, keys)`` -> int32 token ids on the device."""

    def __init__(self, device: torch.device | str, max_rows: int, tokens: torch.Tensor | None = None) -> None:
        """``tokens``: an int32 device buffer of ``max_rows`` entries to sample into (default: one of
        the sampler's own)."""
        self.device = torch.device(device)
        self.max_rows = m = max(1, int(max_rows))
        # int32 words: temperatures [0, m), top-k [m, 2m), top-p [2m, 3m), keys (int64) [4m, 6m)
        self._host = torch.empty(6 * m, dtype=torch.int32, pin_memory=True)
        self._dev = torch.empty(6 * m, dtype=torch.int32, device=self.device)
        if tokens is not None and (tokens.dtype != torch.int32 or tokens.numel() < m or not tokens.is_cuda):
            raise ValueError("the token buffer must be int32 on the device with a place per row")
        self._tokens = tokens if tokens is not None else torch.empty(m, dtype=torch.int32, device=self.device)
        self._argmax_scratch = torch.empty(m * ops.ARGMAX_CHUNKS, dtype=torch.int64, device=self.device)
        self._copied: torch.cuda.Event | None = None

    def _grow(self, rows: int) -> None:
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows to sample, but the sampler was made for {self.max_rows}")

    def sample(
        self,
        logits: torch.Tensor,
        params: Sequence[SamplingParams],
        keys: Sequence[int],
        probs_out: torch.Tensor | None = None,
    ) -> torch.Tensor:
        r = logits.shape[0]
        if len(params) != r or len(keys) != r:
            raise ValueError("one SamplingParams and one key per logits row")
        self._grow(r)
        m = self.max_rows
        tokens = self._tokens[:r]
        if all(p.greedy for p in params):
            if probs_out is None:
                ops.argmax(logits, tokens, self._argmax_scratch)
            else:
                ops.sample(logits, tokens, probs_out=probs_out)
            return tokens
        if self._copied is not None:
            self._copied.synchronize()  # the last call's copy has left the host buffer
        h = self._host.numpy()
        h[0:r] = np.array([p.temperature for p in params], dtype=np.float32).view(np.int32)
        h[m : m + r] = [p.top_k for p in params]
        h[2 * m : 2 * m + r] = np.array([p.top_p for p in params], dtype=np.float32).view(np.int32)
        h[4 * m : 4 * m + 2 * r] = np.array([int(x) & _MASK63 for x in keys], dtype=np.int64).view(np.int32)
        self._dev.copy_(self._host, non_blocking=True)
        if self._copied is None:
            self._copied = torch.cuda.Event()
        self._copied.record()
        d = self._dev
        temps = d[0:r].view(torch.float32)
        top_ks = d[m : m + r]
        top_ps = d[2 * m : 2 * m + r].view(torch.float32)
        rkeys = d[4 * m : 4 * m + 2 * r].view(torch.int64)
        ops.sample(logits, tokens, temps, top_ks, top_ps, rkeys, probs_out)
        return tokens
