"""Device storage of the cache: per group one K and one V tensor
``[entries, num_blocks, kv_heads, block_size, head_dim]`` (an entry per layer call that keeps
a cache), and per stateful mixer call a float tensor ``[num_slots, *state_shape]``.

umarhassan-cloud/kvforge keeps ``[num_blocks, block_size, kv_heads, head_dim]`` per layer
(src/tokenvault/cache/kv_cache.py:27-31).  Here the kv-head index comes before the
position inside a page, so the keys of one head in one page are one contiguous run of
``block_size * head_dim`` elements.
"""

from __future__ import annotations

import torch

from ..parts.base import LayerCache


class KVPool:
    def __init__(self, model, num_blocks: int, block_size: int, num_slots: int, dtype: torch.dtype, device) -> None:
        self.num_blocks, self.block_size, self.dtype = num_blocks, block_size, dtype
        self.k: list[torch.Tensor] = []
        self.v: list[torch.Tensor] = []
        for g in model.groups:
            shape = (len(g.calls), num_blocks, g.need.kv_heads, block_size, g.need.head_dim)
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros(shape, dtype=dtype, device=device))
        self.states: list[torch.Tensor | None] = []
        for shape in model.state_shapes:
            self.states.append(None if shape is None else torch.zeros((num_slots, *shape), dtype=torch.float32, device=device))
        self.caches: list[LayerCache | None] = []
        for idx, call in enumerate(model.spec.execution):
            owner = model.call_group[idx if call.kv_from is None else call.kv_from]
            if owner is None:
                cache = None if self.states[idx] is None else LayerCache(None, None, -1, True, self.states[idx])
            else:
                gi, entry = owner
                cache = LayerCache(self.k[gi][entry], self.v[gi][entry], gi, call.kv_from is None, self.states[idx])
            self.caches.append(cache)

    @property
    def memory_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)

    @property
    def bytes_per_block(self) -> int:
        return self.memory_bytes // max(1, self.num_blocks)

    def clear_state_slots(self, slots: list[int]) -> None:
        if not slots:
            return
        for st in self.states:
            if st is not None:
                st[slots] = 0


def bytes_per_block(model, block_size: int, dtype: torch.dtype) -> int:
    """Bytes that one page index costs over all groups and entries, keys and values
    (src/tokenvault/config.py:91-95 for a single group)."""
    elem = torch.tensor([], dtype=dtype).element_size()
    return sum(2 * len(g.calls) * block_size * g.need.kv_heads * g.need.head_dim * elem for g in model.groups)
