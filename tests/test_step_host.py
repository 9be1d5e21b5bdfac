"""Host-side decisions of the step function that need no device: the list of query tiles a step
hands to the prompt attention kernel, and the shape a step of many tokens is captured for."""

from __future__ import annotations

import random
from types import SimpleNamespace

import numpy as np

from kvforge_b200.engine.step import BatchItem, ModelRunner, _Layout


def layout_with(q_lens, ctx_lens, tile_sizes, n_cap=None, b_cap=None):
    nb = len(q_lens)
    lay = _Layout(n_cap or sum(q_lens), b_cap or nb, 4, 1, nb, tuple(tile_sizes))
    host = np.zeros(lay.total, dtype=np.int32)
    host[lay.off["qsl"] : lay.off["qsl"] + nb + 1] = np.concatenate([[0], np.cumsum(q_lens)])
    host[lay.off["ctx"] : lay.off["ctx"] + nb] = ctx_lens
    return lay, host


def test_query_tiles_cover_every_query_once_longest_walk_first():
    rng = random.Random(4)
    for _ in range(50):
        nb = rng.randint(1, 9)
        q_lens = [rng.choice([1, 1, 2, 5, 31, 32, 33, 100]) for _ in range(nb)]
        ctx_lens = [q + rng.randint(0, 300) for q in q_lens]
        sizes = rng.sample([1, 16, 32, 64, 128], 2)
        lay, host = layout_with(q_lens, ctx_lens, sizes, n_cap=sum(q_lens) + rng.randint(0, 70), b_cap=nb + rng.randint(0, 3))
        counts = ModelRunner._fill_query_tiles(None, host, lay, nb)
        for tq in lay.tile_sizes:
            cap = lay.tile_cap(tq)
            total, n_multi, n_single = counts[tq]
            assert n_single == sum(1 for q in q_lens if q == 1)
            assert total == sum(-(-q // tq) for q in q_lens) <= cap
            for name, n_live, wanted in ((f"qtiles_{tq}", total, q_lens), (f"qtiles_multi_{tq}", n_multi, [q if q > 1 else 0 for q in q_lens])):
                tiles = host[lay.off[name] : lay.off[name] + 2 * cap].reshape(cap, 2)
                assert (tiles[n_live:, 0] == -1).all()
                seen = [set() for _ in range(nb)]
                last_keys = []
                for seq, q0 in tiles[:n_live]:
                    assert q0 % tq == 0 and 0 <= q0 < wanted[seq]
                    assert q0 not in seen[seq]
                    seen[seq].add(int(q0))
                    last_keys.append(ctx_lens[seq] - q_lens[seq] + min(q_lens[seq], q0 + tq))
                assert [len(s) for s in seen] == [-(-w // tq) for w in wanted]
                assert last_keys == sorted(last_keys, reverse=True)


def test_the_shape_a_step_is_captured_for():
    runner = SimpleNamespace(max_model_len=8192)
    items = [BatchItem("a", [1] * 700, 300, "last"), BatchItem("b", [5], 2000, "last")]
    # contexts up to 2,001 tokens: graphs reach the next power of two; a single token is among the sequences
    assert ModelRunner._graph_key(runner, items, 704, 2, False) == (704, 2, 2048, True, False)
    assert ModelRunner._graph_key(runner, items[:1], 704, 1, False) == (704, 1, 1024, False, False)
    # the decode form (one token per sequence) has no such distinction
    assert ModelRunner._graph_key(runner, [BatchItem("b", [5], 5000, "last")], 1, 1, True) == (1, 1, 8192, False, True)
    runner.max_model_len = 4096
    assert ModelRunner._graph_key(runner, [BatchItem("b", [5], 4000, "last")], 1, 1, True)[2] == 4096


def test_a_step_of_many_tokens_padded_to_its_sequence_count_is_no_decode_graph():
    """64 tokens in 64 sequences come two ways: 64 decoding requests (the decode form), or some
    decoding requests beside a short portion of a prompt, padded to 64 and 64.  The two are
    different graphs (the second computes every query of the portion) and must not share a key."""
    runner = SimpleNamespace(max_model_len=4096)
    decoding = [BatchItem(f"d{i}", [3], 100 + i, "last") for i in range(64)]
    mixed = [BatchItem(f"d{i}", [3], 100 + i, "last") for i in range(40)] + [BatchItem("p", [1] * 20, 0, "last")]
    a = ModelRunner._graph_key(runner, decoding, 64, 64, True)
    b = ModelRunner._graph_key(runner, mixed, 64, 64, False)
    assert a != b and a[:3] == b[:3]


def test_when_the_library_product_is_cut_into_slices_of_k():
    from kvforge_b200 import ops

    # a few dozen tokens, an output no wider than K, K of 2,048 or more: 4 slices up to 64 rows, 2 up to 128
    assert ops.library_splits(17, 2048, 2048) == 4 and ops.library_splits(64, 2048, 8192) == 4
    assert ops.library_splits(65, 4096, 14336) == 2 and ops.library_splits(128, 3072, 3072) == 2
    # the decode GEMM's rows, many rows, a wide output, a short K: the plain product
    assert ops.library_splits(16, 2048, 2048) == 1 and ops.library_splits(129, 2048, 8192) == 1
    assert ops.library_splits(32, 16384, 2048) == 1 and ops.library_splits(32, 96, 160) == 1
    assert ops.library_splits(32, 2048, 2048 + 64) == 1  # K that does not cut into 4 slices of whole 64s


def test_slices_of_the_decode_product_and_ranges_of_the_decode_attention():
    import random

    from kvforge_b200 import ops

    # the 1B shape: qkv / output / down up to 8 tokens, and from 9 on
    assert [ops.skinny_splits(n, k, 8) for n, k in ((3072, 2048), (2048, 2048), (2048, 8192))] == [8, 8, 10]
    assert [ops.skinny_splits(n, k, 16) for n, k in ((3072, 2048), (2048, 2048), (2048, 8192))] == [5, 8, 8]
    assert ops.skinny_splits(16384, 2048, 8) == 1 and ops.skinny_splits(96, 128, 4) == 1
    # no slice is ever empty: the kernel cuts K into slices of whole 64s, the same number of them each but the last
    rng = random.Random(0)
    for _ in range(2000):
        n, k, m = rng.randrange(8, 20000), 8 * rng.randrange(1, 2500), rng.choice((1, 8, 9, 16))
        s = ops.skinny_splits(n, k, m)
        per = -(-(-(-k // 64)) // s) * 64
        assert 1 <= s <= ops.SKINNY_MAX_SPLIT and (s - 1) * per < k, (n, k, m, s)
    # key ranges: 128 with 17 to 64 (sequence, kv head) pairs, 512 from 256 on, else 256; one size for one sequence
    sizes = {pairs: ops.attention_split_size(pairs, 1, 4096) for pairs in (1, 8, 16, 17, 64, 65, 255, 256, 2048)}
    assert sizes == {1: 256, 8: 256, 16: 256, 17: 128, 64: 128, 65: 256, 255: 256, 256: 512, 2048: 512}
    assert ops.ATTN_MIN_SPLIT == min(sizes.values())
    assert ops.attention_split_size(64, 1, 1 << 17, reach=4096) == 128 and ops.attention_split_size(64, 1, 1 << 17, reach=8192) == 256
    # heads wider than 64: a CTA holds twice the bytes, so short ranges only up to 32 pairs and half the CTAs a wave
    assert ops.attention_split_size(8, 8, 4096, 4096, head_dim=128) == 256 and ops.attention_split_size(4, 8, 4096, 4096, head_dim=128) == 128
    assert ops.attention_wave_target(8, 8, 64) == 888 and ops.attention_wave_target(8, 8, 128) == 444 and ops.attention_wave_target(64, 8, 128) == 3072
    # and never more ranges than the merge takes
    assert -(-(1 << 20) // ops.attention_split_size(8, 8, 1 << 20)) <= ops.MAX_ATTN_SPLITS
