"""The allocation-free decode attention (kvforge_b200/csrc/kvforge_noalloc.h), called the way
its users call it: through the exported C symbol, with device pointers and nothing else.

Those users are hosts that may not allocate device memory while they run: a plugin inside
another runtime's enqueue call, a server whose device budget was handed out at start-up, a
loop that cannot afford the device-wide synchronisation an allocation may bring.  The
regular entry point makes the caller provide scratch memory for the partial results of the
key ranges; this one keeps that scratch inside the library.  The test checks that both give
the same output on two calls in a row (the second with other shapes, so what the first call
left in the shared scratch must not matter), that an oversized problem is refused with a
message instead of being allocated for, and that no device memory is allocated on the way.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

from __future__ import annotations

import ctypes
import math

import pytest
import torch

from test_gpu_kernels import dev, paged

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 8 * 1024 * 1024
TOO_LARGE = -2


@pytest.fixture(scope="module")
def entry():
    from kvforge_b200 import native

    lib = native.load("noalloc")
    fn = lib.kvf_paged_attention_decode_noalloc_bf16
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [p, p, p, p, p, p, p, i, i, i, i, i, i, i, i, f, i, i, i, p]
    fn.restype = ctypes.c_int
    lib.kvf_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def problem(nh, nkv, d, bs, ctx_lens, seed):
    g = torch.Generator().manual_seed(seed)
    kv = [(torch.randn(c, nkv, d, generator=g).bfloat16(), torch.randn(c, nkv, d, generator=g).bfloat16()) for c in ctx_lens]
    q = torch.randn(len(ctx_lens), nh * d, generator=g).bfloat16()
    kc, vc, tables = paged(kv, nkv, d, bs, torch.bfloat16, seed)
    qsl = torch.arange(len(ctx_lens) + 1, dtype=torch.int32)
    return dev(q), dev(kc), dev(vc), dev(tables), dev(qsl), dev(torch.tensor(ctx_lens, dtype=torch.int32))


def both_ways(entry, nh, nkv, d, bs, ctx_lens, split, window, seed):
    from kvforge_b200 import ops

    _, fn = entry
    q, kc, vc, tables, qsl, ctx = problem(nh, nkv, d, bs, ctx_lens, seed)
    b, bound, scale = len(ctx_lens), max(ctx_lens), 1.0 / math.sqrt(d)
    # the existing entry point, with scratch that the caller allocates
    sa, sm = ops.attention_scratch_shapes(b, nh, d, bound, split)
    want = torch.full((b, nh * d), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.paged_attention(q, want, kc, vc, tables, qsl, ctx, b, 1, nh, nkv, d, scale, window=window,
                        scratch=(torch.empty(sa, device="cuda"), torch.empty(sm, device="cuda")), max_context=bound,
                        split_size=split, kernel="mma")  # fmt: skip
    # the allocation-free one: inputs and outputs only
    got = torch.full((b, nh * d), float("nan"), device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    rc = fn(q.data_ptr(), got.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), qsl.data_ptr(), ctx.data_ptr(),
            b, nh * d, nh * d, tables.shape[1], nh, nkv, d, bs, scale, window, split, bound,
            torch.cuda.current_stream().cuda_stream)  # fmt: skip
    torch.cuda.synchronize()
    after = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    assert rc == 0, entry[0].kvf_noalloc_last_error()
    return got.float().cpu(), want.float().cpu(), before, after


def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row(entry):
    # a first call on this device (it also looks up the scratch array's address), then the checks
    both_ways(entry, 8, 2, 64, 16, [100], 64, 0, seed=0)
    got, want, before, after = both_ways(entry, 32, 8, 64, 16, [700, 1, 256, 257, 33, 2048], 256, 0, seed=1)
    assert not torch.isnan(got).any()
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2)  # the tolerance of the attention kernel tests
    assert torch.equal(got, want)  # same kernels, same ranges: in fact the same bits
    assert after[0] == before[0] and after[1] >= before[1] - (1 << 20), "device memory was allocated"
    # again at once, other shapes and a window: the scratch still holds the last call's partial results
    got, want, _, _ = both_ways(entry, 6, 3, 128, 4, [65, 300, 64], 64, 70, seed=2)
    assert not torch.isnan(got).any()
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2)
    assert torch.equal(got, want)


def test_no_alloc_entry_point_refuses_what_does_not_fit(entry):
    lib, fn = entry
    nh, nkv, d, bs = 32, 8, 128, 16
    q, kc, vc, tables, qsl, ctx = problem(nh, nkv, d, bs, [64] * 8, seed=3)
    out = torch.zeros(8, nh * d, device="cuda", dtype=torch.bfloat16)
    # 8 sequences x 32 heads x 512 ranges x 130 floats is far beyond the 8 MiB inside the library
    rc = fn(q.data_ptr(), out.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), qsl.data_ptr(), ctx.data_ptr(),
            8, nh * d, nh * d, tables.shape[1], nh, nkv, d, bs, 0.1, 0, 64, 32768, torch.cuda.current_stream().cuda_stream)  # fmt: skip
    assert rc == TOO_LARGE
    msg = lib.kvf_noalloc_last_error().decode()
    assert str(SCRATCH_BYTES) in msg and "bytes" in msg
    assert float(out.abs().max()) == 0.0  # nothing ran
    rc = fn(q.data_ptr(), out.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), qsl.data_ptr(), ctx.data_ptr(),
            8, nh * d, nh * d, tables.shape[1], nh, nkv, 80, bs, 0.1, 0, 64, 64, torch.cuda.current_stream().cuda_stream)  # fmt: skip
    assert rc == -3 and "head size" in lib.kvf_noalloc_last_error().decode()
