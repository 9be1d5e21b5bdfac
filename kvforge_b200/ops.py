"""Python faces of the CUDA launchers in ``csrc/`` (loaded through ``native``).

Every function checks device, dtype, layout and size, then launches on torch's current
stream.  A launcher's non-zero return raises with the kernel's name.  Nothing here has a
CPU path: a tensor that is not on a CUDA device is an error.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import native

_SUF = {torch.float32: "f32", torch.bfloat16: "bf16"}

# p = pointer, i = int, l = long long, f = float
_SIGNATURES = {
    "kvf_embed_{s}": "pppppiiipp",
    "kvf_add_rmsnorm_{s}": "pppilpppiifp",
    "kvf_add_residual_{s}": "pplp",
    "kvf_rope_cache_{s}": "ppilppppppiiiiiilpp",
    "kvf_silu_mul_{s}": "ppliip",
    "kvf_cast_from_float_{s}": "pplp",
    "kvf_paged_attention_generic_{s}": "pppppppiiiiiiiiifiiiippp",
    "kvf_paged_attention_mma_bf16": "pppppppiiiiiiiiifiiiippp",
    "kvf_paged_attention_tcgen05_bf16": "pppppppiiiiiiiiilfipipp",
    "kvf_paged_attention_decode_fused_bf16": "pppppppiiiiiiiifiiiipppp",
    "kvf_paged_attention_decode_tma_bf16": "pppppppiiiiiiiilfiiiippppiip",
    "kvf_gemm_nt_f32": "pppiiiiiip",
    "kvf_gemm_skinny_bf16": "pppiiiiiiiilp",
    "kvf_set_pdl": "i",
    "kvf_gemm_tcgen05_bf16": "pppiiiiiiipp",
    "kvf_sample_f32": "pliippppppp",
    "kvf_argmax_f32": "pliipipp",
}
_CTYPES = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "f": ctypes.c_float}

_bound: dict[tuple[str, str], object] = {}


def _fn(name: str, lib: str = "core", signature: str | None = None):
    key = (lib, name)
    f = _bound.get(key)
    if f is None:
        cdll = native.load(lib)
        try:
            f = getattr(cdll, name)
        except AttributeError as e:  # pragma: no cover - a build that lacks a symbol
            raise RuntimeError(f"native library '{lib}' lacks {name}") from e
        sig = signature
        if sig is None:
            for pat, s in _SIGNATURES.items():
                if pat.format(s="f32") == name or pat.format(s="bf16") == name:
                    sig = s
                    break
        if sig is None:
            raise RuntimeError(f"no signature known for {name}")
        f.argtypes = [_CTYPES[c] for c in sig]
        f.restype = ctypes.c_int
        _bound[key] = f
    return f


@dataclass
class Partials:
    """The float slices ``[S, M, N]`` that a split-K product leaves; whoever consumes them
    sums them in slice order."""

    t: torch.Tensor

    @property
    def nsplit(self) -> int:
        return self.t.shape[0]

    @property
    def split_stride(self) -> int:
        return self.t.stride(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  ``torch.cuda.current_stream()`` builds a Python object on every
    call (some 15 us); a step of many tokens launches about 130 kernels from Python, so the raw
    handle is asked for directly where torch offers it."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_pdl_state = None


def set_pdl(enabled: bool) -> None:
    """Ask for programmatic dependent launch on every later launch of this library: a kernel
    may then be scheduled, and prefetch weights, while the kernel ahead of it in the stream is
    still running; it waits before it touches that kernel's results."""
    global _pdl_state
    enabled = bool(enabled)
    if _pdl_state is not enabled:
        _fn("kvf_set_pdl")(1 if enabled else 0)
        _pdl_state = enabled


# Kernels of this library launched so far (library matrix products are not counted).
launch_count = 0


def _check(rc: int, name: str, kernels: int = 1) -> None:
    global launch_count
    if rc != 0:
        raise RuntimeError(f"CUDA launcher {name} failed with cudaError {rc}")
    launch_count += kernels


def _need(t: torch.Tensor, dtype: torch.dtype | None, what: str, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor (this engine has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{what} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous")


def _suffix(dtype: torch.dtype) -> str:
    try:
        return _SUF[dtype]
    except KeyError:
        raise TypeError(f"storage type {dtype} is not supported (float32 or bfloat16)") from None


# ------------------------------------------------------------------ elementwise


def embed(
    table: torch.Tensor,
    ids: torch.Tensor,
    resid: torch.Tensor,
    err: torch.Tensor | None = None,
    feedback_rows: torch.Tensor | None = None,
    feedback: torch.Tensor | None = None,
) -> None:
    """``resid[n, :] = float(table[id, :])``; ``ids`` int32 ``[N]``, ``resid`` float ``[N, H]``.
    Where ``feedback_rows[n] >= 0`` the id is ``feedback[feedback_rows[n]]`` (a token sampled on
    the device in the step before) instead of ``ids[n]``."""
    s = _suffix(table.dtype)
    _need(table, None, "table")
    _need(ids, torch.int32, "ids")
    _need(resid, torch.float32, "resid")
    n, h = resid.shape
    if table.shape[1] != h or ids.numel() < n:
        raise ValueError("embed: shapes do not agree")
    if feedback_rows is not None:
        _need(feedback_rows, torch.int32, "feedback_rows")
        _need(feedback, torch.int32, "feedback")
        if feedback_rows.numel() < n:
            raise ValueError("embed: feedback_rows is too short")
    name = f"kvf_embed_{s}"
    _check(_fn(name)(_ptr(table), _ptr(ids), _ptr(feedback_rows), _ptr(feedback), _ptr(resid), n, h, table.shape[0], _ptr(err), _stream()), name)


def add_rmsnorm(
    resid: torch.Tensor,
    delta: torch.Tensor | Partials | None,
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    rows: torch.Tensor | None = None,
) -> None:
    """``v = resid (+ delta)``; ``out = T(v * rsqrt(mean(v^2) + eps) * weight)``.

    ``delta`` is a tensor in the storage type or the ``Partials`` of a split-K product.
    Without ``rows`` the sum is written back into ``resid``.  With ``rows`` (int32 ``[R]``)
    row ``r`` of ``out`` comes from row ``rows[r]`` and ``resid`` is left as it is.
    """
    s = _suffix(out.dtype)
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "norm weight")
    _need(out, None, "out")
    h = resid.shape[-1]
    n_rows = out.shape[0]
    if out.shape[-1] != h or weight.numel() != h:
        raise ValueError("add_rmsnorm: widths do not agree")
    dptr, pptr, nsplit, stride = None, None, 0, 0
    if delta is ADDED:
        delta = None
    if isinstance(delta, Partials):
        _need(delta.t, torch.float32, "partials", contiguous=False)
        if delta.t.shape[-1] != h or delta.t.stride(1) != h or delta.t.stride(2) != 1:
            raise ValueError("add_rmsnorm: partials must be [S, M, H] with dense rows")
        pptr, nsplit, stride = _ptr(delta.t), delta.nsplit, delta.split_stride
    elif delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[-1] != h:
            raise ValueError("add_rmsnorm: delta width")
        dptr = _ptr(delta)
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if rows.numel() < n_rows:
            raise ValueError("add_rmsnorm: fewer row indices than output rows")
    elif resid.shape[0] < n_rows:
        raise ValueError("add_rmsnorm: fewer residual rows than output rows")
    name = f"kvf_add_rmsnorm_{s}"
    _check(
        _fn(name)(_ptr(resid), dptr, pptr, nsplit, stride, _ptr(weight), _ptr(out), _ptr(rows), n_rows, h, float(eps), _stream()),
        name,
    )


def add_residual(resid: torch.Tensor, delta: torch.Tensor) -> None:
    """``resid += float(delta)`` over the first ``delta.numel()`` elements."""
    s = _suffix(delta.dtype)
    _need(resid, torch.float32, "resid")
    _need(delta, None, "delta")
    if delta.numel() > resid.numel():
        raise ValueError("add_residual: delta is larger than resid")
    name = f"kvf_add_residual_{s}"
    _check(_fn(name)(_ptr(resid), _ptr(delta), delta.numel(), _stream()), name)


def rope_cache_write(
    qkv: torch.Tensor | Partials,
    positions: torch.Tensor,
    inv_freq: torch.Tensor,
    slots: torch.Tensor | None,
    kcache: torch.Tensor | None,
    vcache: torch.Tensor | None,
    nh: int,
    nkv: int,
    d: int,
    block_size: int,
    err: torch.Tensor | None = None,
    q_out: torch.Tensor | None = None,
) -> None:
    """Rotate q and k of ``qkv [N, (nh+2nkv)*d]``; write k and v to their slots.

    ``qkv`` in the storage type: q is rotated in place.  ``qkv`` as ``Partials`` of a split-K
    product: the slices are summed in float and q goes to ``q_out [N, nh*d]``.
    ``inv_freq`` float ``[rot/2]`` fixes how many leading dims turn (``rot <= d``).
    ``kcache/vcache``: ``[num_blocks, nkv, block_size, d]``.  ``slots=None`` rotates q only.
    """
    width = (nh + 2 * nkv) * d
    qptr, pptr, nsplit, stride, qo = None, None, 0, 0, None
    if isinstance(qkv, Partials):
        if q_out is None:
            raise ValueError("rope_cache_write: partials need q_out")
        _need(qkv.t, torch.float32, "partials", contiguous=False)
        if qkv.t.shape[-1] != width or qkv.t.stride(1) != width or qkv.t.stride(2) != 1:
            raise ValueError("rope_cache_write: partials must be [S, N, width] with dense rows")
        n = qkv.t.shape[1]
        dtype = q_out.dtype
        _need(q_out, None, "q_out")
        if tuple(q_out.shape) != (n, nh * d):
            raise ValueError("rope_cache_write: q_out shape")
        pptr, nsplit, stride, qo = _ptr(qkv.t), qkv.nsplit, qkv.split_stride, _ptr(q_out)
    else:
        _need(qkv, None, "qkv")
        n = qkv.shape[0]
        dtype = qkv.dtype
        if qkv.shape[1] != width:
            raise ValueError("rope_cache_write: qkv width")
        qptr = _ptr(qkv)
        if q_out is not None:
            _need(q_out, dtype, "q_out")
            qo = _ptr(q_out)
    s = _suffix(dtype)
    _need(positions, torch.int32, "positions")
    _need(inv_freq, torch.float32, "inv_freq")
    rot = 2 * inv_freq.numel()
    if rot > d:
        raise ValueError("rope_cache_write: more frequencies than head_dim/2")
    num_slots = 0
    if slots is not None:
        _need(slots, torch.int32, "slots")
        _need(kcache, dtype, "kcache")
        _need(vcache, dtype, "vcache")
        if tuple(kcache.shape[1:]) != (nkv, block_size, d) or kcache.shape != vcache.shape:
            raise ValueError("rope_cache_write: cache shape must be [num_blocks, nkv, block_size, d]")
        num_slots = kcache.shape[0] * block_size
    name = f"kvf_rope_cache_{s}"
    _check(
        _fn(name)(
            qptr, pptr, nsplit, stride, qo, _ptr(positions), _ptr(inv_freq), _ptr(slots), _ptr(kcache), _ptr(vcache),
            n, nh, nkv, d, rot, block_size, num_slots, _ptr(err), _stream(),
        ),
        name,
    )  # fmt: skip


GATE_UP_BLOCK = 8  # gate and up rows alternate in blocks of this many in the interleaved layout


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[g0..7, u0..7, g8..15, u8..15, ...]``: the row order in which the skinny product finds
    ``gate_i`` and ``up_i`` in one thread's accumulators."""
    i, h = w_gate.shape
    if i % GATE_UP_BLOCK:
        raise ValueError("interleave_gate_up: the intermediate size must be a multiple of 8")
    b = GATE_UP_BLOCK
    return torch.stack([w_gate.view(i // b, b, h), w_up.view(i // b, b, h)], dim=1).reshape(2 * i, h).contiguous()


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """``out[n, i] = silu(gate_i) * up_i`` computed in float.  Columns of ``gate_up [N, 2I]``:
    all gates then all ups, or (``interleaved``) alternating in blocks of 8."""
    s = _suffix(gate_up.dtype)
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out")
    n, i2 = gate_up.shape
    if out.shape[0] != n or out.shape[1] * 2 != i2:
        raise ValueError("silu_mul: shapes do not agree")
    if interleaved and out.shape[1] % GATE_UP_BLOCK:
        raise ValueError("silu_mul: interleaved layout needs a multiple of 8")
    name = f"kvf_silu_mul_{s}"
    _check(_fn(name)(_ptr(gate_up), _ptr(out), n, out.shape[1], GATE_UP_BLOCK if interleaved else 0, _stream()), name)


def cast_from_float(src: torch.Tensor, out: torch.Tensor) -> None:
    s = _suffix(out.dtype)
    _need(src, torch.float32, "src")
    _need(out, None, "out")
    if src.numel() != out.numel():
        raise ValueError("cast_from_float: sizes differ")
    name = f"kvf_cast_from_float_{s}"
    _check(_fn(name)(_ptr(src), _ptr(out), src.numel(), _stream()), name)


# ------------------------------------------------------------------ attention

MAX_ATTN_SPLITS = 1024  # ranges per (sequence, head) the merge kernel takes


ATTN_ONE_WAVE = 888  # CTAs of the decode attention that run as one wave (six fit an SM, 148 SMs)
ATTN_ONE_WAVE_FEW_PAIRS = 640  # the same with fewer than 32 (sequence, kv head) pairs, whose merges are long: room to spare


ATTN_MIN_SPLIT = 128  # the shortest range any batch gets: scratch is made for it
# With this many (sequence, kv head) pairs (4 to 8 sequences of 8 kv heads) ranges of 128 keys: the
# ranges of 256 keys are too few CTAs to pull the bandwidth, and the last CTA of a pair still merges
# few (decode steps of the 1B shape at 2,088 keys: 4 sequences 0.796 -> 0.773 ms, 6 0.797 -> 0.785,
# 8 0.803 -> 0.789 ms; at 3,040 to 5,040 keys 1.5 to 3 %).  With up to 16 pairs the ranges of a pair
# are a thread-block cluster of at most 16 CTAs, which ranges of 256 keys keep to longer contexts
# (one sequence 0.704 against 0.738 ms); from 96 pairs on shorter ranges lose (12 sequences 0.876
# against 0.928 ms).
ATTN_SHORT_RANGE_PAIRS = (17, 64)
# with heads wider than 64 only up to this many pairs (8 sequences of the 3B shape at 2,074 keys: 1.925 ms a step
# with a grid for ranges of 128 keys, 1.847 ms with one for 256; 4 sequences 1.695 against 1.730 ms)
ATTN_SHORT_RANGE_PAIRS_WIDE_HEADS = 32
# ... and only while the step's reach (the longest context, or what a captured graph was made for) is at most
# this: a grid made for ranges of 128 keys over a long reach is mostly CTAs that leave at once, and they
# cost (8 sequences at 8,030 keys 1.100 against 1.042 ms, at 32,798 keys 2.385 against 2.178 ms)
ATTN_SHORT_RANGE_REACH = 4096


def attention_split_size(num_seqs: int, nkv: int, max_context: int = 0, reach: int = 0, head_dim: int = 64) -> int:
    """Keys per range of the decode form, as the launch fixes it.  A range is a CTA, and a CTA has
    a fixed cost of a few microseconds (its chain of dependent reads, its share of the merge), so
    ranges are not short: 256 keys, 128 with 17 to 64 (sequence, kv head) pairs and a ``reach`` of at most 4,096 keys, 512 with 256 or more
    (measured inside the decode step at 1 to 64 sequences), and more when the context is so long that there would
    be more than ``MAX_ATTN_SPLITS`` of them.  Ranges start at multiples of the size.  (The TMA
    kernel may double the size further at run time, see ``attention_wave_target``.)  Since the
    size follows the number of sequences, so does the order in which a context's keys are merged:
    a caller that wants sums that do not depend on the batch at all (the 32-bit path) passes
    ``num_seqs=1``."""
    pairs = num_seqs * nkv
    if pairs >= 256:
        split = 512 if head_dim <= 64 else 1024  # (64 sequences of the 3B and 8B shapes: 1 % faster than with 512)
    elif ATTN_SHORT_RANGE_PAIRS[0] <= pairs <= (ATTN_SHORT_RANGE_PAIRS[1] if head_dim <= 64 else ATTN_SHORT_RANGE_PAIRS_WIDE_HEADS) and reach <= ATTN_SHORT_RANGE_REACH:
        split = ATTN_MIN_SPLIT
    else:
        split = 256
    while -(-max_context // split) > MAX_ATTN_SPLITS:
        split *= 2
    return split


def attention_wave_target(num_seqs: int, nkv: int, head_dim: int = 64) -> int:
    """How many live CTAs the TMA decode kernel aims at: it doubles the range size, on the
    device, from the step's longest context, until the ranges of all (sequence, kv head) pairs
    are at most this many: one wave of CTAs for few pairs (8 sequences at 4,096 keys: ranges of
    256 make 1,024 CTAs, a wave and a small second one, 21.7 us; ranges of 512 one wave, 15.3 us;
    at 3,026 keys 768 CTAs of 256 keys are still one wave and beat 384 of 512: the batch-8 step
    takes 0.846 instead of 0.871 ms; with 2 sequences at 12,000 keys it is the other way round,
    0.911 against 0.890 ms, since the last CTA of a pair then merges 47 ranges: hence the lower
    number for few pairs), at most six ranges a pair for many (64 sequences at 8,192 keys: ranges
    of 512 take 196 us, ranges of 2,048 take 162 us; four a pair made ranges so long that their
    CTAs no longer ran as even waves).  The launch's grid is made for the smallest size; CTAs of
    ranges that a larger size leaves without keys exit at once."""
    pairs = num_seqs * nkv
    one_wave = ATTN_ONE_WAVE if pairs >= 32 else ATTN_ONE_WAVE_FEW_PAIRS
    if head_dim > 64:
        # a CTA's ring is twice the size and three fit an SM: half the CTAs are a wave (8 sequences of the
        # 3B shape at 4,026 keys: 2.255 -> 2.188 ms a step, of the 8B shape 4.113 -> 4.035 ms)
        one_wave //= 2
    return max(one_wave, 6 * pairs)


def attention_scratch_shapes(max_seqs: int, nh: int, d: int, max_context: int, split_size: int = 256) -> tuple[tuple[int, ...], tuple[int, ...]]:
    """Shapes of the float scratch the decode form needs for contexts up to ``max_context``."""
    splits = max(1, -(-max_context // split_size))
    return (max_seqs, nh, splits, d), (max_seqs, nh, splits, 2)


def check_head_dim(d: int) -> None:
    if d <= 0 or d % 16 != 0 or d > 256:
        raise ValueError(f"head_dim {d} is not supported: it must be a multiple of 16, at most 256")


def mma_attention_supported(dtype: torch.dtype, nh: int, nkv: int, d: int, decode_form: bool) -> bool:
    """Whether the tensor-core kernel (``csrc/attention_mma.cu``) takes this shape."""
    g = nh // max(nkv, 1)
    return dtype == torch.bfloat16 and d in (64, 128) and g <= (16 if decode_form else 64)


TC_ATTN_ROWS = 128  # (token, head of a group) rows of a CTA of the tcgen05 attention kernel


def tcgen05_query_tile(nh: int, nkv: int) -> int:
    """Queries of one sequence that a CTA of the tcgen05 attention kernel takes."""
    return max(1, TC_ATTN_ROWS // max(1, nh // nkv))


def tcgen05_attention_supported(dtype: torch.dtype, nh: int, nkv: int, d: int, decode_form: bool) -> bool:
    """Whether the tcgen05 kernel (``csrc/attention_tcgen05.cu``) takes this shape: many queries
    (not the decode form), bfloat16, head size 64 or 128."""
    return dtype == torch.bfloat16 and d in (64, 128) and not decode_form and nh // max(nkv, 1) <= 128


def tma_decode_supported(dtype: torch.dtype, nh: int, nkv: int, d: int, block_size: int, num_blocks: int) -> bool:
    """Whether the TMA decode kernel (``csrc/attention_decode_tma.cu``) takes this shape."""
    return (
        dtype == torch.bfloat16 and d in (64, 128) and nh // max(nkv, 1) <= 8 and block_size % 16 == 0
        and num_blocks * nkv * block_size < 2**31 - 16
    )  # fmt: skip


def paged_attention(
    q: torch.Tensor,
    out: torch.Tensor,
    kcache: torch.Tensor,
    vcache: torch.Tensor,
    block_tables: torch.Tensor,
    qsl: torch.Tensor,
    ctx_lens: torch.Tensor,
    num_seqs: int,
    max_q_len: int,
    nh: int,
    nkv: int,
    d: int,
    scale: float,
    window: int = 0,
    q_stride: int | None = None,
    scratch: tuple[torch.Tensor, ...] | None = None,
    max_context: int | None = None,
    split_size: int = 256,
    kernel: str = "auto",
    err: torch.Tensor | None = None,
    cluster: bool = True,
    query_tiles: tuple[torch.Tensor, int] | None = None,
    single_only: bool = False,
    wave_target: int = 0,
) -> None:
    """Paged GQA attention of a flat batch (the contract is at the top of
    ``csrc/attention_generic.cu``).

    ``q``: rows of ``q_stride`` elements whose first ``nh*d`` are the query heads; ``out``:
    ``[N, nh*d]``.  With ``scratch`` (and every sequence holding one query) the decode form
    runs: key ranges of ``split_size`` in parallel, then a merge; ``max_context`` bounds the
    contexts.  ``kernel``: ``"auto"`` takes, for bfloat16, the tcgen05 kernel (many queries, head
    size 64) or the mma.sync kernel (decode form; head size 128) and the FP32-pipe kernel
    elsewhere; ``"generic"``, ``"mma"``, ``"tma"`` and ``"tcgen05"`` force one (tests).  ``err``: the
    device error flag (a bounded wait inside a kernel raises it).  ``cluster``: the TMA decode kernel
    merges up to 16 key ranges through a thread-block cluster's shared memory (else through the
    scratch and the tickets).  ``query_tiles``: for the tcgen05 kernel, an int32 array of (sequence or
    -1, first query) pairs, one per tile of ``tcgen05_query_tile`` queries, and how many of them to
    launch; without it the grid spans every sequence times the tiles of the longest query run.
    ``single_only`` (TMA decode kernel): of a mixed batch only the sequences that bring exactly one
    query are computed; the rows of the others are left untouched.  ``wave_target`` (TMA decode
    kernel, 0 = off): the kernel doubles ``split_size`` until the ranges of the step's longest
    context, over all pairs, are at most this many (``attention_wave_target``).
    """
    s = _suffix(q.dtype)
    check_head_dim(d)
    _need(q, None, "q")
    _need(out, q.dtype, "out")
    _need(kcache, q.dtype, "kcache")
    _need(vcache, q.dtype, "vcache")
    _need(block_tables, torch.int32, "block_tables")
    _need(qsl, torch.int32, "query_start_loc")
    _need(ctx_lens, torch.int32, "context_lens")
    if kcache.dim() != 4 or kcache.shape[1] != nkv or kcache.shape[3] != d or kcache.shape != vcache.shape:
        raise ValueError("paged_attention: cache shape must be [num_blocks, nkv, block_size, d]")
    block_size = kcache.shape[2]
    if q_stride is None:
        q_stride = q.shape[-1]
    bt_stride = block_tables.shape[-1] if block_tables.dim() == 2 else block_tables.numel() // max(1, num_seqs)
    split, max_splits, grid_splits, pa, pm, tickets = 0, 0, 0, None, None, None
    if scratch is not None:
        pa, pm = scratch[:2]
        _need(pa, torch.float32, "scratch acc")
        _need(pm, torch.float32, "scratch ml")
        if len(scratch) > 2:
            tickets = scratch[2]
            _need(tickets, torch.int32, "scratch tickets")
            if tickets.numel() < num_seqs * nkv:
                raise ValueError("paged_attention: too few tickets (one per sequence and kv head)")
        if max_q_len != 1:
            raise ValueError("the decode form needs one query per sequence")
        if split_size <= 0 or split_size % 64:
            raise ValueError("split_size must be a positive multiple of 64")
        split = split_size
        max_splits = pa.shape[2]
        if pa.shape[0] < num_seqs or pa.shape[1] != nh or pa.shape[3] != d:
            raise ValueError("paged_attention: scratch shape does not fit")
        if max_context is None or -(-max_context // split) > max_splits:
            raise ValueError("paged_attention: scratch is too small for the longest context")
        grid_splits = max(1, -(-max_context // split))
        if grid_splits > MAX_ATTN_SPLITS:
            raise ValueError("paged_attention: too many key ranges; use a larger split_size")
    decode_form = scratch is not None
    use_tc = tcgen05_attention_supported(q.dtype, nh, nkv, d, decode_form) and q_stride % 8 == 0 and out.shape[-1] % 8 == 0 and max_q_len > 1
    use_mma = mma_attention_supported(q.dtype, nh, nkv, d, decode_form)
    if kernel == "generic":
        use_tc = use_mma = False
    elif kernel == "tma":
        pass
    elif kernel == "mma":
        if not use_mma:
            raise ValueError("the mma.sync attention kernel does not take this shape")
        use_tc = False
    elif kernel == "tcgen05":
        if not tcgen05_attention_supported(q.dtype, nh, nkv, d, decode_form):
            raise ValueError("the tcgen05 attention kernel does not take this shape")
        use_tc = True
    if use_tc:
        name = "kvf_paged_attention_tcgen05_bf16"
        tiles, n_tiles = None, 0
        if query_tiles is not None and 0 < query_tiles[1] <= 65535:
            tiles, n_tiles = query_tiles
            _need(tiles, torch.int32, "query_tiles")
            if tiles.numel() < 2 * n_tiles:
                raise ValueError("paged_attention: the list of query tiles is shorter than the launch")
        _check(
            _fn(name)(
                _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
                num_seqs, max_q_len, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, int(kcache.shape[0]),
                float(scale), int(window), _ptr(tiles), n_tiles, _ptr(err), _stream(),
            ),
            name,
        )  # fmt: skip
        return
    use_tma = tickets is not None and tma_decode_supported(q.dtype, nh, nkv, d, block_size, kcache.shape[0])
    if (kernel == "tma" or single_only) and not use_tma:
        raise ValueError("the TMA decode kernel does not take this shape (or no tickets were given)")
    if use_tma and kernel in ("auto", "tma"):
        name = "kvf_paged_attention_decode_tma_bf16"
        _check(
            _fn(name)(
                _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
                num_seqs, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, int(kcache.shape[0]), float(scale),
                int(window), split, max_splits, grid_splits, _ptr(pa), _ptr(pm), _ptr(tickets), _ptr(err), int(bool(cluster)) | (2 if single_only else 0), int(wave_target), _stream(),
            ),
            name,
        )  # fmt: skip
        return
    if use_mma and tickets is not None:
        name = "kvf_paged_attention_decode_fused_bf16"
        _check(
            _fn(name)(
                _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
                num_seqs, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, float(scale),
                int(window), split, max_splits, grid_splits, _ptr(pa), _ptr(pm), _ptr(tickets), _stream(),
            ),
            name,
        )  # fmt: skip
        return
    name = "kvf_paged_attention_mma_bf16" if use_mma else f"kvf_paged_attention_generic_{s}"
    _check(
        _fn(name)(
            _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), _ptr(qsl), _ptr(ctx_lens),
            num_seqs, max_q_len, q_stride, out.shape[-1], bt_stride, nh, nkv, d, block_size, float(scale),
            int(window), split, max_splits, grid_splits, _ptr(pa), _ptr(pm), _stream(),
        ),
        name,
        2 if scratch is not None else 1,
    )  # fmt: skip


def paged_attention_generic(*args, **kw) -> None:
    """``paged_attention`` on the FP32-pipe kernel whatever the shape."""
    kw["kernel"] = "generic"
    paged_attention(*args, **kw)


# ------------------------------------------------------------------ matrix products


def gemm_nt_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out[M, N] = a[M, K] @ w[N, K]^T`` on the FP32 pipes (no tensor cores).  Row strides
    may exceed the widths (views of wider buffers)."""
    for t, what in ((a, "a"), (w, "w"), (out, "out")):
        _need(t, torch.float32, what, contiguous=False)
        if t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"gemm_nt_f32: {what} must be 2-D with unit inner stride")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n):
        raise ValueError("gemm_nt_f32: shapes do not agree")
    name = "kvf_gemm_nt_f32"
    _check(
        _fn(name)(_ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0), w.stride(0), out.stride(0), _stream()),
        name,
    )


SKINNY_MAX_M = 64  # what the kernel takes
SKINNY_USE_M = 16  # up to here it beats the library product (measured on B200); above, the library is used
SKINNY_MAX_SPLIT = 16


def skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the decode product (``csrc/gemm_skinny_bf16.cu``) takes ``x @ w^T``."""
    return (
        x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= SKINNY_USE_M
        and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
    )  # fmt: skip


def skinny_splits(n_out: int, k: int, m: int = 8) -> int:
    """Slices of K so that a product with few output rows still fills the SMs, each slice at least
    256 wide.  Up to 8 tokens three CTAs of 64 rows fit an SM, and about 384 CTAs (2.6 an SM) were
    best in whole decode steps of all three shapes, with at most 10 slices: the kernel that sums the
    slices is the longer for each one.  (1B shape, 8 sequences: qkv / output / down with 5 / 8 / 8
    slices 0.812 ms a step, with 8 / 8 / 10 slices 0.802 ms, with 8 / 8 / 16 slices 0.845 ms; one
    sequence 0.730 -> 0.703 ms; the 3B shape 2.018 -> 1.974 ms.)  From 9 tokens on a CTA's tiles are
    larger and two fit an SM: about 256 CTAs (with 384 the 16-sequence step took 1.036 instead of
    0.925 ms)."""
    ctas = -(-n_out // 64)
    few = m <= 8
    want = round((384 if few else 256) / ctas)
    while want > 1 and want * ctas > (444 if few else 296):  # more CTAs than are on the SMs at once
        want -= 1
    s = max(1, min(want, k // 256, 10 if few else SKINNY_MAX_SPLIT))
    k_iters = -(-k // 64)
    while s > 1 and (s - 1) * -(-k_iters // s) * 64 >= k:  # the last slice would be empty
        s -= 1
    return s


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | Partials, mode: str = "plain") -> None:
    """``x [M<=64, K] @ w [N, K]^T`` in bfloat16 with float accumulation.

    ``out``: a bfloat16 or float ``[M, N]`` tensor, ``Partials`` (``[S, M, N]`` float, one slice
    of K each), or with ``mode="silu"`` a bfloat16 ``[M, N/2]`` tensor that receives
    ``silu(gate) * up`` for ``w`` in the interleaved gate/up layout.
    """
    m, k = x.shape
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < m <= SKINNY_MAX_M and k % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0):  # fmt: skip
        raise ValueError("gemm_skinny: needs bfloat16, M <= 64, K % 8 == 0, unit inner strides")
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError("gemm_skinny: inner sizes differ")
    ksplit, stride = 1, 0
    if isinstance(out, Partials):
        t = out.t
        _need(t, torch.float32, "partials", contiguous=False)
        if tuple(t.shape[1:]) != (m, n) or t.stride(2) != 1:
            raise ValueError("gemm_skinny: partials must be [S, M, N]")
        code, ksplit, stride, ldo, optr = 2, t.shape[0], t.stride(0), t.stride(1), _ptr(t)
    else:
        _need(out, None, "out", contiguous=False)
        if out.stride(1) != 1:
            raise ValueError("gemm_skinny: out needs unit inner stride")
        if mode == "silu":
            if out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n // 2):
                raise ValueError("gemm_skinny: silu output must be bfloat16 [M, N/2]")
            code = 3
        elif tuple(out.shape) != (m, n):
            raise ValueError("gemm_skinny: out shape")
        elif out.dtype == torch.bfloat16:
            code = 0
        elif out.dtype == torch.float32:
            code = 1
        else:
            raise TypeError("gemm_skinny: out must be bfloat16 or float32")
        ldo, optr = out.stride(0), _ptr(out)
    name = "kvf_gemm_skinny_bf16"
    _check(_fn(name)(_ptr(x), _ptr(w), optr, m, n, k, x.stride(0), w.stride(0), ldo, code, ksplit, stride, _stream()), name)


TCGEN05_MIN_TILES = 120  # below this many 128 x 256 output tiles the persistent grid leaves SMs idle


def tcgen05_ok(x: torch.Tensor, w: torch.Tensor, min_tiles: int = TCGEN05_MIN_TILES) -> bool:
    """Whether the tensor-memory product (``csrc/gemm_tcgen05_bf16.cu``) takes ``x @ w^T`` and
    has enough output tiles to fill the device."""
    tiles = -(-x.shape[0] // 128) * -(-w.shape[0] // 256)
    return tiles >= min_tiles and (
        x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(1) == 1
        and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
        and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
    )  # fmt: skip


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str = "plain", err: torch.Tensor | None = None) -> None:
    """``x [M, K] @ w [N, K]^T`` in bfloat16 on the tcgen05 tensor cores (TMA loads, float
    accumulation in tensor memory).  ``out``: bfloat16 ``[M, N]``, or with ``mode="silu"``
    bfloat16 ``[M, N/2] = silu(gate) * up`` for ``w`` in the interleaved gate/up layout."""
    if not tcgen05_ok(x, w, min_tiles=0):
        raise ValueError("gemm_tcgen05: needs bfloat16, K % 8 == 0, unit inner strides, 16-byte aligned rows")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError("gemm_tcgen05: inner sizes differ")
    _need(out, torch.bfloat16, "out", contiguous=False)
    if out.stride(1) != 1 or out.stride(0) % 8 or out.data_ptr() % 16:
        raise ValueError("gemm_tcgen05: out needs unit inner stride and 16-byte aligned rows")
    if mode == "silu":
        if tuple(out.shape) != (m, n // 2) or n % 16:
            raise ValueError("gemm_tcgen05: silu output must be [M, N/2] with N % 16 == 0")
        code = 3
    else:
        if tuple(out.shape) != (m, n):
            raise ValueError("gemm_tcgen05: out shape")
        code = 0
    name = "kvf_gemm_tcgen05_bf16"
    _check(_fn(name)(_ptr(x), _ptr(w), _ptr(out), m, n, k, x.stride(0), w.stride(0), out.stride(0), code, _ptr(err), _stream()), name)


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ w^T`` for ``x [M, K]``, ``w [N, K]``.

    float32: the engine's own FFMA kernel (true 32-bit).  bfloat16 inputs: cuBLAS through
    ``torch.mm`` with 32-bit accumulation, the library product that umarhassan-cloud/kvforge
    itself uses (``nn.Linear``, src/tokenvault/model.py:70-73); ``out`` may be bfloat16 or
    float32.
    """
    if x.dtype == torch.float32:
        gemm_nt_f32(x, w, out)
        return
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    elif out.dtype == torch.float32:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        raise TypeError("linear: out must be bfloat16 or float32")


class _Added:
    """What a mixer or a feed-forward returns when it has added its result into the step's float
    residual stream (``StepContext.residual``) itself: nothing is left for the norm to add."""

    def __repr__(self) -> str:
        return "ADDED"


ADDED = _Added()


def linear_add(x: torch.Tensor, w: torch.Tensor, acc: torch.Tensor) -> None:
    """``acc += x @ w^T`` for bfloat16 ``x [M, K]``, ``w [N, K]`` and float ``acc [M, N]``: the library
    product with 32-bit accumulation whose epilogue reads and writes ``acc`` in 32-bit, so the sum
    with the residual stream is never rounded to bfloat16 and costs no pass of its own."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    _need(acc, torch.float32, "acc", contiguous=False)
    if tuple(acc.shape) != (x.shape[0], w.shape[0]) or w.shape[1] != x.shape[1]:
        raise ValueError("linear_add: shapes do not agree")
    torch.addmm(acc, x, w.t(), out_dtype=torch.float32, out=acc)


LIBRARY_SPLIT_MAX_M = 128  # up to here the library product of a narrow output gains from slices of K


def library_splits(m: int, n_out: int, k: int) -> int:
    """Slices of K for the library product ``[m, k] x [n_out, k]^T`` of a few dozen tokens.  With
    so few rows and an output no wider than K (the output and down projections) the library
    launches too few CTAs to pull the weights at the rate of HBM; as a batched product over
    slices of K it does (measured on B200 at 32 to 128 rows on the projections of three model
    shapes: 13.3 -> 8.6 us for [2048, 8192] at 64 rows).  1 = no gain expected."""
    if not (SKINNY_USE_M < m <= LIBRARY_SPLIT_MAX_M) or n_out > k or k < 2048:
        return 1
    s = 4 if m <= 64 else 2
    return s if k % (s * 64) == 0 else 1


def linear_split_k(x: torch.Tensor, w: torch.Tensor, part: Partials) -> None:
    """``part[s] = x[:, slice s of K] @ w[:, slice s of K]^T`` in float, one batched library
    product; whoever consumes the slices sums them in slice order."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    m, k = x.shape
    n = w.shape[0]
    t = part.t
    s = t.shape[0]
    if t.dtype != torch.float32 or tuple(t.shape) != (s, m, n) or not t.is_contiguous() or w.shape[1] != k or k % s:
        raise ValueError("linear_split_k: the slices must be contiguous float [S, M, N] with S dividing K")
    ks = k // s
    torch.bmm(x.view(m, s, ks).permute(1, 0, 2), w.view(n, s, ks).permute(1, 2, 0), out_dtype=torch.float32, out=t)


# ------------------------------------------------------------------ sampling


def sample(
    logits: torch.Tensor,
    out_tokens: torch.Tensor,
    temps: torch.Tensor | None = None,
    top_ks: torch.Tensor | None = None,
    top_ps: torch.Tensor | None = None,
    rand_keys: torch.Tensor | None = None,
    probs_out: torch.Tensor | None = None,
) -> None:
    """One token per row of float ``logits [R, V]``.  ``temps=None`` is greedy for all rows.
    ``rand_keys`` int64 ``[R]``: the draw of a row depends on its key alone."""
    _need(logits, torch.float32, "logits", contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("sample: logits must be [R, V] with unit inner stride")
    r, v = logits.shape
    _need(out_tokens, torch.int32, "out_tokens")
    if out_tokens.numel() < r:
        raise ValueError("sample: out_tokens is too short")
    for t, dt, what in (
        (temps, torch.float32, "temps"),
        (top_ks, torch.int32, "top_ks"),
        (top_ps, torch.float32, "top_ps"),
        (rand_keys, torch.int64, "rand_keys"),
    ):
        if t is not None:
            _need(t, dt, what)
            if t.numel() < r:
                raise ValueError(f"sample: {what} is too short")
    if probs_out is not None:
        _need(probs_out, torch.float32, "probs_out")
        if tuple(probs_out.shape) != (r, v):
            raise ValueError("sample: probs_out shape")
    name = "kvf_sample_f32"
    _check(
        _fn(name)(
            _ptr(logits), logits.stride(0), r, v, _ptr(temps), _ptr(top_ks), _ptr(top_ps), _ptr(rand_keys),
            _ptr(out_tokens), _ptr(probs_out), _stream(),
        ),
        name,
    )  # fmt: skip


# stretches of a row of logits that a CTA each looks through (8 rows of 128,256 in the decode step: 32 stretches
# 0.789 ms a step, 128 stretches 0.782 ms; 64 rows the same either way)
ARGMAX_CHUNKS = 128


def argmax(logits: torch.Tensor, out_tokens: torch.Tensor, partial: torch.Tensor) -> None:
    """Greedy tokens of float ``logits [R, V]`` (lowest index among equal maxima) in two short
    kernels; ``partial``: int64 scratch ``[R, ARGMAX_CHUNKS]``."""
    _need(logits, torch.float32, "logits", contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("argmax: logits must be [R, V] with unit inner stride")
    r, v = logits.shape
    _need(out_tokens, torch.int32, "out_tokens")
    _need(partial, torch.int64, "partial")
    if out_tokens.numel() < r or partial.numel() < r * ARGMAX_CHUNKS:
        raise ValueError("argmax: an output or scratch buffer is too small")
    name = "kvf_argmax_f32"
    _check(_fn(name)(_ptr(logits), logits.stride(0), r, v, _ptr(partial), ARGMAX_CHUNKS, _ptr(out_tokens), _stream()), name, 2)


def splitmix64(z: int) -> int:
    """The host twin of the device generator (``csrc/sampling.cu``): the 64-bit value whose
    high-multiply with the total mass picks the token."""
    m = (1 << 64) - 1
    z = (z + 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)
