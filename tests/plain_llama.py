"""Plain, slow implementation of the dense Llama decoder used as the oracle of the tests.

Whole sequences, no cache, no batching, one function per part.  It shares no code with
``kvforge_b200``: it reads ``config.json`` and ``model.safetensors`` itself and works on
ordinary torch tensors on the CPU (or any device it is given).  Every function cites the
place in umarhassan-cloud/kvforge (paths inside that project) whose formula it restates.

The one formula that project does not contain is the llama3 frequency scaling of the
rotary encoding; ``llama3_scaled_inv_freq`` restates the published definition and is
tested against its three regimes in ``tests/test_plain.py``.

``dtype=torch.float32`` computes everything in 32-bit.  ``dtype=torch.bfloat16`` follows the
rounding points of src/tokenvault/model.py when that model is cast to bfloat16: matrix
products, residual sums and activations round to bfloat16, while norms, rotation and
softmax are computed in 32-bit and rounded once.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

# --------------------------------------------------------------------------- files


_ST_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "I32": torch.int32,
    "I64": torch.int64,
}


def read_safetensors(path: str | Path) -> dict[str, torch.Tensor]:
    """Minimal reader of the safetensors container: 8-byte header length, JSON header, raw bytes."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        dt = _ST_DTYPES[meta["dtype"]]
        buf = bytearray(raw[base + lo : base + hi])
        t = torch.frombuffer(buf, dtype=dt).reshape(meta["shape"]).clone()
        out[name] = t
    return out


def read_config(model_dir: str | Path) -> dict:
    return json.loads((Path(model_dir) / "config.json").read_text())


# --------------------------------------------------------------------------- parts


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """src/tokenvault/model.py:35-38 — 32-bit inside, eps added to the mean, weight applied
    in 32-bit before the single rounding back to ``x.dtype``."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * weight.float()).to(x.dtype)


def plain_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """src/tokenvault/model.py:44 — ``1 / theta^(2j/d)`` built in 32-bit."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


def llama3_scaled_inv_freq(
    inv_freq: torch.Tensor,
    factor: float,
    low_freq_factor: float,
    high_freq_factor: float,
    original_max_position: int,
) -> torch.Tensor:
    """llama3 frequency scaling (not in kvforge; the definition published with Llama 3.1).

    With wavelength ``lam = 2*pi/f``: short waves (``lam < P/high``) are kept, long waves
    (``lam > P/low``) are divided by ``factor``, and in between the two are blended with
    ``s = (P/lam - low) / (high - low)`` as ``(1-s)*f/factor + s*f``.
    """
    out = []
    for f in inv_freq.double().tolist():
        lam = 2.0 * math.pi / f
        if lam < original_max_position / high_freq_factor:
            out.append(f)
        elif lam > original_max_position / low_freq_factor:
            out.append(f / factor)
        else:
            s = (original_max_position / lam - low_freq_factor) / (high_freq_factor - low_freq_factor)
            out.append((1.0 - s) * f / factor + s * f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """src/tokenvault/model.py:47-50 — angles ``float(pos) * inv_freq`` in 32-bit, duplicated
    to the full head width."""
    freqs = positions.float()[..., None] * inv_freq.float()
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """src/tokenvault/model.py:53-55."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([-x2, x1], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """src/tokenvault/model.py:58-61 — ``x: [T, heads, d]``, ``cos/sin: [T, d]``; 32-bit, one rounding."""
    cos, sin = cos.unsqueeze(-2), sin.unsqueeze(-2)
    return (x.float() * cos + rotate_half(x.float()) * sin).to(x.dtype)


def causal_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float,
    window: int | None = None,
) -> torch.Tensor:
    """src/tokenvault/cache/paged_attention.py:94-108 (``reference_attention``) for a whole
    sequence: ``q [T, nh, d]``, ``k, v [T, nkv, d]``; scores, softmax and the weighted sum in
    32-bit, the scale applied after the dot product (paged_attention.py:85), one rounding.
    ``window`` (not a kvforge option; used by the tests of the general attention part) lets
    position ``i`` see keys ``i-window+1 .. i`` only.
    """
    t = q.shape[0]
    group = q.shape[1] // k.shape[1]
    kk = k.repeat_interleave(group, dim=1).float()
    vv = v.repeat_interleave(group, dim=1).float()
    scores = torch.einsum("qhd,lhd->hql", q.float(), kk) * scale
    q_pos = torch.arange(t, device=q.device)[:, None]
    k_pos = torch.arange(t, device=q.device)[None, :]
    visible = k_pos <= q_pos
    if window is not None:
        visible = visible & (k_pos > q_pos - window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hql,lhd->qhd", probs, vv).to(q.dtype)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``nn.Linear`` without bias (src/tokenvault/model.py:70-73,121-123): ``y = x W^T``."""
    return x @ w.t()


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """src/tokenvault/model.py:131-132 — ``down(silu(gate(x)) * up(x))``."""
    return linear(torch.nn.functional.silu(linear(x, w_gate)) * linear(x, w_up), w_down)


# --------------------------------------------------------------------------- model


class PlainLlama:
    """Whole-sequence forward of the decoder of src/tokenvault/model.py:146-191 (pre-norm
    blocks, model.py:185-188; logits in 32-bit, model.py:190-191)."""

    def __init__(self, model_dir: str | Path, dtype: torch.dtype = torch.float32, device: str = "cpu"):
        cfg = read_config(model_dir)
        self.cfg = cfg
        self.dtype = dtype
        self.device = device
        self.hidden = cfg["hidden_size"]
        self.n_layers = cfg["num_hidden_layers"]
        self.nh = cfg["num_attention_heads"]
        self.nkv = cfg.get("num_key_value_heads", self.nh)
        self.d = cfg.get("head_dim") or self.hidden // self.nh
        self.eps = cfg["rms_norm_eps"]
        self.vocab = cfg["vocab_size"]
        inv = plain_inv_freq(self.d, cfg.get("rope_theta", 10000.0))
        rs = cfg.get("rope_scaling")
        if rs:
            assert rs.get("rope_type", rs.get("type")) == "llama3"
            inv = llama3_scaled_inv_freq(
                inv,
                rs["factor"],
                rs["low_freq_factor"],
                rs["high_freq_factor"],
                rs["original_max_position_embeddings"],
            )
        self.inv_freq = inv.to(device)
        raw = read_safetensors(Path(model_dir) / "model.safetensors")
        self.w = {}
        for name, t in raw.items():
            name = name.removeprefix("model.")  # src/tokenvault/model_loader.py:104
            self.w[name] = t.to(device=device, dtype=dtype)
        if "lm_head.weight" not in self.w:  # src/tokenvault/model_loader.py:105-106
            self.w["lm_head.weight"] = self.w["embed_tokens.weight"]
        # Which layer runs when, and whose keys and values it reads: [(layer, kv_source_call | None)].
        self.execution = [(i, None) for i in range(self.n_layers)]
        self.window = None

    # One function per part of a layer, so tests can compare parts alone.
    def embed(self, ids: torch.Tensor) -> torch.Tensor:
        return self.w["embed_tokens.weight"][ids]  # model.py:170,183

    def qkv(self, layer: int, x: torch.Tensor, positions: torch.Tensor):
        p = f"layers.{layer}.self_attn."
        t = x.shape[0]
        cos, sin = rope_cos_sin(positions, self.inv_freq)
        q = apply_rope(linear(x, self.w[p + "q_proj.weight"]).view(t, self.nh, self.d), cos, sin)
        k = apply_rope(linear(x, self.w[p + "k_proj.weight"]).view(t, self.nkv, self.d), cos, sin)
        v = linear(x, self.w[p + "v_proj.weight"]).view(t, self.nkv, self.d)
        return q, k, v  # model.py:86-88

    def attention(self, layer: int, x: torch.Tensor, positions: torch.Tensor, kv=None):
        """Returns the mixer's output and the (k, v) it used, so that a later call can read them."""
        q, k, v = self.qkv(layer, x, positions)
        if kv is not None:
            k, v = kv
        o = causal_attention(q, k, v, 1.0 / math.sqrt(self.d), self.window)  # model.py:74
        out = linear(o.reshape(x.shape[0], -1), self.w[f"layers.{layer}.self_attn.o_proj.weight"])
        return out, (k, v)

    def mlp(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        p = f"layers.{layer}.mlp."
        return swiglu(x, self.w[p + "gate_proj.weight"], self.w[p + "up_proj.weight"], self.w[p + "down_proj.weight"])

    def hidden_states(self, ids: list[int] | torch.Tensor) -> torch.Tensor:
        ids = torch.as_tensor(ids, dtype=torch.long, device=self.device)
        positions = torch.arange(ids.shape[0], device=self.device)
        h = self.embed(ids)
        kvs = []
        for layer, src in self.execution:
            x = rms_norm(h, self.w[f"layers.{layer}.input_layernorm.weight"], self.eps)
            a, kv = self.attention(layer, x, positions, None if src is None else kvs[src])
            kvs.append(kv)
            h = h + a  # model.py:186
            x = rms_norm(h, self.w[f"layers.{layer}.post_attention_layernorm.weight"], self.eps)
            h = h + self.mlp(layer, x)  # model.py:187
        return rms_norm(h, self.w["norm.weight"], self.eps)  # model.py:188

    @torch.no_grad()
    def logits(self, ids: list[int] | torch.Tensor) -> torch.Tensor:
        """``[T, vocab]`` 32-bit logits at every position of one whole sequence."""
        return linear(self.hidden_states(ids), self.w["lm_head.weight"]).float()

    @torch.no_grad()
    def greedy(self, prompt: list[int], n: int) -> list[int]:
        """Greedy decoding by full recomputation (tests/conftest.py:22-32 of kvforge)."""
        ids = list(prompt)
        out = []
        for _ in range(n):
            tok = int(self.logits(ids)[-1].argmax())
            out.append(tok)
            ids.append(tok)
        return out


# --------------------------------------------------------------------------- sampling


def processed_probs(
    logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0
) -> torch.Tensor:
    """src/tokenvault/sampling.py:40-66 for one row: the distribution a token is drawn from.
    Temperature 0 gives the one-hot of the argmax; top-k keeps ranks ``< k``; top-p keeps the
    entries whose mass *before* them in descending order is ``< top_p``.  A float64 input is
    kept in float64 (the running sum over a large vocabulary is then free of rounding)."""
    if logits.dtype != torch.float64:
        logits = logits.float()
    if temperature == 0.0:
        out = torch.zeros_like(logits)
        out[logits.argmax()] = 1.0
        return out
    scaled = logits / temperature
    vocab = logits.shape[-1]
    if (0 < top_k < vocab) or top_p < 1.0:
        s, idx = scaled.sort(descending=True)
        remove = torch.arange(vocab) >= (top_k if top_k > 0 else vocab)
        sp = torch.softmax(s.masked_fill(remove, float("-inf")), -1)
        remove |= (sp.cumsum(-1) - sp) >= top_p
        s = s.masked_fill(remove, float("-inf"))
        scaled = torch.full_like(scaled, float("-inf")).scatter(-1, idx, s)
    return torch.softmax(scaled, -1)
