"""The plain implementation against kvforge's own model code (golden logits made on the CPU
by tests/golden/make_golden.py) and against the formulas it restates."""

from __future__ import annotations

import math
from pathlib import Path

import pytest
import torch

from golden.make_golden import GOLDEN_TOKENS
from kvforge_b200 import PRESETS
from kvforge_b200.models.folder import write_random_model
from plain_llama import (
    PlainLlama,
    apply_rope,
    causal_attention,
    llama3_scaled_inv_freq,
    plain_inv_freq,
    processed_probs,
    read_safetensors,
    rms_norm,
    rope_cos_sin,
)

GOLDEN_DIR = Path(__file__).parent / "golden"
GOLDEN = GOLDEN_DIR / "kvforge_reference_logits.safetensors"


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_plain_matches_kvforge_model(name):
    """The committed model folders (``tests/golden/tiny-a``, ``tiny-b``) through the plain
    implementation against the logits kvforge's own model code gave for them."""
    gold = read_safetensors(GOLDEN)
    tokens = gold[f"{name}.tokens"].tolist()
    assert tokens == GOLDEN_TOKENS[name]
    logits = PlainLlama(GOLDEN_DIR / name).logits(tokens)
    ref = gold[f"{name}.logits"]
    assert logits.shape == ref.shape
    assert float((logits - ref).abs().max()) < 2e-5 * max(1.0, float(ref.abs().max()))
    assert torch.equal(logits.argmax(-1), ref.argmax(-1))


def test_llama3_scaling_three_regimes_and_continuity():
    d, theta = 64, 500000.0
    inv = plain_inv_freq(d, theta)
    factor, lo, hi, orig = 8.0, 1.0, 4.0, 8192
    out = llama3_scaled_inv_freq(inv, factor, lo, hi, orig)
    lam = 2 * math.pi / inv.double()
    short, long_ = lam < orig / hi, lam > orig / lo
    assert short.any() and long_.any() and (~short & ~long_).any()
    assert torch.equal(out[short], inv[short])
    assert torch.allclose(out[long_].double(), inv[long_].double() / factor, rtol=1e-7)
    mid = ~short & ~long_
    assert ((out[mid] < inv[mid]) & (out[mid].double() > inv[mid].double() / factor)).all()
    # continuity at both edges of the blend
    for lam_edge, want in ((orig / hi, 1.0), (orig / lo, 1.0 / factor)):
        f = torch.tensor([2 * math.pi / lam_edge], dtype=torch.float32)
        eps = torch.tensor([1e-4], dtype=torch.float32)
        a = llama3_scaled_inv_freq(f * (1 + eps), factor, lo, hi, orig) / (f * (1 + eps))
        b = llama3_scaled_inv_freq(f * (1 - eps), factor, lo, hi, orig) / (f * (1 - eps))
        assert abs(float(a) - want) < 1e-3 and abs(float(b) - want) < 1e-3


# llama3 scaling worked out by hand from its published definition, in plain double arithmetic:
# f = theta^(-2j/d), wavelength lam = 2 pi / f; kept for lam < P/high, f/factor for lam > P/low,
# else s = (P/lam - low)/(high - low) and (1 - s) f/factor + s f.  E.g. the 1B line for j = 16:
# f = 500000^-0.5 = 1.414213562e-3, lam = 4442.88, P/lam = 1.843850, s = 0.2812833,
# (0.7187167/32 + 0.2812833) f = 0.3037432 f = 4.295568e-4.
LLAMA3_LITERALS = [
    # (head_dim, theta, factor, low, high, original context): {pair index: scaled frequency}
    ((64, 500000.0, 32.0, 1.0, 4.0, 8192), {0: 1.0, 7: 5.666962145e-02, 14: 3.211445995e-03, 15: 1.290547928e-03, 16: 4.295567966e-04, 17: 9.708287803e-05, 18: 1.946163818e-05, 31: 9.418306725e-08}),
    ((128, 500000.0, 32.0, 1.0, 4.0, 8192), {28: 3.211445995e-03, 29: 2.118406997e-03, 31: 7.625412034e-04, 34: 9.708287803e-05, 35: 2.389053088e-05, 63: 7.672314972e-08}),
    ((128, 500000.0, 8.0, 1.0, 4.0, 8192), {1: 8.146172339e-01, 29: 2.166570764e-03, 32: 5.248461610e-04, 34: 1.785078128e-04, 35: 9.556212354e-05, 63: 3.068925989e-07}),
    ((32, 500000.0, 8.0, 1.0, 4.0, 64), {0: 1.0, 1: 4.403666027e-01, 2: 7.940300918e-02, 3: 1.067463754e-02, 15: 5.677088101e-07}),
]


@pytest.mark.parametrize("args,literals", LLAMA3_LITERALS)
def test_llama3_scaling_literal_values(args, literals):
    """The plain formula and the engine's (``kvforge_b200/parts/rope.py``) against values worked
    out by hand for the rope parameters of the 1B, 3B and 8B shapes and of tiny-b."""
    from kvforge_b200.parts.rope import llama3_scale, rotary_inv_freq

    d, theta, factor, low, high, orig = args
    plain = llama3_scaled_inv_freq(plain_inv_freq(d, theta), factor, low, high, orig)
    engine = llama3_scale(rotary_inv_freq(d, theta), factor, low, high, orig)
    for j, want in literals.items():
        # 32-bit frequencies: the power is taken in float, so the last digits may differ
        assert abs(float(plain[j]) - want) <= 2e-6 * want, (j, float(plain[j]), want)
        assert abs(float(engine[j]) - want) <= 2e-6 * want, (j, float(engine[j]), want)
    assert torch.allclose(plain, engine, rtol=1e-6, atol=0)


def test_rms_norm_formula():
    x = torch.randn(5, 24, dtype=torch.float64).float()
    w = torch.rand(24) + 0.5
    y = rms_norm(x, w, 1e-5)
    ref = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
    assert torch.allclose(y.double(), ref, atol=1e-6)


def test_rope_is_a_rotation_and_relative():
    d = 16
    inv = plain_inv_freq(d, 10000.0)
    q, k = torch.randn(1, 1, d), torch.randn(1, 1, d)

    def score(pq, pk):
        cq, sq = rope_cos_sin(torch.tensor([pq]), inv)
        ck, sk = rope_cos_sin(torch.tensor([pk]), inv)
        return float((apply_rope(q, cq, sq) * apply_rope(k, ck, sk)).sum())

    cq, sq = rope_cos_sin(torch.tensor([9]), inv)
    assert abs(float(apply_rope(q, cq, sq).norm()) - float(q.norm())) < 1e-5
    assert abs(score(7, 3) - score(107, 103)) < 1e-4  # only the distance matters
    assert abs(score(7, 3) - score(7, 4)) > 1e-4


def test_attention_far_key_and_window():
    # one key among hundreds is made to dominate: the output must be its value
    t, d = 300, 16
    q = torch.zeros(t, 2, d)
    k = torch.randn(t, 1, d) * 0.01
    v = torch.randn(t, 1, d)
    far = 17
    k[far, 0, 0] = 50.0
    q[-1, :, 0] = 50.0
    o = causal_attention(q, k, v, 1.0)
    assert torch.allclose(o[-1, 0], v[far, 0], atol=1e-4)
    # with a window that excludes it, the far key is not seen
    o = causal_attention(q, k, v, 1.0, window=100)
    assert not torch.allclose(o[-1, 0], v[far, 0], atol=1e-2)
    # position 0 sees itself only
    assert torch.allclose(o[0, 0], v[0, 0], atol=1e-6)


def test_processed_probs_options():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 0.0])
    assert processed_probs(logits, 0.0).tolist() == [1.0, 0, 0, 0, 0]
    p = processed_probs(logits, 1.0, top_k=2)
    assert (p[2:] == 0).all() and abs(float(p.sum()) - 1) < 1e-6
    p = processed_probs(logits, 1.0, top_p=0.5)
    assert p[0] == 1.0  # the top entry alone reaches 0.5
    p = processed_probs(logits, 0.5)
    assert torch.allclose(p, torch.softmax(logits / 0.5, -1))


def test_plain_greedy_is_prefix_stable(tmp_path):
    write_random_model(tmp_path / "m", PRESETS["tiny-a"], seed=3, store_dtype=torch.float32, init_std=0.1)
    m = PlainLlama(tmp_path / "m")
    a = m.greedy([5, 6, 7], 6)
    b = m.greedy([5, 6, 7] + a[:3], 3)
    assert a[3:] == b
