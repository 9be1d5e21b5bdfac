"""Makes ``kvforge_reference_logits.safetensors``: logits of umarhassan-cloud/kvforge's own model
code (``Transformer.forward_dense``, src/tokenvault/model.py:193-228) on the CPU for the two
tiny configurations of the tests, so that the plain implementation under ``tests/`` can be
compared with it without that project being present.

    python tests/golden/make_golden.py --reference-src <kvforge checkout>/src

The weights are the ones ``kvforge_b200``'s random-weights mode writes for (preset, seed 7,
init_std 0.1, norm_std 0.1), stored in bfloat16 (both programs then compute in 32-bit on the
same values).  The model folders are written beside the logits (``tiny-a/``, ``tiny-b/``) and
committed with them, so the comparison does not depend on which random numbers a torch build
draws.  kvforge has no llama3 frequency scaling: for tiny-b the
scaled frequencies (computed by the plain implementation's formula) are written into the
model's ``rotary.inv_freq`` buffer, so the check covers everything but that formula, which
has tests of its own.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

GOLDEN_SEED = 7
GOLDEN_TOKENS = {
    "tiny-a": [3, 250, 17, 17, 99, 0, 128, 64, 200, 5, 77, 31, 255, 1, 2, 90, 180, 45, 12, 222, 8],
    "tiny-b": [319, 0, 7, 150, 299, 42, 42, 13, 260, 88, 301, 5, 190, 64, 27, 111, 230, 9, 75, 310, 2, 56, 141],
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True, help="the src/ folder of a kvforge checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference_src)
    from tokenvault import ModelConfig as RefConfig
    from tokenvault.model import Transformer

    from kvforge_b200 import PRESETS
    from kvforge_b200.models.folder import write_random_model
    from kvforge_b200.weights.safetensors_io import write_safetensors
    from plain_llama import llama3_scaled_inv_freq, plain_inv_freq, read_safetensors

    out = {}
    for name, tokens in GOLDEN_TOKENS.items():
        cfg = PRESETS[name]
        write_random_model(HERE / name, cfg, seed=GOLDEN_SEED, store_dtype=torch.bfloat16, init_std=0.1, norm_std=0.1)
        raw = {k: v.float() for k, v in read_safetensors(HERE / name / "model.safetensors").items()}
        ref_cfg = RefConfig(
            vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers,
            num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, intermediate_size=cfg.intermediate_size,
            head_dim=cfg.head_dim, max_position_embeddings=cfg.max_position_embeddings,
            rope_theta=cfg.rope_theta, rms_norm_eps=cfg.rms_norm_eps, tie_word_embeddings=cfg.tie_word_embeddings,
        )  # fmt: skip
        model = Transformer(ref_cfg).eval()
        state = {k.removeprefix("model."): v for k, v in raw.items()}
        if "lm_head.weight" not in state:
            state["lm_head.weight"] = state["embed_tokens.weight"]
        result = model.load_state_dict(state, strict=False)
        assert not result.unexpected_keys and all(k.endswith("inv_freq") for k in result.missing_keys), result
        if cfg.rope_scaling is not None:
            rs = cfg.rope_scaling
            inv = llama3_scaled_inv_freq(
                plain_inv_freq(cfg.head_dim, cfg.rope_theta), rs.factor, rs.low_freq_factor,
                rs.high_freq_factor, rs.original_max_position_embeddings,
            )  # fmt: skip
            model.rotary.inv_freq.copy_(inv)
        with torch.inference_mode():
            logits, _ = model.forward_dense(torch.tensor([tokens]))
        out[f"{name}.logits"] = logits[0].clone()
        out[f"{name}.tokens"] = torch.tensor(tokens, dtype=torch.int32)
    write_safetensors(HERE / "kvforge_reference_logits.safetensors", out)
    print("wrote", HERE / "kvforge_reference_logits.safetensors")


if __name__ == "__main__":
    main()
