#!/usr/bin/env python3
"""Anchor the plain implementation (tests/plain_qwen3.py) on the reference project's own model code.

Run once, on the CPU, with the UESlubei/ondeviceinfer checkout importable:

    python tests/golden/make_golden.py /path/to/ondeviceinfer-checkout

For the tiny random models A and B, and A with biases on the attention projections, it builds the reference's ``Qwen3ForCausalLM``
(ondeviceinfer/model.py:121-163) in fp32, loads the tests' seeded weights into it by
their checkpoint names, runs every prompt alone and whole, and also prefill + token by
token through the reference's resident cache.  It asserts that the plain implementation
agrees with both, then writes ``tests/golden/tiny_{a,b}.npz`` holding, for each prompt,
the reference's logits at the last prompt position and at three other positions,
together with the greedy continuation.  ``tests/test_plain.py`` re-checks the plain
implementation against these files without needing the reference checkout.

The reference's ``Qwen3Config.validate()`` (ondeviceinfer/config.py:73-74) is not called
for model B, whose query width (192) differs from its hidden size (96); the model code
itself has no such restriction.
"""

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import plain_qwen3 as plain  # noqa: E402

CASES = {
    "tiny_a": (plain.TINY_A, 0, [5, 11, 17], 8),
    "tiny_b": (plain.TINY_B, 1, [1, 7, 30, 64], 16),
    "tiny_a_bias": (plain.TINY_A_BIAS, 10, [5, 11, 17], 8),
}


def reference_model(ref_root, cfg, weights):
    sys.path.insert(0, str(ref_root))
    from ondeviceinfer.config import Qwen3Config
    from ondeviceinfer.model import Qwen3ForCausalLM

    config = Qwen3Config(
        vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
        intermediate_size=cfg["intermediate_size"], num_hidden_layers=cfg["num_hidden_layers"],
        num_attention_heads=cfg["num_attention_heads"], num_key_value_heads=cfg["num_key_value_heads"],
        head_dim=cfg["head_dim"], max_position_embeddings=cfg["max_position_embeddings"],
        rms_norm_eps=cfg["rms_norm_eps"], rope_theta=cfg["rope_theta"],
        tie_word_embeddings=cfg["tie_word_embeddings"], attention_bias=cfg.get("attention_bias", False))
    model = Qwen3ForCausalLM(config, dtype=torch.float32).eval()
    state = {k: v.float() for k, v in weights.items()}
    if cfg["tie_word_embeddings"]:
        state["lm_head.weight"] = state["model.embed_tokens.weight"]
    model.load_state_dict(state, strict=True)
    if cfg["tie_word_embeddings"]:
        model.lm_head.weight = model.model.embed_tokens.weight
    return model


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref_root = Path(sys.argv[1])
    for name, (cfg, seed, lengths, new_tokens) in CASES.items():
        weights = plain.random_weights(cfg, seed)
        prompts = plain.random_prompts(cfg, lengths, seed)
        model = reference_model(ref_root, cfg, weights)
        out = {}
        worst = 0.0
        worst_bf16 = 0.0
        with torch.inference_mode():
            for r, prompt in enumerate(prompts):
                ids = torch.tensor([prompt])
                whole = model(ids).logits[0]
                mine = plain.forward_logits(weights, cfg, prompt)
                worst = max(worst, float((whole - mine).abs().max()))
                assert torch.allclose(whole, mine, atol=2e-6, rtol=1e-5), (name, r)
                # the reference's own cache: prefill, then greedy token by token
                from ondeviceinfer.generation import greedy_generate
                cache = model.make_resident_cache(batch_size=1, max_seq_len=len(prompt) + new_tokens)
                gen = greedy_generate(model, ids, max_new_tokens=new_tokens, cache=cache)
                ref_tokens = gen.generated_ids[0].tolist()
                my_tokens = plain.generate(weights, cfg, prompt, new_tokens)
                assert ref_tokens == my_tokens, (name, r, ref_tokens, my_tokens)
                # bf16 arithmetic with the reference's rounding points
                mb = reference_model(ref_root, cfg, weights).to(torch.bfloat16)
                if cfg["tie_word_embeddings"]:
                    mb.lm_head.weight = mb.model.embed_tokens.weight
                whole_bf16 = mb(ids).logits[0].float()
                mine_bf16 = plain.forward_logits(weights, cfg, prompt, torch.bfloat16)
                # bf16 tolerance used throughout the tests: 3e-2 * max(1, max |logit|)
                gap = float((whole_bf16 - mine_bf16).abs().max())
                worst_bf16 = max(worst_bf16, gap)
                assert gap <= 3e-2 * max(1.0, float(whole.abs().max())), (name, r, gap)
                picks = sorted({0, len(prompt) // 3, (2 * len(prompt)) // 3, len(prompt) - 1})
                out[f"prompt_{r}"] = np.asarray(prompt, dtype=np.int32)
                out[f"positions_{r}"] = np.asarray(picks, dtype=np.int32)
                out[f"logits_{r}"] = whole[picks].numpy().astype(np.float32)
                out[f"greedy_{r}"] = np.asarray(ref_tokens, dtype=np.int32)
        target = HERE / f"{name}.npz"
        if target.exists():
            old = np.load(target)
            if sorted(old.files) == sorted(out) and all(np.array_equal(old[k], out[k]) for k in out):
                print(f"{name}: the committed file already holds these outputs")
                continue
        np.savez_compressed(target, **out)
        print(f"{name}: plain vs reference max |dlogit| = {worst:.3e} (fp32), "
              f"{worst_bf16:.3e} (bf16 arithmetic); wrote {name}.npz")


if __name__ == "__main__":
    main()
