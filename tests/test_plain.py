"""The plain implementation itself: against the committed outputs of the reference
project's model code (tests/golden), and the properties the reference's own unit tests
assert (tests/test_foundations.py and tests/test_model.py of UESlubei/ondeviceinfer)."""

from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name,cfg,seed", [("tiny_a", plain.TINY_A, 0), ("tiny_b", plain.TINY_B, 1),
                                           ("tiny_a_bias", plain.TINY_A_BIAS, 10)])
def test_plain_matches_reference_outputs(name, cfg, seed):
    data = np.load(GOLDEN / f"{name}.npz")
    weights = plain.random_weights(cfg, seed)
    r = 0
    while f"prompt_{r}" in data:
        prompt = data[f"prompt_{r}"].tolist()
        logits = plain.forward_logits(weights, cfg, prompt)
        expected = torch.from_numpy(data[f"logits_{r}"])
        picks = data[f"positions_{r}"].tolist()
        assert torch.allclose(logits[picks], expected, atol=2e-6, rtol=1e-5)
        assert plain.generate(weights, cfg, prompt, len(data[f"greedy_{r}"])) == data[f"greedy_{r}"].tolist()
        r += 1
    assert r >= 3


def test_random_prompts_are_the_golden_prompts():
    data = np.load(GOLDEN / "tiny_b.npz")
    prompts = plain.random_prompts(plain.TINY_B, [1, 7, 30, 64], 1)
    assert [data[f"prompt_{r}"].tolist() for r in range(4)] == prompts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_normalises_in_fp32_then_casts_then_scales(dtype):
    torch.manual_seed(0)
    x = torch.randn(2, 5, 128, dtype=dtype)
    w = torch.empty(128, dtype=dtype).uniform_(0.5, 1.5)
    expected = torch.nn.functional.rms_norm(x.float(), (128,), None, 1e-6).to(dtype) * w
    actual = plain.rms_norm(x, w, 1e-6)
    assert actual.dtype == dtype
    assert torch.allclose(actual, expected, atol=2e-3, rtol=2e-3)


def test_rope_position_zero_is_identity_and_norm_is_kept():
    torch.manual_seed(0)
    q = torch.randn(4, 7, 32)
    cos, sin = plain.rope_tables(torch.arange(7), 32, 1e6, torch.float32)
    rotated = plain.apply_rope(q, cos, sin)
    assert cos.shape == (7, 32)
    assert torch.equal(rotated[:, 0], q[:, 0])
    assert torch.allclose(rotated.norm(dim=-1), q.norm(dim=-1), atol=1e-5)


def test_attention_is_causal_and_groups_heads():
    torch.manual_seed(1)
    q, k, v = torch.randn(4, 5, 8), torch.randn(2, 5, 8), torch.randn(2, 5, 8)
    out = plain.causal_gqa_attention(q, k, v)
    expected = torch.nn.functional.scaled_dot_product_attention(
        q[None], k.repeat_interleave(2, 0)[None], v.repeat_interleave(2, 0)[None], is_causal=True)[0]
    assert torch.allclose(out, expected, atol=1e-5, rtol=1e-5)
    # the first position sees only itself
    assert torch.allclose(out[:, 0], v.repeat_interleave(2, 0)[:, 0], atol=1e-6)


def test_swiglu_formula():
    torch.manual_seed(2)
    w = {"gate_proj.weight": torch.randn(16, 8), "up_proj.weight": torch.randn(16, 8),
         "down_proj.weight": torch.randn(8, 16)}
    x = torch.randn(3, 8)
    expected = (torch.nn.functional.silu(x @ w["gate_proj.weight"].t()) * (x @ w["up_proj.weight"].t())) @ w["down_proj.weight"].t()
    assert torch.equal(plain.swiglu(x, w, ""), expected)


def test_uniform_draw_is_a_pure_function_in_unit_interval():
    values = {plain.uniform_draw(s, r, t) for s in range(3) for r in range(5) for t in range(7)}
    assert len(values) == 3 * 5 * 7
    assert all(0.0 <= v < 1.0 for v in values)
    assert plain.uniform_draw(1, 2, 3) == plain.uniform_draw(1, 2, 3)


def test_sample_greedy_takes_first_maximum_and_cdf_order():
    logits = torch.tensor([0.0, 3.0, 3.0, 1.0])
    assert plain.sample(logits, 0.0, 0.9) == 1
    # with a very low temperature the mass sits on indices 1 and 2, half each
    assert plain.sample(logits, 0.01, 0.25) == 1
    assert plain.sample(logits, 0.01, 0.75) == 2
