"""Shared helpers of the tests: tolerances, model folders in temporary directories."""

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

import plain_qwen3 as plain

# Stated once, used everywhere.  fp32: the engine and the plain implementation follow the
# same formulas in the same precision and differ by summation order only (observed
# ~5e-7 on the tiny models).  bf16: the engine keeps fp32 accumulators and rounds once
# per operation, the plain bf16 arithmetic rounds after every elementary operation
# (observed 3e-3 to 7e-3 at |logit| ~ 1).  The bf16 criteria, with s = max(1, max |reference logit|):
# every |d| <= BF16_REL * s, the mean |d| <= BF16_MEAN * s, and every row's cosine with its reference row
# >= BF16_COSINE.  A chosen token counts as the reference's choice if its reference logit is within
# BF16_TIE of the reference maximum; a sampled token if the uniform number lies within BF16_CDF of its
# interval of the reference distribution.
F32_ATOL, F32_RTOL = 2e-5, 2e-5
BF16_REL, BF16_MEAN, BF16_COSINE = 1.5e-2, 3e-3, 0.999
BF16_TIE, BF16_CDF = 1e-2, 1e-2
# The fp32 figure holds for sums of up to 256 terms (the tiny models).  The rounding error of an
# fp32 sum taken in another order grows like the square root of its length, so a model whose
# longest sum has K terms is compared with F32_ATOL * sqrt(K / 256): 1.4e-4 at the 12288-wide
# feed-forward of Qwen3-8B (observed there: 3.2e-5).
F32_SUM_LENGTH = 256


def assert_logits_close(actual: torch.Tensor, expected: torch.Tensor, dtype: str, what: str = "",
                        longest_sum: int = F32_SUM_LENGTH) -> None:
    actual, expected = actual.float().cpu(), expected.float().cpu()
    assert actual.shape == expected.shape, (what, actual.shape, expected.shape)
    assert torch.isfinite(actual).all(), f"{what}: non-finite logits"
    gap = (actual - expected).abs()
    if dtype == "float32":
        atol = F32_ATOL * max(1.0, (longest_sum / F32_SUM_LENGTH) ** 0.5)
        bad = gap > atol + F32_RTOL * expected.abs()
        assert not bad.any(), f"{what}: fp32 max |d| = {float(gap.max()):.3e} at {int(gap.argmax())}"
    else:
        scale = max(1.0, float(expected.abs().max()))
        assert float(gap.max()) <= BF16_REL * scale, f"{what}: bf16 max |d| = {float(gap.max()):.3e} > {BF16_REL * scale:.3e}"
        if gap.numel():
            assert float(gap.mean()) <= BF16_MEAN * scale, f"{what}: bf16 mean |d| = {float(gap.mean()):.3e} > {BF16_MEAN * scale:.3e}"
            cosine = torch.nn.functional.cosine_similarity(actual.double(), expected.double(), dim=-1)
            assert float(cosine.min()) >= BF16_COSINE, f"{what}: bf16 cosine {float(cosine.min()):.6f} in row {int(cosine.argmin())}"


def write_model_folder(folder, cfg: dict, weights: dict) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(cfg))
    return folder


CASES = {
    "A": (plain.TINY_A, 0),
    "B": (plain.TINY_B, 1),
    "C": (plain.TINY_C, 2),
    # with projection biases
    "Ab": (plain.TINY_A_BIAS, 10),
    "Bb": (plain.TINY_B_BIAS, 11),
    "Cb": (plain.TINY_C_BIAS, 12),
    # a width that is no multiple of 8, heads of 48, biases
    "D": (plain.TINY_D, 13),
}


_MODELS = {}


def engine_model(case: str, dtype: str, tmp_root):
    """The engine's model for a tiny case, loaded once per test session from a folder
    written into a temporary directory; returns (model, weights, config dictionary)."""
    import ondeviceinfer_b200 as odi

    key = (case, dtype)
    if key not in _MODELS:
        cfg, seed = CASES[case]
        weights = plain.random_weights(cfg, seed)
        folder = write_model_folder(Path(tmp_root) / f"model_{case}", cfg, weights)
        _MODELS[key] = (odi.load_resident_model(folder, device="cuda:0", dtype=dtype), weights, cfg)
    return _MODELS[key]


_PLAIN = {}


def plain_logits(case: str, tokens, dtype: str = "float32"):
    """Whole-sequence logits of the plain implementation (memoised)."""
    cfg, seed = CASES[case]
    key = (case, tuple(tokens), dtype)
    if key not in _PLAIN:
        weights = plain.random_weights(cfg, seed)
        _PLAIN[key] = plain.forward_logits(weights, cfg, list(tokens),
                                           torch.float32 if dtype == "float32" else torch.bfloat16)
    return _PLAIN[key]
