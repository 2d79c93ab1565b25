"""Generation through the Python entry point and the command line, against the plain implementation."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import ondeviceinfer_b200 as odi
import plain_qwen3 as plain
from helpers import BF16_CDF, BF16_TIE, CASES, engine_model, write_model_folder

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="session")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("models")


def near_tie(weights, cfg, prefix, token, dtype):
    """True if `token` is the plain argmax after `prefix`, or within the bf16 tolerance of it."""
    logits = plain.forward_logits(weights, cfg, prefix)[-1]
    return float(logits.max() - logits[token]) <= (0.0 if dtype == "float32" else BF16_TIE)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_of_model_a(dtype, tmp_root):
    """Three prompts of 5, 11 and 17 tokens, 8 new tokens each, as one batch."""
    model, weights, cfg = engine_model("A", dtype, tmp_root)
    prompts = plain.random_prompts(cfg, [5, 11, 17], 0)
    result = odi.greedy_generate(model, prompts, max_new_tokens=8)
    expected = [plain.generate(weights, cfg, p, 8) for p in prompts]
    if result.generated_ids != expected:          # bf16 may flip a near-tie; then every token must still be one
        assert dtype == "bfloat16"
        for p, g in zip(prompts, result.generated_ids):
            assert all(near_tie(weights, cfg, p + g[:t], g[t], dtype) for t in range(len(g)))
    assert [len(g) for g in result.generated_ids] == [8, 8, 8]
    assert result.token_ids[1] == prompts[1] + result.generated_ids[1]
    assert result.finish_reasons == ["length"] * 3 and result.decode_steps == 7
    assert result.prefill_seconds > 0 and result.decode_seconds > 0 and result.decode_tokens == 21
    tensor_prompts = torch.tensor([prompts[0], prompts[0]])
    twice = odi.greedy_generate(model, tensor_prompts, max_new_tokens=3)
    assert twice.generated_ids[0] == twice.generated_ids[1] == result.generated_ids[0][:3]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_of_model_b_does_not_depend_on_the_batch(dtype, tmp_root):
    """Four prompts of 1, 7, 30 and 64 tokens, temperature 0.8, seed 1, 16 tokens: the same
    tokens as the plain implementation draws with the same uniform numbers, whether the
    requests run as one batch or in batches of two on a small cache."""
    model, weights, cfg = engine_model("B", dtype, tmp_root)
    prompts = plain.random_prompts(cfg, [1, 7, 30, 64], 1)
    together = odi.generate(model, prompts, max_new_tokens=16, temperature=0.8, seed=1)
    small = model.make_cache(max_tokens=2 * 128, max_seqs=2)
    in_pairs = odi.generate(model, prompts, max_new_tokens=16, temperature=0.8, seed=1, cache=small)
    assert in_pairs.batches == [[0, 1], [2, 3]]
    small.check()
    assert small.slots.held_count == 0
    if dtype == "float32":
        assert together.generated_ids == in_pairs.generated_ids
        for r, p in enumerate(prompts):
            expected = plain.generate(weights, cfg, p, 16, temperature=0.8, seed=1, stream=r)
            assert together.generated_ids[r] == expected, r
    else:
        # bf16 logits differ slightly: each token must be what the plain CDF gives for a uniform
        # number within a small distance of the one drawn
        for r, p in enumerate(prompts):
            g = together.generated_ids[r]
            for t, token in enumerate(g):
                logits = plain.forward_logits(weights, cfg, p + g[:t])[-1].double()
                cdf = torch.softmax(logits / 0.8, 0).cumsum(0)
                u = plain.uniform_draw(1, r, t)
                lo = float(cdf[token - 1]) if token > 0 else 0.0
                assert lo - BF16_CDF <= u <= float(cdf[token]) + BF16_CDF, (r, t)
    other_seed = odi.generate(model, prompts, max_new_tokens=16, temperature=0.8, seed=2)
    assert other_seed.generated_ids != together.generated_ids


def test_stop_tokens_end_sequences_early_and_are_kept(tmp_root):
    model, weights, cfg = engine_model("B", "float32", tmp_root)
    prompts = plain.random_prompts(cfg, [1, 7, 30, 64], 1)
    free_run = odi.greedy_generate(model, prompts, max_new_tokens=12)
    stop = free_run.generated_ids[2][3]              # a token that request 2 produces as its fourth
    result = odi.greedy_generate(model, prompts, max_new_tokens=12, eos_token_id=stop)
    for r, (free, got) in enumerate(zip(free_run.generated_ids, result.generated_ids)):
        cut = free.index(stop) + 1 if stop in free else len(free)
        assert got == free[:cut], r
        assert result.finish_reasons[r] == ("stop" if stop in free else "length")
    assert len(result.generated_ids[2]) <= 4
    assert odi.generate(model, prompts, max_new_tokens=12, eos_token_id=[stop, 9999]).generated_ids == result.generated_ids


def test_reference_style_entry_point(tmp_root):
    """load_resident_model / make_resident_cache / greedy_generate with the reference's argument names."""
    cfg, seed = CASES["A"]
    weights = plain.random_weights(cfg, seed)
    folder = write_model_folder(tmp_root / "entry", cfg, weights)
    model = odi.load_resident_model(folder, device="cuda:0", dtype=torch.float32)
    cache = model.make_resident_cache(batch_size=1, max_seq_len=11 + 8)
    assert cache.max_seqs == 1 and cache.max_tokens == 64
    prompt = plain.random_prompts(cfg, [11], 3)
    result = odi.greedy_generate(model, torch.tensor(prompt), max_new_tokens=8, cache=cache, eos_token_id=None)
    assert result.generated_ids[0] == plain.generate(weights, cfg, prompt[0], 8)
    assert result.decode_tokens_per_second > 0
    with pytest.raises(odi.WeightsError):
        bad = dict(weights)
        del bad["model.norm.weight"]
        odi.load_resident_model(write_model_folder(tmp_root / "bad", cfg, bad), dtype="float32")
    with pytest.raises(RuntimeError):
        odi.load_resident_model(folder, device="cpu", dtype="float32")


def test_command_line_generates_and_reports(tmp_root):
    cfg, seed = CASES["B"]
    weights = plain.random_weights(cfg, seed)
    config_path = tmp_root / "cli_config.json"
    config_path.write_text(json.dumps(cfg))
    folder = tmp_root / "cli_model"
    run = lambda *a: subprocess.run([sys.executable, "-m", "ondeviceinfer_b200", *a], cwd=ROOT, text=True,
                                    capture_output=True, timeout=600)
    made = run("random-model", "--config", str(config_path), "--seed", "4", "--out", str(folder))
    assert made.returncode == 0, made.stderr
    prompts = plain.random_prompts(cfg, [7, 30], 1)
    rows = tmp_root / "prompts.jsonl"
    rows.write_text("".join(json.dumps({"id": f"p{i}", "prompt_ids": p}) + "\n" for i, p in enumerate(prompts)))
    report_path = tmp_root / "report.json"
    done = run("generate", "--model", str(folder), "--prompts", str(rows), "--dtype", "float32",
               "--max-new-tokens", "5", "--warmup-runs", "0", "--repeats", "1", "--output", str(report_path))
    assert done.returncode == 0, done.stderr
    report = json.loads(report_path.read_text())
    assert report["summary"]["measurement_count"] == 2 and report["manifest"]["dtype"] == "float32"
    from ondeviceinfer_b200.weights import SafetensorsSource
    source = SafetensorsSource(folder)
    written = {n: source.fetch(n) for n in source.stored()}
    for row, prompt in zip(report["measurements"], prompts):
        assert row["output_token_ids"] == plain.generate(written, cfg, prompt, 5)
        assert row["input_tokens"] == len(prompt) and row["output_tokens"] == 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_gives_the_tokens_of_the_plain_step_path(dtype, tmp_root):
    """Decode steps replayed as CUDA graphs (fixed-width batches with padding rows, counters
    advanced on the device) against the same generation through the generic step function."""
    model, weights, cfg = engine_model("C", dtype, tmp_root)
    prompts = plain.random_prompts(cfg, [3, 60, 77, 129, 64], 31)
    for temperature in (0.0, 0.9):
        kwargs = dict(max_new_tokens=70, temperature=temperature, seed=5, eos_token_id=None)
        stepped = odi.generate(model, prompts, use_graphs=False, **kwargs)
        cache = model.make_cache(max_tokens=5 * 256, max_seqs=5)
        replayed = odi.generate(model, prompts, cache=cache, use_graphs=True, **kwargs)
        again = odi.generate(model, prompts[:3], cache=cache, use_graphs=True, **kwargs)   # width 4 with one padding row
        cache.check()
        assert cache.slots.held_count == 0
        if dtype == "float32":
            assert replayed.generated_ids == stepped.generated_ids
            assert again.generated_ids == stepped.generated_ids[:3]
        elif temperature == 0.0:
            # bf16: the logits of graph replay are compared row by row elsewhere (test_decode_graph_gpu.py); here
            # every token either run chose must be the plain argmax after the same prefix, or within a near-tie of it
            for run in (replayed, stepped, again):
                for p, g in zip(prompts, run.generated_ids):
                    assert all(near_tie(weights, cfg, p + g[:t], g[t], dtype) for t in range(len(g)))
    # sequences that stop at different times: the batch narrows and the runner re-begins
    free_run = odi.generate(model, prompts, max_new_tokens=40, use_graphs=False)
    stop = free_run.generated_ids[1][10]
    a = odi.generate(model, prompts, max_new_tokens=40, eos_token_id=stop, use_graphs=True)
    b = odi.generate(model, prompts, max_new_tokens=40, eos_token_id=stop, use_graphs=False)
    if dtype == "float32":
        assert a.generated_ids == b.generated_ids and a.finish_reasons == b.finish_reasons


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_while_the_longest_sequence_passes_a_power_of_two(dtype, tmp_root):
    """A captured graph fixes how many blocks share a sequence's keys, chosen from the longest
    sequence; when that length passes 256 in the middle of a batch another graph takes over on
    the same buffers, and the tokens stay those of the step path."""
    model, weights, cfg = engine_model("C", dtype, tmp_root)
    prompts = plain.random_prompts(cfg, [200, 250, 17], 77)
    kwargs = dict(max_new_tokens=24, temperature=0.0, eos_token_id=None)
    stepped = odi.generate(model, prompts, use_graphs=False, **kwargs)
    cache = model.make_cache(max_tokens=3 * 320, max_seqs=3)
    replayed = odi.generate(model, prompts, cache=cache, use_graphs=True, **kwargs)
    cache.check()
    if dtype == "float32":
        assert replayed.generated_ids == stepped.generated_ids
        assert replayed.generated_ids[1] == plain.generate(weights, cfg, prompts[1], 24)
    else:
        for p, g in zip(prompts, replayed.generated_ids):
            assert all(near_tie(weights, cfg, p + g[:t], g[t], dtype) for t in range(len(g)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_unequal_requests_that_stop_at_random_steps(dtype, tmp_root):
    """Twenty-five requests of 1 to 700 tokens on a cache of four slots, a stop set of a fifth of the vocabulary, so
    that sequences end at random steps: batches narrow (widths 4, 2, 1), slots and pages are reused, graphs for
    shorter sequences are captured on buffers that held longer ones.  Every request ends for the reason its last
    token gives, nothing is left held, no kernel reports a fault, and in 32-bit graph replay gives the tokens of the
    step function."""
    import random

    from ondeviceinfer_b200.kernels import ops
    model, _, cfg = engine_model("C", dtype, tmp_root)
    rng = random.Random(3)
    lengths = [rng.choice([1, 2, 63, 64, 65, 130, 300, 700]) for _ in range(25)]
    prompts = plain.random_prompts(cfg, lengths, 55)
    stop = list(range(0, cfg["vocab_size"], 5))
    cache = model.make_cache(max_tokens=4 * 896, max_seqs=4)
    runs = {}
    for use_graphs in (True, False):
        for temperature in (0.0, 0.9):
            result = odi.generate(model, prompts, max_new_tokens=90, temperature=temperature, seed=7, cache=cache,
                                  eos_token_id=stop, use_graphs=use_graphs)
            torch.cuda.synchronize()
            ops.raise_on_kernel_fault()
            cache.check()
            assert cache.slots.held_count == 0
            for g, reason in zip(result.generated_ids, result.finish_reasons):
                assert 1 <= len(g) <= 90 and all(t % 5 for t in g[:-1])
                assert reason == ("stop" if g[-1] % 5 == 0 else "length") and (reason == "stop" or len(g) == 90)
            assert result.finish_reasons.count("stop") >= 20
            runs[use_graphs, temperature] = result.generated_ids
    if dtype == "float32":
        assert runs[True, 0.0] == runs[False, 0.0] and runs[True, 0.9] == runs[False, 0.9]
