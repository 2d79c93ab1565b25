"""The arithmetic behind bench.py's roofline and prefill fractions, and its refusals (no GPU)."""

import importlib.util
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
spec = importlib.util.spec_from_file_location("odi_bench", ROOT / "bench.py")
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def test_bytes_of_a_decode_step_and_flops_of_a_prefill_at_qwen3_8b_sizes():
    cfg = dict(bench.QWEN3_8B)
    per_layer, weight_bytes, kv_bytes_per_token = bench.model_figures(cfg, 36)
    # every weight a step uses once: 36 layers and the output head in bf16 (the embedding is only gathered),
    # the norm weights in fp32
    assert per_layer == 6144 * 4096 + 4096 * 4096 + 3 * 12288 * 4096
    assert abs(weight_bytes - 15.137e9) < 0.01e9
    assert kv_bytes_per_token == 147456                     # keys and values of 8 heads of 128 in 36 layers, bf16
    flops = bench.prefill_flops(cfg, 36, 2048)
    assert abs(flops - 29.69e12) < 0.02e12                  # linear 28.45, causal attention 1.24, one row of logits
    # fewer layers scale the per-layer terms only
    assert bench.model_figures(cfg, 2)[2] == 147456 // 18


def test_other_sizes_are_the_named_ones():
    assert bench.OTHER_SIZES["8B"] == {}
    cfg = dict(bench.QWEN3_8B, **bench.OTHER_SIZES["32B"])
    sizes = (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"], cfg["intermediate_size"])
    assert sizes == (64, 5120, 64, 25600)
    _, weight_bytes, kv = bench.model_figures(cfg, 64)
    assert abs(weight_bytes - 63.97e9) < 0.05e9 and kv == 262144


def test_more_than_one_gpu_is_refused():
    many = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"], capture_output=True, text=True)
    assert many.returncode == 2 and "one GPU" in many.stdout


def test_the_reference_arm_imports_a_verbatim_copy_of_the_reference_or_says_why_not(tmp_path):
    """The reference is plain Python without an installer: its arm runs from a copy of its package folder.
    Without such a copy and without the checkout the arm is unavailable and says so; with a copy it is found;
    and the two arms describe one run with the same ``config`` record."""
    folder, why = bench.reference_package(tmp_path / "nothing_here")
    if folder is None:
        assert "cannot be pip-installed" in why
    else:                                                   # the checkout is on this machine: it was copied
        assert (folder / "ondeviceinfer" / "model.py").exists() and why is None
    made = tmp_path / "ref" / "ondeviceinfer"
    made.mkdir(parents=True)
    (made / "model.py").write_text("")
    assert bench.reference_package(tmp_path / "ref") == (tmp_path / "ref", None)

    import argparse
    args = argparse.Namespace(sizes="8B", prompt_len=2048, prompt_range=None, warmup=5, steps=20, context=None,
                              layers=None, batch=8, temperature=0.0)
    cfg, layers, prompt_len, _, context, _, record, metric = bench.plan_run(args, argparse.ArgumentParser())
    assert (layers, prompt_len, context) == (36, 2048, 4096) and "batch 8" in metric
    assert record["untimed_steps"] == 32 and record["layers"] == record["layers_of_model"] == 36
    assert len(record) <= 20 and all(not isinstance(v, (dict, list)) for v in record.values())


def test_measured_peaks_are_read_flat_or_one_level_down_and_absent_ones_fall_back(tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    assert bench.load_peaks() == (bench.FALLBACK_PEAKS, "fallback")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"hbm_gbs": 7000.0, "bf16_tflops": 1600, "bf16_tflops_sustained": 1450.5, "clocks": {"sm_mhz": 1965}}))
    assert bench.load_peaks() == ({"hbm_gbs": 7000.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1450.5}, "measured")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"peaks": {"hbm_gbs": {"value": 6900.0, "unit": "GB/s"}}}))
    peaks, source = bench.load_peaks()
    assert peaks["hbm_gbs"] == 6900.0 and peaks["bf16_tflops"] == bench.FALLBACK_PEAKS["bf16_tflops"]
    assert source.startswith("measured where given")
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert bench.load_peaks()[1] == "fallback"
