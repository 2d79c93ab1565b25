#!/usr/bin/env python3
"""Serving benchmark of ondeviceinfer_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
                    [--layers L] [--batch B] [--no-points]
                    [--sizes 8B|14B|32B] [--prompt-len T] [--context C]

Measures the metric of BASELINE.json: decode tokens per second (and prefill tokens per
second at 2,048 tokens) for the Qwen3-8B layer sizes in bf16 with seeded random weights
and uniform random token ids.  A "step" is one decode step of the whole batch.  The
default run has a batch of 8 sequences with 2,048-token prompts in a cache sized for a
context of 4,096; ``--sizes``, ``--prompt-len`` and ``--context`` give the same run at the
layer sizes of Qwen3-14B or Qwen3-32B and at other lengths.  One JSON line is printed:

* ``value``   decoded tokens per second over K steps, timed on the device with CUDA
              events (sampled tokens stay on the device);
* ``e2e``     the same through the Python entry point: every step copies the step's
              token ids from pinned host memory to the device and reads the sampled
              tokens back to the host;
* ``prefill`` one 2,048-token prompt: tokens/s, ms, and the fraction of the measured
              bf16 tensor-core peak its flops reach;
* ``roofline`` the decode step against HBM: bytes it must read (every weight it uses
              once, plus the cached keys and values of the live requests) / its time;
* ``points``  decode tokens/s at batch 1 and 64.

Every step reads all weights (16 GB) and the cache, far more than the 126 MB L2, so no
explicit L2 flush is needed between timed steps.  The work runs on one GPU only; for
``--gpus N`` with N > 1 a line says so and the exit code is 2.
"""

from __future__ import annotations

import argparse
import json
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "hidden_act": "silu",
}
# other layer sizes of the same architecture, for runs beside the default one (--sizes)
OTHER_SIZES = {
    "8B": {},
    "14B": {"num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "intermediate_size": 17408},
    "32B": {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64, "intermediate_size": 25600},
}
CONTEXT, PROMPT, PREFILL_TOKENS = 4096, 2048, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            tables = [raw] + [v for v in raw.values() if isinstance(v, dict)]     # flat, or one level down
            peaks, found = dict(FALLBACK_PEAKS), 0
            for key in peaks:
                for table in tables:
                    value = table.get(key)
                    if isinstance(value, dict):
                        value = value.get("value")
                    if isinstance(value, (int, float)) and value > 0:
                        peaks[key], found = float(value), found + 1
                        break
            if found:
                return peaks, "measured" if found == len(peaks) else "measured where given, else fallback"
        except (ValueError, TypeError, AttributeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=5)
        clocks, reasons, max_mhz = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 6:
                continue
            try:
                clocks.append(float(cells[0]))
                max_mhz = float(cells[1])
            except ValueError:
                continue
            for name, cell in zip(names, cells[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max_mhz,
                "reasons": sorted(reasons), "samples": len(clocks)}


def model_figures(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * d * H + H * nq * d + 3 * I * H
    weight_bytes = 2 * (layers * per_layer + V * H) + 4 * (layers * (2 * H + 2 * d) + H)
    kv_bytes_per_token = 2 * nkv * d * 2 * layers
    return per_layer, weight_bytes, kv_bytes_per_token


def prefill_flops(cfg, layers, tokens):
    per_layer, _, _ = model_figures(cfg, layers)
    linear = 2 * tokens * layers * per_layer
    attention = 2 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * tokens * layers  # causal half of 4*T^2
    head = 2 * cfg["vocab_size"] * cfg["hidden_size"]
    return linear + attention + head


def run_reference_arm():
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "ondeviceinfer").exists():
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference has neither setup.py nor pyproject.toml, so the offline pip install into "
                          "baseline/_ref fails ('Directory is not installable')"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref exists but no reference arm is wired"}))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--sizes", default="8B", choices=sorted(OTHER_SIZES), help="layer sizes (default: the benchmark's)")
    parser.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens of each prompt before the timed decode steps")
    parser.add_argument("--prompt-range", default=None, metavar="LOW,HIGH",
                        help="unequal prompts: lengths uniform in [LOW, HIGH] from --seed instead of --prompt-len")
    parser.add_argument("--context", type=int, default=None, help="cache positions per sequence (default 4096, or what the prompt needs)")
    args = parser.parse_args()
    if args.impl == "reference":
        return run_reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    import ondeviceinfer_b200 as odi
    from ondeviceinfer_b200.kernels import ops
    from ondeviceinfer_b200.sampling import Sampler

    cfg = dict(QWEN3_8B, **OTHER_SIZES[args.sizes])
    prompt_len = args.prompt_len
    prompt_range = [int(v) for v in args.prompt_range.split(",")] if args.prompt_range else None
    if prompt_range:
        prompt_len = prompt_range[1]
    needed = prompt_len + args.warmup + args.steps + 1
    context = args.context or max(CONTEXT, -(-needed // 64) * 64)
    if context < needed:
        parser.error(f"--context {context} is below the {needed} positions that the prompt and the steps need")
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    peaks, peak_source = load_peaks()
    torch.cuda.set_device(0)
    model = odi.random_resident_model(cfg, args.seed, device="cuda:0", dtype="bfloat16")
    _, weight_bytes, kv_bytes_per_token = model_figures(cfg, layers)
    gen = torch.Generator().manual_seed(args.seed)
    sampler = Sampler(0.0)

    def prompts_for(batch, length):
        if prompt_range:
            lengths = torch.randint(prompt_range[0], prompt_range[1] + 1, (batch,), generator=gen).tolist()
            return [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
        return torch.randint(0, cfg["vocab_size"], (batch, length), generator=gen).tolist()

    def decode_run(batch, steps, warmup, end_to_end):
        """Prefill `batch` prompts of `prompt_len` tokens, then time `steps` decode steps.

        Device-timed: the steps replay back to back, sampled tokens stay on the device.
        End to end: the public decode call per step, which copies the step's token ids from
        pinned host memory to the device and reads the sampled tokens back to the host."""
        cache = model.make_cache(max_tokens=batch * context, max_seqs=batch)
        slots = [cache.alloc() for _ in range(batch)]
        logits = model.step(cache, slots, prompts_for(batch, prompt_len), "last")
        tokens = sampler(logits, range(batch), [0] * batch)
        runner = odi.api.decode_runner(model, cache, temperature=0.0, seed=0)
        runner.begin(slots, tokens, list(range(batch)), [1] * batch)
        for _ in range(warmup):
            tokens = runner.step(tokens)
        torch.cuda.synchronize()
        before = dict(ops.LAUNCHES)
        start_len = sum(cache.length(slot) for slot in slots) / batch
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall = time.perf_counter()
        start.record()
        if end_to_end:
            for _ in range(steps):
                tokens = runner.step(tokens)
        else:
            runner.step_device(steps)
        stop.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall
        ms = start.elapsed_time(stop)
        launches = {k: ops.LAUNCHES[k] - before[k] for k in before}
        mean_ctx = start_len + (steps - 1) / 2.0
        for slot in slots:
            cache.free(slot)
        runner.close()
        del cache, runner
        torch.cuda.empty_cache()
        seconds = wall if end_to_end else ms / 1000.0
        return {"tok_s": batch * steps / seconds, "ms_per_step": seconds * 1000.0 / steps, "launches": launches,
                "bytes_per_step": weight_bytes + batch * mean_ctx * kv_bytes_per_token}

    def prefill_run(repeats=3):
        cache = model.make_cache(max_tokens=PREFILL_TOKENS, max_seqs=1)
        prompt = prompts_for(1, PREFILL_TOKENS)
        best = None
        for i in range(repeats + 1):
            slot = cache.alloc()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            model.step(cache, [slot], prompt, "last")
            stop.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(stop)
            cache.free(slot)
            if i > 0:
                best = ms if best is None else min(best, ms)
        flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
        return {"value": PREFILL_TOKENS / (best / 1000.0), "tokens": PREFILL_TOKENS, "ms": best,
                "frac": flops / (best / 1000.0) / (peaks["bf16_tflops"] * 1e12), "tflops": flops / best / 1e9}

    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(args.batch, args.steps, args.warmup, end_to_end=False)
    clock_record = clocks.stop()
    e2e_run = decode_run(args.batch, args.steps, args.warmup, end_to_end=True)
    result = {
        "metric": "decode tokens/s (Qwen3-%s layer sizes, bf16, batch %d, %s-token prompts)" % (args.sizes, args.batch, format(prompt_len, ",")),
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights normal(0, 0.02), uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "Qwen3-%s layer sizes" % args.sizes, "layers": layers, "layers_of_model": full_layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"],
            "rms_norm_eps": cfg["rms_norm_eps"], "tied_head": False, "global_batch": args.batch,
            "seq_len": context, "prompt_len": args.prompt_range or prompt_len, "parallelism": "single-gpu",
            "l2": "inputs larger than L2: each step reads all weights and the cache",
            "peaks": peak_source},
        "e2e": {"value": e2e_run["tok_s"], "unit": "tokens/s", "ms_per_step": e2e_run["ms_per_step"],
                "h2d_bytes_per_step": 4 * args.batch, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": main_run["launches"]["own"], "library_gemm_launches": main_run["launches"]["library"],
        "clocks": clock_record,
        "roofline": {"bound": "hbm", "achieved": main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1000.0) / 1e9,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s"},
    }
    result["roofline"]["frac"] = result["roofline"]["achieved"] / result["roofline"]["peak"]
    if not args.no_points:
        result["prefill"] = prefill_run()
        points = {}
        for batch in (1, 64):
            run = decode_run(batch, min(args.steps, 64), 3, end_to_end=False)
            points[f"decode_b{batch}"] = run["tok_s"]
            points[f"decode_b{batch}_hbm_frac"] = run["bytes_per_step"] / (run["ms_per_step"] / 1000.0) / 1e9 / peaks["hbm_gbs"]
        result["points"] = points
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
