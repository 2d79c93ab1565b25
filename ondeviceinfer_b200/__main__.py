"""Command line: ``python -m ondeviceinfer_b200 <command> ...``

``generate``      load a model folder, generate for a set of prompts and write a JSON report.
                  Options keep the names and meanings of the reference's scripts
                  (benchmarks/benchmark_resident.py:24-35 and benchmarks/validate_correctness.py:24-31
                  of UESlubei/ondeviceinfer): ``--model --prompts --prompt --dtype --max-new-tokens
                  --warmup-runs --repeats --limit --output --stop-on-eos``; added here:
                  ``--prompt-ids --temperature --seed --batch-size``.
``random-model``  write a model folder with seeded random weights from a ``config.json``.

Prompts are token ids (``--prompt-ids 1,2,3`` or rows ``{"id": ..., "prompt_ids": [...]}``
in the ``--prompts`` file).  Text (``--prompt`` or rows with ``"prompt"``) needs the
tokenizer files in the model folder, as the reference's scripts do.
"""

from __future__ import annotations

import argparse
import json
import platform
import statistics
import sys
import time
from pathlib import Path


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="python -m ondeviceinfer_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate for a set of prompts and report timings")
    g.add_argument("--model", type=Path, required=True, help="folder with config.json and safetensors")
    g.add_argument("--prompts", type=Path, help="JSON-lines file with rows {id, prompt_ids | prompt}")
    g.add_argument("--prompt", help="one text prompt (needs the tokenizer files in --model)")
    g.add_argument("--prompt-ids", help="one prompt as comma-separated token ids")
    g.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    g.add_argument("--max-new-tokens", type=int, default=256)
    g.add_argument("--warmup-runs", type=int, default=1)
    g.add_argument("--repeats", type=int, default=3)
    g.add_argument("--limit", type=int, help="use only the first LIMIT prompts")
    g.add_argument("--output", type=Path, help="write the JSON report here")
    g.add_argument("--stop-on-eos", action="store_true", help="end a sequence at the configuration's eos_token_id")
    g.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--batch-size", type=int, default=1,
                   help="prompts generated together (1 = one after another, as the reference does)")
    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--config", type=Path, required=True, help="a config.json")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", type=Path, required=True)
    return parser


def _tokenize(model_dir: Path, texts):
    try:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(model_dir, local_files_only=True)
    except Exception as error:  # noqa: BLE001
        raise SystemExit(f"text prompts need the tokenizer files in {model_dir}: {error}\n"
                         "give token ids instead (--prompt-ids, or rows with \"prompt_ids\")")
    return [tokenizer(text).input_ids for text in texts]


def _load_prompts(args):
    rows = []
    if args.prompt_ids:
        rows.append({"id": "cli", "prompt_ids": [int(t) for t in args.prompt_ids.split(",") if t.strip()]})
    if args.prompt:
        rows.append({"id": "cli-text", "prompt": args.prompt})
    if args.prompts:
        rows += [json.loads(line) for line in args.prompts.read_text(encoding="utf-8").splitlines() if line.strip()]
    if not rows:
        raise SystemExit("no prompts: give --prompts, --prompt-ids or --prompt")
    rows = rows[:args.limit]
    texts = [i for i, row in enumerate(rows) if "prompt_ids" not in row]
    if texts:
        for i, ids in zip(texts, _tokenize(args.model, [rows[i]["prompt"] for i in texts])):
            rows[i]["prompt_ids"] = ids
    return rows


def _generate(args) -> int:
    import torch

    import ondeviceinfer_b200 as odi
    from ondeviceinfer_b200.cache import PAGE_SIZE, pages_for

    if not torch.cuda.is_available():
        raise SystemExit("CUDA is required: this library has no CPU path")
    rows = _load_prompts(args)
    model = odi.load_resident_model(args.model, device="cuda:0", dtype=args.dtype)
    stop = model.config.stop_token_ids if args.stop_on_eos else None
    measurements = []
    for first in range(0, len(rows), args.batch_size):
        group = rows[first:first + args.batch_size]
        prompts = [row["prompt_ids"] for row in group]
        for repetition in range(args.warmup_runs + args.repeats):
            is_warmup = repetition < args.warmup_runs
            tokens = sum(pages_for(len(p) + args.max_new_tokens) * PAGE_SIZE for p in prompts)
            cache = model.make_cache(max_tokens=tokens, max_seqs=len(prompts))
            torch.cuda.reset_peak_memory_stats()
            result = odi.generate(model, prompts, max_new_tokens=args.max_new_tokens, cache=cache,
                                  temperature=args.temperature, seed=args.seed, eos_token_id=stop)
            for row, generated in zip(group, result.generated_ids):
                measurements.append({
                    "prompt_id": row.get("id"), "repetition": repetition, "is_warmup": is_warmup,
                    "batch_size": len(prompts), "input_tokens": len(row["prompt_ids"]),
                    "output_tokens": len(generated), "prefill_ms": result.prefill_seconds * 1000,
                    "ttft_ms": result.prefill_seconds * 1000, "decode_ms": result.decode_seconds * 1000,
                    "decode_tokens_per_s": result.decode_tokens_per_second,
                    "peak_allocated_bytes": torch.cuda.max_memory_allocated(),
                    "peak_reserved_bytes": torch.cuda.max_memory_reserved(),
                    "kv_cache_bytes": cache.storage_bytes, "output_token_ids": generated})
            label = "warmup" if is_warmup else "measure"
            print(f"{group[0].get('id')} {label} {repetition}: TTFT={result.prefill_seconds * 1000:.2f} ms, "
                  f"decode={result.decode_tokens_per_second:.2f} tok/s", flush=True)
            del cache
    measured = [m for m in measurements if not m["is_warmup"]] or measurements
    report = {
        "manifest": {
            "schema_version": 1, "created_unix_seconds": time.time(), "framework": "ondeviceinfer_b200",
            "hostname": platform.node(), "python_version": platform.python_version(),
            "torch_version": torch.__version__, "cuda_version": torch.version.cuda,
            "gpu_name": torch.cuda.get_device_name(0), "model": str(args.model.resolve()), "dtype": args.dtype,
            "max_new_tokens": args.max_new_tokens, "stop_on_eos": args.stop_on_eos,
            "temperature": args.temperature, "seed": args.seed, "batch_size": args.batch_size,
            "warmup_runs": args.warmup_runs, "measurement_runs": args.repeats},
        "summary": {
            "measurement_count": len(measured),
            "median_ttft_ms": statistics.median(m["ttft_ms"] for m in measured),
            "median_decode_tokens_per_s": statistics.median(m["decode_tokens_per_s"] for m in measured),
            "max_peak_allocated_bytes": max(m["peak_allocated_bytes"] for m in measured)},
        "measurements": measurements}
    if args.output:
        args.output.parent.mkdir(parents=True, exist_ok=True)
        args.output.write_text(json.dumps(report, indent=2) + "\n", encoding="utf-8")
    print(json.dumps(report["summary"], indent=2))
    return 0


def _random_model(args) -> int:
    import ondeviceinfer_b200 as odi

    raw = json.loads(args.config.read_text(encoding="utf-8"))
    folder = odi.write_random_model(args.out, raw, args.seed)
    print(f"wrote {folder}/config.json and {folder}/model.safetensors (seed {args.seed})")
    return 0


def main(argv=None) -> int:
    args = _parser().parse_args(argv)
    return _generate(args) if args.command == "generate" else _random_model(args)


if __name__ == "__main__":
    sys.exit(main())
