"""bin/trace_run as a user runs it: a subprocess fed one JSON line per step, waiting for
``done <step>`` before the next.  The same requests are replayed whole, with the last 32
tokens one by one, and in batches of unequal lengths on a cache too small for all of them
at once (so slots and pages are used again); every logit is compared with the plain
implementation, in 32-bit and in bfloat16."""

import json
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import CASES, assert_logits_close, write_model_folder

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LENGTHS = [1, 7, 30, 64, 65, 130, 40]


class Replay:
    def __init__(self, model_dir, dtype, out_dir, max_tokens):
        self.out = Path(out_dir)
        self.proc = subprocess.Popen(
            [str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd="/")
        self.step = 0

    def run(self, entries, end=()):
        record = {"step": self.step, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(record) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.step}", f"expected 'done {self.step}', got {line!r}"
        wanted = sum(len(e["want"]) for e in entries)
        path = self.out / f"{self.step}.f32"
        self.step += 1
        if wanted == 0:
            assert not path.exists()
            return None
        data = np.fromfile(path, dtype="<f4")
        return torch.from_numpy(data.reshape(wanted, -1).copy())

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_whole_tail_and_batched(dtype, tmp_path):
    cfg, seed = CASES["B"]
    weights = plain.random_weights(cfg, seed)
    model_dir = write_model_folder(tmp_path / "model", cfg, weights)
    requests = plain.random_prompts(cfg, LENGTHS, 21)
    expected = [plain.forward_logits(weights, cfg, r) for r in requests]
    # room for the largest batch below: 130 + 40 + 65 -> 192 + 64 + 128 = 384 tokens in pages of 64
    replay = Replay(model_dir, dtype, tmp_path / "out", max_tokens=384)
    try:
        # 1. whole: each request alone, every position wanted
        for r, tokens in enumerate(requests):
            got = replay.run([{"id": f"w{r}", "tokens": tokens, "want": list(range(len(tokens)))}], end=[f"w{r}"])
            assert got.shape == (len(tokens), cfg["vocab_size"])
            assert_logits_close(got, expected[r], dtype, f"whole {r}")
        # 2. the last 32 tokens one by one
        for r, tokens in enumerate(requests):
            cut = max(1, len(tokens) - 32)
            rows = [replay.run([{"id": f"t{r}", "tokens": tokens[:cut], "want": list(range(cut))}])]
            for t in range(cut, len(tokens)):
                last = t == len(tokens) - 1
                rows.append(replay.run([{"id": f"t{r}", "tokens": [tokens[t]], "want": [0]}],
                                       end=[f"t{r}"] if last else []))
            assert_logits_close(torch.cat(rows), expected[r], dtype, f"tail {r}")
        # 3. batches of unequal lengths; a step that wants nothing; shorter requests end earlier
        for batch in ([5, 6, 4], [0, 1, 2], [3]):
            cut = {r: max(1, len(requests[r]) - 4 - 5 * (r % 3)) for r in batch}
            got = {r: [] for r in batch}
            entries = [{"id": f"b{r}", "tokens": requests[r][:cut[r]],
                        "want": list(range(cut[r])) if r != 6 else []} for r in batch]
            out = replay.run(entries, end=[f"b{r}" for r in batch if cut[r] == len(requests[r])])
            offset = 0
            for e, r in zip(entries, batch):
                got[r].append(out[offset:offset + len(e["want"])])
                offset += len(e["want"])
            live = [r for r in batch if cut[r] < len(requests[r])]
            while live:
                entries = [{"id": f"b{r}", "tokens": [requests[r][cut[r]]], "want": [0]} for r in live]
                for r in live:
                    cut[r] += 1
                ended = [r for r in live if cut[r] == len(requests[r])]
                out = replay.run(entries, end=[f"b{r}" for r in ended])
                for i, r in enumerate(live):
                    got[r].append(out[i:i + 1])
                live = [r for r in live if r not in ended]
            for r in batch:
                skip = (max(1, len(requests[6]) - 4 - 5 * (6 % 3))) if r == 6 else 0
                assert_logits_close(torch.cat(got[r]), expected[r][skip:], dtype, f"batched {r}")
    finally:
        replay.close()


def test_replay_refuses_more_tokens_than_it_was_sized_for(tmp_path):
    cfg, seed = CASES["A"]
    model_dir = write_model_folder(tmp_path / "model", cfg, plain.random_weights(cfg, seed))
    proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", "float32",
                           "--out", str(tmp_path / "out"), "--max-tokens", "64"], text=True, capture_output=True,
                          input=json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": [64]}], "end": []}) + "\n")
    assert proc.returncode != 0 and "capacity" in proc.stderr
