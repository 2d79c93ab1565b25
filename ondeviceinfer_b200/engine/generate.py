"""The generation loop above the step function.

Requests are lists of token ids.  They are served in batches: the prompts of a batch
run in one step, then every live sequence advances by one token per step; a sequence
ends when it produces a stop token (which is kept) or reaches ``max_new_tokens`` (which
counts the token the prompt produces, as ondeviceinfer/generation.py:46-59 does); its
slot is given back at once and the batch goes on without it.  When a batch is finished
the next one starts, on the same cache, until every request is served.  The reference's
loop is batch 1 and greedy only (ondeviceinfer/generation.py:39-40,47); batching, stop
per sequence and temperature sampling are this library's.

The loop talks to the model through four callables (``alloc``, ``free``, ``step``,
``sample``), so its decisions can be tested without a GPU.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Sequence

from ..profiling import nvtx_range


@dataclass
class GenerationResult:
    """``generated_ids[r]`` are the new tokens of request ``r``; ``token_ids[r]`` is its
    prompt followed by them.  Times are wall-clock seconds with the device synchronised;
    ``decode_tokens_per_second`` counts the tokens produced by decode steps only, as
    ondeviceinfer/generation.py:22-25 does."""

    token_ids: List[List[int]]
    generated_ids: List[List[int]]
    finish_reasons: List[str]
    prefill_seconds: float
    decode_seconds: float
    decode_steps: int = 0
    batches: List[List[int]] = field(default_factory=list)
    capture_seconds: float = 0.0    # one-off set-up of a fused decoder (graph captures), not part of decode_seconds
    # wall seconds of every decode step in the order they ran (all batches), from the loop's stop tests to the
    # step's tokens on the host, without set-up: sum(step_seconds) is decode_seconds but for the batches' ends
    step_seconds: List[float] = field(default_factory=list)

    @property
    def decode_tokens(self) -> int:
        return sum(max(0, len(g) - 1) for g in self.generated_ids)

    @property
    def decode_tokens_per_second(self) -> float:
        return self.decode_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, *, max_seqs: int, max_tokens: int,
                 page_size: int) -> List[List[int]]:
    """Cut the requests, in order, into batches that fit the cache: at most ``max_seqs``
    sequences, and room for every sequence at its longest (prompt + max_new_tokens - 1
    cached positions, rounded up to whole pages)."""
    def footprint(n: int) -> int:
        longest = n + max(max_new_tokens - 1, 0)
        return -(-longest // page_size) * page_size

    batches: List[List[int]] = []
    current: List[int] = []
    used = 0
    for r, n in enumerate(prompt_lengths):
        if n <= 0:
            raise ValueError(f"request {r} has an empty prompt")
        need = footprint(n)
        if need > max_tokens:
            raise ValueError(f"request {r} needs room for {need} tokens, the cache holds {max_tokens}")
        if current and (len(current) >= max_seqs or used + need > max_tokens):
            batches.append(current)
            current, used = [], 0
        current.append(r)
        used += need
    if current:
        batches.append(current)
    return batches


def generate_requests(prompts: Sequence[Sequence[int]], *, max_new_tokens: int,
                      alloc: Callable[[], int], free: Callable[[int], None],
                      step: Callable[[List[int], List[List[int]]], object],
                      sample: Callable[[object, List[int], List[int]], List[int]],
                      batches: Sequence[Sequence[int]], stop_token_ids: Sequence[int] = (),
                      synchronize: Callable[[], None] = lambda: None, decoder=None) -> GenerationResult:
    """``step(slots, token_runs)`` returns the logits at each run's last token;
    ``sample(logits, request_indices, step_numbers)`` returns one token per row.

    ``decoder`` (optional) fuses step and sampling for the one-token steps: an object with
    ``begin(slots, last_tokens, request_indices, step_numbers)`` (called whenever the live
    set changed) and ``step(last_tokens) -> tokens`` (one decode step of the live set, in order;
    the host's record of each sequence's last token is what the step is fed).  If it has a
    ``capture_seconds`` counter, what it adds during a batch (one-off set-up such as graph captures)
    is taken out of ``decode_seconds`` and reported apart.

    ``synchronize`` is called where the loop has to wait for the device anyway (around the prompts'
    step and at the end of a batch); it may raise, which ends the generation."""
    if max_new_tokens <= 0:
        raise ValueError("max_new_tokens must be positive")
    stop = set(int(t) for t in stop_token_ids)
    generated: List[List[int]] = [[] for _ in prompts]
    reasons = ["" for _ in prompts]
    prefill_seconds = decode_seconds = capture_seconds = 0.0
    decode_steps = 0
    step_seconds: List[float] = []
    set_up_so_far = lambda: getattr(decoder, "capture_seconds", 0.0)
    for batch in batches:
        live = list(batch)
        slots = {r: alloc() for r in live}
        try:
            synchronize()
            start = time.perf_counter()
            with nvtx_range(f"prefill[{len(live)} requests]"):
                logits = step([slots[r] for r in live], [list(prompts[r]) for r in live])
                tokens = sample(logits, live, [0] * len(live))
                synchronize()
            prefill_seconds += time.perf_counter() - start
            start = time.perf_counter()
            set_up = set_up_so_far()
            changed = True
            while True:
                step_start, step_set_up = time.perf_counter(), set_up_so_far()
                still = []
                for r, tok in zip(live, tokens):
                    generated[r].append(int(tok))
                    if int(tok) in stop:
                        reasons[r] = "stop"
                    elif len(generated[r]) >= max_new_tokens:
                        reasons[r] = "length"
                    else:
                        still.append(r)
                        continue
                    free(slots.pop(r))
                changed = changed or len(still) != len(live)
                live = still
                if not live:
                    break
                if decoder is None:
                    logits = step([slots[r] for r in live], [[generated[r][-1]] for r in live])
                    tokens = sample(logits, live, [len(generated[r]) for r in live])
                else:
                    if changed:
                        decoder.begin([slots[r] for r in live], [generated[r][-1] for r in live], live,
                                      [len(generated[r]) for r in live])
                        changed = False
                    tokens = decoder.step([generated[r][-1] for r in live])
                decode_steps += 1
                step_seconds.append(time.perf_counter() - step_start - (set_up_so_far() - step_set_up))
            synchronize()
            set_up = set_up_so_far() - set_up
            capture_seconds += set_up
            decode_seconds += time.perf_counter() - start - set_up
        finally:
            for slot in slots.values():
                free(slot)
    return GenerationResult(
        token_ids=[list(p) + g for p, g in zip(prompts, generated)], generated_ids=generated,
        finish_reasons=reasons, prefill_seconds=prefill_seconds, decode_seconds=decode_seconds,
        decode_steps=decode_steps, batches=[list(b) for b in batches], capture_seconds=capture_seconds,
        step_seconds=step_seconds)
