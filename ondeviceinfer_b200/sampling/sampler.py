"""Choosing the next token from logits, on the device.

``temperature == 0``: the first index of the maximum, the reference's greedy rule
(ondeviceinfer/generation.py:47,58).  ``temperature > 0``: a draw from
softmax(logits / temperature) by the inverse CDF in vocabulary order, with the uniform
number ``uniform_draw(seed, request, step)``; since that number depends on nothing else,
a request's tokens do not depend on the batch it runs in.  The reference samples
greedily only; temperature sampling is this library's addition.
"""

from __future__ import annotations

from typing import List, Sequence

import torch

from ..kernels import ops

_MASK64 = (1 << 64) - 1


def uniform_draw(seed: int, stream: int, step: int) -> float:
    """Host restatement of the device generator (csrc/sampling.cu): 24 bits of a 64-bit
    mix of (seed, stream, step), as a float in [0, 1)."""
    x = (seed * 0x9E3779B97F4A7C15 + stream * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & _MASK64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _MASK64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _MASK64
    x ^= x >> 31
    return (x >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, temperature: float = 0.0, seed: int = 0) -> None:
        if temperature < 0:
            raise ValueError("temperature must not be negative")
        self.temperature, self.seed = float(temperature), int(seed)

    def sample_device(self, logits: torch.Tensor, streams: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """int32 tokens on the device, one per row of ``logits`` (fp32 [rows, vocab])."""
        n = logits.shape[0]
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
        if self.temperature > 0:
            meta = torch.tensor([list(streams), list(steps)], dtype=torch.int32).to(logits.device)
            ops.sample(logits, out, self.temperature, self.seed, meta[0], meta[1])
        else:
            ops.sample(logits, out, 0.0)
        return out

    def __call__(self, logits: torch.Tensor, streams: Sequence[int], steps: Sequence[int]) -> List[int]:
        return self.sample_device(logits, streams, steps).tolist()
