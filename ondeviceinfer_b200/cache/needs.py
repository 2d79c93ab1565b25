"""What a mixer asks of the cache, declared as data."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVNeed:
    """Keys and values of every cached position (``window`` None) or of the last
    ``window`` positions only."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per sequence, zero when the sequence starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
