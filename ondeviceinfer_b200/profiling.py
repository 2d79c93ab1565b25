"""Opt-in NVTX ranges around steps, layers and the phases of generation.

``ONDEVICEINFER_NVTX=1`` (or ``true`` / ``yes`` / ``on``) in the environment when the package is imported
turns them on, the switch of UESlubei/ondeviceinfer (ondeviceinfer/profiling.py:17-49, read once at
import).  Switched off, ``nvtx_range`` hands out one shared do-nothing context, so the step function
pays a dictionary-free attribute call per range and nothing else.  Ranges are host-side marks: inside a
CUDA-graph capture they describe the capture, and a replayed graph shows as the one range around it.
"""

from __future__ import annotations

import os

_ON = os.environ.get("ONDEVICEINFER_NVTX", "0").strip().lower() in ("1", "true", "yes", "on")


def nvtx_enabled() -> bool:
    """Whether this process was started with NVTX ranges switched on."""
    return _ON


class _Nothing:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _Range:
    __slots__ = ("name",)

    def __init__(self, name: str) -> None:
        self.name = name

    def __enter__(self):
        import torch

        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        import torch

        torch.cuda.nvtx.range_pop()
        return False


_NOTHING = _Nothing()


def nvtx_range(name: str):
    """``with nvtx_range("step"): ...``; a no-op unless the switch is on."""
    return _Range(name) if _ON else _NOTHING
