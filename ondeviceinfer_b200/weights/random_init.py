"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` with exactly the tensors the
architecture's parts declare, under their checkpoint names.  Matrices and the embedding
are normal(0, 0.02), norm weights 1 + normal(0, 0.01), each tensor drawn from a
generator keyed by ``(seed, tensor name)``.  The reference has no such mode; its tests
seed torch's default initialisers (tests/test_model.py:102-104 of UESlubei/ondeviceinfer).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..registry import config_from_dict
from .tensors import RandomSource


def declared_tensors(plan):
    """All tensor declarations of a plan, without touching a device."""
    from ..engine.model import DecoderModel

    return DecoderModel(plan).tensor_decls()


def write_random_model(folder, config, seed: int, *, dtype: torch.dtype = torch.bfloat16) -> Path:
    """``config`` is a typed configuration or a ``config.json`` dictionary."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    if isinstance(config, dict):
        config = config_from_dict(config)
    from safetensors.torch import save_file

    source = RandomSource(declared_tensors(config.to_plan()), seed, dtype=dtype, device="cpu")
    tensors = {name: source.fetch(name).contiguous() for name in source.stored()}
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n", encoding="utf-8")
    return folder
