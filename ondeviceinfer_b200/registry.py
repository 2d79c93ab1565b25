"""One registry from an architecture's name to its model description.

An entry is a configuration class with three members: ``from_dict(raw)`` (typed
configuration from the ``config.json`` dictionary), ``to_plan()`` (the
:class:`~ondeviceinfer_b200.config.specs.ModelPlan` the engine builds) and
``to_dict()`` (a ``config.json`` that reads back equal).  The reference has no
registry: it only checks ``model_type == "qwen3"`` (ondeviceinfer/config.py:40-43);
here the model class is chosen by ``config.json["architectures"][0]``, with
``model_type`` as the fallback for folders that lack that key.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Mapping

_ARCHITECTURES: Dict[str, type] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_cls: type, *, model_type: str | None = None) -> None:
    """Make ``name`` (as written in ``config.json["architectures"]``) loadable."""
    for member in ("from_dict", "to_plan"):
        if not hasattr(config_cls, member):
            raise TypeError(f"{config_cls.__name__} lacks {member}(); see ondeviceinfer_b200.registry")
    _ARCHITECTURES[name] = config_cls
    if model_type is not None:
        _MODEL_TYPES[model_type] = name


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_name(raw: Mapping[str, Any]) -> str:
    archs = raw.get("architectures") or []
    if archs:
        name = archs[0]
    elif raw.get("model_type") in _MODEL_TYPES:
        name = _MODEL_TYPES[raw["model_type"]]
    else:
        raise KeyError(f"config.json names no architecture (architectures={archs!r}, "
                       f"model_type={raw.get('model_type')!r}); known: {known_architectures()}")
    if name not in _ARCHITECTURES:
        raise KeyError(f"unknown architecture {name!r}; known: {known_architectures()}")
    return name


def config_from_dict(raw: Mapping[str, Any]):
    return _ARCHITECTURES[architecture_name(raw)].from_dict(raw)


def config_from_folder(folder):
    path = Path(folder) / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"no config.json in {folder}")
    return config_from_dict(json.loads(path.read_text(encoding="utf-8")))
