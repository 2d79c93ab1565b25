"""Where tensors come from: a safetensors folder, or a seeded random generator.

Both sources answer the same two questions -- which tensors exist (name, shape,
stored dtype) and what one tensor holds -- so that the loader, the random-weights
writer and the benchmark share one binding path.

File discovery follows ondeviceinfer/weights.py:19-30 of UESlubei/ondeviceinfer
(``model.safetensors.index.json`` and its ``weight_map``; without an index, the
safetensors files of the folder), but tensors are read one at a time by name
(ondeviceinfer/weights.py:49-57) instead of loading whole shards into host memory.
"""

from __future__ import annotations

import hashlib
import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Tuple

import torch

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}


@dataclass(frozen=True)
class TensorDecl:
    """A tensor that a part expects in the checkpoint.

    ``init`` is the law of the random-weights mode: ``"normal"`` draws
    normal(0, 0.02), ``"one_plus_normal"`` draws 1 + normal(0, 0.01) (norm weights),
    ``"zeros"`` is all zero.
    """

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class StoredTensor:
    shape: Tuple[int, ...]
    dtype: torch.dtype
    file: str = ""


def _read_header(path: Path) -> Dict[str, StoredTensor]:
    with open(path, "rb") as handle:
        raw = handle.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path} is not a safetensors file (shorter than its header length)")
        (size,) = struct.unpack("<Q", raw)
        if size > 1 << 30:
            raise ValueError(f"{path} is not a safetensors file (header of {size} bytes)")
        header = json.loads(handle.read(size).decode("utf-8"))
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _ST_DTYPES:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        out[name] = StoredTensor(tuple(meta["shape"]), _ST_DTYPES[meta["dtype"]], path.name)
    return out


class SafetensorsSource:
    """The tensors of a model folder, read by name."""

    def __init__(self, folder) -> None:
        self.folder = Path(folder)
        index = self.folder / "model.safetensors.index.json"
        if index.exists():
            weight_map = json.loads(index.read_text(encoding="utf-8"))["weight_map"]
            files = sorted(set(weight_map.values()))
        else:
            files = sorted(p.name for p in self.folder.glob("*.safetensors"))
            if not files:
                raise FileNotFoundError(f"No safetensors index or file found in {self.folder}")
            weight_map = None
        self._stored: Dict[str, StoredTensor] = {}
        for file in files:
            path = self.folder / file
            if not path.exists():
                raise FileNotFoundError(f"{index.name} names {file}, which is not in {self.folder}")
            for name, stored in _read_header(path).items():
                if weight_map is not None and weight_map.get(name) != file:
                    continue
                self._stored[name] = stored
        if weight_map is not None:
            absent = sorted(set(weight_map) - set(self._stored))
            if absent:
                raise KeyError(f"{index.name} lists tensors that its files do not hold: {absent[:8]}")
        self._handles: dict = {}

    def stored(self) -> Dict[str, StoredTensor]:
        return self._stored

    def fetch(self, name: str) -> torch.Tensor:
        """The tensor as stored, on the CPU."""
        from safetensors import safe_open

        try:
            file = self._stored[name].file
        except KeyError as error:
            raise KeyError(f"Tensor {name!r} is not present in the checkpoint") from error
        if file not in self._handles:
            self._handles[file] = safe_open(str(self.folder / file), framework="pt", device="cpu")
        return self._handles[file].get_tensor(name)

    def close(self) -> None:
        self._handles.clear()


def _name_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


class RandomSource:
    """Seeded random tensors for a list of declarations.

    Each tensor has a generator of its own, keyed by ``(seed, name)``, so the value of
    a tensor does not depend on which others are drawn or in which order.  Values are
    drawn in fp32 on ``device`` and rounded to ``dtype``.
    """

    def __init__(self, decls, seed: int, *, dtype: torch.dtype = torch.bfloat16, device="cpu",
                 std: float = 0.02, norm_std: float = 0.01) -> None:
        self._decls = {d.name: d for d in decls}
        self.seed, self.dtype, self.device = seed, dtype, torch.device(device)
        self.std, self.norm_std = std, norm_std

    def stored(self) -> Dict[str, StoredTensor]:
        return {n: StoredTensor(tuple(d.shape), self.dtype) for n, d in self._decls.items()}

    def fetch(self, name: str) -> torch.Tensor:
        decl = self._decls[name]
        if decl.init == "zeros":
            return torch.zeros(decl.shape, dtype=self.dtype, device=self.device)
        gen = torch.Generator(device=self.device).manual_seed(_name_seed(self.seed, name))
        t = torch.randn(decl.shape, generator=gen, dtype=torch.float32, device=self.device)
        if decl.init == "one_plus_normal":
            t.mul_(self.norm_std).add_(1.0)
        elif decl.init == "normal":
            t.mul_(self.std)
        else:
            raise ValueError(f"tensor {name!r}: unknown init law {decl.init!r}")
        return t.to(self.dtype)

    def close(self) -> None:
        pass
