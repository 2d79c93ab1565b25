"""Binding checkpoint tensors to the parts of a model, by name.

The parts declare the tensors they expect (name and shape); the source says what it
holds.  All disagreements -- missing tensors, tensors nobody asked for, wrong shapes --
are collected and raised as ONE :class:`WeightsError` before any tensor is read.  The
reference gets the same strictness from ``load_state_dict(strict=True)``
(ondeviceinfer/weights.py:72-74).

What is kept in which precision:

* matrices and tables that feed the matrix kernels are held in the run's compute dtype
  (bfloat16 for serving, float32 for the 32-bit path);
* other floating tensors (norm weights and the like) are held in float32: for a tensor
  stored in bfloat16 that is exact, and a tensor stored in 32-bit stays so;
* integer tensors are held as int32.
"""

from __future__ import annotations

import weakref
from typing import Dict, Iterable, List

import torch

from .tensors import StoredTensor, TensorDecl


class WeightsError(RuntimeError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the full lists; the message shows them."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[str]) -> None:
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        super().__init__("\n".join(lines))


def check(decls: Iterable[TensorDecl], stored: Dict[str, StoredTensor], ignored: Iterable[str] = ()) -> None:
    expected: Dict[str, TensorDecl] = {}
    wrong: List[str] = []
    for decl in decls:
        seen = expected.get(decl.name)
        if seen is not None and tuple(seen.shape) != tuple(decl.shape):
            wrong.append(f"{decl.name}: two parts expect {tuple(seen.shape)} and {tuple(decl.shape)}")
        expected[decl.name] = decl
    missing = sorted(n for n in expected if n not in stored)
    unexpected = sorted(n for n in stored if n not in expected and n not in set(ignored))
    for name, decl in expected.items():
        if name in stored and tuple(stored[name].shape) != tuple(decl.shape):
            wrong.append(f"{name}: expected {tuple(decl.shape)}, found {tuple(stored[name].shape)}")
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, sorted(wrong))


class Fetcher:
    """What a part's ``load`` receives: tensors by name, on the device, in the held precision."""

    def __init__(self, source, compute_dtype: torch.dtype, device) -> None:
        self.source, self.compute_dtype, self.device = source, compute_dtype, torch.device(device)
        # One tensor per name for as long as somebody holds it: two parts that bind the same matrix (a head tied
        # to the embedding table) share its storage; a matrix that its part only concatenates into another is
        # not kept alive by this table.
        self._matrices = weakref.WeakValueDictionary()

    def matrix(self, name: str) -> torch.Tensor:
        """A matrix or table in the compute dtype (the same tensor for the same name while it is held)."""
        held = self._matrices.get(name)
        if held is not None:
            return held
        t = self.source.fetch(name)
        if not t.is_floating_point():
            raise TypeError(f"tensor {name!r} is stored as {t.dtype}, a floating matrix was expected")
        t = t.to(device=self.device, dtype=self.compute_dtype, non_blocking=False).contiguous()
        self._matrices[name] = t
        return t

    def vector(self, name: str) -> torch.Tensor:
        """A small floating tensor, held in float32."""
        t = self.source.fetch(name)
        if not t.is_floating_point():
            raise TypeError(f"tensor {name!r} is stored as {t.dtype}, a floating tensor was expected")
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def integer(self, name: str) -> torch.Tensor:
        t = self.source.fetch(name)
        if t.is_floating_point():
            raise TypeError(f"tensor {name!r} is stored as {t.dtype}, an integer table was expected")
        return t.to(device=self.device, dtype=torch.int32).contiguous()
