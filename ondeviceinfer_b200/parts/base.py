"""Interfaces of the parts a decoder layer is put together from, and their registries.

A part is built from its spec alone (``Part(spec)``: no device work, no checkpoint
access), declares the checkpoint tensors it binds, and later receives them:

``tensor_decls() -> list[TensorDecl]``
    names and shapes of the checkpoint tensors the part expects.
``load(fetch, runtime) -> None``
    fetch the tensors (``fetch.matrix(name)`` in the compute dtype, ``fetch.vector(name)``
    in fp32, ``fetch.integer(name)`` as int32), fuse or re-lay them as the kernels want,
    keep ``runtime`` (compute dtype, device).

On top of that each kind of part has one call:

**Norm**       ``__call__(x, rows=None) -> Tensor``: x is the fp32 residual stream
               ``[tokens, hidden]``; the result is in the compute dtype; ``rows`` (int32
               indices) restricts the output to those rows.
**Position**   ``rotary_tables(ctx) -> (cos, sin) | None``: fp32 ``[tokens, rot_dim/2]``
               tables for the step's token positions (``ctx.tok_pos``), memoised per
               step with ``ctx.memo``; None for "no rotation".  ``rot_dim`` attribute.
**Mixer**      ``cache_needs() -> tuple`` of :class:`KVNeed` / :class:`StateNeed`;
               ``forward(x, ctx, view, residual) -> None``: x ``[tokens, hidden]`` in the
               compute dtype (already normed); must ADD its output to ``residual``
               (fp32 ``[tokens, hidden]``) in place.  ``ctx`` describes the step's
               sequences (:class:`~ondeviceinfer_b200.engine.step.StepContext`), ``view``
               is the cache of this layer execution
               (:class:`~ondeviceinfer_b200.cache.CacheView`).  A mixer with a state of
               its own must advance it over all tokens a sequence brings in the step,
               so that cutting a sequence into steps changes no result.
**FeedForward** ``forward(x, ctx, residual) -> None``: same contract without a cache.
**Block**      ``cache_needs()`` and ``forward(hidden, ctx, view) -> None`` on the fp32
               residual stream in place; owns the arrangement of norms, mixer and
               feed-forward.

Optional, for speed only (a part that knows nothing of it loses nothing but a fusion): a mixer or
feed-forward that ends with ``linear(..., residual=residual, track=ctx)`` lets that product leave the
sums of squares of the rows it wrote (``ctx.residual_sumsq``); the block then gives the next part, if
it says ``takes_lazy_norm = True`` and the norm has ``lazy(x, parts)``, a
:class:`~ondeviceinfer_b200.parts.linear.NormedRows` instead of a tensor, which ``linear`` and
``gated_linear`` turn into the normed operand inside the tensor-core kernel (``.materialize()`` gives
the tensor).  A part that passes ``track`` must not touch ``residual`` after that product.

Also optional, between a block and the model: a block with ``finishes_residual_adds = True`` may set
``ctx.defers_residual_add`` while its parts run; a product that the vendor library computed then leaves its
residual add pending (``ctx.pending_residual_add``) and the block's next norm does it in its own pass
(``norm(x, add=product)`` for a norm with ``adds = True``), the add after its last product being taken over by
the next such block or by the model.  Whoever calls such a block directly finishes with
``parts.linear.flush_residual_add(ctx)``.  A block that knows nothing of this never sees a pending add.

Also optional: a mixer whose single-token kernel cuts each sequence's keys among several blocks may ask the
context how (``ctx.key_splits(blocks_per_cut) -> (tiles_per_split, splits)``): the number of 64-key tiles
that a block takes, as one int32 on the device that follows the step's sequences (also under graph replay,
where the host refreshes it), and a bound on the cuts of one sequence, which is what a captured graph fixes.

Parts are chosen by the *type* of their spec.  ``register_part(SpecType, PartClass)``
adds a kind; nothing else in the library has to change for it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch

from ..weights.tensors import TensorDecl

_PARTS: Dict[type, type] = {}


def register_part(spec_type: type, part_cls: type) -> None:
    for member in ("tensor_decls", "load"):
        if not hasattr(part_cls, member):
            raise TypeError(f"{part_cls.__name__} lacks {member}(); see ondeviceinfer_b200.parts.base")
    _PARTS[spec_type] = part_cls


def build_part(spec):
    try:
        cls = _PARTS[type(spec)]
    except KeyError:
        known = sorted(t.__name__ for t in _PARTS)
        raise KeyError(f"no part is registered for spec type {type(spec).__name__}; known: {known}") from None
    return cls(spec)


@dataclass
class Runtime:
    """What a loaded part needs to know about the run."""

    dtype: torch.dtype      # compute dtype: torch.bfloat16 or torch.float32
    device: torch.device


class Part:
    """Convenience base: a part without tensors."""

    def __init__(self, spec) -> None:
        self.spec = spec
        self.runtime: Runtime | None = None

    def tensor_decls(self) -> List[TensorDecl]:
        return []

    def load(self, fetch, runtime: Runtime) -> None:
        self.runtime = runtime
