"""Architecture-neutral descriptions of a decoder: what each layer is made of and in which order layers run.

A model is data before it is code.  An architecture's configuration class turns its
``config.json`` into a :class:`ModelPlan`; the engine builds parts from the plan through
the part registries (``ondeviceinfer_b200.parts``).  Nothing in a spec names a model:
every size and constant is a field, and the checkpoint tensor names a part binds are
given to it by the plan (``names`` / ``prefix``), not known by the part.

Specs are frozen dataclasses.  A new kind of part brings its own spec class; the
registries key on the spec's *type*, so nothing here has to change for it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


def _frozen_names(names: Mapping[str, str]) -> Tuple[Tuple[str, str], ...]:
    return tuple(sorted(names.items()))


@dataclass(frozen=True)
class RMSNormSpec:
    """y = weight * cast(x * rsqrt(mean(x^2) + eps)); statistics in fp32."""

    size: int
    eps: float
    weight_name: str  # full checkpoint name of the [size] weight


@dataclass(frozen=True)
class RotarySpec:
    """Half-split rotary position encoding over the first ``rotary_dim`` lanes of a head."""

    head_dim: int
    theta: float
    rotary_dim: Optional[int] = None  # None: the whole head

    @property
    def dim(self) -> int:
        return self.head_dim if self.rotary_dim is None else self.rotary_dim


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding inside the mixer."""


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal self-attention over cached keys and values.

    ``qk_norm_eps`` not None adds an RMSNorm over each query and key head (one [head_dim]
    weight shared by the heads) before the position encoding.  ``window`` not None keeps
    only the last ``window`` keys visible (the query's own position included).
    ``names`` maps the roles q, k, v, o, q_norm, k_norm to tensor names below ``prefix``; when it also
    names q_bias, k_bias, v_bias or o_bias, that projection adds the [out] bias of that name.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: object  # RotarySpec | NoPositionSpec | any registered position spec
    prefix: str
    names: Tuple[Tuple[str, str], ...]
    qk_norm_eps: Optional[float] = None
    window: Optional[int] = None
    scale: Optional[float] = None  # None: 1/sqrt(head_dim)

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]

    def has(self, role: str) -> bool:
        return role in dict(self.names)


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases."""

    hidden_size: int
    intermediate_size: int
    activation: str  # "silu"
    prefix: str
    names: Tuple[Tuple[str, str], ...]

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]


@dataclass(frozen=True)
class PreNormBlockSpec:
    """h += mixer(norm1(h)); h += feed_forward(norm2(h))."""

    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object


@dataclass(frozen=True)
class OrderEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelPlan.layers``; the same layer may appear in several
    entries (its weights are then shared, each execution has a cache of its own).
    ``cache_from`` not None makes this execution read the cache that the earlier order
    entry with that index wrote, instead of writing one itself.
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token embedding: hidden[t] = table[token[t]], no scaling, nothing added."""

    vocab_size: int
    hidden_size: int
    weight_name: str


@dataclass(frozen=True)
class HeadSpec:
    """Output head: logits = rows W^T on the rows the final norm gives it.  ``weight_name`` None ties it to the
    embedding table (the model then fills in that tensor's name and sets ``tied``); with ``tied`` the head
    binds ``weight_name`` without declaring it, because another part already does."""

    vocab_size: int
    hidden_size: int
    weight_name: Optional[str]
    tied: bool = False


@dataclass(frozen=True)
class ModelPlan:
    """``embedding`` and ``head`` are specs of registered parts like the layers' (any spec whose part has
    ``forward(ctx) -> hidden`` resp. ``forward(rows, ctx) -> logits`` and the sizes ``vocab_size`` /
    ``hidden_size``); :class:`EmbeddingSpec` and :class:`HeadSpec` are the plain ones."""

    embedding: object
    layers: Tuple[object, ...]
    order: Tuple[OrderEntry, ...]
    final_norm: object
    head: object
    # tensors that may be present in a checkpoint and are deliberately not used
    ignored_tensors: Tuple[str, ...] = field(default_factory=tuple)

    def validate(self) -> None:
        for i, entry in enumerate(self.order):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {entry.layer}, the plan has {len(self.layers)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < i:
                    raise ValueError(f"order[{i}] reads the cache of entry {entry.cache_from}, "
                                     "which must be an earlier entry")
                if self.order[entry.cache_from].cache_from is not None:
                    raise ValueError(f"order[{i}] reads the cache of entry {entry.cache_from}, "
                                     "which owns no cache itself")


def names(**roles: str) -> Tuple[Tuple[str, str], ...]:
    """Helper for plans: ``names(q="q_proj.weight", ...)``."""
    return _frozen_names(roles)
