"""Arrangement of norms, mixer and feed-forward in a layer."""

from __future__ import annotations

from ..config.specs import PreNormBlockSpec
from .base import Part, build_part, register_part


def ops_residual_add(residual, product) -> None:
    from ..kernels import ops
    ops.residual_add(residual, product)


class PreNormBlock(Part):
    """h += mixer(norm(h)); h += feed_forward(norm(h))  (ondeviceinfer/model.py:49-63)."""

    finishes_residual_adds = True     # its norms take over a residual add that a product left pending

    def __init__(self, spec: PreNormBlockSpec) -> None:
        super().__init__(spec)
        self.mixer_norm = build_part(spec.mixer_norm)
        self.mixer = build_part(spec.mixer)
        self.ffn_norm = build_part(spec.ffn_norm)
        self.ffn = build_part(spec.ffn)

    def _children(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def tensor_decls(self):
        return [d for part in self._children() for d in part.tensor_decls()]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        for part in self._children():
            part.load(fetch, runtime)

    def cache_needs(self):
        return tuple(self.mixer.cache_needs())

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self._children())

    @staticmethod
    def _normed(norm, consumer, hidden, ctx):
        """norm(hidden); left to the consumer's first product when the product that wrote ``hidden``
        has left the rows' sums of squares in ``ctx.residual_sumsq`` and both sides know how."""
        known = getattr(ctx, "residual_sumsq", None)
        ctx.residual_sumsq = None
        pending = getattr(ctx, "pending_residual_add", None)
        if pending is not None:
            # a product of the part before is still to be added to the stream: in this norm's pass if it is
            # this stream and the norm knows how, else now
            ctx.pending_residual_add = None
            if pending[0] is hidden and getattr(norm, "adds", False):
                return norm(hidden, add=pending[1])
            ops_residual_add(*pending)
        if known is not None and known[0] is hidden and hasattr(norm, "lazy") and getattr(consumer, "takes_lazy_norm", False):
            return norm.lazy(hidden, known[1])
        return norm(hidden)

    def forward(self, hidden, ctx, view) -> None:
        # This block finishes residual adds that its parts' last products leave pending (in the norm that follows,
        # here or in the next block; the model flushes the last one): it says so, and only then is an add deferred.
        ctx.defers_residual_add = True
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, hidden, ctx), ctx, view, hidden)
        self.ffn.forward(self._normed(self.ffn_norm, self.ffn, hidden, ctx), ctx, hidden)


register_part(PreNormBlockSpec, PreNormBlock)
