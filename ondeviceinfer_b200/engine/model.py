"""A decoder built from a :class:`~ondeviceinfer_b200.config.specs.ModelPlan`.

The model is an embedding part, a tuple of layers (blocks), the order in which layers run
(data: it may name a layer twice, or let an execution read the cache of an earlier one), a
final norm and a head part, every one of them built from its spec through the part
registries.  It does not know which architecture it is, nor what its ends do.
"""

from __future__ import annotations

from dataclasses import replace
from typing import List, Optional

import torch

from ..cache import SequenceCache
from ..config.specs import ModelPlan
from ..parts import Runtime, build_part
from ..parts.linear import flush_residual_add
from ..profiling import nvtx_range
from ..weights import loader
from ..weights.tensors import TensorDecl


class DecoderModel:
    def __init__(self, plan: ModelPlan) -> None:
        plan.validate()
        self.plan = plan
        self.embedding = build_part(plan.embedding)
        self.layers = [build_part(spec) for spec in plan.layers]
        self.final_norm = build_part(plan.final_norm)
        head = plan.head
        if getattr(head, "weight_name", "") is None:        # tied: the head binds the embedding's tensor
            head = replace(head, weight_name=plan.embedding.weight_name, tied=True)
        self.head = build_part(head)
        self.vocab_size = plan.embedding.vocab_size          # token ids a step may bring
        self.logits_size = head.vocab_size                   # width of the logits the head returns
        self.hidden_size = plan.embedding.hidden_size
        self.runtime: Optional[Runtime] = None
        for i, entry in enumerate(plan.order):
            if entry.cache_from is not None:
                mine = self.layers[entry.layer].cache_needs()
                theirs = self.layers[plan.order[entry.cache_from].layer].cache_needs()
                if mine != theirs:
                    raise ValueError(f"order[{i}] reads the cache of entry {entry.cache_from}, whose layer keeps "
                                     f"{theirs}, but its own layer needs {mine}")

    # ------------------------------------------------------------------ weights

    def tensor_decls(self) -> List[TensorDecl]:
        decls = list(self.embedding.tensor_decls())
        for layer in self.layers:
            decls += layer.tensor_decls()
        return decls + list(self.final_norm.tensor_decls()) + list(self.head.tensor_decls())

    def load(self, source, *, dtype: torch.dtype, device) -> "DecoderModel":
        """Check the source against the declarations (one error for everything that does
        not fit), then bind every tensor on ``device``."""
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError(f"ondeviceinfer_b200 runs on CUDA devices only (got {device}); there is no CPU path")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be torch.bfloat16 or torch.float32, not {dtype}")
        loader.check(self.tensor_decls(), source.stored(), self.plan.ignored_tensors)
        self.runtime = Runtime(dtype=dtype, device=device)
        fetch = loader.Fetcher(source, dtype, device)
        self.embedding.load(fetch, self.runtime)
        for layer in self.layers:
            layer.load(fetch, self.runtime)
        self.final_norm.load(fetch, self.runtime)
        self.head.load(fetch, self.runtime)
        return self

    @property
    def device(self) -> torch.device:
        self._require_loaded()
        return self.runtime.device

    @property
    def dtype(self) -> torch.dtype:
        self._require_loaded()
        return self.runtime.dtype

    def _require_loaded(self) -> None:
        if self.runtime is None:
            raise RuntimeError("the model has no weights yet: call load() first")

    @property
    def graph_safe(self) -> bool:
        """True if every part may be captured in a CUDA graph (no host work per step)."""
        return all(getattr(part, "graph_safe", False)
                   for part in (self.embedding, *self.layers, self.final_norm, self.head))

    # ------------------------------------------------------------------ cache

    def make_cache(self, *, max_tokens: int, max_seqs: int, max_step_tokens: int = 256) -> SequenceCache:
        self._require_loaded()
        needs = [self.layers[e.layer].cache_needs() if e.cache_from is None else () for e in self.plan.order]
        return SequenceCache(needs, [e.cache_from for e in self.plan.order], dtype=self.runtime.dtype,
                             device=self.runtime.device, max_tokens=max_tokens, max_seqs=max_seqs,
                             max_step_tokens=max_step_tokens)

    # ------------------------------------------------------------------ forward

    def forward(self, ctx, cache) -> torch.Tensor:
        """Run the step described by ``ctx``; return fp32 logits at ``ctx.want_rows``."""
        with nvtx_range("embed"):
            hidden = self.embedding.forward(ctx)           # the fp32 residual stream [tokens, hidden]
        ctx.residual_sumsq = None          # nothing is known about the rows of `hidden` yet
        ctx.pending_residual_add = None
        for index, entry in enumerate(self.plan.order):
            layer = self.layers[entry.layer]
            # A block that finishes deferred residual adds (parts/block.py) sets the flag for its own parts and
            # takes over an add that the block before left; any other block finds the stream complete.
            ctx.defers_residual_add = False
            if not getattr(layer, "finishes_residual_adds", False):
                flush_residual_add(ctx)
            with nvtx_range(f"layer_{entry.layer}"):
                layer.forward(hidden, ctx, cache.view(index))
        flush_residual_add(ctx)                # the last block's last product
        if ctx.n_want == 0:
            return torch.empty((0, self.logits_size), dtype=torch.float32, device=self.runtime.device)
        with nvtx_range("head"):
            return self.head.forward(self.final_norm(hidden, rows=ctx.want_rows), ctx)
