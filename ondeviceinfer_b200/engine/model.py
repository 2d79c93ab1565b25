"""A decoder built from a :class:`~ondeviceinfer_b200.config.specs.ModelPlan`.

The model is the embedding, a tuple of layers (blocks built from the plan through the
part registries), the order in which layers run (data: it may name a layer twice, or let
an execution read the cache of an earlier one), the final norm and the output head.
It does not know which architecture it is.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from ..cache import SequenceCache
from ..config.specs import ModelPlan
from ..kernels import ops
from ..parts import Runtime, build_part, linear
from ..profiling import nvtx_range
from ..weights import loader
from ..weights.tensors import TensorDecl


class DecoderModel:
    def __init__(self, plan: ModelPlan) -> None:
        plan.validate()
        self.plan = plan
        self.layers = [build_part(spec) for spec in plan.layers]
        self.final_norm = build_part(plan.final_norm)
        self.vocab_size = plan.embedding.vocab_size
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
        e, h = self.plan.embedding, self.plan.head
        decls = [TensorDecl(e.weight_name, (e.vocab_size, e.hidden_size))]
        for layer in self.layers:
            decls += layer.tensor_decls()
        decls += self.final_norm.tensor_decls()
        if h.weight_name is not None:
            decls.append(TensorDecl(h.weight_name, (h.vocab_size, h.hidden_size)))
        return decls

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
        self.embedding = fetch.matrix(self.plan.embedding.weight_name)
        for layer in self.layers:
            layer.load(fetch, self.runtime)
        self.final_norm.load(fetch, self.runtime)
        head_name = self.plan.head.weight_name
        self.head = self.embedding if head_name is None else fetch.matrix(head_name)
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
        return all(getattr(layer, "graph_safe", False) for layer in self.layers) and \
            getattr(self.final_norm, "graph_safe", False)

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
        hidden = torch.empty((ctx.n_tokens, self.hidden_size), dtype=torch.float32, device=self.runtime.device)
        with nvtx_range("embed"):
            ops.embed(self.embedding, ctx.token_ids, hidden)
        ctx.residual_sumsq = None          # nothing is known about the rows of `hidden` yet
        for index, entry in enumerate(self.plan.order):
            with nvtx_range(f"layer_{entry.layer}"):
                self.layers[entry.layer].forward(hidden, ctx, cache.view(index))
        if ctx.n_want == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.runtime.device)
        with nvtx_range("head"):
            final = self.final_norm(hidden, rows=ctx.want_rows)
            return linear(final, self.head, out_dtype=torch.float32)
