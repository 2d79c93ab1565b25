"""The two ends of a decoder as parts: the token embedding and the output head.

Like every part they are chosen by the type of their spec, so an architecture whose ends differ (a scaled
embedding, learned positions added to it, logits with a soft cap, several heads) brings a spec and a class
of its own and registers them; the model only calls ``embedding.forward(ctx)`` and
``head.forward(rows, ctx)``.

Reference: ``nn.Embedding`` lookup without scaling (ondeviceinfer/model.py:77-82,100) and a bias-free
``lm_head`` (ondeviceinfer/model.py:138-144,163), tied to the embedding table when the configuration says
so (ondeviceinfer/weights.py:77-78).
"""

from __future__ import annotations

import torch

from ..config.specs import EmbeddingSpec, HeadSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import linear


class TokenEmbedding(Part):
    """hidden[t, :] = table[token[t], :], widened into the fp32 residual stream."""

    graph_safe = True

    def tensor_decls(self):
        return [TensorDecl(self.spec.weight_name, (self.spec.vocab_size, self.spec.hidden_size))]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.table = fetch.matrix(self.spec.weight_name)

    def forward(self, ctx) -> torch.Tensor:
        hidden = torch.empty((ctx.n_tokens, self.spec.hidden_size), dtype=torch.float32, device=self.runtime.device)
        ops.embed(self.table, ctx.token_ids, hidden)
        return hidden


class OutputHead(Part):
    """logits = rows W^T in fp32.  A tied head binds the embedding's tensor (the loader hands out one tensor
    per name, so the table is held once) and declares nothing of its own."""

    graph_safe = True

    def tensor_decls(self):
        if self.spec.tied:
            return []
        return [TensorDecl(self.spec.weight_name, (self.spec.vocab_size, self.spec.hidden_size))]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.weight = fetch.matrix(self.spec.weight_name)
        if tuple(self.weight.shape) != (self.spec.vocab_size, self.spec.hidden_size):
            raise ValueError(f"the head's weight {self.spec.weight_name!r} is {tuple(self.weight.shape)}, expected "
                             f"{(self.spec.vocab_size, self.spec.hidden_size)}")

    def forward(self, rows: torch.Tensor, ctx) -> torch.Tensor:
        """``rows`` [wanted, hidden] in the compute dtype (already normed) -> fp32 logits [wanted, vocab]."""
        return linear(rows, self.weight, out_dtype=torch.float32)


register_part(EmbeddingSpec, TokenEmbedding)
register_part(HeadSpec, OutputHead)
