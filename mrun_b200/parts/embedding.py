"""Embedding parts: what fills the residual streams from the token ids in place of the plain
table lookup (``ModelSpec.embedding``).

``hashed_bigram_embedding`` (the formulas are with :class:`HashedBigramEmbeddingSpec`): the token's
row times a scale plus a row of a second table chosen by a hash of the token and the one before
it.  The token before a step's first token of a request is per-request state (one int32 a state
slot, written by the kernel that embeds the request's last token of the step), so a prompt may be
cut anywhere and a decoded token that is still on the device needs no trip to the host.
"""
from __future__ import annotations

import torch

from ..cache.needs import FixedState
from ..config.spec import HashedBigramEmbeddingSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_embedding


@register_embedding("hashed_bigram_embedding")
class HashedBigramEmbedding:
    graph_safe = True

    @staticmethod
    def tensor_specs(spec: HashedBigramEmbeddingSpec, prefix: str):
        out = [TensorSpec(prefix, (spec.vocab, spec.hidden))]
        if spec.buckets:
            out.append(TensorSpec(spec.table_name, (spec.buckets + 1, spec.hidden)))
        return out

    def __init__(self, spec: HashedBigramEmbeddingSpec, tensors, runtime: Runtime):
        self.spec = spec
        self.table = tensors[""]                    # the token table as the model holds it
        self.pairs = runtime.matrix(tensors[spec.table_name]) if spec.buckets else None
        if self.pairs is not None and self.pairs.shape != (spec.buckets + 1, spec.hidden):
            raise ValueError("the bigram table does not have the spec's shape")

    def cache_need(self):
        if not self.spec.buckets:
            return None
        return FixedState((1,), "int32", name="previous_token")

    def forward(self, ctx, cache, out: torch.Tensor, streams: int) -> torch.Tensor:
        s = self.spec
        state = cache.states["previous_token"] if self.pairs is not None else None
        return ops.embed_bigram(self.table, self.pairs, ctx.token_ids, ctx.positions, ctx.token_slot, state, out, streams,
                                s.scale, s.buckets, s.mul_prev, s.mul_cur)
