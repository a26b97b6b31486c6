"""Latent attention over a paged cache of one latent row per token.

The cache row of a token is ``[c | r | 0...]``: its key/value latent c (``kv_rank`` features,
RMS-normed), the rotated key part r that all heads share (``rot_dim`` features) and zeros up to a
width the attention kernels take.  Keys and values of the heads are never made: with
K_h = U_h c and V_h = W_h c (the two up-projections), a head's score is

    q_plain . (U_h c) + q_rot . r  =  (U_h^T q_plain) . c + q_rot . r,

so the query row ``[U_h^T q_plain | q_rot | 0...]`` meets the cache row as one key of a single
key/value head, and the head's output is W_h (sum_j p_j c_j): the same cache row is the value,
and W_h runs on the weighted latent.  The framework's paged attention kernels therefore serve
this mixer unchanged (``heads`` query heads over one kv head whose K and V are the same pages);
prefill, decode and mixed steps take the paths they take for grouped-query attention.  Rows wider
than those kernels' 256 features (a latent of 512, say) go to a tensor-core kernel of their own
(``csrc/attention_latent.cu``: a block a token and 16 heads, a quarter of the value columns a warp).

A layer without a query latent (``q_rank`` = 0) has one query projection ``q`` straight from the
input; it rides in the same product as the key/value down-projection.  ``window`` reaches the
attention kernels as it does for grouped-query attention.

Per step: one product for both down-projections (their weights stacked), one kernel that norms
the two latents, rotates r and writes the cache row, the query up-projection, a per-head product
with U_h^T, one kernel that rotates the queries' rotated parts into the query rows, attention, a
per-head product with W_h, the output projection (left pending for the norm after it).
"""
from __future__ import annotations

import torch

from ..cache.needs import PagedLatent
from ..config.spec import LatentAttentionSpec, TensorSpec
from ..kernels import ops
from ..kernels.attention import paged_attention, supports_tensor_cores
from .base import POSITIONS, Runtime, register_mixer


@register_mixer("latent_attention")
class LatentAttention:
    can_defer_output = True         # ``forward(..., defer_output=True)`` may return ``ops.PendingLinear``

    @staticmethod
    def tensor_specs(spec: LatentAttentionSpec, prefix: str):
        s = spec
        if s.q_rank:
            query = [TensorSpec(f"{prefix}.dq", (s.q_rank, s.hidden)),
                     TensorSpec(f"{prefix}.dq.norm", (s.q_rank,), "norm"),
                     TensorSpec(f"{prefix}.uq", (s.heads * (s.dim + s.rot_dim), s.q_rank))]
        else:
            query = [TensorSpec(f"{prefix}.q", (s.heads * (s.dim + s.rot_dim), s.hidden))]
        return query + [
            TensorSpec(f"{prefix}.dkv", (s.kv_rank + s.rot_dim, s.hidden)),
            TensorSpec(f"{prefix}.dkv.norm", (s.kv_rank,), "norm"),
            TensorSpec(f"{prefix}.uk", (s.heads * s.dim, s.kv_rank)),
            TensorSpec(f"{prefix}.uv", (s.heads * s.vdim, s.kv_rank)),
            TensorSpec(f"{prefix}.o", (s.hidden, s.heads * s.vdim)),
        ]

    def __init__(self, spec: LatentAttentionSpec, tensors, runtime: Runtime):
        s = self.spec = spec
        self.runtime = runtime
        if s.window is not None and s.window < 1:
            raise ValueError("a window holds at least one position")
        # the first product: [query latent | key/value latent | shared key part], or, without a
        # query latent, [queries | key/value latent | shared key part]
        self.w_down = runtime.matrix(torch.cat([tensors["dq" if s.q_rank else "q"], tensors["dkv"]], dim=0))
        self.q_norm = runtime.vector_f32(tensors["dq.norm"]) if s.q_rank else None
        self.kv_norm = runtime.vector_f32(tensors["dkv.norm"])
        self.w_uq = runtime.matrix(tensors["uq"]) if s.q_rank else None
        # U_h^T per head, [heads, kv_rank, dim]: the per-head product takes weights as [out, in]
        self.w_uk_t = runtime.matrix(tensors["uk"].view(s.heads, s.dim, s.kv_rank).transpose(1, 2))
        self.w_uv = runtime.matrix(tensors["uv"].view(s.heads, s.vdim, s.kv_rank))
        self.w_o = runtime.matrix(tensors["o"])
        self.position = POSITIONS.build(s.position, {}, runtime) if s.position is not None else None
        self.rot_dims = self.position.rotary_dim if self.position is not None else 0
        self.pairing = getattr(self.position, "pairing", "half")
        if self.rot_dims > s.rot_dim:
            raise ValueError(f"{self.rot_dims} rotating features do not fit the rotated part of {s.rot_dim}")
        # the cache row's width: a size the tensor-core attention kernels are built for
        self.width = -(-(s.kv_rank + s.rot_dim) // 16) * 16
        # the tiled kernel that very wide groups fall to needs a tile list made on the host
        self.graph_safe = not (supports_tensor_cores(runtime.precision.act, self.width, s.heads) and s.heads > 16)

    def cache_need(self):
        return PagedLatent(self.width, self.spec.window)

    def activation_elements(self) -> int:
        s = self.spec
        return s.q_rank + s.kv_rank + s.rot_dim + s.heads * (s.dim + s.rot_dim + 2 * self.width + s.vdim)

    def forward(self, x, ctx, cache, defer_output: bool = False):
        s, width = self.spec, self.width
        tokens = x.shape[0]
        group = ctx.group(cache.group_key)
        down = ops.linear(x, self.w_down)
        rot = self.position.rotation(ctx) if self.position is not None else None
        slots = group.slot_mapping if cache.writable else None
        if s.q_rank:
            cq = torch.empty((tokens, s.q_rank), dtype=x.dtype, device=x.device)
            ops.latent_prepare(down, self.q_norm, self.kv_norm, s.eps, rot, self.rot_dims, self.pairing, slots, cq,
                               cache.k, s.q_rank, s.kv_rank, s.rot_dim)
            q = ops.linear(cq, self.w_uq)
        else:
            nq = s.heads * (s.dim + s.rot_dim)
            q = down[:, :nq]
            ops.latent_prepare(down[:, nq:], None, self.kv_norm, s.eps, rot, self.rot_dims, self.pairing, slots, None,
                               cache.k, 0, s.kv_rank, s.rot_dim)
        q_att = torch.empty((tokens, s.heads, width), dtype=x.dtype, device=x.device)
        ops.linear_per_head(q.unflatten(1, (s.heads, s.dim + s.rot_dim))[:, :, :s.dim], self.w_uk_t,
                            q_att[:, :, :s.kv_rank])
        ops.latent_query(q, rot, self.rot_dims, self.pairing, q_att, s.heads, s.dim, s.rot_dim, s.kv_rank)
        mixed = torch.empty((tokens, s.heads * width), dtype=x.dtype, device=x.device)
        paged_attention(q_att.view(tokens, s.heads * width), s.heads * width, mixed, cache, group, ctx, s.heads,
                        s.softmax_scale, s.window or 0, value_dim=s.kv_rank)
        value = torch.empty((tokens, s.heads, s.vdim), dtype=x.dtype, device=x.device)
        ops.linear_per_head(mixed.view(tokens, s.heads, width)[:, :, :s.kv_rank], self.w_uv, value)
        value = value.view(tokens, s.heads * s.vdim)
        if defer_output:
            return ops.linear_or_pending(value, self.w_o)
        return ops.linear(value, self.w_o)
