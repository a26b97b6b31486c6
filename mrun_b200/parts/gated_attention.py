"""Grouped-query attention with keys and values of different sizes, a norm of q and k (over the
whole projection, or head by head), a sink term in the softmax, an output gate per head, values
that may be the unnormed keys, and a causal, sliding-window or chunked mask (the formulas are
with :class:`GatedAttentionSpec`).

One product makes [q | k | v | gate] (or [q | gate] for a layer that reads another layer's pages,
[q | k] for one whose values are its keys); ``ops.proj_norm_rope_cache`` or
``ops.head_norm_rope_cache`` norms q and k, rotates them and writes k and v into the pages; the
attention kernel applies the sink and the gate's sigmoid to every head's output; the output
projection follows.  In a step of single tokens the tensor-core decode kernels take the rows of
a layer with a norm per head raw and do the norm, the rotation and the page write themselves, as
they do for :class:`Attention`.  Scores, softmax, the sink and the gate are 32-bit in both
precisions.  A chunked mask reaches the attention kernels as a negative window (minus the chunk's size).

Kernels: bfloat16 with keys and values of one size that the tensor-core attention takes go
through the framework's paged kernels (tcgen05 prompt tiles, TMA decode; the sink enters their
final normalisation, the gate is one more kernel); every other shape, and the 32-bit path, runs
on CUDA cores in 32-bit arithmetic with sink and gate inside the kernel.
"""
from __future__ import annotations

import os

import torch

from ..cache.needs import PagedKV
from ..config.spec import GatedAttentionSpec, TensorSpec
from ..kernels import ops
from ..kernels.attention import decode_fuses_input, paged_attention, supports_tensor_cores
from .base import POSITIONS, Runtime, register_mixer


# False (``MRUN_GATED_ATTENTION_TENSOR_CORES=0`` in the environment): the CUDA-core kernel for every
# shape (tests compare the two)
TENSOR_CORES = os.environ.get("MRUN_GATED_ATTENTION_TENSOR_CORES", "1") != "0"


@register_mixer("gated_attention")
class GatedAttention:
    can_defer_output = True

    @staticmethod
    def tensor_specs(spec: GatedAttentionSpec, prefix: str):
        nq, nk, nv = spec.heads * spec.dim, spec.kv_heads * spec.dim, spec.kv_heads * spec.vdim
        out = [TensorSpec(f"{prefix}.q", (nq, spec.hidden)),
               TensorSpec(f"{prefix}.o", (spec.hidden, spec.heads * spec.vdim))]
        if spec.own_kv:
            out.append(TensorSpec(f"{prefix}.k", (nk, spec.hidden)))
            if spec.values != "keys":
                out.append(TensorSpec(f"{prefix}.v", (nv, spec.hidden)))
        if spec.qk_norm is not None:
            per_head = spec.qk_norm == "head"
            out.append(TensorSpec(f"{prefix}.q.norm", (spec.dim if per_head else nq,), "norm"))
            if spec.own_kv:
                out.append(TensorSpec(f"{prefix}.k.norm", (spec.dim if per_head else nk,), "norm"))
        if spec.head_gate:
            out.append(TensorSpec(f"{prefix}.g", (spec.heads, spec.hidden)))
        return out

    def __init__(self, spec: GatedAttentionSpec, tensors, runtime: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads={spec.heads} is not a multiple of kv_heads={spec.kv_heads}")
        if spec.qk_norm not in (None, "projection", "head"):
            raise ValueError(f"the q/k norm of this attention works over the whole projection or head by head, "
                             f"not {spec.qk_norm!r}")
        if spec.values not in ("projection", "keys"):
            raise ValueError(f"values come from a projection of their own or are the keys, not {spec.values!r}")
        self.keys_as_values = spec.values == "keys"
        if self.keys_as_values and (spec.vdim != spec.dim or not spec.own_kv):
            raise ValueError("values that are the keys have the keys' size and belong to a layer with keys of its own")
        if spec.window is not None and spec.chunk is not None:
            raise ValueError("an attention has a sliding window or a chunked mask, not both")
        if (spec.window is not None and spec.window < 1) or (spec.chunk is not None and spec.chunk < 1):
            raise ValueError("a window or a chunk holds at least one position")
        self.spec = spec
        self.runtime = runtime
        # what the attention kernels take as their window: W, 0 for none, -C for chunks of C
        self.mask = -spec.chunk if spec.chunk is not None else (spec.window or 0)
        self.nq, self.nk, self.nv = spec.heads * spec.dim, spec.kv_heads * spec.dim, spec.kv_heads * spec.vdim
        parts = [tensors["q"]] + ([tensors["k"]] + ([] if self.keys_as_values else [tensors["v"]]) if spec.own_kv else [])
        self.k_off, self.v_off = (self.nq, -1 if self.keys_as_values else self.nq + self.nk) if spec.own_kv else (-1, -1)
        # the kernel that norms head by head also serves the layers that norm nothing special
        self.per_head = spec.qk_norm == "head" or self.keys_as_values
        self.gate_off = sum(p.shape[0] for p in parts)
        if spec.head_gate:
            parts.append(tensors["g"])
        rows = sum(p.shape[0] for p in parts)
        if rows % 8:        # rows of the product's output start on 16 bytes, as the tensor-core kernels read q
            parts.append(torch.zeros((8 - rows % 8, spec.hidden), dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = runtime.matrix(torch.cat(parts, dim=0))
        self.w_o = runtime.matrix(tensors["o"])
        self.q_weight = self.k_weight = None
        if spec.qk_norm is not None:
            self.q_weight = runtime.vector_f32(tensors["q.norm"])
            self.k_weight = runtime.vector_f32(tensors["k.norm"]) if spec.own_kv else None
        self.position = POSITIONS.build(spec.position, {}, runtime) if spec.position is not None else None
        self.pairing = getattr(self.position, "pairing", "half")
        ratio = spec.heads // spec.kv_heads
        self.tensor_cores = (TENSOR_CORES and spec.dim == spec.vdim
                             and supports_tensor_cores(runtime.precision.act, spec.dim, ratio))
        # the tiled kernel that very wide groups fall to needs a tile list made on the host
        self.graph_safe = not (self.tensor_cores and ratio > 16)
        # rows laid out [q | k | v] with a norm per head and half-split pairs are what the decode
        # attention kernels take raw (they norm, rotate and store the step's q, k and v themselves)
        self.fusable = (self.tensor_cores and spec.qk_norm == "head" and spec.own_kv and not self.keys_as_values
                        and self.pairing == "half")

    def cache_need(self):
        s = self.spec
        if not s.own_kv:
            return None
        # a chunk's keys lie within the last `chunk` positions: the pages before them are given back
        return PagedKV(s.kv_heads, s.dim, s.chunk if s.chunk is not None else s.window,
                       value_dim=s.vdim if s.vdim != s.dim else None)

    def activation_elements(self) -> int:
        s = self.spec
        return 2 * self.nq + self.nk + self.nv + s.heads * (1 + 2 * s.vdim)

    def forward(self, x, ctx, cache, defer_output: bool = False):
        s = self.spec
        if cache is None or cache.k is None:
            raise ValueError("this attention has no pages to read: a layer without keys and values of its own "
                             "runs as a schedule entry that names the cache of another")
        if s.own_kv != bool(cache.writable):
            raise ValueError("an attention with keys and values of its own writes its own pages, one without reads another's")
        group = ctx.group(cache.group_key)
        y = ops.linear(x, self.w_in)
        rot = self.position.rotation(ctx) if self.position is not None else None
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        gate = y[:, self.gate_off:self.gate_off + s.heads] if s.head_gate else None
        out = torch.empty((x.shape[0], s.heads * s.vdim), dtype=x.dtype, device=x.device)
        if self.fusable and decode_fuses_input(ctx, x.dtype, s.heads, s.kv_heads, s.dim, self.runtime.page_size):
            # a pure decode step: the attention kernel norms, rotates and stores q, k, v itself
            paged_attention(y, y.stride(0), out, cache, group, ctx, s.heads, s.softmax_scale, self.mask, sink=s.sink,
                            raw=(self.q_weight, self.k_weight, s.eps, rot, rotary_dim, group.slot_mapping))
            if gate is not None:
                ops.head_gate(out, gate, s.heads)
            if defer_output:
                return ops.linear_or_pending(out, self.w_o)
            return ops.linear(out, self.w_o)
        if self.per_head:
            ops.head_norm_rope_cache(y, 0, max(self.k_off, 0), self.v_off, s.heads, s.kv_heads, s.dim, s.vdim,
                                     self.q_weight, self.k_weight, s.eps, rot, rotary_dim, self.pairing,
                                     group.slot_mapping if s.own_kv else None, cache.k, cache.v, self.runtime.page_size)
        else:
            ops.proj_norm_rope_cache(y, 0, self.k_off, self.v_off, s.heads, s.kv_heads, s.dim, s.vdim, self.q_weight,
                                     self.k_weight, s.eps, rot, rotary_dim, self.pairing,
                                     group.slot_mapping if s.own_kv else None, cache.k, cache.v, self.runtime.page_size)
        if self.tensor_cores:
            paged_attention(y, y.stride(0), out, cache, group, ctx, s.heads, s.softmax_scale, self.mask, sink=s.sink)
            if gate is not None:
                ops.head_gate(out, gate, s.heads)
        else:
            ops.paged_attention_generic(y, y.stride(0), out, cache.k, cache.v, group.block_tables, ctx.token_slot,
                                        ctx.positions, s.heads, s.softmax_scale, self.mask, sink=s.sink, gate=gate)
        if defer_output:
            return ops.linear_or_pending(out, self.w_o)
        return ops.linear(out, self.w_o)
