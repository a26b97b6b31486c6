"""Linear attention with a decay per head and key channel (the formulas are with
:class:`GatedLinearAttentionSpec`).

One product makes [q | k | v | gate | a1 x]; a small product finishes the low-rank decay
projection with 32-bit output, as it enters the recurrence.  ``ops.gated_scan`` scales q, forms the
decays sigmoid(. + bias)^(1/tau) and walks each request's tokens from the state it left (float32
[heads, dim, vdim] per request); ``ops.gated_norm`` norms every head's output with the shared
weight and applies SiLU of the gate; the output projection follows.  The state and everything
inside the recurrence are 32-bit in both precisions.
"""
from __future__ import annotations

import torch

from ..cache.needs import FixedState
from ..config.spec import GatedLinearAttentionSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_mixer


@register_mixer("gated_linear_attention")
class GatedLinearAttention:
    can_defer_output = True
    graph_safe = True

    @staticmethod
    def tensor_specs(spec: GatedLinearAttentionSpec, prefix: str):
        keyed, inner = spec.heads * spec.dim, spec.heads * spec.vdim
        return [TensorSpec(f"{prefix}.q", (keyed, spec.hidden)),
                TensorSpec(f"{prefix}.k", (keyed, spec.hidden)),
                TensorSpec(f"{prefix}.v", (inner, spec.hidden)),
                TensorSpec(f"{prefix}.g", (inner, spec.hidden)),
                TensorSpec(f"{prefix}.o", (spec.hidden, inner)),
                TensorSpec(f"{prefix}.norm", (spec.vdim,), "norm"),
                TensorSpec(f"{prefix}.a1", (spec.rank, spec.hidden)),
                TensorSpec(f"{prefix}.a2", (keyed, spec.rank)),
                TensorSpec(f"{prefix}.a2.b", (keyed,))]

    def __init__(self, spec: GatedLinearAttentionSpec, tensors, runtime: Runtime):
        if not spec.tau > 0:
            raise ValueError(f"tau must be positive, got {spec.tau}")
        self.spec = spec
        self.w_in = runtime.matrix(torch.cat([tensors[n] for n in ("q", "k", "v", "g", "a1")], dim=0))
        self.w_a2 = runtime.matrix(tensors["a2"])
        self.bias = runtime.vector_f32(tensors["a2.b"])
        self.w_o = runtime.matrix(tensors["o"])
        self.norm_weight = runtime.vector_f32(tensors["norm"])
        self.act = runtime.precision.act

    def activation_elements(self) -> int:
        s = self.spec
        return s.heads * (5 * s.dim + 5 * s.vdim) + s.rank

    def cache_need(self):
        s = self.spec
        return FixedState((s.heads, s.dim, s.vdim), "float32", name="state")

    def forward(self, x, ctx, cache, defer_output: bool = False):
        s = self.spec
        if cache is None or not cache.writable:
            raise ValueError("a recurrent mixer needs a state of its own")
        keyed, inner = s.heads * s.dim, s.heads * s.vdim
        y = ops.linear(x, self.w_in)
        gate = y[:, 2 * keyed + inner:2 * keyed + 2 * inner]
        a = ops.linear(y[:, 2 * keyed + 2 * inner:], self.w_a2, out_dtype=torch.float32)    # a column slice: the products take row strides
        o = ops.gated_scan(y[:, :keyed], y[:, keyed:2 * keyed], y[:, 2 * keyed:2 * keyed + inner], a, self.bias, s.tau,
                           cache.states["state"], ctx, s.heads, s.dim, s.vdim)
        o = ops.gated_norm(o, self.norm_weight, gate, s.eps, s.heads, self.act, gate_function="silu")
        if defer_output:
            return ops.linear_or_pending(o, self.w_o)
        return ops.linear(o, self.w_o)
