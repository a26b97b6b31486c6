"""A mixture of gated experts behind a sigmoid router with a group-limited choice, and a shared
expert with a gate of its own (the formulas are with :class:`GroupedRoutedMLPSpec`).

The router's rows and the shared expert's gate row are one product with 32-bit output;
``ops.route_grouped`` makes the dense weight row (score / sum * scale at the chosen experts), the
chosen list and the shared expert's sigmoid weight.  The experts' [gate | up] rows are stacked
expert by expert with the shared expert's after them, and so are the columns of the down
matrices, as :mod:`routed` and :mod:`table_routed` stack theirs.  A small step, and every 32-bit
step, runs one product up over all experts, the gated activation with the token's weight of each
expert (zero for an expert it did not choose), and one product down whose 32-bit accumulator sums
the weighted experts and the shared expert: a row's result depends on the row only, and the step
can be captured.  A bfloat16 step that would spend ``routed.SORT_MIN_SAVED_FLOPS`` or more on
experts nobody chose sorts its (token, expert) pairs by expert and runs grouped products over the
chosen experts only, as the other routed feed-forwards do.
"""
from __future__ import annotations

import math

import torch

from ..config.spec import GroupedRoutedMLPSpec, TensorSpec
from ..kernels import ops
from . import routed
from .base import Runtime, register_feed_forward

SCORES = ("sigmoid", "logit")
ACTIVATIONS = {"silu": 1.0}       # the gate's function as the factor inside its sigmoid: g * sigmoid(factor * g)


@register_feed_forward("grouped_routed_mlp")
class GroupedRoutedMLP:
    can_defer_output = True

    @staticmethod
    def tensor_specs(spec: GroupedRoutedMLPSpec, prefix: str):
        out = [TensorSpec(f"{prefix}.router", (spec.experts, spec.hidden))]
        if spec.router_bias:
            out.append(TensorSpec(f"{prefix}.router.b", (spec.experts,)))
        sizes = [(f"e{e}", spec.expert_ff) for e in range(spec.experts)] + ([("shared", spec.shared_ff)] if spec.shared_ff else [])
        for name, ff in sizes:
            out += [TensorSpec(f"{prefix}.{name}.gate", (ff, spec.hidden)),
                    TensorSpec(f"{prefix}.{name}.up", (ff, spec.hidden)),
                    TensorSpec(f"{prefix}.{name}.down", (spec.hidden, ff))]
        if spec.shared_ff and spec.shared_gate:
            out.append(TensorSpec(f"{prefix}.shared.sg", (1, spec.hidden)))
        return out

    def __init__(self, spec: GroupedRoutedMLPSpec, tensors, runtime: Runtime):
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"no kernel has the expert activation {spec.activation!r} (known: {', '.join(ACTIVATIONS)})")
        if spec.experts % spec.groups or not 1 <= spec.keep_groups <= spec.groups \
                or not 1 <= spec.top <= spec.keep_groups * (spec.experts // spec.groups):
            raise ValueError(f"{spec.experts} experts in {spec.groups} groups of which {spec.keep_groups} stay "
                             f"cannot give {spec.top} choices")
        if spec.score not in SCORES:
            raise ValueError(f"no kernel has the router score {spec.score!r} (known: {', '.join(SCORES)})")
        if spec.score == "logit" and (spec.groups != 1 or (spec.shared_ff and spec.shared_gate)):
            raise ValueError("a router that ranks its logits has no groups and no gated shared expert")
        self.spec = spec
        self.router_bias = runtime.vector_f32(tensors["router.b"]) if spec.router_bias else None
        self.alpha = ACTIVATIONS[spec.activation]
        names = [f"e{e}" for e in range(spec.experts)] + (["shared"] if spec.shared_ff else [])
        self.gated_shared = bool(spec.shared_ff and spec.shared_gate)
        router = torch.cat([tensors["router"]] + ([tensors["shared.sg"]] if self.gated_shared else []), dim=0)
        self.router_rows = router.shape[0]
        if runtime.precision.act == torch.bfloat16 and router.shape[0] % 8:
            # zero rows up to a multiple of 8: the vendor library's tensor-core kernels of this
            # architecture want rows of 16 bytes; the route kernel reads the first columns only
            router = torch.cat([router, router.new_zeros(-router.shape[0] % 8, router.shape[1])], dim=0)
        self.w_router = runtime.matrix(router)
        self.w_up = runtime.matrix(torch.cat([t for n in names for t in (tensors[f"{n}.gate"], tensors[f"{n}.up"])], dim=0))
        self.w_down = runtime.matrix(torch.cat([tensors[f"{n}.down"] for n in names], dim=1))
        routed_rows, routed_cols = 2 * spec.experts * spec.expert_ff, spec.experts * spec.expert_ff
        self.routed_rows, self.routed_cols = routed_rows, routed_cols
        # the same memory seen expert by expert, for the grouped products: [experts, out, in]
        self.w_up_experts = self.w_up[:routed_rows].view(spec.experts, 2 * spec.expert_ff, spec.hidden)
        self.w_down_experts = self.w_down[:, :routed_cols].view(spec.hidden, spec.experts, spec.expert_ff).permute(1, 0, 2)
        self.w_up_shared = self.w_up[routed_rows:] if spec.shared_ff else None
        self.w_down_shared = self.w_down[:, routed_cols:] if spec.shared_ff else None
        self.sortable = (runtime.precision.act == torch.bfloat16 and spec.top < spec.experts
                         and spec.hidden % 8 == 0 and spec.expert_ff % 8 == 0 and self.w_down.shape[1] % 8 == 0)

    def activation_elements(self) -> int:
        s = self.spec
        return 3 * (s.experts * s.expert_ff + s.shared_ff) + 2 * s.experts + 1

    def _route(self, x, chosen=None):
        s = self.spec
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)[:, :self.router_rows]
        if s.score == "logit":      # the softmax over the chosen logits only
            return ops.route_top_k(logits, s.top, "logit", chosen=chosen, bias=self.router_bias), None
        if self.router_bias is not None:
            logits = ops.add_bias(logits.contiguous(), self.router_bias)
        return ops.route_grouped(logits, s.experts, s.top, s.groups, s.keep_groups, s.group_top, s.route_scale, chosen=chosen)

    def _sorted_forward(self, x):
        """Only the chosen experts: float32 [tokens, hidden]."""
        s = self.spec
        chosen = torch.empty((x.shape[0], s.top), dtype=torch.int32, device=x.device)
        weights, shared_weight = self._route(x, chosen)
        ends, source, row_weight, dest = ops.moe_sort(chosen, weights)
        rows = ops.gather_rows(x, source)
        act = ops.clamped_glu(ops.grouped_linear(rows, self.w_up_experts, ends), row_weight, 1, s.expert_ff, math.inf,
                              self.alpha, up_offset=0.0)
        rows = ops.grouped_linear(act, self.w_down_experts, ends)
        base = None
        if s.shared_ff:
            shared = ops.clamped_glu(ops.linear(x, self.w_up_shared), shared_weight, 1, s.shared_ff, math.inf, self.alpha,
                                     up_offset=0.0)
            base = torch.mm(shared, self.w_down_shared.t(), out_dtype=torch.float32)
        return ops.combine_rows(base, rows, dest)

    def forward(self, x, ctx, defer_output: bool = False):
        s = self.spec
        saved = 6.0 * x.shape[0] * (s.experts - s.top) * s.expert_ff * s.hidden
        if self.sortable and saved >= routed.SORT_MIN_SAVED_FLOPS and x.shape[0] > 16 \
                and not torch.cuda.is_current_stream_capturing():
            return self._sorted_forward(x)
        weights, shared_weight = self._route(x)
        u = ops.linear(x, self.w_up)
        act = torch.empty((x.shape[0], self.routed_cols + s.shared_ff), dtype=u.dtype, device=u.device)
        ops.clamped_glu(u[:, :self.routed_rows], weights, s.experts, s.expert_ff, math.inf, self.alpha, up_offset=0.0,
                        out=act[:, :self.routed_cols])
        if s.shared_ff:
            ops.clamped_glu(u[:, self.routed_rows:], shared_weight, 1, s.shared_ff, math.inf, self.alpha, up_offset=0.0,
                            out=act[:, self.routed_cols:])
        if defer_output:
            return ops.linear_or_pending(act, self.w_down)
        return ops.linear(act, self.w_down)
