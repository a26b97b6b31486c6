"""A routed feed-forward: a mixture of small experts ``down(act(up(x)))`` and an optional shared
expert of the same form.

The router's logits and scores are 32-bit (``ops.route_top_k``: the score of every expert, the
``top`` largest chosen, their scores kept as the experts' weights and zero for the rest).  The
experts' up-projections are stacked into one matrix, the shared expert's rows after them, and so
are the columns of the down-projections: a step is the router product, the routing kernel, one
product up, one kernel that applies relu^2 and the token's weight of the column's expert (zero
for an expert the token did not choose, one for the shared expert), and one product down, which
sums the weighted experts and the shared expert in its 32-bit accumulator.  Every token's result
depends on its own row only.

A bfloat16 step that would spend ``SORT_MIN_SAVED_FLOPS`` or more on experts nobody chose computes
only the experts a token chose: the (token, expert) pairs are sorted by expert (``ops.moe_sort``), the tokens' rows gathered
in that order, both products run as grouped products over the experts' row ranges with relu^2 and
the row's weight between them, and one kernel adds each token's rows, in the order its experts
were chosen, to the shared expert's output.  Smaller steps, and the 32-bit path, compute every
expert with zero weights as above: the sort, the gather and the grouped products' set-up cost a few
hundred microseconds of a step (measured on B200 at 2,048 rows and 8 experts of which 2 are
chosen: at width 2,048 and experts of 2,048 the sorted step loses 3 % with two products an
expert, 2.1e11 FLOPs saved, and wins 8 to 10 % with three, 3.1e11; at width 4,096 and experts of
3,072 it wins 12 % with two),
with a handful of rows most experts' weights are read either way, and the 32-bit path keeps one
summation order for every cutting.  ``MRUN_MOE_SORT_MIN_FLOPS`` in the environment overrides the
threshold (0: every bfloat16 step sorts).
"""
from __future__ import annotations

import os

import torch

from ..config.spec import RoutedMLPSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_feed_forward

ACTIVATIONS = ("relu2",)
# FLOPs a step would spend on experts nobody chose, from which its pairs are sorted by expert
SORT_MIN_SAVED_FLOPS = float(os.environ.get("MRUN_MOE_SORT_MIN_FLOPS", 2.5e11))


@register_feed_forward("routed_mlp")
class RoutedMLP:
    can_defer_output = True         # ``forward(..., defer_output=True)`` may return ``ops.PendingLinear``

    @staticmethod
    def tensor_specs(spec: RoutedMLPSpec, prefix: str):
        out = [TensorSpec(f"{prefix}.router", (spec.experts, spec.hidden))]
        for e in range(spec.experts):
            out += [TensorSpec(f"{prefix}.e{e}.up", (spec.expert_ff, spec.hidden)),
                    TensorSpec(f"{prefix}.e{e}.down", (spec.hidden, spec.expert_ff))]
        if spec.shared_ff:
            out += [TensorSpec(f"{prefix}.shared.up", (spec.shared_ff, spec.hidden)),
                    TensorSpec(f"{prefix}.shared.down", (spec.hidden, spec.shared_ff))]
        return out

    def __init__(self, spec: RoutedMLPSpec, tensors, runtime: Runtime):
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"no kernel has the expert activation {spec.activation!r} (known: {', '.join(ACTIVATIONS)})")
        if spec.score not in ops.ROUTER_SCORES:
            raise ValueError(f"no kernel has the router score {spec.score!r}")
        self.spec = spec
        names = [f"e{e}" for e in range(spec.experts)] + (["shared"] if spec.shared_ff else [])
        self.w_router = runtime.matrix(tensors["router"])
        self.w_up = runtime.matrix(torch.cat([tensors[f"{n}.up"] for n in names], dim=0))
        self.w_down = runtime.matrix(torch.cat([tensors[f"{n}.down"] for n in names], dim=1))
        # the same memory seen expert by expert, for the grouped products: [experts, out, in]
        routed = spec.experts * spec.expert_ff
        self.w_up_experts = self.w_up[:routed].view(spec.experts, spec.expert_ff, spec.hidden)
        self.w_down_experts = self.w_down[:, :routed].view(spec.hidden, spec.experts, spec.expert_ff).permute(1, 0, 2)
        self.w_up_shared = self.w_up[routed:] if spec.shared_ff else None
        self.w_down_shared = self.w_down[:, routed:] if spec.shared_ff else None
        self.sortable = (runtime.precision.act == torch.bfloat16 and spec.top < spec.experts
                         and spec.hidden % 8 == 0 and spec.expert_ff % 8 == 0 and self.w_down.shape[1] % 8 == 0)

    def activation_elements(self) -> int:
        return 2 * (self.spec.experts * self.spec.expert_ff + self.spec.shared_ff) + self.spec.experts

    def _sorted_forward(self, x, logits):
        """Only the chosen experts: float32 [tokens, hidden]."""
        s = self.spec
        chosen = torch.empty((x.shape[0], s.top), dtype=torch.int32, device=x.device)
        weights = ops.route_top_k(logits, s.top, s.score, s.renormalize, chosen=chosen)
        ends, source, row_weight, dest = ops.moe_sort(chosen, weights)
        rows = ops.gather_rows(x, source)
        act = ops.relu2_rows(ops.grouped_linear(rows, self.w_up_experts, ends), row_weight)
        rows = ops.grouped_linear(act, self.w_down_experts, ends)
        base = None
        if s.shared_ff:
            shared = ops.relu2_scaled(ops.linear(x, self.w_up_shared), None, 0, 1)
            base = torch.mm(shared, self.w_down_shared.t(), out_dtype=torch.float32)
        return ops.combine_rows(base, rows, dest)

    def forward(self, x, ctx, defer_output: bool = False):
        s = self.spec
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)
        saved = 4.0 * x.shape[0] * (s.experts - s.top) * s.expert_ff * s.hidden
        if self.sortable and saved >= SORT_MIN_SAVED_FLOPS and x.shape[0] > 16 \
                and not torch.cuda.is_current_stream_capturing():
            return self._sorted_forward(x, logits)
        weights = ops.route_top_k(logits, s.top, s.score, s.renormalize)
        act = ops.relu2_scaled(ops.linear(x, self.w_up), weights, s.experts, s.expert_ff)
        if defer_output:
            return ops.linear_or_pending(act, self.w_down)
        return ops.linear(act, self.w_down)
