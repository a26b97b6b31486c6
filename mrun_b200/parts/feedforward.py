"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``, act = SiLU for Qwen3
(crates/mrun-engine/src/models/common.rs:312-345, crates/mrun-engine/src/models/activations.rs:46-59).
gate and up run as one product with the weights stacked (this file's own concatenation); with at
most 16 rows the activation is applied in that product's epilogue.  The gate's function is a name
the kernels know by a code (``ops.GATE_FUNCTIONS``); a projection's ``.bias`` is bound and added
when the checkpoint has one (crates/mrun-engine/src/load.rs:281,302-305)."""
from __future__ import annotations

import torch

from ..config.spec import ClampedGatedMLPSpec, GatedMLPSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_feed_forward


def _bias_name(weight_name: str):
    """``x.weight`` -> ``x.bias``; a name without that ending has no bias beside it (None)."""
    return weight_name[:-len("weight")] + "bias" if weight_name.endswith(".weight") else None


@register_feed_forward("gated_mlp")
class GatedMLP:
    accepts_normed_rows = True      # its first product takes ``ops.NormedRows`` as x
    can_defer_output = True         # ``forward(..., defer_output=True)`` may return ``ops.PendingLinear``
    @staticmethod
    def tensor_specs(spec: GatedMLPSpec, prefix: str):
        gate, up, down = spec.tensor_names
        out = [TensorSpec(f"{prefix}.{gate}", (spec.intermediate, spec.hidden)),
               TensorSpec(f"{prefix}.{up}", (spec.intermediate, spec.hidden)),
               TensorSpec(f"{prefix}.{down}", (spec.hidden, spec.intermediate))]
        for name, size in ((gate, spec.intermediate), (up, spec.intermediate), (down, spec.hidden)):
            if name.endswith(".weight"):
                out.append(TensorSpec(f"{prefix}.{_bias_name(name)}", (size,), optional=True))
        return out

    def __init__(self, spec: GatedMLPSpec, tensors, runtime: Runtime):
        ops.gate_code(spec.activation)       # refuses a gate function no kernel has
        self.spec = spec
        gate_name, up_name, down_name = spec.tensor_names
        gate, up = tensors[gate_name], tensors[up_name]
        # bfloat16: gate and up rows interleaved in runs of eight, so that the decode GEMM's
        # epilogue finds a gate and its up in one thread and applies the activation itself
        self.interleaved = runtime.precision.act == torch.bfloat16 and spec.intermediate % 8 == 0
        if self.interleaved:
            stacked = torch.stack([gate.view(-1, 8, spec.hidden), up.view(-1, 8, spec.hidden)], dim=1)
            self.w_gate_up = runtime.matrix(stacked.reshape(2 * spec.intermediate, spec.hidden))
        else:
            self.w_gate_up = runtime.matrix(torch.cat([gate, up], dim=0))
        self.w_down = runtime.matrix(tensors[down_name])
        self.b_gate_up = None
        gate_bias, up_bias = tensors.get(_bias_name(gate_name)), tensors.get(_bias_name(up_name))
        if gate_bias is not None or up_bias is not None:
            zeros = torch.zeros(spec.intermediate, dtype=torch.float32)
            gate_bias = zeros if gate_bias is None else gate_bias.to(torch.float32)
            up_bias = zeros if up_bias is None else up_bias.to(torch.float32)
            if self.interleaved:
                both = torch.stack([gate_bias.view(-1, 8), up_bias.view(-1, 8)], dim=1).reshape(-1)
            else:
                both = torch.cat([gate_bias, up_bias])
            self.b_gate_up = runtime.vector_f32(both)
        down_bias = tensors.get(_bias_name(down_name))
        self.b_down = runtime.vector_f32(down_bias) if down_bias is not None else None

    def activation_elements(self) -> int:
        """Elements per token of the temporaries alive at once (gate, up and their product)."""
        return 3 * self.spec.intermediate

    def forward(self, x, ctx, defer_output: bool = False):
        name = self.spec.activation
        if self.interleaved and self.b_gate_up is None and ops.skinny_ok(x, self.w_gate_up):
            act = ops.gemm_skinny(x, self.w_gate_up, swiglu_rows=True, activation=name)
        elif self.interleaved and self.b_gate_up is None and ops.tc5_ok(x, self.w_gate_up):
            act = ops.gemm_tc5(x, self.w_gate_up, swiglu_rows=True, activation=name)
        else:
            gate_up = ops.linear(x, self.w_gate_up, bias=self.b_gate_up)
            act = torch.empty((gate_up.shape[0], self.spec.intermediate), dtype=gate_up.dtype, device=gate_up.device)
            ops.swiglu(gate_up, act, interleaved=self.interleaved, activation=name)
        if defer_output:
            return ops.linear_or_pending(act, self.w_down, self.b_down)
        return ops.linear(act, self.w_down, bias=self.b_down)


@register_feed_forward("clamped_gated_mlp")
class ClampedGatedMLP:
    """Dense gated feed-forward with clamped branches (the formulas are with
    :class:`ClampedGatedMLPSpec`): one product makes [gate | up], ``ops.clamped_glu`` adds their
    biases in 32-bit and applies min / clamp, the gate's sigmoid and the +1, one product goes down
    with its bias.  The checkpoint names the matrices ``gate``, ``up``, ``down`` and their biases
    ``gate.b``, ``up.b``, ``down.b``."""

    can_defer_output = True

    @staticmethod
    def tensor_specs(spec: ClampedGatedMLPSpec, prefix: str):
        out = [TensorSpec(f"{prefix}.gate", (spec.intermediate, spec.hidden)),
               TensorSpec(f"{prefix}.up", (spec.intermediate, spec.hidden)),
               TensorSpec(f"{prefix}.down", (spec.hidden, spec.intermediate))]
        if spec.biases:
            out += [TensorSpec(f"{prefix}.gate.b", (spec.intermediate,)), TensorSpec(f"{prefix}.up.b", (spec.intermediate,)),
                    TensorSpec(f"{prefix}.down.b", (spec.hidden,))]
        return out

    def __init__(self, spec: ClampedGatedMLPSpec, tensors, runtime: Runtime):
        self.spec = spec
        self.w_gate_up = runtime.matrix(torch.cat([tensors["gate"], tensors["up"]], dim=0))
        self.w_down = runtime.matrix(tensors["down"])
        self.b_gate_up = self.b_down = None
        if spec.biases:
            self.b_gate_up = runtime.vector_f32(torch.cat([tensors["gate.b"].to(torch.float32), tensors["up.b"].to(torch.float32)]))
            self.b_down = runtime.vector_f32(tensors["down.b"])

    def activation_elements(self) -> int:
        return 3 * self.spec.intermediate

    def forward(self, x, ctx, defer_output: bool = False):
        s = self.spec
        u = ops.linear(x, self.w_gate_up)
        act = ops.clamped_glu(u, None, 1, s.intermediate, s.limit, s.alpha, bias=self.b_gate_up)
        if defer_output:
            return ops.linear_or_pending(act, self.w_down, self.b_down)
        return ops.linear(act, self.w_down, bias=self.b_down)
