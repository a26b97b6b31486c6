"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * w`` in 32-bit
(crates/mrun-engine/src/load.rs:348-364; the form with eps added to the mean is stated at
crates/mrun-engine/src/models/gated_delta.rs:11-13)."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import LayerNormSpec, RMSNormSpec, TensorSpec
from ..kernels import ops
from .base import Runtime, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    @staticmethod
    def tensor_specs(spec: RMSNormSpec, prefix: str):
        # a scale stored minus an offset lies around zero, not around one
        return [TensorSpec(prefix if spec.bare else f"{prefix}.weight", () if spec.scalar else (spec.size,),
                           "norm_zero" if spec.offset else "norm")]

    # ``delta`` may be a product that has not run yet (``ops.PendingLinear``): with a handful
    # of rows it runs with the residual sum and this norm folded into its epilogue, and what
    # comes back is ``ops.NormedRows`` (the row scale is applied by the product that reads it);
    # with more rows the vendor GEMM adds it into the 32-bit stream itself.
    accepts_pending = True

    def __init__(self, spec: RMSNormSpec, tensors, runtime: Runtime):
        self.size, self.eps = spec.size, float(spec.eps)
        weight = tensors["" if spec.bare else "weight"]
        if spec.scalar:             # one number for all coordinates: the kernels take it as a vector of equal entries
            weight = weight.reshape(1).expand(spec.size)
        if spec.offset:             # stored around zero: the kernels take the scale itself
            weight = weight.to(torch.float32) + float(spec.offset)
        self.weight = runtime.vector_f32(weight)
        self.act = runtime.precision.act

    def add_forward(self, resid: torch.Tensor, delta):
        if isinstance(delta, ops.PendingPostNorm):
            # a branch output that is normed and scaled before it joins the stream: one kernel
            # norms it, adds it and norms the new rows with this norm's weight
            out = torch.empty(resid.shape, dtype=self.act, device=resid.device)
            return ops.post_norm_add(resid, delta.branch, delta.weight, delta.scale, delta.eps, self.weight,
                                     self.eps, out)
        if isinstance(delta, ops.PendingPairNorm):
            delta = delta.compute().to(self.act)        # no fused form with this norm: the addend, in the activation type
        if isinstance(delta, ops.PendingLinear):
            if ops.norm_fusable(delta, resid, self.weight):
                return ops.linear_into_norm(delta, resid, self.weight, self.eps)
            if ops.accumulate_ok(delta, resid):
                ops.linear_add_into(resid, delta)          # the sum rides in the vendor GEMM
                delta = None
            else:
                delta = delta.compute()
        out = torch.empty(resid.shape, dtype=self.act, device=resid.device)
        return ops.add_rmsnorm(resid, delta, self.weight, self.eps, out)

    def rows_forward(self, resid: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        if isinstance(delta, ops.PendingPostNorm):
            out = torch.empty((rows.numel(), self.size), dtype=self.act, device=resid.device)
            return ops.post_norm_add(resid, delta.branch, delta.weight, delta.scale, delta.eps, self.weight,
                                     self.eps, out, rows=rows)
        if isinstance(delta, ops.PendingPairNorm):
            delta = delta.compute().to(self.act)
        if isinstance(delta, ops.PendingLinear):
            delta = delta.compute()
        out = torch.empty((rows.numel(), self.size), dtype=self.act, device=resid.device)
        return ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows=rows)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_forward(x.to(torch.float32), None)


@register_norm("layernorm")
class LayerNorm:
    """Layer norm with a weight and no bias, in 32-bit: ``y = (x - mean) * rsqrt(var + eps) * w``,
    the variance taken from the deviations.  The residual sum rides in the same kernel; a branch
    output may come in 32-bit or in the activation type."""

    @staticmethod
    def tensor_specs(spec: LayerNormSpec, prefix: str):
        return [TensorSpec(prefix if spec.bare else f"{prefix}.weight", (spec.size,), "norm")]

    # ``delta`` may be a product that has not run yet: above 16 bfloat16 rows the vendor GEMM adds
    # it into the 32-bit stream itself, otherwise it is computed first
    accepts_pending = True
    accepts_wide_delta = True       # ``delta`` may be 32-bit where the activations are not

    def __init__(self, spec: LayerNormSpec, tensors, runtime: Runtime):
        self.size, self.eps = spec.size, float(spec.eps)
        self.weight = runtime.vector_f32(tensors["" if spec.bare else "weight"])
        self.act = runtime.precision.act

    def _settle(self, resid: torch.Tensor, delta, in_place: bool):
        if isinstance(delta, ops.PendingLinear):
            if in_place and ops.accumulate_ok(delta, resid):
                ops.linear_add_into(resid, delta)
                return None
            return delta.compute()
        if isinstance(delta, ops.PENDING):
            return delta.compute()
        return delta

    def add_forward(self, resid: torch.Tensor, delta):
        out = torch.empty(resid.shape, dtype=self.act, device=resid.device)
        if isinstance(delta, ops.PendingPairNorm):      # two branches still to be normed and averaged: one kernel
            return ops.pair_norm_add_layernorm(resid, delta, self.weight, self.eps, out)
        delta = self._settle(resid, delta, True)
        return ops.add_layernorm(resid, delta, self.weight, self.eps, out)

    def rows_forward(self, resid: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty((rows.numel(), self.size), dtype=self.act, device=resid.device)
        if isinstance(delta, ops.PendingPairNorm):
            return ops.pair_norm_add_layernorm(resid, delta, self.weight, self.eps, out, rows=rows)
        delta = self._settle(resid, delta, False)
        return ops.add_layernorm(resid, delta, self.weight, self.eps, out, rows=rows)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_forward(x.to(torch.float32), None)
