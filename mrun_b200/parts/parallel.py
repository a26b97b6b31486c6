"""Two mixers side by side (the formulas are with :class:`ParallelMixerSpec`).

Both read the same normed rows.  Each runs as it would alone, with its own kinds of cache: the
schedule entry's need is the two needs together (at most one of them paged; fixed-size states
under different names), and both see the entry's one :class:`EntryCache`, of which each uses its
own members.  Their last products write 32-bit sums; each branch is divided by its root mean
square over the model width, multiplied by its weight, and ``share`` of their sum joins the
stream.  A caller that takes pending outputs (``defer_output=True``) gets the two branches as
they are (``ops.PendingPairNorm``): a layer norm behind it does the branch norms, the average,
the residual sum and its own norm in one kernel; otherwise ``ops.pair_norm_mean`` makes the
32-bit addend.
"""
from __future__ import annotations

import torch

from ..cache.needs import split_need
from ..config.spec import ParallelMixerSpec, TensorSpec
from ..kernels import ops
from .base import MIXERS, Runtime, local, register_mixer


@register_mixer("parallel")
class ParallelMixer:
    can_defer_output = True         # ``forward(..., defer_output=True)`` may return ``ops.PendingPairNorm``

    @staticmethod
    def tensor_specs(spec: ParallelMixerSpec, prefix: str):
        out = []
        for side, name in ((spec.left, spec.left_prefix), (spec.right, spec.right_prefix)):
            out += MIXERS.tensor_specs(side, f"{prefix}.{name}")
            out.append(TensorSpec(f"{prefix}.{name}.{spec.out_name}", (spec.hidden,), "norm"))
        return out

    def __init__(self, spec: ParallelMixerSpec, tensors, runtime: Runtime):
        self.spec = spec
        self.sides = []
        for side, name in ((spec.left, spec.left_prefix), (spec.right, spec.right_prefix)):
            mine = local(tensors, name)
            mixer = MIXERS.build(side, mine, runtime)
            self.sides.append((mixer, runtime.vector_f32(mine[spec.out_name]),
                               bool(getattr(mixer, "can_defer_output", False))))
        split_need(self.cache_need())       # refuses two paged needs, and states of one name
        self.graph_safe = all(getattr(mixer, "graph_safe", False) for mixer, _, _ in self.sides)

    def cache_need(self):
        needs = []
        for mixer, _, _ in self.sides:
            need = mixer.cache_need()
            if need is not None:
                needs += list(need) if isinstance(need, (tuple, list)) else [need]
        return tuple(needs) if needs else None

    def activation_elements(self) -> int:
        total = 2 * self.spec.hidden
        for mixer, _, _ in self.sides:
            hint = getattr(mixer, "activation_elements", None)
            total += int(hint()) if hint is not None else 0
        return total

    def _branch(self, mixer, defers: bool, x, ctx, cache) -> torch.Tensor:
        """One side's output as 32-bit rows."""
        if defers:
            y = mixer.forward(x, ctx, cache, defer_output=True)
            if isinstance(y, ops.PendingLinear):
                return ops.linear(y.x, y.w, out_dtype=torch.float32)
        else:
            y = mixer.forward(x, ctx, cache)
        if isinstance(y, ops.PENDING):
            y = y.compute()
        return y if y.dtype == torch.float32 else y.to(torch.float32)

    def forward(self, x, ctx, cache, defer_output: bool = False):
        (left, w_left, left_defers), (right, w_right, right_defers) = self.sides
        a = self._branch(left, left_defers, x, ctx, cache)
        b = self._branch(right, right_defers, x, ctx, cache)
        pending = ops.PendingPairNorm(a, b, w_left, w_right, self.spec.eps, self.spec.share)
        return pending if defer_output else pending.compute()
