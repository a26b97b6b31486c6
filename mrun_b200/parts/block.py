"""The pre-norm arrangement of a layer: ``x += mixer(norm(x)); x += ff(norm(x))``
(crates/mrun-engine/src/models/qwen3.rs:133-145).

The residual sum is fused with the norm that follows it: a block receives the 32-bit stream and the
previous branch's output that has not been added yet, and returns its own feed-forward output
unadded.  The sum itself is 32-bit.

Two optional capabilities let a decode step fold that sum and norm into the products around
them; a part that does not declare them gets and gives plain tensors.  A mixer or feed-forward
with ``can_defer_output`` may return its last product unrun (``ops.PendingLinear``) when called
with ``defer_output=True``; a norm with ``accepts_pending`` takes it as ``delta`` and may answer
with ``ops.NormedRows``; a part with ``accepts_normed_rows`` takes those as its ``x``.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.needs import FixedState
from ..config.spec import LayerSpec, TensorSpec
from ..kernels import ops
from .base import FEED_FORWARDS, MIXERS, NORMS, Runtime, local, register_arrangement


def norm_add(norm, resid: torch.Tensor, delta):
    """``norm.add_forward`` for a ``delta`` that may be pending: computed first unless the norm
    takes it as it is."""
    if isinstance(delta, ops.PENDING) and not getattr(norm, "accepts_pending", False):
        delta = delta.compute()
    if isinstance(delta, torch.Tensor) and delta.dtype == torch.float32 and resid.dtype == torch.float32 \
            and getattr(norm, "act", torch.float32) != torch.float32 and not getattr(norm, "accepts_wide_delta", False):
        delta = delta.to(norm.act)      # a 32-bit branch output in front of a norm that takes the activation type
    return norm.add_forward(resid, delta)


def part_input(part, h):
    """Normed rows for a part: finished into a plain tensor unless the part takes them as they are."""
    if isinstance(h, ops.NormedRows) and not getattr(part, "accepts_normed_rows", False):
        h = h.finish()
    return h


@register_arrangement("pre_norm")
class PreNormBlock:
    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str = "") -> list[TensorSpec]:
        p = spec.prefix
        out = (NORMS.tensor_specs(spec.mixer_norm, f"{p}.{spec.mixer_norm_prefix}")
               + MIXERS.tensor_specs(spec.mixer, f"{p}.{spec.mixer_prefix}"))
        if spec.feed_forward is not None:       # a layer may be a mixer only
            out += (NORMS.tensor_specs(spec.feed_forward_norm, f"{p}.{spec.feed_forward_norm_prefix}")
                    + FEED_FORWARDS.tensor_specs(spec.feed_forward, f"{p}.{spec.feed_forward_prefix}"))
        return out

    def __init__(self, spec: LayerSpec, tensors, runtime: Runtime):
        mine = local(tensors, spec.prefix)
        self.mixer_norm = NORMS.build(spec.mixer_norm, local(mine, spec.mixer_norm_prefix), runtime)
        self.mixer = MIXERS.build(spec.mixer, local(mine, spec.mixer_prefix), runtime)
        self.feed_forward_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, local(mine, spec.feed_forward_norm_prefix), runtime)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, local(mine, spec.feed_forward_prefix), runtime)
        self._mixer_defers = bool(getattr(self.mixer, "can_defer_output", False))
        self._feed_forward_defers = bool(getattr(self.feed_forward, "can_defer_output", False))

    accepts_pending = True      # ``delta`` may be an ``ops.PendingLinear``, and so may the result

    def forward(self, resid: torch.Tensor, delta, ctx, cache):
        h = part_input(self.mixer, norm_add(self.mixer_norm, resid, delta))
        if self._mixer_defers:
            a = self.mixer.forward(h, ctx, cache, defer_output=True)
        else:
            a = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            return a
        h = part_input(self.feed_forward, norm_add(self.feed_forward_norm, resid, a))
        if self._feed_forward_defers:
            return self.feed_forward.forward(h, ctx, defer_output=True)
        return self.feed_forward.forward(h, ctx)


@register_arrangement("sandwich")
class SandwichBlock:
    """``x += s * post_norm_1(mixer(norm_1(x))); x += s * post_norm_2(ff(norm_2(x)))``: every branch
    is normed on its way in and on its way out, and its normed output is multiplied by the
    layer's ``residual_scale`` s before it joins the 32-bit stream.  A layer without a
    feed-forward has the first half only.

    The branch's last product writes 32-bit sums; the post-norm of the branch, the residual sum
    and the norm in front of the next branch are one kernel (``ops.post_norm_add``), so the block
    hands its own last branch output on unadded, as the pre-norm arrangement does."""

    accepts_pending = True

    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str = "") -> list[TensorSpec]:
        p = spec.prefix
        out = (NORMS.tensor_specs(spec.mixer_norm, f"{p}.{spec.mixer_norm_prefix}")
               + NORMS.tensor_specs(spec.mixer_post_norm, f"{p}.{spec.mixer_post_norm_prefix}")
               + MIXERS.tensor_specs(spec.mixer, f"{p}.{spec.mixer_prefix}"))
        if spec.feed_forward is not None:
            out += (NORMS.tensor_specs(spec.feed_forward_norm, f"{p}.{spec.feed_forward_norm_prefix}")
                    + NORMS.tensor_specs(spec.feed_forward_post_norm, f"{p}.{spec.feed_forward_post_norm_prefix}")
                    + FEED_FORWARDS.tensor_specs(spec.feed_forward, f"{p}.{spec.feed_forward_prefix}"))
        return out

    def __init__(self, spec: LayerSpec, tensors, runtime: Runtime):
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and spec.feed_forward_post_norm is None):
            raise ValueError("the sandwich arrangement needs a post-norm for every branch")
        mine = local(tensors, spec.prefix)
        build = lambda norm_spec, prefix: NORMS.build(norm_spec, local(mine, prefix), runtime)
        self.scale = float(spec.residual_scale)
        self.act = runtime.precision.act
        self.mixer_norm = build(spec.mixer_norm, spec.mixer_norm_prefix)
        self.mixer_post_norm = build(spec.mixer_post_norm, spec.mixer_post_norm_prefix)
        self.mixer = MIXERS.build(spec.mixer, local(mine, spec.mixer_prefix), runtime)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = build(spec.feed_forward_norm, spec.feed_forward_norm_prefix)
            self.feed_forward_post_norm = build(spec.feed_forward_post_norm, spec.feed_forward_post_norm_prefix)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, local(mine, spec.feed_forward_prefix), runtime)
        self._mixer_defers = bool(getattr(self.mixer, "can_defer_output", False))
        self._feed_forward_defers = bool(getattr(self.feed_forward, "can_defer_output", False))

    def _branch(self, y, post_norm) -> "ops.PendingPostNorm":
        """The branch output as 32-bit rows, with the post-norm that it still has to pass."""
        if isinstance(y, ops.PendingLinear):
            y = ops.linear(y.x, y.w, out_dtype=torch.float32)
        elif isinstance(y, ops.PENDING):
            y = y.compute()
        if y.dtype != torch.float32:
            y = y.to(torch.float32)
        return ops.PendingPostNorm(y, post_norm.weight, post_norm.eps, self.scale, self.act)

    def forward(self, resid: torch.Tensor, delta, ctx, cache):
        h = part_input(self.mixer, norm_add(self.mixer_norm, resid, delta))
        if self._mixer_defers:
            a = self.mixer.forward(h, ctx, cache, defer_output=True)
        else:
            a = self.mixer.forward(h, ctx, cache)
        a = self._branch(a, self.mixer_post_norm)
        if self.feed_forward is None:
            return a
        h = part_input(self.feed_forward, norm_add(self.feed_forward_norm, resid, a))
        if self._feed_forward_defers:
            f = self.feed_forward.forward(h, ctx, defer_output=True)
        else:
            f = self.feed_forward.forward(h, ctx)
        return self._branch(f, self.feed_forward_post_norm)


@register_arrangement("streams")
class StreamsBlock:
    """A pre-norm layer over several residual streams a token (hyper-connections).  The stream
    tensor is float32 [tokens, S * width].  Sublayer i (1: the mixer, 2: the feed-forward) reads u =
    sum_s in_i[s] x_s through its norm and writes x_t <- sum_s mix_i[s, t] x_s + out_i[t] * y into
    all streams at once.  The write is handed on unapplied (``ops.PendingStreams``) and runs in
    the kernel that makes the next sublayer's input, so a sublayer boundary is one kernel.  With
    ``LayerSpec.streams`` = 0 the layer has no coefficients and this is ``x += y`` over one
    stream.

    ``LayerSpec.input_conv_taps`` > 0: what the mixer reads is h + conv(h), a causal convolution
    per channel over the request's tokens; the last taps - 1 rows of h are per-request state of
    this layer run, kept beside the mixer's own cache (``cache.states['input_conv']``).  A layer
    without a feed-forward has the first half only."""

    accepts_pending = False

    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str = "") -> list[TensorSpec]:
        p, s = spec.prefix, spec.streams
        out = (NORMS.tensor_specs(spec.mixer_norm, f"{p}.{spec.mixer_norm_prefix}")
               + MIXERS.tensor_specs(spec.mixer, f"{p}.{spec.mixer_prefix}"))
        halves = [spec.mixer_streams_prefix]
        if spec.feed_forward is not None:
            out += (NORMS.tensor_specs(spec.feed_forward_norm, f"{p}.{spec.feed_forward_norm_prefix}")
                    + FEED_FORWARDS.tensor_specs(spec.feed_forward, f"{p}.{spec.feed_forward_prefix}"))
            halves.append(spec.feed_forward_streams_prefix)
        if s:
            for half in halves:
                out += [TensorSpec(f"{p}.{half}.in", (s,), "streams_in"), TensorSpec(f"{p}.{half}.out", (s,), "norm"),
                        TensorSpec(f"{p}.{half}.mix", (s, s), "streams_mix")]
        if spec.input_conv_taps:
            out.append(TensorSpec(f"{p}.{spec.input_conv_name}", (spec.mixer_norm.size, spec.input_conv_taps)))
        return out

    def __init__(self, spec: LayerSpec, tensors, runtime: Runtime):
        mine = local(tensors, spec.prefix)
        self.count = max(1, spec.streams)
        self.act = runtime.precision.act
        self.mixer_norm = NORMS.build(spec.mixer_norm, local(mine, spec.mixer_norm_prefix), runtime)
        self.mixer = MIXERS.build(spec.mixer, local(mine, spec.mixer_prefix), runtime)
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, local(mine, spec.feed_forward_norm_prefix), runtime)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, local(mine, spec.feed_forward_prefix), runtime)
        self._feed_forward_defers = bool(getattr(self.feed_forward, "can_defer_output", False))
        self._mixer_defers = bool(getattr(self.mixer, "can_defer_output", False))

        def coefficients(prefix):
            if not spec.streams:
                return None, None, None
            c = local(mine, prefix)
            return runtime.vector_f32(c["in"]), runtime.vector_f32(c["mix"]), runtime.vector_f32(c["out"])

        self.in1, self.mix1, self.out1 = coefficients(spec.mixer_streams_prefix)
        self.in2, self.mix2, self.out2 = coefficients(spec.feed_forward_streams_prefix) if self.feed_forward else (None,) * 3
        self.taps = int(spec.input_conv_taps)
        self.width = spec.mixer_norm.size
        self.conv_weight = runtime.vector_f32(mine[spec.input_conv_name]) if self.taps else None
        self._state_dtype = runtime.precision.name

    def cache_need(self):
        """The mixer's need and, with an input convolution, the state of its last inputs."""
        need = self.mixer.cache_need()
        if not self.taps:
            return need
        own = FixedState((self.taps - 1, self.width), self._state_dtype, name="input_conv")
        if need is None:
            return (own,)
        return (tuple(need) if isinstance(need, (tuple, list)) else (need,)) + (own,)

    @staticmethod
    def _rows(y) -> torch.Tensor:
        """A sublayer's output as 32-bit rows (its last product writes them where it was left unrun)."""
        if isinstance(y, ops.PendingLinear):
            return ops.linear(y.x, y.w, out_dtype=torch.float32)
        if isinstance(y, ops.PENDING):
            y = y.compute()
        return y if y.dtype == torch.float32 else y.to(torch.float32)

    def forward(self, resid: torch.Tensor, delta, ctx, cache):
        if delta is not None and not isinstance(delta, ops.PendingStreams):
            delta = ops.PendingStreams(self._rows(delta), None, None)
        h = ops.streams_step(resid, delta, self.in1, self.mixer_norm.weight, self.mixer_norm.eps, self.act, self.count)
        if self.taps:
            if cache is None or not cache.writable:
                raise ValueError("a layer with an input convolution needs a cache of its own")
            h = ops.causal_conv(h, self.conv_weight, cache.states["input_conv"], ctx, residual=True, silu=False)
        if self._mixer_defers:
            a = self.mixer.forward(h, ctx, cache, defer_output=True)
        else:
            a = self.mixer.forward(h, ctx, cache)
        a = ops.PendingStreams(self._rows(a), self.mix1, self.out1)
        if self.feed_forward is None:
            return a
        h = ops.streams_step(resid, a, self.in2, self.feed_forward_norm.weight, self.feed_forward_norm.eps, self.act,
                             self.count)
        if self._feed_forward_defers:
            f = self.feed_forward.forward(h, ctx, defer_output=True)
        else:
            f = self.feed_forward.forward(h, ctx)
        return ops.PendingStreams(self._rows(f), self.mix2, self.out2)
