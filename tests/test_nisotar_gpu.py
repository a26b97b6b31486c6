"""Nisotar on the GPU against the plain implementation (``plain_nisotar``): every new kernel and
every part alone (whole requests, token by token, portions down to one and two tokens, unequal
requests side by side, state slots and pages given back and used again), inputs made so that one
key just inside or just outside a window or a chunk, or the sink, decides the result, then whole
models replayed through ``bin/trace_run`` cut in every way, then greedy generation through
``Engine.generate`` and the command line."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_nisotar as plain
from test_fikudra_gpu import (CLOSE_CALL, FLIP_CALL, LENGTHS, SIZES, TRACE_LENGTHS, Steps, check_rows, close, named,
                              random_tensors, runtime)
from tiny_nisotar import NTINY, load_folder, make_folder, tokens_of
from trace_tools import TraceBuilder, TraceRunner, cut_decode_tail, cut_mixed, cut_portions, cut_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


# ------------------------------------------------------------------ kernels alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [8, 100, 192, 1027, 4096, 9000])
def test_add_layernorm_kernel(dtype, hidden):
    """With and without a branch output (32-bit or of the activation type), in place and at chosen
    rows; a large common offset must not cost the variance its digits."""
    from mrun_b200.kernels import ops
    act = getattr(torch, dtype)
    gen = torch.Generator().manual_seed(hidden)
    resid = torch.randn(13, hidden, generator=gen) * 2 + 50.0
    w = 1 + 0.3 * torch.randn(hidden, generator=gen)
    for delta_dtype in (None, torch.float32, act):
        delta = None if delta_dtype is None else (torch.randn(13, hidden, generator=gen)).to(delta_dtype)
        total = resid.double() + (0 if delta is None else delta.double())
        want = plain.layer_norm(total, w.double(), 1e-5)
        stream = resid.to(DEV)
        out = torch.empty((13, hidden), dtype=act, device=DEV)
        ops.add_layernorm(stream, None if delta is None else delta.to(DEV), w.to(DEV), 1e-5, out)
        close(out, want, dtype, "all rows", bound=2e-5 if dtype == "float32" else 1e-2)
        assert torch.allclose(stream.cpu().double(), total, atol=1e-5)              # the stream advanced
        rows = torch.tensor([12, 0, 5], dtype=torch.int32)
        stream = resid.to(DEV)
        out = torch.empty((3, hidden), dtype=act, device=DEV)
        ops.add_layernorm(stream, None if delta is None else delta.to(DEV), w.to(DEV), 1e-5, out, rows=rows.to(DEV))
        close(out, want[rows.long()], dtype, "chosen rows", bound=2e-5 if dtype == "float32" else 1e-2)
        assert torch.equal(stream.cpu(), resid)                                      # and stayed where it was


@pytest.mark.parametrize("hidden", [8, 100, 1024, 5000])
def test_pair_norm_mean_kernel(hidden):
    from mrun_b200.kernels import ops
    gen = torch.Generator().manual_seed(hidden)
    a, b = torch.randn(9, hidden, generator=gen) * 3, torch.randn(9, hidden, generator=gen) * 0.01
    wa, wb = 1 + 0.3 * torch.randn(hidden, generator=gen), 0.5 * torch.randn(hidden, generator=gen)
    got = ops.pair_norm_mean(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 1e-6, 0.5)
    want = 0.5 * (plain.unit_rms(a.double(), 1e-6) * wa.double() + plain.unit_rms(b.double(), 1e-6) * wb.double())
    close(got, want, "float32", "pair norm", bound=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [8, 100, 1024, 13000])
def test_pair_norm_add_layernorm_kernel(dtype, hidden):
    """The two branch norms, their average, the residual sum and the layer norm as one kernel: the
    stream advances by the addend and the normed rows are the plain ones; at chosen rows the stream
    stays."""
    from mrun_b200.kernels import ops
    act = getattr(torch, dtype)
    gen = torch.Generator().manual_seed(hidden + 1)
    resid = torch.randn(9, hidden, generator=gen) * 2 - 20.0
    a, b = torch.randn(9, hidden, generator=gen) * 3, torch.randn(9, hidden, generator=gen) * 0.01
    wa, wb = 1 + 0.3 * torch.randn(hidden, generator=gen), 0.5 * torch.randn(hidden, generator=gen)
    w = 1 + 0.3 * torch.randn(hidden, generator=gen)
    addend = 0.5 * (plain.unit_rms(a.double(), 1e-6) * wa.double() + plain.unit_rms(b.double(), 1e-6) * wb.double())
    want = plain.layer_norm(resid.double() + addend, w.double(), 1e-5)
    pending = ops.PendingPairNorm(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 1e-6, 0.5)
    close(pending.compute(), addend, "float32", "the addend alone", bound=1e-5)
    stream = resid.to(DEV)
    out = torch.empty((9, hidden), dtype=act, device=DEV)
    ops.pair_norm_add_layernorm(stream, pending, w.to(DEV), 1e-5, out)
    close(out, want, dtype, "all rows", bound=2e-5 if dtype == "float32" else 1e-2)
    assert torch.allclose(stream.cpu().double(), resid.double() + addend, atol=1e-5)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    stream = resid.to(DEV)
    out = torch.empty((3, hidden), dtype=act, device=DEV)
    ops.pair_norm_add_layernorm(stream, pending, w.to(DEV), 1e-5, out, rows=rows.to(DEV))
    close(out, want[rows.long()], dtype, "chosen rows", bound=2e-5 if dtype == "float32" else 1e-2)
    assert torch.equal(stream.cpu(), resid)


@pytest.mark.parametrize("experts, top", [(3, 1), (8, 3), (16, 16), (40, 5), (130, 7), (300, 2)])
@pytest.mark.parametrize("bias", [False, True])
def test_route_by_logits_kernel(experts, top, bias):
    """The largest logits (bias included) are chosen and weigh the softmax over themselves only;
    the logits may be the first columns of wider rows."""
    from mrun_b200.kernels import ops
    gen = torch.Generator().manual_seed(experts * 7 + top)
    tokens = 150
    wide = torch.randn(tokens, experts + 5, generator=gen) * 3.0
    wide[0, :experts] -= 200.0                        # logits far below zero still give weights that sum to one
    wide[1, :experts] += 200.0
    b = torch.randn(experts, generator=gen) * 2.0 if bias else None
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=DEV)
    weights = ops.route_top_k(wide.to(DEV)[:, :experts], top, "logit", chosen=chosen, bias=None if b is None else b.to(DEV))
    weights, chosen = weights.cpu().double(), chosen.cpu()
    z = wide[:, :experts].float() + (b if b is not None else 0)
    for t in range(tokens):
        ranked = z[t].double().sort(descending=True)
        assert chosen[t].tolist() == ranked.indices[:top].tolist(), f"token {t}"
        dense = torch.zeros(experts, dtype=F64)
        dense[ranked.indices[:top]] = torch.softmax(ranked.values[:top], dim=0)
        assert torch.allclose(weights[t], dense, rtol=2e-5, atol=1e-7), f"token {t}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot_dims, pairing, own_values",
                         [(4, 2, 32, 32, 16, "half", False), (3, 3, 20, 12, 20, "half", True), (6, 1, 64, 64, 0, "half", False),
                          (2, 2, 24, 40, 8, "interleaved", True), (5, 1, 130, 130, 64, "half", False),
                          (3, 1, 128, 128, 64, "half", True), (2, 2, 256, 256, 256, "half", False), (4, 4, 16, 16, 16, "half", True),
                          (2, 1, 64, 64, 8, "half", True), (2, 1, 64, 64, 32, "interleaved", False)])
def test_head_norm_rope_cache_kernel(dtype, heads, kv_heads, dim, vdim, rot_dims, pairing, own_values):
    """q normed and rotated in place; the pages get the normed, rotated keys and the values: a
    projection of their own, or the keys as they came in.  Heads of 16 to 256 features in rows that
    start on 16 bytes take the kernel that moves 16 bytes a lane, the others an element a lane."""
    from mrun_b200.kernels import ops
    act = getattr(torch, dtype)
    gen = torch.Generator().manual_seed(dim)
    tokens, page = 11, 4
    nq, nk, nv = heads * dim, kv_heads * dim, kv_heads * vdim
    width = nq + nk + (nv if own_values else 0) + (8 if dim % 8 == 0 else 3)
    x = (torch.randn(tokens, width, generator=gen) * 2).to(act)
    wq, wk = 1 + 0.3 * torch.randn(dim, generator=gen), 1 + 0.3 * torch.randn(dim, generator=gen)
    positions = torch.arange(tokens) * 7
    rot = None
    if rot_dims:
        freq = 100.0 ** (-2.0 * torch.arange(rot_dims // 2, dtype=F64) / rot_dims)
        angle = positions.double()[:, None] * freq
        rot = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).float()
    slots = torch.tensor([9, 2, 40, 41, 17, -1, 0, 5, 30, 31, 22], dtype=torch.int32)
    k_cache = torch.zeros((12, kv_heads, page, dim), dtype=act, device=DEV)
    v_cache = torch.zeros((12, kv_heads, page, vdim), dtype=act, device=DEV)
    xd = x.to(DEV)
    ops.head_norm_rope_cache(xd, 0, nq, nq + nk if own_values else -1, heads, kv_heads, dim, vdim, wq.to(DEV), wk.to(DEV),
                             1e-5, None if rot is None else rot.to(DEV), rot_dims, pairing, slots.to(DEV), k_cache, v_cache, page)

    def turned(v, weight):
        y = plain.unit_rms(v.double(), 1e-5) * weight.double()
        if rot is None:
            return y
        c, s = rot[:, None, :, 0].double(), rot[:, None, :, 1].double()
        out = y.clone()
        first = slice(0, rot_dims, 2) if pairing == "interleaved" else slice(0, rot_dims // 2)
        second = slice(1, rot_dims, 2) if pairing == "interleaved" else slice(rot_dims // 2, rot_dims)
        out[..., first] = y[..., first] * c - y[..., second] * s
        out[..., second] = y[..., second] * c + y[..., first] * s
        return out
    bound = 1e-5 if dtype == "float32" else 1e-2
    close(xd[:, :nq].view(tokens, heads, dim), turned(x[:, :nq].view(tokens, heads, dim), wq), dtype, "q", bound=bound)
    assert torch.equal(xd[:, nq:].cpu(), x[:, nq:])                                   # nothing else in the rows moved
    want_k = turned(x[:, nq:nq + nk].view(tokens, kv_heads, dim), wk)
    raw_v = x[:, nq + nk:nq + nk + nv] if own_values else x[:, nq:nq + nk]
    raw_v = raw_v.reshape(tokens, kv_heads, vdim)
    flat_k = k_cache.permute(0, 2, 1, 3).reshape(-1, kv_heads, dim).cpu()
    flat_v = v_cache.permute(0, 2, 1, 3).reshape(-1, kv_heads, vdim).cpu()
    written = [int(s) for s in slots if s >= 0]
    rows = [i for i, s in enumerate(slots.tolist()) if s >= 0]
    close(flat_k[written], want_k[rows], dtype, "keys in the pages", bound=bound)
    assert torch.equal(flat_v[written], raw_v[rows])                                  # values are copied, never rounded again
    untouched = sorted(set(range(12 * page)) - set(written))
    assert not flat_k[untouched].any() and not flat_v[untouched].any()


# ------------------------------------------------------------------ specs and entries of the mixers

def attention_spec(hidden, heads, kv_heads, dim, vdim, size, rot_dims, scaling=None, chunked=False, keys=False, scale=0.3):
    from mrun_b200.config.spec import GatedAttentionSpec, ScaledRotarySpec
    position = ScaledRotarySpec(dims=rot_dims, base=300.0, pairing="half", scaling=scaling) if rot_dims else None
    return GatedAttentionSpec(hidden=hidden, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, softmax_scale=scale, eps=1e-5,
                              qk_norm="head", sink=True, head_gate=False, position=position,
                              window=None if chunked else size, chunk=size if chunked else None,
                              values="keys" if keys else "projection")


def attention_entry(heads, kv_heads, dim, vdim, size, rot_dims, scaling=None, scale=0.3):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": 300.0}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def latent_spec(hidden, heads, dim, rot_dim, vdim, kv_rank, size, scale=0.2):
    from mrun_b200.config.spec import LatentAttentionSpec, ScaledRotarySpec
    position = ScaledRotarySpec(dims=rot_dim, base=300.0, pairing="half") if rot_dim else None
    return LatentAttentionSpec(hidden=hidden, heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=0, kv_rank=kv_rank,
                               softmax_scale=scale, eps=1e-5, position=position, window=size)


def latent_entry(heads, dim, rot_dim, vdim, kv_rank, size, scale=0.2):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "mask": {"size": size}}
    if rot_dim:
        m["rot"] = {"dims": rot_dim, "base": 300.0}
    return m


def delta_spec(hidden, heads, kv_heads, dim, vdim, conv, decay_rank=4, gate_rank=3):
    from mrun_b200.config.spec import ChannelDeltaSpec
    return ChannelDeltaSpec(hidden=hidden, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, decay_rank=decay_rank,
                            gate_rank=gate_rank, eps=1e-5)


ATTENTION_SHAPES = [  # heads, kv heads, key size, value size, window or chunk, rotating features, stretch, page size
    (6, 3, 24, 48, 30, 8, (4.0, 64, 8.0, 1.0), 16),
    (5, 5, 20, 20, 1, 0, None, 8),
    (4, 1, 12, 12, 7, 12, None, 4),
    (4, 2, 64, 64, 37, 32, (8.0, 128, 16.0, 2.0), 16),      # bfloat16: the tensor-core kernels at 64
    (3, 1, 128, 128, 50, 64, None, 16),                     # the same at 128
    (2, 2, 80, 80, 16, 40, None, 8),
    (34, 2, 16, 16, 9, 4, None, 16),                        # seventeen query heads a kv head
    (4, 4, 32, 32, 1000, 16, None, 8),                      # longer than every request
]


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("chunked, keys", [(False, False), (True, True), (True, False)])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, size, rot_dims, scaling, page", ATTENTION_SHAPES)
def test_attention_alone(dtype, tensor_cores, chunked, keys, heads, kv_heads, dim, vdim, size, rot_dims, scaling, page, monkeypatch):
    """A sliding window with values of their own, a chunked mask with the unnormed keys as values,
    and a chunked mask with values of their own, on the CUDA-core and the tensor-core kernels."""
    from mrun_b200.parts import MIXERS, gated_attention
    monkeypatch.setattr(gated_attention, "TENSOR_CORES", tensor_cores)
    if keys and vdim != dim:
        pytest.skip("values that are the keys have the keys' size")
    rt = runtime(dtype, page)
    spec = attention_spec(40, heads, kv_heads, dim, vdim, size, rot_dims, scaling, chunked=chunked, keys=keys)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", torch.Generator().manual_seed(dim + vdim + size))
    assert ("v" in w) == (not keys) and w["q.norm"].shape == (dim,)
    part = MIXERS.build(spec, w, rt)
    if tensor_cores and not part.tensor_cores:
        pytest.skip("the tensor-core kernels do not take this shape")
    W = named(w, "m.")
    m = attention_entry(heads, kv_heads, dim, vdim, size, rot_dims, scaling)
    need = part.cache_need()
    assert need.window == size and (need.value_dim or dim) == vdim

    def fn(h, _):
        return plain.softmax_attention(m, W, "m.", h, 1e-5, torch.arange(h.shape[0]), values_are_keys=keys, chunked=chunked)
    check_rows(lambda rows, ctx, caches: part.forward(rows, ctx, caches[0]), 40, dtype, LENGTHS, fn, [need], rt)


LATENT_SHAPES = [  # heads, plain size, rotated size, value size, latent size, window, page size
    (3, 24, 8, 20, 40, 20, 16),
    (2, 10, 6, 14, 270, 9, 8),          # a row wider than 256 features: the CUDA-core kernel
    (4, 32, 16, 32, 48, 45, 4),         # bfloat16: a row of 64 features on the tensor-core kernels
    (5, 16, 0, 8, 32, 100000, 16),      # no rotated part, a window longer than every request
    (20, 16, 16, 24, 112, 33, 16),      # twenty query heads over the one latent row
    (2, 64, 32, 64, 96, 1, 8),          # a window of one position
    (3, 48, 16, 40, 128, 27, 16),       # a row of 144 features
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, rot_dim, vdim, kv_rank, size, page", LATENT_SHAPES)
def test_latent_attention_alone(dtype, heads, dim, rot_dim, vdim, kv_rank, size, page):
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype, page)
    spec = latent_spec(40, heads, dim, rot_dim, vdim, kv_rank, size)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", torch.Generator().manual_seed(dim + kv_rank))
    assert "dq" not in w and w["q"].shape == (heads * (dim + rot_dim), 40)
    part = MIXERS.build(spec, w, rt)
    W = named(w, "m.")
    m = latent_entry(heads, dim, rot_dim, vdim, kv_rank, size)
    assert part.cache_need().window == size
    check_rows(lambda rows, ctx, caches: part.forward(rows, ctx, caches[0]), 40, dtype, LENGTHS,
               lambda h, _: plain.latent_attention(m, W, "m.", h, 1e-5, torch.arange(h.shape[0])), [part.cache_need()], rt)


DELTA_SHAPES = [(4, 2, 16, 24, 4), (1, 1, 72, 33, 1), (5, 5, 10, 7, 2), (2, 1, 160, 16, 3), (2, 2, 128, 128, 3)]


def delta_weights(spec, prefix, gen):
    from mrun_b200.parts import MIXERS
    w = random_tensors(MIXERS.tensor_specs(spec, prefix), prefix, gen)
    w["A_log"] = (torch.rand(w["A_log"].shape, generator=gen) * 3 - 3).to(torch.bfloat16).float()
    w["dt_bias"] = (w["dt_bias"] * 6).to(torch.bfloat16).float()          # decays from near 0 to near 1
    return w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, conv", DELTA_SHAPES)
def test_delta_rule_alone(dtype, heads, kv_heads, dim, vdim, conv):
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype)
    spec = delta_spec(48, heads, kv_heads, dim, vdim, conv)
    w = delta_weights(spec, "m", torch.Generator().manual_seed(heads + dim))
    part = MIXERS.build(spec, w, rt)
    W = named(w, "m.")
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim}
    check_rows(lambda rows, ctx, caches: part.forward(rows, ctx, caches[0]), 48, dtype, LENGTHS,
               lambda h, _: plain.delta_rule(m, W, "m.", h, 1e-5), [part.cache_need()], rt)


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("left, right, page", [((4, 2, 32, 32, 24, 16, None), (4, 2, 16, 24, 4), 16),
                                               ((3, 1, 12, 12, 1, 12, None), (1, 1, 72, 33, 1), 8),
                                               ((2, 1, 128, 128, 50, 64, None), (2, 2, 32, 16, 3), 4),
                                               ((4, 2, 64, 64, 33, 16, (2.0, 32, 4.0, 1.0)), (3, 1, 8, 12, 2), 16)])
def test_parallel_mixer_alone(dtype, tensor_cores, left, right, page, monkeypatch):
    """Both sides read the same rows; the pages of the left and the two states of the right belong
    to one schedule entry; each output is normed over the width before the two are averaged."""
    from mrun_b200.cache.needs import split_need
    from mrun_b200.config.spec import ParallelMixerSpec
    from mrun_b200.parts import MIXERS, gated_attention
    monkeypatch.setattr(gated_attention, "TENSOR_CORES", tensor_cores)
    rt = runtime(dtype, page)
    hidden = 56
    spec = ParallelMixerSpec(hidden=hidden, left=attention_spec(hidden, *left, chunked=True, keys=True),
                             right=delta_spec(hidden, *right), eps=1e-5)
    gen = torch.Generator().manual_seed(left[2] + right[2])
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", gen)
    w.update({f"right.{k}": v for k, v in delta_weights(spec.right, "m.right", gen).items() if k in ("A_log", "dt_bias")})
    w["right.o"] = w["right.o"] * 0.01                  # sides of very different sizes: the norms make them equal partners
    part = MIXERS.build(spec, w, rt)
    if tensor_cores and not part.sides[0][0].tensor_cores:
        pytest.skip("the tensor-core kernels do not take this shape")
    paged, states = split_need(part.cache_need())
    assert paged.window == left[4] and sorted(s.name for s in states) == ["conv", "state"]
    W = named(w, "m.")
    m = {"left": attention_entry(*left), "right": dict(zip(("heads", "kv_heads", "dim", "vdim", "conv"), right))}

    def fn(h, _):
        full = plain.parallel_mixer(m, W, "m.", h, 1e-5, torch.arange(h.shape[0]))
        # each side contributes about half of the result
        lone = 0.5 * plain.unit_rms(plain.delta_rule(m["right"], W, "m.right.", h, 1e-5), 1e-5) * W["m.right.out"]
        assert 0.2 < float(lone.norm() / full.norm()) < 5.0
        return full
    check_rows(lambda rows, ctx, caches: part.forward(rows, ctx, caches[0]), hidden, dtype, LENGTHS, fn, [part.cache_need()], rt)
    # left pending for the layer norm behind it: the branch norms, the average, the sum into a stream
    # of zeros and the norm are one kernel
    from mrun_b200.config.spec import LayerNormSpec
    from mrun_b200.kernels import ops
    from mrun_b200.parts import NORMS
    norm_weight = (1 + 0.2 * torch.randn(hidden, generator=gen)).to(torch.bfloat16).float()
    norm = NORMS.build(LayerNormSpec(hidden, 1e-5, bare=True), {"": norm_weight}, rt)

    def through_norm(rows, ctx, caches):
        pending = part.forward(rows, ctx, caches[0], defer_output=True)
        assert isinstance(pending, ops.PendingPairNorm)
        return norm.add_forward(torch.zeros((rows.shape[0], hidden), dtype=torch.float32, device=DEV), pending)
    check_rows(through_norm, hidden, dtype, LENGTHS, lambda h, _: plain.layer_norm(fn(h, _), norm_weight.double(), 1e-5),
               [part.cache_need()], rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden, ff, limit", [(40, 48, 1.5), (100, 90, 0.25), (64, 256, 30.0)])
def test_clamped_dense_feed_forward_alone(dtype, hidden, ff, limit):
    from mrun_b200.config.spec import ClampedGatedMLPSpec
    from mrun_b200.parts import FEED_FORWARDS
    rt = runtime(dtype)
    spec = ClampedGatedMLPSpec(hidden=hidden, intermediate=ff, limit=limit)
    w = random_tensors(FEED_FORWARDS.tensor_specs(spec, "f"), "f", torch.Generator().manual_seed(ff), std=0.4)
    part = FEED_FORWARDS.build(spec, w, rt)
    W = named(w, "f.")
    gen = torch.Generator().manual_seed(1)
    x = (torch.randn(70, hidden, generator=gen) * 2).to(rt.precision.act)
    want = plain.dense_feed_forward({"limit": limit}, W, "f.", x.double())
    g = x.double() @ W["f.gate"].T + W["f.gate.b"]
    assert limit > 10 or (bool((g > limit).any()) and bool((g < -limit).any()))       # both sides of the clamp are met
    for rows in (70, 3):                                                              # the vendor product and the decode product
        close(part.forward(x[:rows].to(DEV), None), want[:rows], dtype, f"{rows} rows")


@pytest.mark.parametrize("dtype, sorted_experts", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("hidden, experts, top, ff", [(40, 8, 3, 24), (48, 3, 1, 16), (64, 40, 5, 8), (32, 4, 4, 16)])
def test_routed_feed_forward_alone(dtype, sorted_experts, hidden, experts, top, ff, monkeypatch):
    """Rows alone against rows in a batch, the chosen experts only against every expert with zero
    weights; the router's logits are spread so that no choice is a close call."""
    from mrun_b200.config.spec import GroupedRoutedMLPSpec
    from mrun_b200.engine.batch import StepContext
    from mrun_b200.parts import FEED_FORWARDS, routed
    monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 0.0 if sorted_experts else 1e30)
    rt = runtime(dtype)
    spec = GroupedRoutedMLPSpec(hidden=hidden, experts=experts, top=top, expert_ff=ff, score="logit", router_bias=True)
    gen = torch.Generator().manual_seed(experts + ff)
    w = random_tensors(FEED_FORWARDS.tensor_specs(spec, "f"), "f", gen, std=0.3)
    w["router"] = (w["router"] * 4).to(torch.bfloat16).float()
    w["router.b"] = (torch.randn(experts, generator=gen) * 2).to(torch.bfloat16).float()
    part = FEED_FORWARDS.build(spec, w, rt)
    W = named(w, "f.")
    x = torch.randn(90, hidden, generator=gen).to(rt.precision.act)
    margins = []
    want = plain.routed_feed_forward({"router": {"experts": experts, "top": top}}, W, "f.", x.double(), margins)
    sure = margins[0] > (1e-4 if dtype == "float32" else 0.15)
    assert int(sure.sum()) > 40
    got = part.forward(x.to(DEV), None)
    got = (got.compute() if hasattr(got, "compute") else got).float().cpu()
    close(got[sure], want[sure], dtype, "a batch of rows")
    for t in [i for i in range(90) if sure[i]][:5]:
        one = part.forward(x[t:t + 1].to(DEV), None)
        one = (one.compute() if hasattr(one, "compute") else one).float().cpu()
        close(one, want[t:t + 1], dtype, f"row {t} alone", bound=3e-5 * float(want.abs().max() / want[t].abs().max())
              if dtype == "float32" else 3e-2 * float(want.abs().max() / want[t].abs().max()))


# ------------------------------------------------------------------ one key decides

def run_cut(part, rt, x, portions, pages):
    """Feeds the rows ``x`` of one request in ``portions`` through a mixer alone: float32 rows."""
    book = Steps([part.cache_need()], rt, pages=pages, slots=1)
    got, at = [], 0
    for n in portions:
        def run(ctx, places):
            return part.forward(x[at:at + n].to(DEV, rt.precision.act), ctx, book.caches[0]).float().cpu()
        got.append(book.run([("r", [0] * n)], run))
        at += n
    book.release("r")
    return torch.cat(got)


def edge_cuts(total, edge):
    """Whole; a prompt up to just before the edge, the tokens around it decoded alone, the rest as
    one portion; portions of two and three tokens across it."""
    alone = [1] * 6
    small = [2, 3] * ((total // 5) + 1)
    cut, at = [], 0
    for n in small:
        n = min(n, total - at)
        if n:
            cut.append(n); at += n
    return [[total], [edge - 3] + alone + [total - edge - 3], cut]


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("dim, size, page", [(16, 21, 8), (64, 37, 16), (128, 64, 16), (20, 16, 4)])
def test_one_key_at_the_edge_of_a_window_or_chunk_and_the_sink(dtype, tensor_cores, chunked, dim, size, page, monkeypatch):
    """One key and the queries that look for it are made so that its score dominates a head: at the
    first token, on both sides of a page border and far into the request.  A query on the last
    position that still sees it (the window's last, the chunk's last) takes its value; the query one
    position further on does not, and both are asked from inside a prompt portion, by tokens
    decoded alone and from portions of two and three tokens.  Then queries that score far below
    zero against every key: the sink takes the weight and the output all but vanishes."""
    from mrun_b200.parts import MIXERS, gated_attention
    monkeypatch.setattr(gated_attention, "TENSOR_CORES", tensor_cores)
    rt = runtime(dtype, page)
    hidden, heads = 32, 2
    spec = attention_spec(hidden, heads, 1, dim, dim, size, 8, chunked=chunked, keys=chunked, scale=0.5)
    gen = torch.Generator().manual_seed(17 + dim)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", gen, std=0.1)
    # the last (unrotated) feature of both heads' queries reads input column 1 alone, the key's reads
    # column 0 alone, and the norms weigh that feature: it carries the score
    w["q"][:, :2] = 0; w["k"][:, :2] = 0
    for row in (dim - 1, 2 * dim - 1):
        w["q"][row] = 0; w["q"][row, 1] = 1
    w["k"][dim - 1] = 0; w["k"][dim - 1, 0] = 1
    w["q.norm"][dim - 1] = 3.0
    w["k.norm"][dim - 1] = 3.0
    part = MIXERS.build(spec, w, rt)
    if tensor_cores and not part.tensor_cores:
        pytest.skip("the tensor-core kernels do not take this shape")
    W = named(w, "m.")
    m = attention_entry(heads, 1, dim, dim, size, 8, scale=0.5)
    total = 6 * size + 40

    def reference(x):
        h = x.to(rt.precision.act).double()
        return plain.softmax_attention(m, W, "m.", h, 1e-5, torch.arange(total), values_are_keys=chunked, chunked=chunked)
    starts = [0, page - 1, page, 4 * size + 3] if not chunked else [0, size, 2 * size + size // 2, 4 * size + 1]
    for far in starts:
        last_seen = (far // size + 1) * size - 1 if chunked else far + size - 1
        x = torch.randn(total, hidden, generator=gen) * 0.5
        x[:, 0] = 0; x[:, 1] = 0
        x[far, 0] = 30.0                                    # the key
        inside = sorted({min(far + 1, last_seen), last_seen})
        outside = [last_seen + 1, last_seen + 2]
        x[inside + outside, 1] = 30.0
        want = reference(x)
        lost = x.clone(); lost[far, 0] = 0
        blind = reference(lost)
        change = (want - blind).abs().max(1).values / want.abs().max()
        assert float(change[inside].min()) > 0.2, "the plain run does not depend on the key where it should"
        assert float(change[outside].max()) == 0.0, "the plain run sees the key where it should not"
        for portions in edge_cuts(total, last_seen + 1):
            got = run_cut(part, rt, x, portions, pages=-(-total // page) + 2)
            what = f"key at {far}, last seen at {last_seen}, portions {portions[:8]}"
            close(got[inside + outside], want[inside + outside], dtype, what + ": the queries at the edge")
            close(got, want, dtype, what + ": all tokens")
    # the sink: every key leans the same way on the feature that carries the score, and some queries
    # lean the other way, so that all their scores lie far below zero
    x = torch.randn(total, hidden, generator=gen) * 0.5
    x[:, 0] = 0.3; x[:, 1] = 0
    deniers = [0, 1, size, 2 * size + 5, total - 4, total - 1]
    x[deniers, 1] = -30.0
    want = reference(x)
    assert float(want[deniers].abs().max() / want.abs().max()) < 1e-3
    for portions in ([total], [total - 6] + [1] * 6, edge_cuts(total, size)[2]):
        got = run_cut(part, rt, x, portions, pages=-(-total // page) + 2)
        close(got, want, dtype, f"the sink, portions {portions[:8]}")
        assert float(got[deniers].abs().max() / want.abs().max()) < (1e-3 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim, rot_dim, kv_rank, size, page", [(16, 8, 40, 21, 8), (32, 16, 48, 37, 16), (24, 8, 264, 16, 4)])
def test_latent_attention_one_key_at_the_edge_of_the_window(dtype, dim, rot_dim, kv_rank, size, page):
    """The same for the attention over the latent: one latent channel carries the key, the heads'
    key up-projection passes it to their last plain feature, and the queries that look for it are
    large on that feature."""
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype, page)
    hidden, heads, vdim = 32, 2, 12
    spec = latent_spec(hidden, heads, dim, rot_dim, vdim, kv_rank, size, scale=0.5)
    gen = torch.Generator().manual_seed(5 + dim)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", gen, std=0.1)
    w["q"][:, :2] = 0; w["dkv"][:, :2] = 0
    w["dkv"][kv_rank - 1] = 0; w["dkv"][kv_rank - 1, 0] = 1           # the last latent channel reads column 0 alone
    w["dkv.norm"][kv_rank - 1] = 2.0
    uk = w["uk"].view(heads, dim, kv_rank)
    uq = w["q"].view(heads, dim + rot_dim, hidden)
    for h in range(heads):
        uk[h, dim - 1] = 0; uk[h, dim - 1, kv_rank - 1] = 1           # and reaches the head's last plain key feature
        uk[h, :dim - 1, kv_rank - 1] = 0
        uq[h, dim - 1] = 0; uq[h, dim - 1, 1] = 1                     # which the query's column 1 meets
    part = MIXERS.build(spec, w, rt)
    W = named(w, "m.")
    m = latent_entry(heads, dim, rot_dim, vdim, kv_rank, size, scale=0.5)
    total = 5 * size + 30

    def reference(x):
        return plain.latent_attention(m, W, "m.", x.to(rt.precision.act).double(), 1e-5, torch.arange(total))
    for far in (0, page - 1, page, 3 * size + 2):
        last_seen = far + size - 1
        x = torch.randn(total, hidden, generator=gen) * 0.5
        x[:, 0] = 0; x[:, 1] = 0
        x[far, 0] = 30.0
        inside, outside = sorted({far + 1, last_seen}), [last_seen + 1, last_seen + 2]
        x[inside + outside, 1] = 8.0
        want = reference(x)
        lost = x.clone(); lost[far, 0] = 0
        change = (want - reference(lost)).abs().max(1).values / want.abs().max()
        assert float(change[inside].min()) > 0.2 and float(change[outside].max()) == 0.0
        for portions in edge_cuts(total, last_seen + 1):
            got = run_cut(part, rt, x, portions, pages=-(-total // page) + 2)
            what = f"key at {far}, last seen at {last_seen}, portions {portions[:8]}"
            close(got[inside + outside], want[inside + outside], dtype, what + ": the queries at the edge")
            close(got, want, dtype, what + ": all tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_delta_rule_keeps_a_far_key_by_channel_and_overwrites_it(dtype):
    """Key channel 0 of head 0 never decays, channel 1 decays at once.  A key written into both
    early in the prompt still answers a query on channel 0 hundreds of tokens later (in the prompt,
    in a later portion and decoded alone) and is gone for a query on channel 1."""
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype)
    hidden, heads, dim, vdim = 32, 2, 16, 24
    spec = delta_spec(hidden, heads, heads, dim, vdim, 1, decay_rank=2, gate_rank=2)
    gen = torch.Generator().manual_seed(23)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", gen, std=0.05)
    for name in ("q.conv", "k.conv", "v.conv"):
        w[name] = torch.ones_like(w[name])              # one tap of weight 1: the projections pass through SiLU only
    w["a1"].zero_(); w["a2"].zero_()
    w["A_log"] = torch.zeros(heads)
    w["dt_bias"] = torch.full((heads * dim,), -3.0)     # softplus(-3) = 0.049: a slow decay everywhere else
    w["dt_bias"][0] = -60.0                             # no decay at all in 32-bit
    w["dt_bias"][1] = 60.0                              # gone after one token
    w["b"].zero_()                                      # beta = 1/2
    for name, row, column in (("k", 0, 0), ("k", 1, 0), ("q", 0, 1), ("q", 1, 2)):
        w[name][row] = 0; w[name][row, column] = 1      # both channels' keys read column 0; the queries columns 1 and 2
    w["k"][2:, 0] = 0; w["q"][2:, 1:3] = 0
    w["k"][:, 1:3] = 0; w["q"][:, 0] = 0
    w["v"][:, :3] = 0; w["g1"][:, :3] = 0; w["b"][:, :3] = 0
    part = MIXERS.build(spec, w, rt)
    W = named(w, "m.")
    m = {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": vdim}
    total = 420
    x = torch.randn(total, hidden, generator=gen) * 0.3
    x[:, :3] = 0
    x[5, 0] = 8.0                                       # the key, into channels 0 and 1 of head 0
    keepers, forgetters = [6, 130, 300, 401, 419], [7, 131, 402]
    x[keepers, 1] = 8.0
    x[forgetters, 2] = 8.0
    x = x.to(rt.precision.act).float()
    want = plain.delta_rule(m, W, "m.", x.double(), 1e-5)
    lost = x.clone(); lost[5, 0] = 0
    change = (want - plain.delta_rule(m, W, "m.", lost.double(), 1e-5)).abs().max(1).values / want.abs().max()
    # (the lost key's other channels grow to unit length, which the slow channels carry on for a while)
    assert float(change[keepers].min()) > 0.1 and float(change[forgetters].max()) < 1e-2
    for portions in ([400] + [1] * 20, [3, 2, 2, 100, 193, 100] + [1] * 20):
        got = run_cut(part, rt, x, portions, pages=8)
        close(got[keepers], want[keepers], dtype, "queries on the kept channel")
        close(got, want, dtype, "all tokens")


# ------------------------------------------------------------------ whole models

@pytest.fixture(scope="module", params=sorted(NTINY))
def ntiny(request, tmp_path_factory):
    name = request.param
    return name, make_folder(name, str(tmp_path_factory.mktemp(f"nisotar_{name}"))), NTINY[name]


def close_calls(margins, count):
    """[count] flags: the position's own choice of experts is within CLOSE_CALL of another one, or
    an earlier position of the sequence chose within FLIP_CALL (keys, values and states made after
    another choice there reach every later position)."""
    gap = np.full(count, np.inf)
    for m in margins:
        gap = np.minimum(gap, m.numpy())
    return (gap < CLOSE_CALL) | (np.minimum.accumulate(gap) < FLIP_CALL)


def plain_logits(cfg, weights, tokens):
    margins = []
    logits = plain.forward(cfg, weights, tokens, margins=margins).to(torch.float32).numpy()
    return logits, close_calls(margins, len(tokens))


def test_layers_of_the_plain_run_and_the_engine_agree(ntiny):
    """The engine's 32-bit residual stream after every layer is the plain run's, and the plain
    run's last layer, normed and projected, gives its logits."""
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.loading import executor_from_folder
    from mrun_b200.kernels import ops
    name, folder, settings = ntiny
    cfg, weights = load_folder(folder)
    tokens = tokens_of(cfg["vocab"], 41, seed=4)
    logits, layers = plain.forward(cfg, weights, tokens, want_layers=True)
    assert layers.shape == (len(cfg["layers"]), 41, cfg["width"])
    W = plain.as_double(weights)
    assert torch.allclose(plain.layer_norm(layers[-1], W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T, logits)
    ex = executor_from_folder(folder, dtype="float32", page_size=settings["page_size"], num_pages=32, max_requests=1)
    seen = []
    for block in ex.model.blocks:
        def forward(resid, delta, ctx, cache, inner=block.forward):
            out = inner(resid, delta, ctx, cache)
            pending = out.compute() if isinstance(out, ops.PENDING) else out
            seen.append((resid + pending.float()).cpu().double())
            return out
        block.forward = forward
    request = ex.admit("r")
    got = ex.step([StepEntry(request, tokens, list(range(41)))]).cpu().double()
    for i, layer in enumerate(seen):
        error = float((layer - layers[i]).abs().max() / layers[i].abs().max())
        assert error < 2e-5, f"{name}: after layer {i} ({cfg['layers'][i]['type']}): {error:.3e}"
    assert float((got - logits).abs().max() / logits.abs().max()) < 2e-5


@pytest.mark.parametrize("dtype, sorted_experts, tensor_cores", [("float32", False, False), ("bfloat16", False, False),
                                                                ("bfloat16", True, True)])
def test_every_cutting_matches_plain(ntiny, dtype, sorted_experts, tensor_cores, tmp_path, monkeypatch):
    """Whole prompts, a prefix and then token by token (long where the pool allows), portions of
    changing size down to one and two tokens, and up to four requests side by side in a pool so
    small that pages and state slots are used again."""
    name, folder, settings = ntiny
    cfg, weights = load_folder(folder)
    vocab = cfg["vocab"]
    requests = {f"r{i}": tokens_of(vocab, n, seed=200 + i) for i, n in enumerate(TRACE_LENGTHS)}
    both = {rid: plain_logits(cfg, weights, tokens) for rid, tokens in requests.items()}
    want = {rid: logits for rid, (logits, _) in both.items()}
    unsure = {rid: flags for rid, (_, flags) in both.items()}
    if name == "R":                                    # every expert of every layer is chosen: nothing is left out
        assert not any(bool(f.any()) for f in unsure.values())
    cuts = {}
    b = TraceBuilder()
    def section(label):
        cuts[label] = len(b.where)
    section("whole")
    for rid in ("r0", "r1", "r3", "r5"):
        cut_whole(b, rid, requests[rid])
    section("decode_tail")
    cut_decode_tail(b, "r0", requests["r0"])
    cut_decode_tail(b, "r7", requests["r7"], tail=2)
    cut_decode_tail(b, "r5", requests["r5"], tail=200 if name == "P" else 40)          # long decoding
    section("portions")
    for k, rid in enumerate(("r2", "r4", "r5", "r3")):
        cut_portions(b, rid, requests[rid], SIZES[k:] + SIZES[:k])
    section("mixed")
    cut_mixed(b, requests, SIZES, live=4, seed=6)
    section("end")
    rounded = sorted((-(-n // 64) * 64 for n in TRACE_LENGTHS), reverse=True)
    monkeypatch.setenv("MRUN_MOE_SORT_MIN_FLOPS", "0" if sorted_experts else "1e30")
    monkeypatch.setenv("MRUN_GATED_ATTENTION_TENSOR_CORES", "1" if tensor_cores else "0")
    runner = TraceRunner(folder, dtype, str(tmp_path / "out"), sum(rounded[:4]), settings["page_size"], max_requests=4)
    try:
        runner.run(b.steps)
    finally:
        assert runner.close() == 0
    scale = max(float(np.max(np.abs(w))) for w in want.values())
    bound = 2e-5 if dtype == "float32" else 4e-2
    files, worst, first_seen, compared, over, every = {}, {}, {}, {}, {}, {}
    labels = list(cuts)
    for index, (step, row, rid, position) in enumerate(b.where):
        if step not in files:
            files[step] = runner.logits(step, vocab)
        got = files[step][row]
        if dtype == "float32":
            seen = first_seen.setdefault((rid, position), (got, step))
            assert np.array_equal(seen[0], got), (f"{name}: request {rid}, position {position}: steps {seen[1]} and "
                                                  f"{step} differ in bits")
        error = float(np.max(np.abs(got - want[rid][position]))) / scale
        label = [l for l in labels[:-1] if cuts[l] <= index][-1]
        every.setdefault(label, []).append(error)
        if dtype == "bfloat16" and unsure[rid][position]:
            continue
        compared[label] = compared.get(label, 0) + 1
        if error > bound:
            over[label] = over.get(label, 0) + 1
        if error > worst.get(label, (0.0,))[0]:
            worst[label] = (error, step, rid, position)
    print(name, dtype, {k: f"{v[0]:.2e}" for k, v in worst.items()}, over)
    # A bfloat16 run may leave the bound at a few ill-conditioned positions (the first tokens of a
    # request, where the delta rule's read-out is all but zero before its norm takes the size
    # away): two, or one in fifty of a section, and never by more than three times.  32-bit: none.
    for label, (error, step, rid, position) in worst.items():
        where = f"{name}/{dtype}/{label}: error {error:.3e} at step {step}, request {rid}, position {position}"
        assert error <= (bound if dtype == "float32" else 3 * bound), where
        few = 0 if dtype == "float32" else max(2, compared[label] // 50)
        assert over.get(label, 0) <= few, f"{where}; {over[label]} of {compared[label]} over {bound}"
    # Positions at or after a close call of a router are not held to the bound one by one, but a
    # fault of the cache, the state or the batch would move most of them
    for label, errors in every.items():
        within = sum(e <= bound for e in errors)
        assert within >= 0.8 * len(errors), f"{name}/{dtype}/{label}: only {within} of {len(errors)} positions within {bound}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(ntiny, dtype):
    """Greedy generation through ``Engine.generate``: the scheduler cuts prompts into portions of
    seven tokens beside decoded tokens of other requests, with four state slots for five requests."""
    from mrun_b200 import Engine
    name, folder, settings = ntiny
    cfg, weights = load_folder(folder)
    prompts = [tokens_of(cfg["vocab"], n, seed=300 + n) for n in (1, 9, 40, 71, 5)]
    engine = Engine.from_folder(folder, dtype=dtype, page_size=settings["page_size"], context=512,
                                max_batch_tokens=7, max_requests=4)
    results = engine.generate(prompts, max_tokens=10, ignore_eos=True)
    assert bool(engine.executor._graphs) == engine.executor.model.graph_safe
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and len(result.tokens) == 10
        tokens = list(prompt)
        for n, token in enumerate(result.tokens):
            margins = []
            logits = plain.forward(cfg, weights, tokens, margins=margins)[-1]
            best = int(torch.argmax(logits))
            margin = 1e-3 if dtype == "float32" else 2 * 4e-2 * float(logits.abs().max())
            unsure = dtype == "bfloat16" and bool(close_calls(margins, len(tokens))[-1])
            assert token == best or unsure or float(logits[best] - logits[token]) < margin, \
                f"{name}: output token {n}: engine {token}, plain {best}, behind by {float(logits[best] - logits[token]):.4f}"
            tokens.append(token)
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live


def test_command_line_random_then_run(tmp_path):
    """``mrun random`` writes a Nisotar folder from its config.json (the low-rank projections' inner
    sizes from the rank keys), ``mrun run`` reads them back from the checkpoint and generates."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
    mrun = os.path.join(root, "bin", "mrun")
    run = lambda *args: subprocess.run([sys.executable, mrun, *args], capture_output=True, text=True, timeout=600)
    (tmp_path / "cfg.json").write_text(json.dumps(NTINY["T"]["config"]))
    folder = str(tmp_path / "model")
    made = run("random", folder, "--config", str(tmp_path / "cfg.json"), "--seed", "21", "--std", "0.1")
    assert made.returncode == 0, made.stderr
    cfg, weights = load_folder(folder)
    for entry in cfg["layers"]:                        # the sizes are read from the checkpoint's shapes from here on
        if entry["type"] == "parallel":
            entry["mixer"]["right"].pop("decay_rank"); entry["mixer"]["right"].pop("gate_rank")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    prompt = tokens_of(cfg["vocab"], 19, seed=8)
    result = run("run", folder, "--prompt", ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32",
                 "--ignore-eos", "--context", "1K")
    assert result.returncode == 0, result.stderr
    tokens = list(prompt)
    for token in (int(t) for t in result.stdout.strip().split(",")):
        logits = plain.forward(cfg, weights, tokens)[-1]
        best = int(torch.argmax(logits))
        assert token == best or float(logits[best] - logits[token]) < 1e-3
        tokens.append(token)
    assert len(tokens) == 19 + 6 and "Nisotar" in result.stderr


# ------------------------------------------------------------------ layer sizes of a real model

REAL_MOE = {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": 512}}
REAL_SIZES = {"architecture": "Nisotar", "vocab": 4096, "width": 1024, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
              "layers": [{"type": "latent_attention", "mlp": {"kind": "dense", "ff": 2048, "limit": 7.0},
                          "mixer": {"heads": 8, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 192, "scale": 192 ** -0.5,
                                    "mask": {"size": 128}, "rot": {"base": 10000.0, "dims": 64}}},
                         {"type": "parallel", "mlp": REAL_MOE,
                          "mixer": {"left": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                             "mask": {"size": 96}, "rot": {"base": 500000.0, "dims": 64}},
                                    "right": {"heads": 8, "kv_heads": 4, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64,
                                              "gate_rank": 64}}},
                         {"type": "attention", "mlp": REAL_MOE,
                          "mixer": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 200},
                                    "rot": {"base": 10000.0, "dims": 128,
                                            "scaling": {"factor": 8.0, "original": 256, "fast": 32.0, "slow": 1.0}}}}]}


@pytest.mark.parametrize("dtype, sorted_experts, top", [("float32", False, 2), ("bfloat16", False, 8), ("bfloat16", True, 2)])
def test_real_layer_sizes(dtype, sorted_experts, top, tmp_path, monkeypatch):
    """Heads of 128 (in bfloat16 the tcgen05 and TMA attention kernels under a window and under a
    chunk, the latent row of 256 features), a width of 1,024, eight experts of 512: a prompt whole
    and in portions, then decoded token by token, against the plain model.  With two experts chosen
    a bfloat16 run is held to the bound where no choice up to the position was a close call, and
    at seven in ten of all positions; with every expert chosen at every position."""
    import copy
    from mrun_b200.config.nisotar import NisotarConfig
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.loading import executor_from_folder
    from mrun_b200.parts import routed
    from mrun_b200.weights import write_random_model
    monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 0.0 if sorted_experts else 1e30)
    sizes = copy.deepcopy(REAL_SIZES)
    for entry in sizes["layers"]:
        if entry["mlp"]["kind"] == "moe":
            entry["mlp"]["router"]["top"] = top
    folder = write_random_model(NisotarConfig.from_dict(sizes), str(tmp_path / "real"), seed=7, std=0.03, norm_noise=0.1)
    cfg, weights = load_folder(folder)
    tokens = tokens_of(cfg["vocab"], 330, seed=77)
    margins = []
    want = plain.forward(cfg, weights, tokens, margins=margins).to(torch.float32)
    sure = torch.from_numpy(~close_calls(margins, len(tokens))) if dtype == "bfloat16" else torch.ones(330, dtype=torch.bool)
    ex = executor_from_folder(folder, dtype=dtype, page_size=16, num_pages=64, max_requests=2)
    seen = {}
    for label, portions in (("whole", [330]), ("portions", [200, 3, 65, 30] + [1] * 32)):
        request, at, got = ex.admit(label), 0, []
        for n in portions:
            got.append(ex.step([StepEntry(request, tokens[at:at + n], list(range(n)))]).cpu())
            at += n
        ex.release(request)
        got = torch.cat(got)
        errors = (got - want).abs().max(1).values / want.abs().max()
        print(dtype, sorted_experts, label, f"{float(errors[sure].max()):.2e} at the {int(sure.sum())} sure positions, "
              f"{float(errors.max()):.2e} at all")
        if dtype == "float32":
            assert float(errors.max()) <= 2e-5, f"{label}: {float(errors.max()):.3e}"
            assert torch.equal(seen.setdefault("logits", got), got), "the cuttings differ in bits"
        else:
            assert int(sure.sum()) >= (5 if top == 2 else 330) and float(errors[sure].max()) <= 4e-2, f"{label}: {float(errors[sure].max()):.3e}"
            assert int((errors <= 4e-2).sum()) >= 0.7 * len(tokens), f"{label}: {int((errors <= 4e-2).sum())} of {len(tokens)} within the bound"
    ex.check()
