"""Fikudra on the GPU against the plain implementation (``plain_fikudra``): every new kernel and
every part alone (whole requests, token by token, portions down to one and two tokens, unequal
requests side by side, state slots and pages given back and used again), inputs made so that one
far key, the sink or a kept state decides the result, then whole models replayed through
``bin/trace_run`` cut in every way, then greedy generation through ``Engine.generate`` and the
command line."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_fikudra as plain
from tiny_fikudra import FTINY, load_folder, make_folder, tokens_of
from trace_tools import TraceBuilder, TraceRunner, cut_decode_tail, cut_mixed, cut_portions, cut_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def runtime(dtype, page_size=8):
    from mrun_b200.parts import Precision, Runtime
    return Runtime(torch.device(DEV), Precision.of(dtype), page_size)


def tolerance(dtype):
    return 3e-5 if dtype == "float32" else 3e-2


def close(got, want, dtype, what="", bound=None):
    got, want = got.detach().to("cpu", F64), want.to(F64)
    error = float((got - want).abs().max() / want.abs().max())
    assert error <= (bound or tolerance(dtype)), f"{what}: relative error {error:.3e}"


class Steps:
    """A cache manager for a few schedule entries' needs and step contexts for several requests."""

    def __init__(self, needs, rt, pages=96, slots=3, shares=None):
        from mrun_b200.cache import CacheManager
        from mrun_b200.engine.batch import HostStaging
        self.manager = CacheManager(list(needs), list(shares or [None] * len(needs)), rt.page_size, pages, slots,
                                    device=rt.device, dtype=rt.precision.act)
        self.staging = HostStaging(rt.device)
        self.caches = self.manager.entries
        self.requests = {}

    def run(self, entries, fn):
        """entries: [(request id, token ids)]; ``fn(ctx, places)`` runs the step, places = [(id,
        first position, first row, tokens)]; the step is committed after it."""
        from mrun_b200.engine.batch import StepEntry, build_context
        for rid, _ in entries:
            if rid not in self.requests:
                self.requests[rid] = self.manager.admit(rid)
        items = [(self.requests[rid], len(ids)) for rid, ids in entries]
        starts = [r.length for r, _ in items]
        plan = self.manager.plan_append(items)
        ctx = build_context([StepEntry(self.requests[rid], list(ids)) for rid, ids in entries], self.manager, self.staging)
        places = [(rid, start, seg.q_start, len(ids)) for (rid, ids), start, seg in zip(entries, starts, ctx.segments)]
        out = fn(ctx, places)
        self.manager.commit(plan)
        return out

    def release(self, rid):
        self.manager.release(self.requests.pop(rid))


SIZES = [2, 7, 1, 3, 16, 5, 2, 33, 9, 64, 4, 1]


def schedules(lengths):
    """Ways of feeding the same requests: (label, steps, slots); a step is [(id, tokens)]."""
    ids = list(lengths)
    out = [("whole", [[(r, lengths[r])] for r in ids], 2)]
    steps = []
    for r in ids:                               # a prefix, then token by token
        head = max(1, lengths[r] - 40)
        steps += [[(r, head)]] + [[(r, 1)] for _ in range(lengths[r] - head)]
    out.append(("token by token", steps, 2))
    steps, k = [], 0
    for r in ids:                               # portions of changing size
        at = 0
        while at < lengths[r]:
            n = min(SIZES[k % len(SIZES)], lengths[r] - at)
            k += 1
            steps.append([(r, n)])
            at += n
    out.append(("portions", steps, 2))
    # unequal requests side by side, three at a time: portions of some beside single tokens of others
    rng = np.random.default_rng(5)
    waiting, running, steps = list(ids), {}, []
    while waiting or running:
        while waiting and len(running) < 3:
            running[waiting.pop(0)] = 0
        step = []
        for r in list(running):
            left = lengths[r] - running[r]
            if rng.random() < 0.25 and len(running) > 1:
                continue
            n = 1 if left <= 6 else min(int(rng.choice(SIZES)), left - 6)
            step.append((r, n))
            running[r] += n
            if running[r] == lengths[r]:
                del running[r]
        if step:
            steps.append(step)
    out.append(("side by side", steps, 3))
    return out


LENGTHS = {"a": 75, "b": 2, "c": 140, "d": 1, "e": 37}


def check_rows(run_rows, hidden, dtype, lengths, plain_fn, needs, rt, shares=None, bound=None, ids=None, scale_of=None):
    """Feeds random inputs by every schedule to ``run_rows(rows, ctx, caches, token ids)`` and
    compares each request's rows with ``plain_fn(x, ids)`` of the whole request; in 32-bit all
    schedules must give the same bits."""
    gen = torch.Generator().manual_seed(11)
    act = rt.precision.act
    x = {r: torch.randn(n, hidden, generator=gen).to(act).to(torch.float32) for r, n in lengths.items()}
    ids = ids or {r: [0] * n for r, n in lengths.items()}
    want = {r: plain_fn(v.to(F64), ids[r]) for r, v in x.items()}
    scale = max(float(w.abs().max()) for w in want.values())
    first = {}
    for label, steps, slots in schedules(lengths):
        book = Steps(needs, rt, slots=slots, shares=shares)
        fed = {r: 0 for r in lengths}

        def run(ctx, places):
            rows = torch.cat([x[rid][start:start + n] for rid, start, _, n in places]).to(DEV, act)
            return run_rows(rows, ctx, book.caches).float().cpu()

        for step in steps:
            out = book.run([(rid, ids[rid][fed[rid]:fed[rid] + n]) for rid, n in step], run)
            at = 0
            for rid, n in step:
                got, start = out[at:at + n], fed[rid]
                error = float((got.to(F64) - want[rid][start:start + n]).abs().max()) / scale
                assert error <= (bound or tolerance(dtype)), f"{label}: request {rid}, tokens {start}..{start + n}: {error:.3e}"
                if dtype == "float32":
                    for i in range(n):
                        seen = first.setdefault((rid, start + i), got[i])
                        assert torch.equal(seen, got[i]), f"{label}: request {rid}, position {start + i} differs in bits"
                at += n
                fed[rid] += n
                if fed[rid] == lengths[rid]:
                    book.release(rid)                              # its slot and pages are used again
        book.manager.check_invariants()


def random_tensors(specs, prefix, gen, std=0.3):
    out = {}
    for t in specs:
        name = t.name[len(prefix) + 1:]
        if t.init == "norm":
            out[name] = 1 + 0.2 * torch.randn(t.shape, generator=gen)
        elif t.init == "norm_zero":
            out[name] = 0.2 * torch.randn(t.shape, generator=gen)
        else:
            out[name] = torch.randn(t.shape, generator=gen) * std
        out[name] = out[name].to(torch.bfloat16).float()           # values both precisions hold exactly
    return out


def named(w, prefix):
    return {f"{prefix}{k}": v.double() for k, v in w.items()}


# ------------------------------------------------------------------ kernels alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams, buckets, mul_prev, mul_cur, vocab, hidden",
                         [(1, 101, 7, 13, 300, 64), (3, 7, 3, 5, 90, 100), (4, 64, 1000003, 1, 70000, 24), (2, 0, 0, 0, 50, 33),
                          (8, 1, 5, 9, 20, 8)])
def test_bigram_embedding(dtype, streams, buckets, mul_prev, mul_cur, vocab, hidden):
    """The pair row of a portion's first token comes from the request's state: cut anywhere, beside
    other requests, in slots used again; a sequence's first token takes the table's last row."""
    from mrun_b200.config.spec import HashedBigramEmbeddingSpec
    from mrun_b200.parts import EMBEDDINGS
    rt = runtime(dtype)
    gen = torch.Generator().manual_seed(vocab)
    spec = HashedBigramEmbeddingSpec(vocab=vocab, hidden=hidden, scale=3.0, buckets=buckets, mul_prev=mul_prev,
                                     mul_cur=mul_cur, table_name="pairs")
    table = torch.randn(vocab, hidden, generator=gen).to(torch.bfloat16).float()
    pairs = torch.randn(buckets + 1, hidden, generator=gen).to(torch.bfloat16).float()
    part = EMBEDDINGS.build(spec, {"": rt.matrix(table), "pairs": pairs}, rt)
    cfg = {"embedding": {"scale": 3.0}}
    if buckets:
        cfg["embedding"]["bigram"] = {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}
    W = {"embed": table.double(), "bigram": pairs.double()}
    ids = {r: torch.randint(0, vocab, (n,), generator=gen).tolist() for r, n in LENGTHS.items()}
    ids["c"][:4] = [vocab - 1, vocab - 1, 0, vocab - 1]             # the largest products of the hash

    def run_rows(rows, ctx, caches):
        out = torch.empty((ctx.num_tokens, streams * hidden), dtype=torch.float32, device=DEV)
        part.forward(ctx, caches[0], out, streams)
        assert all(torch.equal(out[:, :hidden], out[:, s * hidden:(s + 1) * hidden]) for s in range(streams))
        return out[:, -hidden:]
    need = part.cache_need()
    assert (need is None) == (buckets == 0)
    from mrun_b200.cache.needs import FixedState
    check_rows(run_rows, hidden, dtype, LENGTHS, lambda x, tokens: plain.embedding(cfg, W, tokens),
               [need if need is not None else FixedState((1,), "int32", name="unused")], rt, ids=ids, bound=1e-6)


@pytest.mark.parametrize("experts, top, groups, keep", [(8, 3, 4, 2), (6, 2, 6, 3), (12, 2, 3, 1), (4, 4, 1, 1), (3, 1, 1, 1),
                                                        (64, 6, 8, 3), (5, 2, 5, 5), (10, 5, 2, 1)])
@pytest.mark.parametrize("shared", [False, True])
def test_route_grouped_kernel(experts, top, groups, keep, shared):
    from mrun_b200.kernels import ops
    gen = torch.Generator().manual_seed(experts * 7 + top)
    tokens = 200
    logits = torch.randn(tokens, experts + (1 if shared else 0), generator=gen) * 2.0
    logits[0, :experts] -= 30.0                       # scores that all but vanish still give weights that sum to the scale
    logits[1, :experts] = 30.0                        # scores that are all 1 in 32-bit: a tie, any valid choice
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=DEV)
    weights, gate = ops.route_grouped(logits.to(DEV), experts, top, groups, keep, 2, 1.75, chosen=chosen)
    router = {"experts": experts, "top": top, "scale": 1.75}
    if groups > 1 or keep != 1:
        router["groups"] = {"count": groups, "keep": keep}
    weights, chosen = weights.cpu(), chosen.cpu()
    assert (gate is not None) == shared
    if shared:
        assert torch.allclose(gate.cpu().double(), torch.sigmoid(logits[:, experts].double()), atol=1e-6)
    for t in range(tokens):
        if t == 1:
            picked = chosen[t].tolist()
            assert len(set(picked)) == top and all(0 <= e < experts for e in picked)
            assert len({e // (experts // groups) for e in picked}) <= keep
            assert float(weights[t].sum()) == pytest.approx(1.75, rel=1e-5) and int((weights[t] > 0).sum()) == top
            continue
        picks = plain.choose_experts(router, torch.sigmoid(logits[t, :experts].double()))
        assert sorted(chosen[t].tolist()) == sorted(e for e, _ in picks), f"token {t}"
        dense = torch.zeros(experts, dtype=F64)
        for e, w in picks:
            dense[e] = w
        assert torch.allclose(weights[t].double(), dense, rtol=2e-5, atol=1e-7), f"token {t}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("groups, n", [(3, 40), (2, 33), (5, 7), (8, 128), (1, 1500)])
def test_gated_norm_with_silu_gate(dtype, groups, n):
    from mrun_b200.kernels import ops
    gen = torch.Generator().manual_seed(n)
    act = getattr(torch, dtype)
    o = torch.randn(19, groups * n, generator=gen) * 3
    w = 1 + 0.3 * torch.randn(n, generator=gen)
    wide = torch.randn(19, 2 * groups * n + 8, generator=gen).to(act)
    gate = wide[:, 8:8 + groups * n]                                   # a column slice: rows are strided
    got = ops.gated_norm(o.to(DEV), w.to(DEV), wide.to(DEV)[:, 8:8 + groups * n], 1e-5, groups, act, gate_function="silu")
    g = gate.double()
    want = (plain.unit_rms(o.double().view(19, groups, n), 1e-5) * w.double()).view(19, -1) * g * torch.sigmoid(g)
    close(got, want, dtype, "gated norm", bound=1e-5 if dtype == "float32" else 1e-2)


# ------------------------------------------------------------------ mixers alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, vdim, tau, rank", [(3, 24, 40, 4.0, 8), (2, 72, 33, 16.0, 5), (1, 160, 16, 8.0, 6),
                                                         (5, 10, 7, 2.5, 3), (2, 128, 64, 1.0, 16), (4, 32, 32, 32.0, 1)])
def test_gated_linear_attention_alone(dtype, heads, dim, vdim, tau, rank):
    from mrun_b200.config.spec import GatedLinearAttentionSpec
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype)
    spec = GatedLinearAttentionSpec(hidden=48, heads=heads, dim=dim, vdim=vdim, tau=tau, rank=rank, eps=1e-5)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", torch.Generator().manual_seed(heads + dim))
    w["a2.b"] = (w["a2.b"] * 10).to(torch.bfloat16).float()            # decays from near 0 to near 1
    part = MIXERS.build(spec, w, rt)
    W = named(w, "m.")
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    check_rows(lambda rows, ctx, caches: part.forward(rows, ctx, caches[0]), 48, dtype, LENGTHS,
               lambda h, _: plain.gated_linear_attention(m, W, "m.", h, 1e-5), [part.cache_need()], rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_linear_attention_keeps_a_far_key_and_forgets_by_channel(dtype):
    """Key channel 0 never decays, channel 1 decays at once.  A key written into both early in the
    prompt must still answer a query on channel 0 hundreds of tokens later (in the prompt, in a
    later portion and in tokens decoded alone), and must be gone for a query on channel 1."""
    from mrun_b200.config.spec import GatedLinearAttentionSpec
    from mrun_b200.parts import MIXERS
    rt = runtime(dtype)
    hidden, heads, dim, vdim = 32, 2, 16, 24
    spec = GatedLinearAttentionSpec(hidden=hidden, heads=heads, dim=dim, vdim=vdim, tau=1.0, rank=2, eps=1e-5)
    gen = torch.Generator().manual_seed(23)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", gen, std=0.05)
    w["a1"].zero_(); w["a2"].zero_()
    w["a2.b"] = torch.full((heads * dim,), 2.0)
    w["a2.b"][0] = 40.0                                # sigmoid = 1 in 32-bit: kept for ever
    w["a2.b"][1] = -40.0                               # gone after one token
    for name, row, column in (("k", 0, 0), ("k", 1, 0), ("q", 0, 1), ("q", 1, 2)):
        w[name][row] = 0; w[name][row, column] = 1     # both channels' keys read column 0; the queries 1 and 2
    w["k"][:, 0][2:] = 0; w["q"][:, 1:3][2:] = 0
    w["v"][:, :3] = 0; w["g"][:, :3] = 0               # the three columns reach the result through these keys and queries only
    part = MIXERS.build(spec, w, rt)
    W = named(w, "m.")
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": 1.0}
    total = 420
    x = torch.randn(total, hidden, generator=gen) * 0.3
    x[:, :3] = 0
    x[5, 0] = 6.0                                       # the key, into channels 0 and 1 of head 0
    keepers, forgetters = [6, 130, 300, 401, 419], [7, 131, 402]
    x[keepers, 1] = 6.0
    x[forgetters, 2] = 6.0
    x = x.to(rt.precision.act).float()
    want = plain.gated_linear_attention(m, W, "m.", x.double(), 1e-5)
    lost = x.clone(); lost[5, 0] = 0
    blind = plain.gated_linear_attention(m, W, "m.", lost.double(), 1e-5)
    change = (want - blind).abs().max(1).values / want.abs().max()
    assert float(change[keepers].min()) > 0.1 and float(change[forgetters].max()) < 1e-6
    for portions in ([400] + [1] * 20, [3, 2, 2, 100, 193, 100] + [1] * 20):
        book = Steps([part.cache_need()], rt, slots=1)
        got, at = [], 0
        for n in portions:
            def run(ctx, places):
                return part.forward(x[at:at + n].to(DEV, rt.precision.act), ctx, book.caches[0]).float().cpu()
            got.append(book.run([("r", [0] * n)], run))
            at += n
        got = torch.cat(got)
        close(got[keepers], want[keepers], dtype, "queries on the kept channel")
        close(got, want, dtype, "all tokens")
        book.release("r")


ATTENTION_SHAPES = [  # heads, kv heads, key size, value size, rotating features, stretch, page size
    (6, 3, 24, 48, 8, 4.0, 16),
    (5, 5, 20, 28, 0, None, 8),
    (4, 1, 12, 36, 12, None, 4),
    (4, 2, 64, 64, 64, None, 16),       # bfloat16: the tensor-core kernels at 64
    (8, 1, 32, 16, 16, 1.5, 16),
    (3, 1, 128, 128, 32, 2.0, 16),      # the same at 128
    (2, 2, 80, 48, 80, 8.0, 8),
    (34, 2, 16, 16, 4, None, 16),       # seventeen query heads a kv head
]


def attention_spec(hidden, heads, kv_heads, dim, vdim, rot, factor, own_kv=True, scale=0.3):
    from mrun_b200.config.spec import GatedAttentionSpec, ScaledRotarySpec
    position = ScaledRotarySpec(dims=rot, base=300.0, pairing="interleaved", linear_factor=factor) if rot else None
    return GatedAttentionSpec(hidden=hidden, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, softmax_scale=scale, eps=1e-5,
                              qk_norm="projection", sink=True, head_gate=True, own_kv=own_kv, position=position)


def attention_entry(heads, kv_heads, dim, vdim, rot, factor, scale=0.3):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = {"dims": rot, "base": 300.0}
        if factor:
            m["rot"]["scaling"] = {"factor": factor}
    return m


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot, factor, page", ATTENTION_SHAPES)
def test_gated_attention_alone(dtype, tensor_cores, heads, kv_heads, dim, vdim, rot, factor, page, monkeypatch):
    from mrun_b200.parts import MIXERS, gated_attention
    monkeypatch.setattr(gated_attention, "TENSOR_CORES", tensor_cores)
    rt = runtime(dtype, page)
    spec = attention_spec(40, heads, kv_heads, dim, vdim, rot, factor)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", torch.Generator().manual_seed(dim + vdim))
    part = MIXERS.build(spec, w, rt)
    if tensor_cores and not part.tensor_cores:
        pytest.skip("the tensor-core kernels do not take this shape")
    W = named(w, "m.")
    m = attention_entry(heads, kv_heads, dim, vdim, rot, factor)

    def fn(h, _):
        positions = torch.arange(h.shape[0])
        return plain.attention(m, W, "m.", h, 1e-5, positions, plain.attention_keys_values(m, W, "m.", h, 1e-5, positions))
    check_rows(lambda rows, ctx, caches: part.forward(rows, ctx, caches[0]), 40, dtype, LENGTHS, fn, [part.cache_need()], rt)


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot, factor, page", [ATTENTION_SHAPES[0], ATTENTION_SHAPES[3], ATTENTION_SHAPES[4]])
def test_gated_attention_reading_another_layers_pages(dtype, tensor_cores, heads, kv_heads, dim, vdim, rot, factor, page, monkeypatch):
    """Two layers in one step: the first writes its keys and values, the second has none of its own
    and reads the first one's pages with its own queries, gate and softmax scale.  The second
    layer's input is another function of the rows than the first one's, so that keys made from the
    wrong input would show."""
    from mrun_b200.parts import MIXERS, gated_attention
    monkeypatch.setattr(gated_attention, "TENSOR_CORES", tensor_cores)
    rt = runtime(dtype, page)
    owner_spec = attention_spec(40, heads, kv_heads, dim, vdim, rot, factor)
    reader_spec = attention_spec(40, heads, kv_heads, dim, vdim, rot, factor, own_kv=False, scale=0.45)
    gen = torch.Generator().manual_seed(dim)
    wo = random_tensors(MIXERS.tensor_specs(owner_spec, "a"), "a", gen)
    wr = random_tensors(MIXERS.tensor_specs(reader_spec, "b"), "b", gen)
    assert "k" not in wr and "v" not in wr and "k.norm" not in wr
    owner, reader = MIXERS.build(owner_spec, wo, rt), MIXERS.build(reader_spec, wr, rt)
    if tensor_cores and not reader.tensor_cores:
        pytest.skip("the tensor-core kernels do not take this shape")
    assert reader.cache_need() is None
    W = {**named(wo, "a."), **named(wr, "b.")}
    mo = attention_entry(heads, kv_heads, dim, vdim, rot, factor)
    mr = attention_entry(heads, kv_heads, dim, vdim, rot, factor, scale=0.45)
    act = rt.precision.act

    def second_input(rows):
        return (rows.flip(1) * 0.5).to(act)

    def fn(h, _):
        positions = torch.arange(h.shape[0])
        kept = plain.attention_keys_values(mo, W, "a.", h, 1e-5, positions)
        return plain.attention(mr, W, "b.", second_input(h.float()).double(), 1e-5, positions, kept)

    def run_rows(rows, ctx, caches):
        assert caches[0].writable and not caches[1].writable
        owner.forward(rows, ctx, caches[0])
        return reader.forward(second_input(rows), ctx, caches[1])
    check_rows(run_rows, 40, dtype, LENGTHS, fn, [owner.cache_need(), None], rt, shares=[None, 0])


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("dim, vdim, page", [(16, 32, 16), (20, 28, 8), (64, 64, 16)])
def test_gated_attention_one_key_stands_out_and_the_sink(dtype, tensor_cores, dim, vdim, page, monkeypatch):
    """One far key and the queries that look for it are scaled so that its score dominates a head:
    at the first token, on both sides of a page border and a hundred tokens back, asked for from
    inside a prompt portion and by tokens decoded alone.  Losing that key, or taking the one beside
    it, changes the head's output by about its size.  Other queries are scaled the other way, so
    that every score is far below zero: the sink then holds nearly all the weight and the output
    all but vanishes, where a softmax without it would return an average of the values."""
    from mrun_b200.parts import MIXERS, gated_attention
    monkeypatch.setattr(gated_attention, "TENSOR_CORES", tensor_cores)
    rt = runtime(dtype, page)
    hidden, heads = 32, 2
    spec = attention_spec(hidden, heads, 1, dim, vdim, 8, 2.0, scale=0.5)
    gen = torch.Generator().manual_seed(17)
    w = random_tensors(MIXERS.tensor_specs(spec, "m"), "m", gen, std=0.1)
    # the last (unrotated) feature of both heads' queries reads input column 1 alone, the key's reads
    # column 0 alone; the norm over the whole projection keeps the ratio of a row's features, and
    # its weights at those features are large, so that these features carry the score
    w["q"][:, :2] = 0; w["k"][:, :2] = 0
    for row in (dim - 1, 2 * dim - 1):
        w["q"][row] = 0; w["q"][row, 1] = 1
    w["k"][dim - 1] = 0; w["k"][dim - 1, 0] = 1
    w["q.norm"][[dim - 1, 2 * dim - 1]] = 8.0
    w["k.norm"][dim - 1] = 8.0
    w["g"] = w["g"] * 0 ; w["g"][:, 3] = 1.0            # the gate reads column 3, held at 2: sigmoid(2) for every head
    part = MIXERS.build(spec, w, rt)
    if tensor_cores and not part.tensor_cores:
        pytest.skip("the tensor-core kernels do not take this shape")
    W = named(w, "m.")
    m = attention_entry(heads, 1, dim, vdim, 8, 2.0, scale=0.5)
    total = 420

    def reference(x):
        positions = torch.arange(total)
        h = x.to(rt.precision.act).double()
        return plain.attention(m, W, "m.", h, 1e-5, positions, plain.attention_keys_values(m, W, "m.", h, 1e-5, positions))
    for far in (0, page - 1, page, 2 * page + 1, 100):
        x = torch.randn(total, hidden, generator=gen) * 0.5
        x[:, 0] = 0; x[:, 1] = 0; x[:, 3] = 2.0
        x[far, 0] = 30.0                                    # the key
        askers = [far + 1, far + page, 300, 401, 419]       # in the prompt portion and decoded alone
        x[askers, 1] = 30.0
        deniers = [far + 2, 350, 410]                       # every score far below zero
        x[deniers, 1] = -30.0
        # all keys lean the same way on that feature, so that a denier's scores are all negative
        x[:, 0] = torch.where(x[:, 0] == 0, torch.full((total,), 4.0), x[:, 0])
        want = reference(x)
        lost = x.clone(); lost[far, 0] = 4.0
        blind = reference(lost)
        assert float((want - blind)[askers].abs().max(1).values.min() / want.abs().max()) > 0.2     # every asker sees the key
        assert float(want[deniers].abs().max() / want.abs().max()) < 1e-3                            # the sink takes it all
        book = Steps([part.cache_need()], rt, pages=-(-total // page) + 2, slots=1)
        got, at = [], 0
        for n in [400] + [1] * 20:
            def run(ctx, places):
                return part.forward(x[at:at + n].to(DEV, rt.precision.act), ctx, book.caches[0]).float().cpu()
            got.append(book.run([("r", [0] * n)], run))
            at += n
        got = torch.cat(got)
        close(got[askers], want[askers], dtype, f"key at {far}")
        close(got, want, dtype, f"key at {far}, all tokens")
        assert float(got[deniers].abs().max() / want.abs().max()) < 2e-3
        book.release("r")


# ------------------------------------------------------------------ feed-forward and layer alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts, top, groups, keep, shared, scale", [(8, 3, 4, 2, 40, 1.5), (6, 2, 2, 1, 0, 0.5), (4, 4, 1, 1, 24, 1.0),
                                                                        (3, 1, 1, 1, 0, 1.0), (6, 2, 6, 3, 16, 1.0), (40, 6, 8, 3, 8, 2.5)])
def test_grouped_routed_feed_forward_alone(dtype, experts, top, groups, keep, shared, scale, monkeypatch):
    """All rows at once against the plain feed-forward, rows alone against rows in a batch, and the
    step that sorts its rows by expert against the step that computes every expert.  Rows whose
    choice is a close call in the plain run are left out of the bfloat16 comparison."""
    from mrun_b200.config.spec import GroupedRoutedMLPSpec
    from mrun_b200.parts import FEED_FORWARDS, routed
    rt = runtime(dtype)
    hidden, ff = 72, 24
    spec = GroupedRoutedMLPSpec(hidden=hidden, experts=experts, top=top, expert_ff=ff, groups=groups, keep_groups=keep,
                                route_scale=scale, shared_ff=shared)
    gen = torch.Generator().manual_seed(experts + top)
    w = random_tensors(FEED_FORWARDS.tensor_specs(spec, "f"), "f", gen, std=0.2)
    part = FEED_FORWARDS.build(spec, w, rt)
    W = named(w, "f.")
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}},
           "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}
    h = torch.randn(300, hidden, generator=gen).to(torch.bfloat16)
    margins = []
    want = plain.routed_feed_forward(mlp, W, "f.", h.double(), margins)
    sure = torch.ones(300, dtype=torch.bool) if dtype == "float32" else margins[0] > 0.02
    assert int(sure.sum()) > 150
    monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 1e30)
    got = part.forward(h.to(DEV, rt.precision.act), None)
    close(got[sure.to(DEV)], want[sure], dtype, "every expert computed")
    assert torch.equal(part.forward(h.to(DEV, rt.precision.act), None), got), "the same step twice must give the same bits"
    for rows in ([0], [7, 8], list(range(20, 37))):                  # a row's result is its own
        alone = part.forward(h[rows].to(DEV, rt.precision.act), None)
        if dtype == "float32":
            assert torch.equal(alone, got[rows])
        keep_rows = sure[rows]
        if bool(keep_rows.any()):
            close(alone[keep_rows.to(DEV)], want[rows][keep_rows], dtype, f"rows {rows[:3]}", bound=None if dtype == "float32" else 5e-2)
    assert part.sortable == (dtype == "bfloat16" and top < experts)
    if part.sortable:
        monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 0.0)
        close(part.forward(h.to(DEV, rt.precision.act), None)[sure.to(DEV)], want[sure], dtype, "sorted by expert")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams, mixer_kind, with_ff", [(3, "gla", True), (0, "attention", True), (1, "gla", False), (4, "attention", True)])
def test_layer_under_streams_alone(dtype, streams, mixer_kind, with_ff):
    """One layer of the design: norms that add 1 to their weights, either mixer, the grouped experts,
    several streams that each sublayer reads as one weighted sum and writes all at once from the
    old ones.  The streams after the layer's last write, fed whole and in portions."""
    from mrun_b200.config.spec import GatedLinearAttentionSpec, GroupedRoutedMLPSpec, LayerSpec, RMSNormSpec
    from mrun_b200.kernels import ops
    from mrun_b200.parts import ARRANGEMENTS
    rt = runtime(dtype)
    width, count = 56, max(1, streams)
    norm = RMSNormSpec(width, 1e-5, bare=True, offset=1.0)
    if mixer_kind == "gla":
        mixer = GatedLinearAttentionSpec(hidden=width, heads=2, dim=16, vdim=24, tau=4.0, rank=4, eps=1e-5)
        m = {"heads": 2, "dim": 16, "vdim": 24, "tau": 4.0}
    else:
        mixer = attention_spec(width, 4, 2, 16, 24, 8, 2.0)
        m = attention_entry(4, 2, 16, 24, 8, 2.0)
    ff = GroupedRoutedMLPSpec(hidden=width, experts=4, top=4, expert_ff=16, shared_ff=8) if with_ff else None    # every expert chosen: no close calls
    spec = LayerSpec(prefix="b", mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm if with_ff else None,
                     arrangement="streams", mixer_prefix="mix", feed_forward_prefix="mlp", mixer_norm_prefix="norm1",
                     feed_forward_norm_prefix="norm2", streams=streams, mixer_streams_prefix="hc1", feed_forward_streams_prefix="hc2")
    cls = ARRANGEMENTS.get("streams")
    gen = torch.Generator().manual_seed(streams + 40)
    w = {}
    for t in cls.tensor_specs(spec):
        if t.init == "streams_in":
            w[t.name] = 1.0 / count + 0.2 * torch.randn(t.shape, generator=gen)
        elif t.init == "streams_mix":
            w[t.name] = torch.eye(count) + 0.2 * torch.randn(t.shape, generator=gen)
        elif t.init == "norm":
            w[t.name] = 1 + 0.2 * torch.randn(t.shape, generator=gen)
        elif t.init == "norm_zero":
            w[t.name] = 0.3 * torch.randn(t.shape, generator=gen)
        else:
            w[t.name] = torch.randn(t.shape, generator=gen) * 0.3
        w[t.name] = w[t.name].to(torch.bfloat16).float()
    assert float(w["b.norm1"].abs().max()) < 1.5                       # stored around zero
    block = cls(spec, w, rt)
    W = {k: v.double() for k, v in w.items()}
    total = 50
    x0 = torch.randn(total, count, width, generator=gen)
    positions = torch.arange(total)

    def mix(h):
        if mixer_kind == "gla":
            return plain.gated_linear_attention(m, W, "b.mix.", h, 1e-5)
        return plain.attention(m, W, "b.mix.", h, 1e-5, positions, plain.attention_keys_values(m, W, "b.mix.", h, 1e-5, positions))
    mlp = {"kind": "moe", "router": {"experts": 4, "top": 4}, "expert": {"ff": 16}, "shared": {"ff": 8}}
    s = [x0[:, i].double() for i in range(count)]
    s = plain.streams_sublayer(s, W, "b.", 1, mix, 1e-5)
    if with_ff:
        s = plain.streams_sublayer(s, W, "b.", 2, lambda h: plain.feed_forward(mlp, W, "b.mlp.", h), 1e-5)
    want = torch.stack(s, 1)
    for chunks in ([total], [2, 1, 30, 17]):
        book = Steps([block.cache_need()], rt, slots=1)
        got = []
        for n in chunks:
            def run(ctx, places):
                (_, start, _, count_), = places
                resid = x0[start:start + count_].reshape(count_, -1).to(DEV)
                pending = block.forward(resid, None, ctx, book.caches[0])
                assert isinstance(pending, ops.PendingStreams)
                ops.streams_step(resid, pending, None, None, 0.0, torch.float32, count, want_sum=True)
                return resid.cpu()
            got.append(book.run([("r", [0] * n)], run))
        close(torch.cat(got).view(total, count, width), want, dtype, f"streams after the layer, fed as {chunks}",
              bound=None if dtype == "float32" else 2e-2)


# ------------------------------------------------------------------ whole models, cut in every way

TRACE_LENGTHS = [70, 1, 133, 2, 45, 260, 97, 3, 161]
CLOSE_CALL = 0.02      # router scores: a bfloat16 run may choose otherwise below this gap
FLIP_CALL = 0.01       # and is taken to have done so at an earlier position below this one


@pytest.fixture(scope="module", params=sorted(FTINY))
def ftiny(request, tmp_path_factory):
    name = request.param
    return name, make_folder(name, str(tmp_path_factory.mktemp(f"fikudra_{name}"))), FTINY[name]


def plain_logits(cfg, weights, tokens):
    """float32 logits of every position, and which positions have a router whose choice (of groups
    or of experts) is a close call in some layer, at the position or before it: there a bfloat16
    run may rightly choose otherwise, and its logits are not compared."""
    margins = []
    logits = plain.forward(cfg, weights, tokens, margins=margins).to(torch.float32).numpy()
    return logits, close_calls(margins, len(tokens))


def close_calls(margins, count):
    """[count] flags: the position's own choice is within CLOSE_CALL of another one, or an earlier
    position of the sequence chose within FLIP_CALL: keys, values and states made after another
    choice there reach every later position."""
    gap = np.full(count, np.inf)
    for m in margins:
        gap = np.minimum(gap, m.numpy())
    before = np.minimum.accumulate(gap)
    return (gap < CLOSE_CALL) | (before < FLIP_CALL)


def test_layers_of_the_plain_run_and_the_engine_agree(ftiny):
    """The sum of the streams after the last layer, normed and projected, is what the engine's
    logits are: the plain run's per-layer record ends where the logits start."""
    name, folder, settings = ftiny
    cfg, weights = load_folder(folder)
    tokens = tokens_of(cfg["vocab"], 12, seed=4)
    logits, layers = plain.forward(cfg, weights, tokens, want_layers=True)
    assert layers.shape == (len(cfg["layers"]), 12, cfg["width"])
    W = plain.as_double(weights)
    again = plain.offset_norm(layers[-1], W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
    assert torch.allclose(again, logits)


@pytest.mark.parametrize("dtype, sorted_experts, tensor_cores", [("float32", False, False), ("bfloat16", False, False),
                                                                ("bfloat16", True, True)])
def test_every_cutting_matches_plain(ftiny, dtype, sorted_experts, tensor_cores, tmp_path, monkeypatch):
    """Whole prompts, a prefix and then token by token (long where the pool allows), portions of
    changing size down to one and two tokens, and up to four requests side by side in a pool so
    small that pages and state slots are used again.  ``sorted_experts``: routed steps of more than
    16 rows compute the chosen experts only; ``tensor_cores``: attention of a fitting shape runs
    through the tcgen05 and TMA kernels."""
    name, folder, settings = ftiny
    cfg, weights = load_folder(folder)
    vocab = cfg["vocab"]
    requests = {f"r{i}": tokens_of(vocab, n, seed=200 + i) for i, n in enumerate(TRACE_LENGTHS)}
    both = {rid: plain_logits(cfg, weights, tokens) for rid, tokens in requests.items()}
    want = {rid: logits for rid, (logits, _) in both.items()}
    unsure = {rid: flags for rid, (_, flags) in both.items()}
    if name == "T":                                    # every expert of every layer is chosen: nothing is left out
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
    # A bfloat16 run may leave the bound at a few ill-conditioned positions (a first token whose
    # linear-attention read-out, (q.k) v, is all but zero before its norm takes the size away): one,
    # or one in fifty of a section, and never by more than three times.  32-bit: none.
    for label, (error, step, rid, position) in worst.items():
        where = f"{name}/{dtype}/{label}: error {error:.3e} at step {step}, request {rid}, position {position}"
        assert error <= (bound if dtype == "float32" else 3 * bound), where
        few = 0 if dtype == "float32" else max(1, compared[label] // 50)
        assert over.get(label, 0) <= few, f"{where}; {over[label]} of {compared[label]} over {bound}"
    # Positions at or after a close call are not held to the bound one by one (another expert there
    # is another function), but a fault of the cache, the state or the batch would move most of them:
    # four in five of all positions of a section stay within the bound all the same.
    for label, errors in every.items():
        within = sum(e <= bound for e in errors)
        assert within >= 0.8 * len(errors), f"{name}/{dtype}/{label}: only {within} of {len(errors)} positions within {bound}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(ftiny, dtype):
    """Greedy generation through ``Engine.generate``: the scheduler cuts prompts into portions of
    seven tokens beside decoded tokens of other requests, with four state slots for five requests."""
    from mrun_b200 import Engine
    name, folder, settings = ftiny
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
    """``mrun random`` writes a Fikudra folder from its config.json (the decay projection's inner
    size from the ``rank`` key), ``mrun run`` reads that size back from the checkpoint and generates."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))
    mrun = os.path.join(root, "bin", "mrun")
    run = lambda *args: subprocess.run([sys.executable, mrun, *args], capture_output=True, text=True, timeout=600)
    (tmp_path / "cfg.json").write_text(json.dumps(FTINY["S"]["config"]))
    folder = str(tmp_path / "model")
    made = run("random", folder, "--config", str(tmp_path / "cfg.json"), "--seed", "21", "--std", "0.1")
    assert made.returncode == 0, made.stderr
    cfg, weights = load_folder(folder)
    for entry in cfg["layers"]:                        # the size is read from the checkpoint's shapes from here on
        entry["mixer"].pop("rank", None)
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
    assert len(tokens) == 19 + 6 and "Fikudra" in result.stderr


# ------------------------------------------------------------------ layer sizes of a real model

REAL_MOE = {"kind": "moe", "router": {"experts": 8, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}},
            "expert": {"ff": 512}, "shared": {"ff": 512}}
REAL_ATTENTION = {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                  "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 2.0}}}
REAL_SIZES = {"architecture": "Fikudra", "vocab": 4096, "width": 1024, "norm": {"eps": 1e-6}, "streams": 4,
              "embedding": {"scale": 4.0, "bigram": {"buckets": 1021, "mul_prev": 1000003, "mul_cur": 7}},
              "layers": [{"type": "attention", "mixer": REAL_ATTENTION, "mlp": REAL_MOE},
                         {"type": "gla", "mixer": {"heads": 8, "dim": 128, "vdim": 128, "tau": 8.0, "rank": 64}, "mlp": REAL_MOE},
                         {"type": "attention", "mixer": dict(REAL_ATTENTION, kv_from=0), "mlp": None}]}


@pytest.mark.parametrize("dtype, sorted_experts, top", [("float32", False, 2), ("bfloat16", False, 8), ("bfloat16", True, 2)])
def test_real_layer_sizes(dtype, sorted_experts, top, tmp_path, monkeypatch):
    """Heads of 128 x 128 (full row slices of the scan; in bfloat16 the tcgen05 and TMA attention
    kernels with the sink and the head gate in 16-byte steps), four streams of 1,024, eight experts
    of 512 in four groups with a shared one, a router product padded to 16 rows: a prompt whole and
    in portions, then decoded token by token, against the plain model.  With two experts chosen a
    bfloat16 run is held to the bound where no choice up to the position was a close call, and at
    seven in ten of all positions; with every expert chosen (all groups kept) at every position."""
    import copy
    from mrun_b200.config.fikudra import FikudraConfig
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.loading import executor_from_folder
    from mrun_b200.parts import routed
    from mrun_b200.weights import write_random_model
    monkeypatch.setattr(routed, "SORT_MIN_SAVED_FLOPS", 0.0 if sorted_experts else 1e30)
    sizes = copy.deepcopy(REAL_SIZES)
    for entry in sizes["layers"]:
        if entry["mlp"] is not None:
            entry["mlp"]["router"]["top"] = top
            entry["mlp"]["router"]["groups"]["keep"] = 2 if top == 2 else 4
    folder = write_random_model(FikudraConfig.from_dict(sizes), str(tmp_path / "real"), seed=7, std=0.03, norm_noise=0.1)
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
