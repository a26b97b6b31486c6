"""The Fikudra decoder in plain torch on the CPU in 64-bit, one function per mechanism, written from
the design's equations and sharing nothing with the engine.  Slow on purpose: attention as a full
score matrix, the linear attention as a token-by-token loop, experts one token at a time.

Notation: h is what a sublayer reads (already normed), W the checkpoint's tensors by name (64-bit),
p a tensor-name prefix ending in a dot, m / mlp the layer's ``mixer`` / ``mlp`` entry of config.json.
"""
from __future__ import annotations

import torch

F = torch.float64


def as_double(weights):
    return {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The layers' norm: the stored weight lies around zero and 1 is added to it."""
    return unit_rms(x, eps) * (1.0 + w)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every token: the last row (number ``buckets``) for the first."""
    return [buckets] + [(tokens[i - 1] * mul_prev + tokens[i] * mul_cur) % buckets for i in range(1, len(tokens))]


def embedding(cfg, W, tokens):
    e = cfg.get("embedding") or {}
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * float(e.get("scale", 1.0))
    b = e.get("bigram")
    if b is not None:
        rows = bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])
        x = x + W["bigram"][torch.tensor(rows, dtype=torch.long)]
    return x


def rotate(x, positions, rot):
    """x: [T, heads, dim].  Pair i = features (2i, 2i + 1) of the first rot['dims'] features turns by
    the angle position * base^(-2i/dims) / factor."""
    if rot is None or not rot.get("dims"):
        return x
    dims = rot["dims"]
    f = float(rot["base"]) ** (-2.0 * torch.arange(dims // 2, dtype=F) / dims)
    factor = (rot.get("scaling") or {}).get("factor")
    if factor:
        f = f / float(factor)
    a = positions.to(F)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def attention_keys_values(m, W, p, h, eps, positions):
    """(k [T, G, dim] normed over the whole projection and rotated, v [T, G, vdim])."""
    G, T = m.get("kv_heads") or m["heads"], h.shape[0]
    k = unit_rms(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    return rotate(k.view(T, G, m["dim"]), positions, m.get("rot")), (h @ W[p + "v"].T).view(T, G, m["vdim"])


def sink_softmax(s, mask):
    """exp(s_j) / (1 + sum over the visible j of exp(s_j)) along the last axis."""
    s = torch.where(mask, s, torch.full_like(s, float("-inf")))
    top = s.max(-1, keepdim=True).values.clamp_min(0.0)         # the sink's score 0 takes part in the maximum
    e = torch.exp(s - top)
    return e / (torch.exp(-top) + e.sum(-1, keepdim=True))


def attention(m, W, p, h, eps, positions, keys_values):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    G, T = m.get("kv_heads") or H, h.shape[0]
    q = unit_rms(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    q = rotate(q.view(T, H, D), positions, m.get("rot"))
    k, v = keys_values
    gate = torch.sigmoid(h @ W[p + "g"].T)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, V, dtype=F)
    for head in range(H):
        g = head // (H // G)
        weights = sink_softmax((q[:, head] @ k[:, g].T) * float(m["scale"]), mask)
        out[:, head] = (weights @ v[:, g]) * gate[:, head:head + 1]
    return out.reshape(T, H * V) @ W[p + "o"].T


def channel_decay(m, W, p, h):
    """sigmoid(a2 (a1 h) + bias)^(1 / tau), [T, heads, dim]."""
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    return torch.sigmoid(z).pow(1.0 / float(m["tau"])).view(h.shape[0], m["heads"], m["dim"])


def gated_linear_attention(m, W, p, h, eps):
    H, D, V, T = m["heads"], m["dim"], m["vdim"], h.shape[0]
    q = (h @ W[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, D)
    v = (h @ W[p + "v"].T).view(T, H, V)
    decay = channel_decay(m, W, p, h)
    S = torch.zeros(H, D, V, dtype=F)
    o = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps) * W[p + "norm"]
    g = h @ W[p + "g"].T
    return (o.reshape(T, H * V) * (g * torch.sigmoid(g))) @ W[p + "o"].T


def expert(W, p, h):
    g = h @ W[p + "gate"].T
    return ((g * torch.sigmoid(g)) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def choose_experts(router, scores, margin=None):
    """scores: [experts] of one token -> [(expert, weight)] in the order of choice.  ``margin``, a
    list, receives how far the choice was from another one: the gap between the last group kept and
    the first one dropped, and between the last expert chosen and the best one left out."""
    E, top = router["experts"], router["top"]
    allowed = torch.ones(E, dtype=torch.bool)
    groups = router.get("groups")
    if groups is not None:
        size = E // groups["count"]
        group_scores = torch.stack([scores[g * size:(g + 1) * size].topk(min(2, size)).values.sum()
                                    for g in range(groups["count"])])
        allowed[:] = False
        for g in group_scores.topk(groups["keep"]).indices.tolist():
            allowed[g * size:(g + 1) * size] = True
        if margin is not None and groups["keep"] < groups["count"]:
            ranked = group_scores.sort(descending=True).values
            margin.append(float(ranked[groups["keep"] - 1] - ranked[groups["keep"]]))
    masked = torch.where(allowed, scores, torch.full_like(scores, -1.0))
    picks = masked.topk(top).indices
    if margin is not None and top < int(allowed.sum()):
        ranked = masked.sort(descending=True).values
        margin.append(float(ranked[top - 1] - ranked[top]))
    weights = scores[picks] / (scores[picks].sum() + 1e-20) * float(router.get("scale", 1.0))
    return list(zip(picks.tolist(), weights.tolist()))


def routed_feed_forward(mlp, W, p, h, margins=None):
    """``margins``, a list, receives one tensor [T]: each token's smallest gap of choice."""
    scores = torch.sigmoid(h @ W[p + "router"].T)
    y = torch.zeros_like(h)
    gaps = torch.full((h.shape[0],), float("inf"), dtype=F)
    for t in range(h.shape[0]):
        margin = []
        for e, w in choose_experts(mlp["router"], scores[t], margin):
            y[t] += w * expert(W, f"{p}e{e}.", h[t:t + 1])[0]
        if margin:
            gaps[t] = min(margin)
    if margins is not None:
        margins.append(gaps)
    if mlp.get("shared") is not None:
        y = y + torch.sigmoid(h @ W[p + "shared.sg"].T) * expert(W, p + "shared.", h)
    return y


def feed_forward(mlp, W, p, h, margins=None):
    if mlp.get("kind") == "dense":
        return expert(W, p, h)
    return routed_feed_forward(mlp, W, p, h, margins)


def streams_sublayer(streams, W, p, q, fn, eps):
    """One sublayer over the residual streams (a list of [T, width]); q = 1 (mixer) or 2.  Without
    coefficients in the checkpoint: the plain residual sum over one stream."""
    norm_w = W[f"{p}norm{q}"]
    if f"{p}hc{q}.in" not in W:
        return [streams[0] + fn(offset_norm(streams[0], norm_w, eps))]
    c_in, c_out, mix = W[f"{p}hc{q}.in"], W[f"{p}hc{q}.out"], W[f"{p}hc{q}.mix"]
    n = len(streams)
    y = fn(offset_norm(sum(c_in[s] * streams[s] for s in range(n)), norm_w, eps))
    return [sum(mix[s, t] * streams[s] for s in range(n)) + c_out[t] * y for t in range(n)]


def forward(cfg, weights, tokens, want_layers=False, margins=None):
    """float64 logits [T, vocab] of one sequence (and the sum of the streams after every layer).
    ``margins``, a list, receives one tensor [T] for every routed feed-forward."""
    W = as_double(weights)
    eps = float(cfg["norm"]["eps"])
    positions = torch.arange(len(tokens))
    x0 = embedding(cfg, W, tokens)
    streams = [x0.clone() for _ in range(cfg.get("streams") or 1)]
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "attention":
            def mixer(h, i=i, m=m, p=p):
                source = m.get("kv_from")
                if source is None:
                    kept[i] = attention_keys_values(m, W, p, h, eps, positions)
                    source = i
                return attention(m, W, p, h, eps, positions, kept[source])
        elif layer["type"] == "gla":
            def mixer(h, m=m, p=p):
                return gated_linear_attention(m, W, p, h, eps)
        else:
            raise ValueError(layer["type"])
        streams = streams_sublayer(streams, W, f"l{i}.", 1, mixer, eps)
        if layer.get("mlp") is not None:
            streams = streams_sublayer(streams, W, f"l{i}.", 2, lambda h: feed_forward(layer["mlp"], W, f"l{i}.mlp.", h, margins), eps)
        after.append(sum(streams))
    logits = offset_norm(sum(streams), W["final.norm"], eps) @ W["head"].T
    return (logits, torch.stack(after)) if want_layers else logits
