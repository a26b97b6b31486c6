"""The Nisotar decoder in plain torch on the CPU in 64-bit, one function per mechanism, written from
the design's equations and sharing nothing with the engine.  Slow on purpose: attention as a full
score matrix, the delta rule as a token-by-token loop, experts one token at a time.

Notation: h is what a sublayer reads (already normed), W the checkpoint's tensors by name (64-bit),
p a tensor-name prefix ending in a dot, m / mlp the layer's ``mixer`` / ``mlp`` entry of config.json.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def as_double(weights):
    return {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * w, no bias."""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def frequencies(rot):
    """Frequency of every pair of a rotation and the factor on cos and sin."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])
    at = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(at(float(sc["fast"]))), 0)
    hi = min(math.ceil(at(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x: [T, heads, dim].  Feature i pairs with feature i + dims/2 among the first ``dims``."""
    if rot is None or not rot.get("dims"):
        return x
    half = rot["dims"] // 2
    f, mag = frequencies(rot)
    a = positions.to(F)[:, None] * f[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:2 * half]
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


def window_mask(T, size):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def chunk_mask(T, size):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_rows(s, mask, sink):
    """Softmax over the visible keys of every row; ``sink``: one more term of score 0 in the
    denominator."""
    s = torch.where(mask, s, torch.full_like(s, float("-inf")))
    top = s.max(-1, keepdim=True).values
    if sink:
        top = top.clamp_min(0.0)
    e = torch.exp(s - top)
    total = e.sum(-1, keepdim=True)
    if sink:
        total = total + torch.exp(-top)
    return e / total


def heads_attention(q, k, v, scale, mask, sink):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H * V]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for head in range(H):
        g = head // (H // G)
        out[:, head] = softmax_rows((q[:, head] @ k[:, g].T) * scale, mask, sink) @ v[:, g]
    return out.reshape(T, -1)


def softmax_attention(m, W, p, h, eps, positions, values_are_keys=False, chunked=False):
    """The grouped-query attention with per-head q/k norm, partial rotation and a sink.  With
    ``values_are_keys`` the values are the key projection as it comes out (before norm and
    rotation); ``chunked``: keys of the query's own chunk instead of a sliding window."""
    H, D, T = m["heads"], m["dim"], h.shape[0]
    G = m.get("kv_heads") or H
    q = (h @ W[p + "q"].T).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, G, D)
    v = k.clone() if values_are_keys else (h @ W[p + "v"].T).view(T, G, m["vdim"])
    q = rotate(unit_rms(q, eps) * W[p + "q.norm"], positions, m.get("rot"))
    k = rotate(unit_rms(k, eps) * W[p + "k.norm"], positions, m.get("rot"))
    size = m["mask"]["size"]
    mask = chunk_mask(T, size) if chunked else window_mask(T, size)
    return heads_attention(q, k, v, float(m["scale"]), mask, sink=True) @ W[p + "o"].T


def latent_attention(m, W, p, h, eps, positions):
    H, D, R, V, C, T = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], h.shape[0]
    q = (h @ W[p + "q"].T).view(T, H, D + R)
    down = h @ W[p + "dkv"].T
    c = unit_rms(down[:, :C], eps) * W[p + "dkv.norm"]
    rot = dict(m["rot"], dims=R) if R else None          # the rotated part turns as a whole
    shared = rotate(down[:, C:].view(T, 1, R), positions, rot)
    q_rot = rotate(q[:, :, D:], positions, rot)
    k_plain = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, V)
    qq = torch.cat([q[:, :, :D], q_rot], dim=-1)
    kk = torch.cat([k_plain, shared.expand(T, H, R)], dim=-1)
    mask = window_mask(T, m["mask"]["size"])
    return heads_attention(qq, kk, v, float(m["scale"]), mask, sink=False) @ W[p + "o"].T


def short_conv(x, w):
    """Causal convolution over time per channel: x [T, C], w [C, taps], the last column weighs
    the current token, zeros before the start; then SiLU."""
    T, taps = x.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F), x], dim=0)
    y = sum(padded[j:j + T] * w[:, j] for j in range(taps))
    return y * torch.sigmoid(y)


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(m, W, p, h, eps):
    """The gated delta rule with a decay per head and key channel."""
    H, G, D, V, T = m["heads"], m["kv_heads"], m["dim"], m["vdim"], h.shape[0]
    q = short_conv(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, D)
    k = short_conv(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, D)
    v = short_conv(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, V)
    q, k = unit_vector(q) * D ** -0.5, unit_vector(k)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    decay = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(z).view(T, H, D))
    S = torch.zeros(H, D, V, dtype=F)
    o = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head][:, None] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + k[t, g][:, None] * u[None, :]
            o[t, head] = S[head].T @ q[t, g]
    o = unit_rms(o, eps) * W[p + "norm"]
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T)
    return (o.reshape(T, H * V) * gate) @ W[p + "o"].T


def parallel_mixer(m, W, p, h, eps, positions):
    left = softmax_attention(m["left"], W, p + "left.", h, eps, positions, values_are_keys=True, chunked=True)
    right = delta_rule(m["right"], W, p + "right.", h, eps)
    return 0.5 * (unit_rms(left, eps) * W[p + "left.out"] + unit_rms(right, eps) * W[p + "right.out"])


def dense_feed_forward(mlp, W, p, h):
    limit = float(mlp["limit"])
    g = (h @ W[p + "gate"].T + W[p + "gate.b"]).clamp(max=limit)
    u = (h @ W[p + "up"].T + W[p + "up.b"]).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T + W[p + "down.b"]


def expert(W, p, h):
    g = h @ W[p + "gate"].T
    return ((g * torch.sigmoid(g)) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def routed_feed_forward(mlp, W, p, h, margins=None):
    """``margins``, a list, receives one tensor [T]: the gap between the last logit chosen and the
    best one left out."""
    top = mlp["router"]["top"]
    z = h @ W[p + "router"].T + W[p + "router.b"]
    y = torch.zeros_like(h)
    gaps = torch.full((h.shape[0],), float("inf"), dtype=F)
    for t in range(h.shape[0]):
        ranked = z[t].sort(descending=True)
        weights = torch.softmax(ranked.values[:top], dim=0)
        for e, w in zip(ranked.indices[:top].tolist(), weights.tolist()):
            y[t] += w * expert(W, f"{p}e{e}.", h[t:t + 1])[0]
        if top < z.shape[1]:
            gaps[t] = ranked.values[top - 1] - ranked.values[top]
    if margins is not None:
        margins.append(gaps)
    return y


def feed_forward(mlp, W, p, h, margins=None):
    if mlp["kind"] == "dense":
        return dense_feed_forward(mlp, W, p, h)
    return routed_feed_forward(mlp, W, p, h, margins)


def mixer(layer, W, p, h, eps, positions):
    kind, m = layer["type"], layer["mixer"]
    if kind == "attention":
        return softmax_attention(m, W, p, h, eps, positions)
    if kind == "latent_attention":
        return latent_attention(m, W, p, h, eps, positions)
    if kind == "parallel":
        return parallel_mixer(m, W, p, h, eps, positions)
    raise ValueError(kind)


def forward(cfg, weights, tokens, want_layers=False, margins=None):
    """float64 logits [T, vocab] of one sequence (and the residual stream after every layer).
    ``margins``, a list, receives one tensor [T] for every routed feed-forward."""
    W = as_double(weights)
    eps = float(cfg["norm"]["eps"])
    positions = torch.arange(len(tokens))
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    after = []
    for i, layer in enumerate(cfg["layers"]):
        x = x + mixer(layer, W, f"l{i}.mix.", layer_norm(x, W[f"l{i}.norm1"], eps), eps, positions)
        if layer.get("mlp") is not None:
            x = x + feed_forward(layer["mlp"], W, f"l{i}.mlp.", layer_norm(x, W[f"l{i}.norm2"], eps), margins)
        after.append(x)
    logits = layer_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, torch.stack(after)) if want_layers else logits
