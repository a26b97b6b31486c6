"""Small Nisotar configurations for the tests, none like another: the three mixers in several
sizes (grouped and ungrouped heads, keys and values of equal and of different sizes, head sizes
that the tensor-core kernels take and sizes that fit no vector width, rotation of some, of all and
of no features, with and without a stretch of the frequencies, windows and chunks from one
position to longer than any request, latent rows narrower and wider than 256 features, delta rules
with one to four convolution taps and grouped keys), dense, routed and absent feed-forwards, from
one expert chosen to all of them, more than 32 experts."""
from __future__ import annotations

import json
import os

import numpy as np


def rot(dims, base, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def attention(heads, kv_heads, dim, vdim, scale, size, rotation=None):
    out = {"heads": heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if kv_heads is not None:
        out["kv_heads"] = kv_heads
    if rotation is not None:
        out["rot"] = rotation
    return out


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, size, base=10000.0):
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
           "mask": {"size": size}}
    if rot_dim:
        out["rot"] = {"base": base, "dims": rot_dim}
    return out


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
            "gate_rank": gate_rank}


def parallel(left, right):
    return {"left": left, "right": right}


def layer(kind, mix, mlp):
    return {"type": kind, "mixer": mix, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


NTINY = {
    # every mixer once; grouped heads; an attention whose values are twice its keys (the CUDA-core
    # kernel in both precisions) with a stretched rotation of a third of the features; a latent row
    # of 48 features; a chunk of 24 positions over pages of 16; three experts of eight
    "P": dict(
        config={"architecture": "Nisotar", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
                "layers": [layer("latent_attention", latent(3, 24, 8, 20, 40, 0.2, 20, base=300.0), dense(48, 1.5)),
                           layer("parallel", parallel(attention(4, 2, 32, 32, 0.2, 24, rot(16, 5000.0)),
                                                      delta(4, 2, 16, 24, 4, 6, 5)), moe(8, 3, 24)),
                           layer("attention", attention(6, 3, 24, 48, 0.25, 30, rot(8, 100.0, (4.0, 64, 8.0, 1.0))),
                                 moe(5, 2, 16))]},
        seed=3, std=0.1, norm_noise=0.2, page_size=16),
    # sizes that fit no vector width: an odd width, heads of 20 and 12 features, kv_heads left out,
    # no rotation in one attention, all features rotated in another; a window of one position and a
    # chunk of one position (a token sees itself only); a latent row wider than 256 features under
    # a window; one tap (no convolution state) and one delta-rule head; a layer without a
    # feed-forward; one expert of three; no embedding scale
    "Q": dict(
        config={"architecture": "Nisotar", "vocab": 131, "width": 100, "norm": {"eps": 1e-5},
                "layers": [layer("attention", attention(5, None, 20, 20, 0.22, 1), moe(3, 1, 22)),
                           layer("parallel", parallel(attention(3, 1, 12, 12, 0.3, 1, rot(12, 100.0)),
                                                      delta(1, 1, 72, 33, 1, 3, 2)), None),
                           layer("latent_attention", latent(2, 10, 6, 14, 270, 0.1, 9, base=50.0), dense(90, 3.0)),
                           layer("parallel", parallel(attention(2, 2, 20, 20, 0.2, 7),
                                                      delta(5, 5, 10, 7, 2, 4, 3)), moe(4, 2, 18))]},
        seed=5, std=0.1, norm_noise=0.1, page_size=8),
    # shapes the tensor-core kernels take in bfloat16: attention heads of 64 and 128 (tcgen05 prompt
    # tiles, TMA decode) under a window and under a chunk, a latent row of 64 features; windows and
    # chunks that are no multiple of the page of four tokens; every expert chosen, so that a
    # bfloat16 run is compared at every position
    "R": dict(
        config={"architecture": "Nisotar", "vocab": 257, "width": 96, "norm": {"eps": 1e-4}, "embedding": {"scale": 0.25},
                "layers": [layer("parallel", parallel(attention(2, 1, 128, 128, 0.09, 50, rot(64, 1000000.0)),
                                                      delta(2, 2, 32, 16, 3, 8, 8)), moe(4, 4, 16)),
                           layer("attention", attention(4, 2, 64, 64, 0.125, 37, rot(32, 10000.0, (8.0, 128, 16.0, 2.0))),
                                 dense(64, 2.5)),
                           layer("latent_attention", latent(4, 32, 16, 32, 48, 0.14, 45), moe(3, 3, 24))]},
        seed=9, std=0.1, norm_noise=0.3, page_size=4),
    # windows and chunks longer than every request (plain causal attention); 40 experts of which
    # five are chosen; one key/value head for eight query heads; a latent attention without a
    # rotated part; two taps; delta-rule keys of 160 features (several row slices of the scan)
    "S": dict(
        config={"architecture": "Nisotar", "vocab": 128, "width": 80, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
                "layers": [layer("attention", attention(8, 1, 32, 16, 0.18, 4096, rot(16, 10000.0)), moe(40, 5, 8)),
                           layer("latent_attention", latent(5, 16, 0, 8, 32, 0.25, 100000), None),
                           layer("parallel", parallel(attention(4, 4, 16, 16, 0.25, 5000, rot(8, 20.0, (2.0, 32, 4.0, 1.0))),
                                                      delta(2, 1, 160, 16, 2, 5, 7)), dense(40, 1.0))]},
        seed=13, std=0.1, norm_noise=0.2, page_size=16),
    # two parallel layers in a row and two attentions of different windows in a row; all experts of
    # two chosen; a chunk of two positions; a window as long as a page
    "T": dict(
        config={"architecture": "Nisotar", "vocab": 200, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
                "layers": [layer("parallel", parallel(attention(3, 3, 16, 16, 0.3, 2, rot(4, 30.0)),
                                                      delta(3, 1, 8, 12, 3, 2, 2)), moe(2, 2, 20)),
                           layer("parallel", parallel(attention(6, 2, 48, 48, 0.15, 33, rot(48, 700.0)),
                                                      delta(4, 4, 24, 8, 4, 9, 1)), dense(30, 0.5)),
                           layer("attention", attention(2, 2, 80, 80, 0.11, 8, rot(40, 9000.0)), moe(6, 6, 8)),
                           layer("attention", attention(4, 1, 16, 24, 0.25, 19), None)]},
        seed=21, std=0.1, norm_noise=0.2, page_size=8),
}


def nconfig(name: str):
    from mrun_b200.config.nisotar import NisotarConfig
    return NisotarConfig.from_dict(NTINY[name]["config"])


def make_folder(name: str, folder: str) -> str:
    from mrun_b200.weights import write_random_model
    t = NTINY[name]
    return write_random_model(nconfig(name), folder, seed=t["seed"], std=t["std"], norm_noise=t["norm_noise"])


def load_folder(folder: str):
    """config.json as a dict and every tensor as stored."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, dict(load_file(os.path.join(folder, "model.safetensors")))


def tokens_of(vocab: int, length: int, seed: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, size=length).tolist()
