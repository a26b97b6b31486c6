"""Small Fikudra configurations for the tests, none like another: both mixer kinds in several sizes
(keys and values of equal and of different sizes, grouped and ungrouped heads, rotation of all, of
some and of no features, with and without a stretch), layers that read the pages of an earlier one,
one to four residual streams and none, expert groups from one to as many as there are experts, with
and without a shared expert, a dense feed-forward and none, with and without the bigram table."""
from __future__ import annotations

import json
import os

import numpy as np


def attention(heads, kv_heads, dim, vdim, scale, rot_dims=None, base=10000.0, factor=None, kv_from=None):
    out = {"heads": heads, "dim": dim, "vdim": vdim, "scale": scale}
    if kv_heads is not None:
        out["kv_heads"] = kv_heads
    if rot_dims is not None:
        out["rot"] = {"base": base, "dims": rot_dims}
        if factor is not None:
            out["rot"]["scaling"] = {"factor": factor}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def layer(kind, mix, mlp):
    return {"type": kind, "mixer": mix, "mlp": mlp}


def moe(experts, top, ff, groups=None, keep=None, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups, "keep": keep}
    if scale is not None:
        router["scale"] = scale
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


FTINY = {
    # two streams; grouped heads with values twice the keys' size, a third of the features rotated
    # and stretched; the third layer reads the first layer's pages; four groups of which two stay,
    # three experts chosen; a layer without a feed-forward; key rows of the scan in two slices
    "P": dict(
        config={"architecture": "Fikudra", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "streams": 2,
                "embedding": {"scale": 8.0, "bigram": {"buckets": 101, "mul_prev": 7, "mul_cur": 13}},
                "layers": [layer("attention", attention(6, 3, 24, 48, 0.2, rot_dims=8, base=500.0, factor=4.0),
                                 moe(8, 3, 24, groups=4, keep=2, scale=1.5, shared=40)),
                           layer("gla", gla(3, 24, 40, 4.0, 8), None),
                           layer("attention", attention(6, 3, 24, 48, 0.2, rot_dims=8, base=500.0, factor=4.0, kv_from=0),
                                 moe(6, 2, 16, groups=2, keep=1, scale=0.5)),
                           layer("gla", gla(2, 16, 16, 1.0, 4), moe(4, 4, 8, shared=24))]},
        seed=3, std=0.1, norm_noise=0.2, page_size=16),
    # no streams, no bigram table, no groups, no shared expert, no rotation in one layer and all
    # features rotated without a stretch in the other; sizes that fit no vector width: an odd
    # width, key and value sizes that are no multiple of 8, a key size of 72 in the scan, one expert
    # of three; kv_heads left out (as many as heads); a dense feed-forward
    "Q": dict(
        config={"architecture": "Fikudra", "vocab": 131, "width": 100, "norm": {"eps": 1e-5},
                "embedding": {"scale": 1.0},
                "layers": [layer("gla", gla(2, 72, 33, 16.0, 5), moe(3, 1, 22)),
                           layer("attention", attention(5, None, 20, 28, 0.22), {"kind": "dense", "ff": 90}),
                           layer("attention", attention(4, 1, 12, 36, 0.3, rot_dims=12, base=100.0), None),
                           layer("gla", gla(5, 10, 7, 2.5, 3), moe(5, 2, 18, groups=5, keep=3, scale=2.0, shared=10))]},
        seed=5, std=0.1, norm_noise=0.1, page_size=8),
    # one stream with coefficients of its own; keys and values of 64 (the tensor-core kernels in
    # bfloat16: tcgen05 prompt tiles, TMA decode), two layers reading the pages of the first; as
    # many groups as experts; a key size of 160 in the scan; pages of four tokens
    "R": dict(
        config={"architecture": "Fikudra", "vocab": 257, "width": 96, "norm": {"eps": 1e-4}, "streams": 1,
                "embedding": {"scale": 3.0, "bigram": {"buckets": 64, "mul_prev": 1000003, "mul_cur": 1}},
                "layers": [layer("attention", attention(4, 2, 64, 64, 0.125, rot_dims=64, base=1000000.0),
                                 moe(6, 2, 24, groups=6, keep=3, scale=1.0, shared=16)),
                           layer("gla", gla(2, 160, 16, 8.0, 6), moe(2, 1, 48, groups=1, keep=1)),
                           layer("attention", attention(4, 2, 64, 64, 0.125, rot_dims=64, base=1000000.0, kv_from=0), None),
                           layer("attention", attention(4, 2, 64, 64, 0.1, rot_dims=64, base=1000000.0, kv_from=0),
                                 moe(4, 2, 32, shared=32))]},
        seed=9, std=0.1, norm_noise=0.3, page_size=4),
    # four streams; a linear attention first; one key/value head for eight query heads; keys of 32
    # with values of 16 (the CUDA-core kernel with padding-free pages); every expert of the kept
    # groups chosen
    "S": dict(
        config={"architecture": "Fikudra", "vocab": 128, "width": 80, "norm": {"eps": 1e-5}, "streams": 4,
                "embedding": {"scale": 0.5, "bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 5}},
                "layers": [layer("gla", gla(5, 16, 16, 32.0, 10), moe(8, 4, 16, groups=4, keep=2, scale=2.5, shared=8)),
                           layer("attention", attention(8, 1, 32, 16, 0.18, rot_dims=16, base=10000.0, factor=1.5), None)]},
        seed=13, std=0.1, norm_noise=0.2, page_size=16),
    # every expert of every routed layer is chosen (as many groups kept as there are), so that no
    # choice is a close call and a bfloat16 run is compared at every position; keys and values of
    # 64 with half of the features rotated; three streams; a dense feed-forward under the reading layer
    "T": dict(
        config={"architecture": "Fikudra", "vocab": 200, "width": 72, "norm": {"eps": 1e-5}, "streams": 3,
                "embedding": {"scale": 2.0, "bigram": {"buckets": 37, "mul_prev": 11, "mul_cur": 29}},
                "layers": [layer("attention", attention(4, 2, 64, 64, 0.15, rot_dims=32, base=5000.0, factor=2.5),
                                 moe(4, 4, 16, shared=16)),
                           layer("gla", gla(3, 32, 24, 8.0, 6), moe(6, 6, 8, groups=3, keep=3, scale=1.5)),
                           layer("attention", attention(4, 2, 64, 64, 0.15, rot_dims=32, base=5000.0, factor=2.5, kv_from=0),
                                 {"kind": "dense", "ff": 48}),
                           layer("gla", gla(2, 16, 48, 2.0, 4), None)]},
        seed=21, std=0.1, norm_noise=0.2, page_size=16),
    # six layers with two page owners of different sizes, each read by a later layer, the readers in
    # the other order than the owners; a linear attention first and last, one with a single head as
    # wide as the model; one expert chosen of two; nine experts in three groups; a table of two rows
    "U": dict(
        config={"architecture": "Fikudra", "vocab": 90, "width": 48, "norm": {"eps": 1e-6}, "streams": 2,
                "embedding": {"scale": 4.0, "bigram": {"buckets": 2, "mul_prev": 5, "mul_cur": 3}},
                "layers": [layer("gla", gla(2, 8, 12, 1.5, 2), moe(2, 1, 8)),
                           layer("attention", attention(2, 2, 32, 32, 0.2, rot_dims=16, base=1000.0), None),
                           layer("attention", attention(4, 1, 16, 8, 0.3, rot_dims=16, base=50.0, factor=3.0),
                                 moe(9, 3, 8, groups=3, keep=2, scale=0.7, shared=8)),
                           layer("attention", attention(4, 1, 16, 8, 0.25, rot_dims=16, base=50.0, factor=3.0, kv_from=2),
                                 {"kind": "dense", "ff": 32}),
                           layer("attention", attention(2, 2, 32, 32, 0.2, rot_dims=16, base=1000.0, kv_from=1), None),
                           layer("gla", gla(1, 48, 48, 64.0, 3), moe(4, 2, 8, shared=4))]},
        seed=33, std=0.15, norm_noise=0.2, page_size=8),
}


def fconfig(name: str):
    from mrun_b200.config.fikudra import FikudraConfig
    return FikudraConfig.from_dict(FTINY[name]["config"])


def make_folder(name: str, folder: str) -> str:
    from mrun_b200.weights import write_random_model
    t = FTINY[name]
    return write_random_model(fconfig(name), folder, seed=t["seed"], std=t["std"], norm_noise=t["norm_noise"])


def load_folder(folder: str):
    """config.json as a dict and every tensor as stored."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, dict(load_file(os.path.join(folder, "model.safetensors")))


def tokens_of(vocab: int, length: int, seed: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, size=length).tolist()
