"""Nisotar without a GPU: the registry, the configuration read back from its own dictionary, its
refusals, the tensor names and shapes of every part, the random-weights folder, and hand-worked
values of the plain implementation's functions."""
from __future__ import annotations

import copy
import json
import math
import os

import pytest
import torch

import plain_nisotar as plain
from tiny_nisotar import NTINY, load_folder, make_folder, nconfig

F = torch.float64


def test_registry_resolves_the_architecture():
    from mrun_b200 import registry
    from mrun_b200.config.nisotar import NisotarConfig
    assert registry.resolve({"architecture": "Nisotar"}) is NisotarConfig
    assert "nisotar" in registry.supported()


def attention_names(names, p, m, width, keys_as_values):
    groups = m.get("kv_heads") or m["heads"]
    assert names[f"{p}.q"] == (m["heads"] * m["dim"], width)
    assert names[f"{p}.k"] == (groups * m["dim"], width)
    assert names[f"{p}.q.norm"] == names[f"{p}.k.norm"] == (m["dim"],)
    assert names[f"{p}.o"] == (width, m["heads"] * m["vdim"])
    assert (f"{p}.v" in names) == (not keys_as_values)
    if not keys_as_values:
        assert names[f"{p}.v"] == (groups * m["vdim"], width)
    assert f"{p}.g" not in names


@pytest.mark.parametrize("name", sorted(NTINY))
def test_read_back_and_spec(name):
    from mrun_b200.config.nisotar import NisotarConfig
    from mrun_b200.config.spec import LayerNormSpec
    from mrun_b200.weights.loader import expected_tensors
    config = nconfig(name)
    raw = NTINY[name]["config"]
    expected = dict(raw, embedding={"scale": (raw.get("embedding") or {}).get("scale", 1.0)})
    assert config.to_dict() == expected
    assert NisotarConfig.from_dict(json.loads(json.dumps(config.to_dict()))) == config
    spec = config.to_spec()
    assert isinstance(spec.final_norm, LayerNormSpec) and spec.streams == 1
    assert (spec.embedding_transform is not None) == (config.embedding_scale != 1.0)
    names = {t.name: t.shape for t in expected_tensors(spec)}
    width = raw["width"]
    assert names["embed"] == names["head"] == (raw["vocab"], width) and names["final.norm"] == (width,)
    for i, layer in enumerate(raw["layers"]):
        m, p = layer["mixer"], f"l{i}"
        assert names[f"{p}.norm1"] == (width,)
        assert (f"{p}.norm2" in names) == (layer["mlp"] is not None)
        if layer["type"] == "attention":
            attention_names(names, f"{p}.mix", m, width, keys_as_values=False)
        elif layer["type"] == "latent_attention":
            assert names[f"{p}.mix.q"] == (m["heads"] * (m["dim"] + m["rot_dim"]), width)
            assert names[f"{p}.mix.dkv"] == (m["kv_rank"] + m["rot_dim"], width)
            assert names[f"{p}.mix.dkv.norm"] == (m["kv_rank"],)
            assert names[f"{p}.mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"])
            assert names[f"{p}.mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
            assert names[f"{p}.mix.o"] == (width, m["heads"] * m["vdim"])
            assert f"{p}.mix.dq" not in names and f"{p}.mix.uq" not in names
        else:
            attention_names(names, f"{p}.mix.left", m["left"], width, keys_as_values=True)
            r = m["right"]
            keyed, inner, qk = r["heads"] * r["dim"], r["heads"] * r["vdim"], r["kv_heads"] * r["dim"]
            assert names[f"{p}.mix.right.q"] == names[f"{p}.mix.right.k"] == (qk, width)
            assert names[f"{p}.mix.right.v"] == (inner, width)
            assert names[f"{p}.mix.right.q.conv"] == (qk, r["conv"]) and names[f"{p}.mix.right.v.conv"] == (inner, r["conv"])
            assert names[f"{p}.mix.right.b"] == (r["heads"], width) and names[f"{p}.mix.right.A_log"] == (r["heads"],)
            assert names[f"{p}.mix.right.a1"] == (r["decay_rank"], width) and names[f"{p}.mix.right.a2"] == (keyed, r["decay_rank"])
            assert names[f"{p}.mix.right.g1"] == (r["gate_rank"], width) and names[f"{p}.mix.right.g2"] == (inner, r["gate_rank"])
            assert names[f"{p}.mix.right.dt_bias"] == (keyed,) and names[f"{p}.mix.right.norm"] == (r["vdim"],)
            assert names[f"{p}.mix.right.o"] == (width, inner)
            assert names[f"{p}.mix.left.out"] == names[f"{p}.mix.right.out"] == (width,)
        mlp = layer["mlp"]
        if mlp is None:
            assert not any(n.startswith(f"{p}.mlp.") for n in names)
        elif mlp["kind"] == "moe":
            r, ff = mlp["router"], mlp["expert"]["ff"]
            assert names[f"{p}.mlp.router"] == (r["experts"], width) and names[f"{p}.mlp.router.b"] == (r["experts"],)
            assert names[f"{p}.mlp.e{r['experts'] - 1}.gate"] == names[f"{p}.mlp.e0.up"] == (ff, width)
            assert names[f"{p}.mlp.e0.down"] == (width, ff) and f"{p}.mlp.e{r['experts']}.gate" not in names
        else:
            assert names[f"{p}.mlp.gate"] == names[f"{p}.mlp.up"] == (mlp["ff"], width)
            assert names[f"{p}.mlp.gate.b"] == names[f"{p}.mlp.up.b"] == (mlp["ff"],)
            assert names[f"{p}.mlp.down"] == (width, mlp["ff"]) and names[f"{p}.mlp.down.b"] == (width,)
    assert config.num_parameters() == sum(math.prod(s) for s in names.values())


def test_the_parts_take_their_constants_from_the_configuration():
    from mrun_b200.config.spec import (ChannelDeltaSpec, ClampedGatedMLPSpec, GatedAttentionSpec, GroupedRoutedMLPSpec,
                                       LatentAttentionSpec, ParallelMixerSpec)
    latent, both, attention = (layer for layer in nconfig("P").layers)
    m = latent.mixer
    assert isinstance(m, LatentAttentionSpec) and (m.q_rank, m.kv_rank, m.rot_dim, m.window) == (0, 40, 8, 20)
    assert m.position.dims == 8 and m.position.pairing == "half" and m.position.base == 300.0
    assert isinstance(latent.feed_forward, ClampedGatedMLPSpec) and latent.feed_forward.limit == 1.5
    assert latent.feed_forward.alpha == 1.702 and latent.feed_forward.biases
    assert isinstance(both.mixer, ParallelMixerSpec) and both.mixer.share == 0.5
    left, right = both.mixer.left, both.mixer.right
    assert isinstance(left, GatedAttentionSpec) and (left.chunk, left.window, left.values) == (24, None, "keys")
    assert left.qk_norm == "head" and left.sink and not left.head_gate
    assert isinstance(right, ChannelDeltaSpec) and (right.conv, right.decay_rank, right.gate_rank) == (4, 6, 5)
    ff = both.feed_forward
    assert isinstance(ff, GroupedRoutedMLPSpec) and (ff.score, ff.router_bias, ff.groups, ff.shared_ff) == ("logit", True, 1, 0)
    a = attention.mixer
    assert (a.window, a.chunk, a.values, a.dim, a.vdim) == (30, None, "projection", 24, 48)
    assert a.position.scaling == (4.0, 64.0, 8.0, 1.0)


@pytest.mark.parametrize("change, key", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c["layers"][0].update(type="gla"), "layers[0].type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "layers[0].mixer.kv_rank"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "layers[0].mixer.mask"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "layers[0].mlp.limit"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(heads=3), "layers[1].mixer.left.heads"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(vdim=16), "layers[1].mixer.left.vdim"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=34), "layers[1].mixer.left.rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("decay_rank"), "layers[1].mixer.right.decay_rank"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(kv_heads=3), "layers[1].mixer.right.heads"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "layers[1].mlp.router.top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="table"), "layers[1].mlp.kind"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("slow"), "layers[2].mixer.rot.scaling.slow"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), "layers[2].mixer.mask.size"),
])
def test_refusals_name_the_key(change, key):
    from mrun_b200.config.base import ConfigError
    from mrun_b200.config.nisotar import NisotarConfig
    cfg = copy.deepcopy(NTINY["P"]["config"])
    change(cfg)
    with pytest.raises(ConfigError) as error:
        NisotarConfig.from_dict(cfg)
    assert error.value.key == key, str(error.value)


def test_random_folder_and_ranks_from_the_checkpoint(tmp_path):
    """The folder's tensors are the spec's; with the rank keys gone from config.json the inner sizes
    of the delta rule's low-rank projections come from the checkpoint's shapes."""
    from mrun_b200 import registry
    from mrun_b200.weights.loader import expected_tensors
    folder = make_folder("P", str(tmp_path / "m"))
    cfg, weights = load_folder(folder)
    spec = nconfig("P").to_spec()
    assert {t.name: tuple(t.shape) for t in expected_tensors(spec)} == {k: tuple(v.shape) for k, v in weights.items()}
    right = cfg["layers"][1]["mixer"]["right"]
    right.pop("decay_rank"); right.pop("gate_rank")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    again = registry.load_config(folder)
    assert again.layers[1].mixer.right.decay_rank == 6 and again.layers[1].mixer.right.gate_rank == 5
    assert again.to_spec().layers == spec.layers


# ------------------------------------------------------------------ the plain functions, by hand

def test_layer_norm_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=F)
    w = torch.tensor([1.0, 2.0, 0.5, -1.0], dtype=F)
    d = torch.tensor([-2.0, -1.0, 0.0, 3.0], dtype=F)
    want = d / math.sqrt(14.0 / 4.0 + 0.25) * w
    assert torch.allclose(plain.layer_norm(x, w, 0.25)[0], want)
    assert abs(float(plain.layer_norm(x + 100.0, w, 0.25).sum() - want.sum())) < 1e-9      # a shift changes nothing


def test_masks_by_hand():
    w = plain.window_mask(6, 3)
    assert w[5].tolist() == [False, False, False, True, True, True] and w[1].tolist() == [True, True] + [False] * 4
    c = plain.chunk_mask(7, 3)
    assert c[2].tolist() == [True, True, True, False, False, False, False]
    assert c[3].tolist() == [False, False, False, True, False, False, False]           # the first of its chunk sees itself only
    assert c[6].tolist() == [False] * 6 + [True]
    assert plain.chunk_mask(5, 1).tolist() == torch.eye(5, dtype=torch.bool).tolist()
    assert plain.window_mask(5, 9).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()


def test_softmax_with_and_without_a_sink_by_hand():
    s = torch.tensor([[0.0, math.log(3.0), 5.0]], dtype=F)
    mask = torch.tensor([[True, True, False]])
    assert torch.allclose(plain.softmax_rows(s, mask, sink=False), torch.tensor([[0.25, 0.75, 0.0]], dtype=F))
    assert torch.allclose(plain.softmax_rows(s, mask, sink=True), torch.tensor([[0.2, 0.6, 0.0]], dtype=F))
    far_below = plain.softmax_rows(torch.tensor([[-800.0, -900.0]], dtype=F), torch.tensor([[True, True]]), sink=True)
    assert float(far_below.sum()) < 1e-300 or float(far_below.sum()) == 0.0               # the sink takes all the weight


def test_stretched_frequencies_by_hand():
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, magnitude = plain.frequencies(rot)
    plain_f = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    at = lambda turns: 8 * math.log(64 / (2 * math.pi * turns)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(at(8.0)), 0), min(math.ceil(at(1.0)), 7)
    assert (lo, hi) == (0, 3)
    for i in range(4):
        ramp = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert float(f[i]) == pytest.approx(plain_f[i] / 4.0 * ramp + plain_f[i] * (1 - ramp))
    assert magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 0.0, 1.0, 0.0, 0.0, 7.0]]], dtype=F)      # pair (0, 4): (1, 0); pair (1, 5): (0, 1)
    y = plain.rotate(x, torch.tensor([3]), rot)[0, 0]
    a0, a1 = 3 * float(f[0]), 3 * float(f[1])
    assert float(y[0]) == pytest.approx(magnitude * math.cos(a0)) and float(y[4]) == pytest.approx(magnitude * math.sin(a0))
    assert float(y[1]) == pytest.approx(-magnitude * math.sin(a1)) and float(y[5]) == pytest.approx(magnitude * math.cos(a1))
    assert float(y[8]) == 7.0                                                          # beyond the rotating features


def test_short_convolution_by_hand():
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=F)
    w = torch.tensor([[0.5, -1.0, 2.0]], dtype=F)                                       # the last column is the current token's
    y = torch.tensor([2.0, 4.0 - 1.0, 8.0 - 2.0 + 0.5], dtype=F)
    assert torch.allclose(plain.short_conv(x, w)[:, 0], y * torch.sigmoid(y))


def test_delta_rule_first_tokens_by_hand():
    """One head, no convolution history (one tap of weight 1): after the first token S = beta k v^T
    and the read-out is beta (q . k) v; the second token first decays the rows, then corrects."""
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2}
    eye = torch.eye(2, dtype=F)
    W = {"m.q": eye, "m.k": eye, "m.v": eye, "m.q.conv": torch.ones(2, 1, dtype=F), "m.k.conv": torch.ones(2, 1, dtype=F),
         "m.v.conv": torch.ones(2, 1, dtype=F), "m.b": torch.zeros(1, 2, dtype=F), "m.a1": torch.zeros(1, 2, dtype=F),
         "m.a2": torch.zeros(2, 1, dtype=F), "m.dt_bias": torch.tensor([0.0, 50.0], dtype=F), "m.A_log": torch.zeros(1, dtype=F),
         "m.norm": torch.ones(2, dtype=F), "m.g1": torch.zeros(1, 2, dtype=F), "m.g2": torch.zeros(2, 1, dtype=F), "m.o": eye}
    h = torch.tensor([[3.0, 4.0], [1.0, 0.0]], dtype=F)
    silu = lambda t: t * torch.sigmoid(t)
    a = silu(h)
    unit = lambda t: t / torch.sqrt((t * t).sum() + 1e-6)
    k0, k1 = unit(a[0]), unit(a[1])
    S = 0.5 * k0[:, None] * a[0][None, :]                                               # beta = sigmoid(0)
    o0 = S.T @ (k0 * 2 ** -0.5)
    decay = torch.exp(-torch.nn.functional.softplus(torch.tensor([0.0, 50.0], dtype=F)))    # channel 1 is forgotten at once
    S = decay[:, None] * S
    S = S + k1[:, None] * (0.5 * (a[1] - S.T @ k1))[None, :]
    o1 = S.T @ (k1 * 2 ** -0.5)
    want = torch.stack([plain.unit_rms(o0, 1e-5), plain.unit_rms(o1, 1e-5)]) * 0.5       # the gate is sigmoid(0)
    assert torch.allclose(plain.delta_rule(dict(m), W, "m.", h, 1e-5), want)


def test_routed_feed_forward_by_hand():
    """Three experts, two chosen by the largest logits (bias included), weighed by the softmax over
    the two logits only."""
    W = {"f.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=F), "f.router.b": torch.tensor([0.0, 2.5, 0.0], dtype=F)}
    for e in range(3):
        W[f"f.e{e}.gate"] = torch.full((1, 2), float(e + 1), dtype=F)
        W[f"f.e{e}.up"] = torch.ones(1, 2, dtype=F)
        W[f"f.e{e}.down"] = torch.tensor([[1.0], [0.0]], dtype=F)
    h = torch.tensor([[1.0, 1.0]], dtype=F)                  # logits 1, 3.5, 2: experts 1 and 2
    margins = []
    y = plain.routed_feed_forward({"router": {"experts": 3, "top": 2}}, W, "f.", h, margins)
    w1, w2 = math.exp(3.5) / (math.exp(3.5) + math.exp(2.0)), math.exp(2.0) / (math.exp(3.5) + math.exp(2.0))
    silu = lambda z: z / (1 + math.exp(-z))
    assert float(y[0, 0]) == pytest.approx(w1 * silu(4.0) * 2.0 + w2 * silu(6.0) * 2.0) and float(y[0, 1]) == 0.0
    assert float(margins[0][0]) == pytest.approx(1.0)


def test_dense_feed_forward_clamps_by_hand():
    W = {"f.gate": torch.tensor([[1.0], [1.0]], dtype=F), "f.gate.b": torch.tensor([0.0, -10.0], dtype=F),
         "f.up": torch.tensor([[1.0], [-1.0]], dtype=F), "f.up.b": torch.zeros(2, dtype=F),
         "f.down": torch.tensor([[1.0, 1.0]], dtype=F), "f.down.b": torch.tensor([0.25], dtype=F)}
    h = torch.tensor([[5.0]], dtype=F)                      # gate 5 -> 2 (clamped above), -5 (not clamped below); up 5 -> 2, -5 -> -2
    g0, g1 = 2.0, -5.0
    want = g0 / (1 + math.exp(-1.702 * g0)) * 3.0 + g1 / (1 + math.exp(-1.702 * g1)) * (-1.0) + 0.25
    assert float(plain.dense_feed_forward({"limit": 2.0}, W, "f.", h)) == pytest.approx(want)
