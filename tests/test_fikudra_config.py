"""Fikudra without a GPU: the registry, the configuration read back from its own dictionary, its
refusals, the tensor names and shapes of every part, the random-weights folder, and hand-worked
values of the plain implementation's functions."""
from __future__ import annotations

import copy
import json
import math
import os

import pytest
import torch

import plain_fikudra as plain
from tiny_fikudra import FTINY, fconfig, load_folder, make_folder, tokens_of

F = torch.float64


def test_registry_resolves_the_architecture():
    from mrun_b200 import registry
    from mrun_b200.config.fikudra import FikudraConfig
    assert registry.resolve({"architecture": "Fikudra"}) is FikudraConfig
    assert "fikudra" in registry.supported()


@pytest.mark.parametrize("name", sorted(FTINY))
def test_read_back_and_spec(name):
    from mrun_b200.config.fikudra import FikudraConfig
    from mrun_b200.weights.loader import expected_tensors
    config = fconfig(name)
    raw = FTINY[name]["config"]
    assert config.to_dict() == raw
    assert FikudraConfig.from_dict(json.loads(json.dumps(config.to_dict()))) == config
    spec = config.to_spec()
    assert spec.streams == (raw.get("streams") or 1)
    assert [e.cache_of for e in spec.run_order()] == [l["mixer"].get("kv_from") for l in raw["layers"]]
    names = {t.name: t.shape for t in expected_tensors(spec)}
    width = raw["width"]
    assert names["embed"] == names["head"] == (raw["vocab"], width) and names["final.norm"] == (width,)
    bigram = raw["embedding"].get("bigram")
    assert ("bigram" in names) == (bigram is not None)
    if bigram is not None:
        assert names["bigram"] == (bigram["buckets"] + 1, width)
    for i, layer in enumerate(raw["layers"]):
        m, p = layer["mixer"], f"l{i}"
        assert names[f"{p}.norm1"] == (width,)
        assert (f"{p}.hc1.mix" in names) == ("streams" in raw)
        if "streams" in raw:
            s = raw["streams"]
            assert names[f"{p}.hc1.in"] == names[f"{p}.hc1.out"] == (s,) and names[f"{p}.hc1.mix"] == (s, s)
            assert (f"{p}.hc2.mix" in names) == (layer["mlp"] is not None)
        assert (f"{p}.norm2" in names) == (layer["mlp"] is not None)
        if layer["type"] == "attention":
            groups = m.get("kv_heads") or m["heads"]
            own = m.get("kv_from") is None
            assert names[f"{p}.mix.q"] == (m["heads"] * m["dim"], width)
            assert names[f"{p}.mix.q.norm"] == (m["heads"] * m["dim"],)
            assert names[f"{p}.mix.g"] == (m["heads"], width)
            assert names[f"{p}.mix.o"] == (width, m["heads"] * m["vdim"])
            for tensor in ("k", "v", "k.norm"):
                assert (f"{p}.mix.{tensor}" in names) == own
            if own:
                assert names[f"{p}.mix.k"] == (groups * m["dim"], width)
                assert names[f"{p}.mix.v"] == (groups * m["vdim"], width)
                assert names[f"{p}.mix.k.norm"] == (groups * m["dim"],)
        else:
            keyed, inner = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            assert names[f"{p}.mix.q"] == names[f"{p}.mix.k"] == (keyed, width)
            assert names[f"{p}.mix.v"] == names[f"{p}.mix.g"] == (inner, width)
            assert names[f"{p}.mix.o"] == (width, inner) and names[f"{p}.mix.norm"] == (m["vdim"],)
            assert names[f"{p}.mix.a1"] == (m["rank"], width) and names[f"{p}.mix.a2"] == (keyed, m["rank"])
            assert names[f"{p}.mix.a2.b"] == (keyed,)
        mlp = layer["mlp"]
        if mlp is not None and mlp["kind"] == "moe":
            r, ff = mlp["router"], mlp["expert"]["ff"]
            assert names[f"{p}.mlp.router"] == (r["experts"], width)
            assert names[f"{p}.mlp.e{r['experts'] - 1}.gate"] == names[f"{p}.mlp.e0.up"] == (ff, width)
            assert names[f"{p}.mlp.e0.down"] == (width, ff) and f"{p}.mlp.e{r['experts']}.gate" not in names
            assert (f"{p}.mlp.shared.sg" in names) == (f"{p}.mlp.shared.up" in names) == ("shared" in mlp)
            if "shared" in mlp:
                assert names[f"{p}.mlp.shared.down"] == (width, mlp["shared"]["ff"]) and names[f"{p}.mlp.shared.sg"] == (1, width)
        elif mlp is not None:
            assert names[f"{p}.mlp.gate"] == (mlp["ff"], width) and names[f"{p}.mlp.down"] == (width, mlp["ff"])
    total = sum(math.prod(shape) for shape in names.values())
    assert config.num_parameters() == total


def test_refusals_name_the_key():
    from mrun_b200.config.base import ConfigError
    from mrun_b200.config.fikudra import FikudraConfig
    base = FTINY["P"]["config"]

    def refused(change, key):
        cfg = copy.deepcopy(base)
        change(cfg)
        with pytest.raises(ConfigError) as error:
            FikudraConfig.from_dict(cfg)
        assert key in str(error.value), str(error.value)

    refused(lambda c: c["layers"][0].update(type="mamba"), "layers[0].type")
    refused(lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "layers[0].mixer.heads")
    refused(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "layers[0].mixer.rot.dims")
    refused(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "layers[0].mixer.rot.dims")
    refused(lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0), "layers[0].mixer.rot.scaling.factor")
    refused(lambda c: c["layers"][0]["mixer"].pop("scale"), "layers[0].mixer.scale")
    refused(lambda c: c["layers"][1]["mixer"].pop("tau"), "layers[1].mixer.tau")
    refused(lambda c: c["layers"][1]["mixer"].pop("rank"), "layers[1].mixer.rank")
    refused(lambda c: c["layers"][2]["mixer"].update(kv_from=2), "layers[2].mixer.kv_from")        # itself
    refused(lambda c: c["layers"][2]["mixer"].update(kv_from=1), "layers[2].mixer.kv_from")        # no attention
    refused(lambda c: c["layers"][2]["mixer"].update(vdim=24), "layers[2].mixer.kv_from")          # other sizes
    refused(lambda c: c["layers"][2]["mixer"]["rot"].update(base=7.0), "layers[2].mixer.kv_from")  # other rotation
    refused(lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "layers[0].mlp.router.top")   # 2 groups of 2 stay
    refused(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "layers[0].mlp.router.groups.count")
    refused(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=5), "layers[0].mlp.router.groups.keep")
    refused(lambda c: c["layers"][0]["mlp"].update(kind="conv"), "layers[0].mlp.kind")
    refused(lambda c: c["layers"][0]["mlp"].pop("expert"), "layers[0].mlp.expert")
    refused(lambda c: c["embedding"]["bigram"].pop("buckets"), "embedding.bigram.buckets")
    refused(lambda c: c.update(streams=9), "streams")
    refused(lambda c: c["norm"].pop("eps"), "norm.eps")
    refused(lambda c: c.pop("width"), "width")
    refused(lambda c: c.update(layers=[]), "layers")


def test_defaults_of_keys_a_config_may_leave_out():
    config = fconfig("Q")
    assert config.streams is None and config.bigram is None and config.embedding_scale == 1.0
    assert config.layers[1].mixer.kv_heads == 5 and config.layers[1].mixer.position is None
    assert config.layers[2].mixer.position.linear_factor is None and config.layers[2].mixer.position.pairing == "interleaved"
    first = config.layers[0].feed_forward
    assert (first.groups, first.keep_groups, first.route_scale, first.shared_ff) == (1, 1, 1.0, 0)
    assert config.layers[2].feed_forward is None
    spec = config.to_spec()
    assert spec.streams == 1 and all(l.streams == 0 for l in spec.layers)
    assert spec.layers[2].feed_forward_norm is None
    # a feed-forward entry without "kind" is what its keys say
    from mrun_b200.config.fikudra import FikudraConfig
    cfg = copy.deepcopy(FTINY["Q"]["config"])
    for entry in cfg["layers"]:
        if entry["mlp"] is not None:
            entry["mlp"].pop("kind")
    again = FikudraConfig.from_dict(cfg)
    assert [type(l.feed_forward) for l in again.layers] == [type(l.feed_forward) for l in config.layers]


def test_random_folder_and_rank_from_the_checkpoint(tmp_path):
    """The inner size of the decay projection is the shape of a checkpoint tensor when config.json
    does not give it; the norms' weights are stored around zero."""
    from mrun_b200 import registry
    from mrun_b200.weights import load_tensors
    folder = make_folder("P", str(tmp_path / "p"))
    cfg, weights = load_folder(folder)
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    config = registry.load_config(folder)
    assert config.layers[1].mixer.rank == 8 and config.layers[3].mixer.rank == 4
    tensors = load_tensors(folder, config.to_spec())
    assert tensors["bigram"].shape == (102, 64) and tensors["l0.hc1.mix"].shape == (2, 2)
    assert "l2.mix.k" not in tensors and "l2.mix.q.norm" in tensors
    assert float(tensors["l0.norm1"].float().abs().mean()) < 0.5 < float(tensors["l0.mix.q.norm"].float().abs().mean())


# ------------------------------------------------------------------ hand-worked values of the plain functions

def test_plain_norm_adds_one_to_its_weight():
    x = torch.tensor([[3.0, 4.0]], dtype=F)
    w = torch.tensor([0.0, -0.5], dtype=F)
    rms = math.sqrt(12.5 + 0.5)
    assert torch.allclose(plain.offset_norm(x, w, 0.5), torch.tensor([[3.0 / rms, 2.0 / rms]], dtype=F))


def test_plain_bigram_rows_and_embedding():
    assert plain.bigram_rows([5, 2, 9], 7, 3, 4) == [7, (15 + 8) % 7, (6 + 36) % 7]
    W = {"embed": torch.arange(20, dtype=F).view(10, 2), "bigram": 100.0 + torch.arange(16, dtype=F).view(8, 2)}
    cfg = {"embedding": {"scale": 2.0, "bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 4}}}
    x = plain.embedding(cfg, W, [5, 2, 9])
    assert x.tolist() == [[20.0 + 114.0, 22.0 + 115.0], [8.0 + 104.0, 10.0 + 105.0], [36.0 + 100.0, 38.0 + 101.0]]


def test_plain_rotation_pairs_neighbours_and_stretches():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]]], dtype=F).repeat(2, 1, 1)
    out = plain.rotate(x, torch.tensor([0, 3]), {"dims": 4, "base": 100.0, "scaling": {"factor": 2.0}})
    assert torch.equal(out[0], x[0])                                  # position 0 turns nothing
    a0, a1 = 3 * 1.0 / 2.0, 3 * 100.0 ** -0.5 / 2.0
    want = [math.cos(a0), math.sin(a0), -2.0 * math.sin(a1), 2.0 * math.cos(a1), 5.0, 6.0]
    assert torch.allclose(out[1, 0], torch.tensor(want, dtype=F))


def test_plain_sink_softmax():
    s = torch.tensor([[0.0, 9.0], [math.log(3.0), 0.0]], dtype=F)
    mask = torch.tensor([[True, False], [True, True]])
    p = plain.sink_softmax(s, mask)
    assert torch.allclose(p, torch.tensor([[0.5, 0.0], [0.6, 0.2]], dtype=F))


def test_plain_gated_linear_attention_two_tokens():
    # one head, two key channels, one value column; identity-like projections over a width of 2
    W = {"m.q": torch.eye(2, dtype=F), "m.k": torch.eye(2, dtype=F), "m.v": torch.tensor([[1.0, 1.0]], dtype=F),
         "m.g": torch.tensor([[0.0, 0.0]], dtype=F), "m.o": torch.tensor([[1.0], [0.0]], dtype=F),
         "m.norm": torch.tensor([1.0], dtype=F), "m.a1": torch.zeros(1, 2, dtype=F), "m.a2": torch.zeros(2, 1, dtype=F),
         "m.a2.b": torch.tensor([0.0, math.log(3.0)], dtype=F)}
    m = {"heads": 1, "dim": 2, "vdim": 1, "tau": 2.0}
    decay = plain.channel_decay(m, W, "m.", torch.zeros(1, 2, dtype=F))
    assert torch.allclose(decay[0, 0], torch.tensor([0.5 ** 0.5, 0.75 ** 0.5], dtype=F))
    # the gate's SiLU of 0 is 0: the output vanishes whatever the state
    assert float(plain.gated_linear_attention(m, W, "m.", torch.ones(2, 2, dtype=F), 0.0).abs().max()) == 0.0
    # a gate row that gives SiLU(g) = g * sigmoid(g); the head norm leaves the sign of o only (one column, eps 0)
    W["m.g"] = torch.tensor([[1.0, 0.0]], dtype=F)
    h = torch.tensor([[1.0, 2.0], [-3.0, 1.0]], dtype=F)
    # S1 = k1 v1 = [1, 2] * 3; o1 = S1 . q1 / sqrt(2) > 0; S2 = decay * S1 + k2 v2 = [0.707 * 3 + 6, 0.866 * 6 - 2]
    # o2 = (-3 * 8.121 + 1 * 3.196) / sqrt(2) < 0
    out = plain.gated_linear_attention(m, W, "m.", h, 0.0)
    silu = lambda g: g / (1.0 + math.exp(-g))
    assert torch.allclose(out[:, 0], torch.tensor([silu(1.0), -silu(-3.0)], dtype=F)) and float(out[:, 1].abs().max()) == 0.0


def test_plain_choice_among_the_best_groups():
    router = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}, "scale": 2.0}
    # the largest score sits in group 0, but group 1 has the largest sum of two
    scores = torch.tensor([0.9, 0.1, 0.6, 0.7, 0.2, 0.3], dtype=F)
    picks = plain.choose_experts(router, scores)
    assert [e for e, _ in picks] == [3, 2]
    assert picks[0][1] == pytest.approx(2.0 * 0.7 / 1.3) and picks[1][1] == pytest.approx(2.0 * 0.6 / 1.3)
    router["groups"]["keep"] = 2                      # groups 1 (1.3) and 0 (1.0) stay, group 2 (0.5) does not
    assert [e for e, _ in plain.choose_experts(router, scores)] == [0, 3]
    del router["groups"]                              # no groups: the two largest of all
    scores[5] = 0.8
    assert [e for e, _ in plain.choose_experts(router, scores)] == [0, 5]
    # groups of one expert: a group's score is that expert's score
    single = {"experts": 3, "top": 1, "groups": {"count": 3, "keep": 1}}
    assert plain.choose_experts(single, torch.tensor([0.2, 0.5, 0.4], dtype=F)) == [(1, pytest.approx(1.0))]


def test_plain_streams_mix_from_the_old_ones():
    W = {"l0.norm1": torch.zeros(2, dtype=F), "l0.hc1.in": torch.tensor([1.0, 0.0], dtype=F),
         "l0.hc1.out": torch.tensor([0.0, 10.0], dtype=F), "l0.hc1.mix": torch.tensor([[0.0, 1.0], [1.0, 0.0]], dtype=F)}
    a, b = torch.tensor([[3.0, 4.0]], dtype=F), torch.tensor([[1.0, 1.0]], dtype=F)
    seen = []

    def sublayer(h):
        seen.append(h)
        return torch.ones_like(h)
    out = plain.streams_sublayer([a, b], W, "l0.", 1, sublayer, 0.0)
    assert torch.allclose(seen[0], a / math.sqrt(12.5))               # reads the first stream alone
    assert torch.equal(out[0], b) and torch.equal(out[1], a + 10.0)   # the streams swap; the output joins the second


def test_plain_layers_that_share_keys_differ_from_layers_that_do_not(tmp_path):
    """Reading the first layer's keys and values is not the same as having one's own: the plain
    model with the sharing layer pointed at itself (given copies of the tensors) gives other logits."""
    folder = make_folder("P", str(tmp_path / "p"))
    cfg, weights = load_folder(folder)
    tokens = tokens_of(cfg["vocab"], 12, seed=1)
    shared = plain.forward(cfg, weights, tokens)
    own = copy.deepcopy(cfg)
    own["layers"][2]["mixer"].pop("kv_from")
    for tensor in ("k", "v", "k.norm"):
        weights[f"l2.mix.{tensor}"] = weights[f"l0.mix.{tensor}"]
    assert float((plain.forward(own, weights, tokens) - shared).abs().max()) > 1e-3
