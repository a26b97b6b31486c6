"""Typed configuration of the Nisotar decoder: pre-norm layers under layer norms without a bias,
each with one of three mixers and a dense, a routed or no feed-forward.

Mixers (``layers[i].type``):

* ``attention``: grouped-query attention with a q/k norm per head, a rotation of the first
  ``rot.dims`` features in the half-split pairing with an optional band-wise stretch of the
  frequencies (``rot.scaling``), a sliding window (``mask.size``) and a sink in the softmax;
* ``latent_attention``: attention over a cached latent (``kv_rank`` features) and one rotated key
  part all heads share (``rot_dim``), queries straight from the input, a sliding window and the
  ordinary softmax;
* ``parallel``: two mixers that read the same input, ``left`` an attention whose values are its
  unnormed keys and whose mask is chunked (``mask.size`` positions a chunk), ``right`` a gated
  delta rule with short convolutions and a decay per key channel; each output is RMS-normed over
  the model width and the two are averaged.

Feed-forwards (``layers[i].mlp``, or null): ``dense`` with clamped branches and biases (``ff``,
``limit``), or ``moe``: ``router.experts`` gated experts of ``expert.ff`` features of which a token
takes the ``router.top`` with the largest logits (router with a bias), weighed by the softmax over
the chosen logits.

config.json is nested: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``layers``.  The
inner sizes of the delta rule's two low-rank projections are not in config.json: they are the
shapes of ``l<i>.mix.right.a1`` and ``l<i>.mix.right.g1`` in the checkpoint (or, for a
configuration made without one, the keys ``decay_rank`` and ``gate_rank`` of the mixer).
Checkpoint tensors are named ``embed``, ``head``, ``final.norm`` and ``l<i>.<part>`` without a
``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .balivik import _number, checkpoint_shapes
from .base import ConfigError, eos_token_ids, req_int
from .spec import (ChannelDeltaSpec, ClampedGatedMLPSpec, GatedAttentionSpec, GroupedRoutedMLPSpec, LatentAttentionSpec,
                   LayerNormSpec, LayerSpec, ModelSpec, ParallelMixerSpec, ScaledRotarySpec, ScaleSpec)
from .zasesun import _count, _positive, _section

# the gate of the dense feed-forward: g * sigmoid(1.702 g)
DENSE_GATE_ALPHA = 1.702


@dataclass(frozen=True)
class NisotarLayer:
    mixer: Any                       # GatedAttentionSpec | LatentAttentionSpec | ParallelMixerSpec
    feed_forward: Optional[Any]      # ClampedGatedMLPSpec | GroupedRoutedMLPSpec | None
    raw: Any                         # the layer's entry of config.json, kept for to_dict()


@dataclass(frozen=True)
class NisotarConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[NisotarLayer, ...]
    embedding_scale: float = 1.0
    max_positions: int = 1 << 20
    eos_token_id: Tuple[int, ...] = ()

    architecture = "Nisotar"
    model_type = "nisotar"

    # ------------------------------------------------------------------ reading
    @staticmethod
    def _rotary(m: Mapping[str, Any], mw: str, limit: int, dims: Optional[int] = None) -> Optional[ScaledRotarySpec]:
        """The rotation of a mixer: the first ``rot.dims`` features of a vector of ``limit`` (or
        ``dims``, where the mixer fixes how many turn), half-split pairing."""
        rot = m.get("rot")
        if rot is None:
            return None
        if not isinstance(rot, dict):
            raise ConfigError(f"{mw}rot", "is not an object")
        if dims is None:
            dims = _count(rot, "dims", f"{mw}rot.", 0)
        if dims == 0:
            return None
        if dims % 2 or dims > limit:
            raise ConfigError(f"{mw}rot.dims", f"must be even and at most {limit}, got {dims}")
        scaling = rot.get("scaling")
        stretch = None
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"{mw}rot.scaling", "is not an object")
            sw = f"{mw}rot.scaling."
            stretch = (_positive(scaling, "factor", sw), _positive(scaling, "original", sw),
                       _positive(scaling, "fast", sw), _positive(scaling, "slow", sw))
        return ScaledRotarySpec(dims=dims, base=_positive(rot, "base", f"{mw}rot."), pairing="half", scaling=stretch)

    @staticmethod
    def _mask(m: Mapping[str, Any], mw: str) -> int:
        return _count(_section(m, "mask", mw), "size", f"{mw}mask.")

    @classmethod
    def _attention(cls, m: Mapping[str, Any], mw: str, width: int, eps: float, chunked: bool, keys_as_values: bool):
        heads = _count(m, "heads", mw)
        kv_heads = _count(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError(f"{mw}heads", f"({heads}) is not a multiple of kv_heads ({kv_heads})")
        dim = _count(m, "dim", mw)
        vdim = _count(m, "vdim", mw) if m.get("vdim") is not None else dim
        if keys_as_values and vdim != dim:
            raise ConfigError(f"{mw}vdim", f"({vdim}) differs from dim ({dim}) where the values are the keys")
        size = cls._mask(m, mw)
        return GatedAttentionSpec(hidden=width, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                                  softmax_scale=_positive(m, "scale", mw), eps=eps, qk_norm="head", sink=True,
                                  head_gate=False, position=cls._rotary(m, mw, dim),
                                  window=None if chunked else size, chunk=size if chunked else None,
                                  values="keys" if keys_as_values else "projection")

    @classmethod
    def _delta_rule(cls, m: Mapping[str, Any], mw: str, prefix: str, width: int, eps: float, shapes: dict):
        heads = _count(m, "heads", mw)
        kv_heads = _count(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError(f"{mw}heads", f"({heads}) is not a multiple of kv_heads ({kv_heads})")
        ranks = {}
        for key, tensor in (("decay_rank", f"{prefix}.a1"), ("gate_rank", f"{prefix}.g1")):
            if tensor in shapes and len(shapes[tensor]) == 2:
                ranks[key] = int(shapes[tensor][0])
            elif m.get(key) is not None:
                ranks[key] = _count(m, key, mw)
            else:
                raise ConfigError(f"{mw}{key}", f"is given neither by the checkpoint tensor {tensor} nor by the key")
        return ChannelDeltaSpec(hidden=width, heads=heads, kv_heads=kv_heads, dim=_count(m, "dim", mw),
                                vdim=_count(m, "vdim", mw), conv=_count(m, "conv", mw), eps=eps, **ranks)

    @classmethod
    def _mixer(cls, i: int, layer: Mapping[str, Any], where: str, width: int, eps: float, shapes: dict):
        kind = layer.get("type")
        m = _section(layer, "mixer", where)
        mw = f"{where}mixer."
        if kind == "attention":
            return cls._attention(m, mw, width, eps, chunked=False, keys_as_values=False)
        if kind == "latent_attention":
            rot_dim = _count(m, "rot_dim", mw, 0)
            # the rotated part turns as a whole: rot.dims is rot_dim
            position = cls._rotary(m, mw, rot_dim, dims=rot_dim) if rot_dim else None
            return LatentAttentionSpec(hidden=width, heads=_count(m, "heads", mw), dim=_count(m, "dim", mw),
                                       rot_dim=rot_dim, vdim=_count(m, "vdim", mw), q_rank=0,
                                       kv_rank=_count(m, "kv_rank", mw), softmax_scale=_positive(m, "scale", mw),
                                       eps=eps, position=position, window=cls._mask(m, mw))
        if kind == "parallel":
            left = cls._attention(_section(m, "left", mw), f"{mw}left.", width, eps, chunked=True, keys_as_values=True)
            right = cls._delta_rule(_section(m, "right", mw), f"{mw}right.", f"l{i}.mix.right", width, eps, shapes)
            return ParallelMixerSpec(hidden=width, left=left, right=right, eps=eps, share=0.5)
        raise ConfigError(f"{where}type", f"names the unknown mixer {kind!r}")

    @staticmethod
    def _feed_forward(layer: Mapping[str, Any], where: str, width: int):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        if not isinstance(mlp, dict):
            raise ConfigError(f"{where}mlp", "is neither an object nor null")
        fw = f"{where}mlp."
        kind = mlp.get("kind")
        if kind is None:        # left out: what the entry holds says which it is
            kind = "moe" if "router" in mlp else "dense" if "ff" in mlp else None
        if kind == "dense":
            return ClampedGatedMLPSpec(hidden=width, intermediate=_count(mlp, "ff", fw), limit=_positive(mlp, "limit", fw),
                                       alpha=DENSE_GATE_ALPHA, biases=True)
        if kind != "moe":
            raise ConfigError(f"{fw}kind", f"names the unknown feed-forward {kind!r}")
        router = _section(mlp, "router", fw)
        rw = f"{fw}router."
        experts, top = _count(router, "experts", rw), _count(router, "top", rw)
        if top > experts:
            raise ConfigError(f"{rw}top", f"({top}) exceeds the {experts} experts")
        return GroupedRoutedMLPSpec(hidden=width, experts=experts, top=top,
                                    expert_ff=_count(_section(mlp, "expert", fw), "ff", f"{fw}expert."),
                                    score="logit", router_bias=True)

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any], model_dir: Optional[str] = None) -> "NisotarConfig":
        vocab, width = req_int(cfg, "vocab"), req_int(cfg, "width")
        eps = _positive(_section(cfg, "norm", ""), "eps", "norm.")
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers", "is missing or empty")
        shapes = checkpoint_shapes(model_dir)
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}]", "is not an object")
            layers.append(NisotarLayer(cls._mixer(i, entry, where, width, eps, shapes),
                                       cls._feed_forward(entry, where, width), entry))
        scale = 1.0
        if cfg.get("embedding") is not None:
            section = _section(cfg, "embedding", "")
            if section.get("scale") is not None:
                scale = _number(section, "scale", "embedding.")
        positions = cfg.get("max_positions")
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers), embedding_scale=scale,
                   max_positions=req_int(cfg, "max_positions") if positions is not None else 1 << 20,
                   eos_token_id=eos_token_ids(model_dir, cfg))

    def to_dict(self) -> dict:
        """config.json contents that :meth:`from_dict` reads back to an equal configuration."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embedding_scale}, "layers": [layer.raw for layer in self.layers]}
        if self.max_positions != 1 << 20:
            out["max_positions"] = self.max_positions
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out

    # ------------------------------------------------------------------ derived
    def num_parameters(self) -> int:
        from ..weights.loader import expected_tensors
        total = 0
        for t in expected_tensors(self.to_spec()):
            count = 1
            for extent in t.shape:
                count *= extent
            total += count
        return total

    def to_spec(self) -> ModelSpec:
        norm = LayerNormSpec(self.width, self.eps, bare=True)
        layers = tuple(
            LayerSpec(prefix=f"l{i}", mixer=layer.mixer, feed_forward=layer.feed_forward,
                      mixer_norm=norm, feed_forward_norm=norm if layer.feed_forward is not None else None,
                      arrangement="pre_norm", mixer_prefix="mix", feed_forward_prefix="mlp",
                      mixer_norm_prefix="norm1", feed_forward_norm_prefix="norm2")
            for i, layer in enumerate(self.layers))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=self.max_positions, layers=layers, final_norm=norm, tie_embeddings=False,
            embedding_name="embed", final_norm_prefix="final.norm", head_name="head",
            eos_token_ids=self.eos_token_id,
            embedding_transform=ScaleSpec(self.embedding_scale) if self.embedding_scale != 1.0 else None,
            ignored_prefixes=(), ignored_containing=())
