"""Typed configuration of the Fikudra decoder: layers that are each a softmax attention (query
and key norm over the whole projection, partial interleaved rotary positions with linear scaling,
a sink term in the softmax, an output gate per head, optionally the keys and values of an earlier
layer) or a gated linear attention with a decay per key channel, under hyper-connections (several
residual streams a token); mixtures of gated experts behind a sigmoid router with group-limited
choice and a gated shared expert; norms whose weights are stored around zero; a scaled token
embedding with a hashed bigram table added.

config.json of this design is nested: ``layers`` lists the layers (``type``, ``mixer`` with the
mixer's sizes, ``mlp`` with the feed-forward's or null), beside ``vocab``, ``width``, ``norm.eps``,
``embedding`` (``scale``, ``bigram``: ``buckets``, ``mul_prev``, ``mul_cur``) and the optional
``streams``.  The inner size of a linear attention's decay projection is not in config.json: it is
the shape of ``l<i>.mix.a1`` in the checkpoint (or, for a configuration made without one, the
mixer's ``rank`` key).  Checkpoint tensors are named ``embed``, ``bigram``, ``head``,
``final.norm`` and ``l<i>.<part>`` without a ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .balivik import _number, checkpoint_shapes
from .base import ConfigError, eos_token_ids, req_int
from .spec import (GatedAttentionSpec, GatedLinearAttentionSpec, GatedMLPSpec, GroupedRoutedMLPSpec,
                   HashedBigramEmbeddingSpec, LayerSpec, ModelSpec, RMSNormSpec, ScaledRotarySpec, ScheduleEntry)
from .zasesun import _count, _positive, _section


@dataclass(frozen=True)
class FikudraLayer:
    mixer: Any                       # GatedAttentionSpec | GatedLinearAttentionSpec
    feed_forward: Optional[Any]      # GroupedRoutedMLPSpec | GatedMLPSpec | None
    kv_from: Optional[int]           # the layer whose keys and values an attention reads
    raw: Any                         # the layer's entry of config.json, kept for to_dict()


@dataclass(frozen=True)
class FikudraConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[FikudraLayer, ...]
    embedding_scale: float = 1.0
    bigram: Optional[Tuple[int, int, int]] = None       # (buckets, mul_prev, mul_cur)
    streams: Optional[int] = None
    max_positions: int = 1 << 20
    eos_token_id: Tuple[int, ...] = ()

    architecture = "Fikudra"
    model_type = "fikudra"

    # ------------------------------------------------------------------ reading
    @staticmethod
    def _rotary(m: Mapping[str, Any], mw: str, dim: int) -> Optional[ScaledRotarySpec]:
        rot = m.get("rot")
        if rot is None:
            return None
        if not isinstance(rot, dict):
            raise ConfigError(f"{mw}rot", "is not an object")
        dims = _count(rot, "dims", f"{mw}rot.", 0)
        if dims == 0:
            return None
        if dims % 2 or dims > dim:
            raise ConfigError(f"{mw}rot.dims", f"must be even and at most dim={dim}, got {dims}")
        factor = None
        scaling = rot.get("scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"{mw}rot.scaling", "is not an object")
            factor = _positive(scaling, "factor", f"{mw}rot.scaling.")
        return ScaledRotarySpec(dims=dims, base=_positive(rot, "base", f"{mw}rot."), pairing="interleaved",
                                linear_factor=factor)

    @classmethod
    def _mixer(cls, i: int, layer: Mapping[str, Any], where: str, width: int, eps: float, shapes: dict):
        kind = layer.get("type")
        m = _section(layer, "mixer", where)
        mw = f"{where}mixer."
        heads = _count(m, "heads", mw)
        dim, vdim = _count(m, "dim", mw), _count(m, "vdim", mw)
        if kind == "attention":
            kv_heads = _count(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
            if heads % kv_heads:
                raise ConfigError(f"{mw}heads", f"({heads}) is not a multiple of kv_heads ({kv_heads})")
            source = m.get("kv_from")
            if source is not None and (isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i):
                raise ConfigError(f"{mw}kv_from", f"must name an earlier layer, got {source!r}")
            spec = GatedAttentionSpec(hidden=width, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                                      softmax_scale=_positive(m, "scale", mw), eps=eps, qk_norm="projection", sink=True,
                                      head_gate=True, own_kv=source is None, position=cls._rotary(m, mw, dim))
            return spec, source
        if kind == "gla":
            tensor = f"l{i}.mix.a1"
            if tensor in shapes and len(shapes[tensor]) == 2:
                rank = int(shapes[tensor][0])
            elif m.get("rank") is not None:
                rank = _count(m, "rank", mw)
            else:
                raise ConfigError(f"{mw}rank", f"is given neither by the checkpoint tensor {tensor} nor by the key")
            return GatedLinearAttentionSpec(hidden=width, heads=heads, dim=dim, vdim=vdim, tau=_positive(m, "tau", mw),
                                            rank=rank, eps=eps), None
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
            return GatedMLPSpec(width, _count(mlp, "ff", fw), "silu", tensor_names=("gate", "up", "down"))
        if kind != "moe":
            raise ConfigError(f"{fw}kind", f"names the unknown feed-forward {kind!r}")
        router = _section(mlp, "router", fw)
        rw = f"{fw}router."
        experts, top = _count(router, "experts", rw), _count(router, "top", rw)
        groups = keep = 1
        if router.get("groups") is not None:
            section = _section(router, "groups", rw)
            groups, keep = _count(section, "count", f"{rw}groups."), _count(section, "keep", f"{rw}groups.")
            if experts % groups:
                raise ConfigError(f"{rw}groups.count", f"({groups}) does not divide the {experts} experts")
            if keep > groups:
                raise ConfigError(f"{rw}groups.keep", f"({keep}) exceeds the {groups} groups")
        if top > keep * (experts // groups):
            raise ConfigError(f"{rw}top", f"({top}) exceeds the {keep * (experts // groups)} experts that can be chosen")
        shared_ff = 0
        if mlp.get("shared") is not None:
            shared_ff = _count(_section(mlp, "shared", fw), "ff", f"{fw}shared.")
        return GroupedRoutedMLPSpec(hidden=width, experts=experts, top=top,
                                    expert_ff=_count(_section(mlp, "expert", fw), "ff", f"{fw}expert."),
                                    groups=groups, keep_groups=keep, group_top=2,
                                    route_scale=_number(router, "scale", rw) if router.get("scale") is not None else 1.0,
                                    shared_ff=shared_ff, shared_gate=True)

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any], model_dir: Optional[str] = None) -> "FikudraConfig":
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
            mixer, source = cls._mixer(i, entry, where, width, eps, shapes)
            if source is not None:
                other = layers[source]
                if not isinstance(other.mixer, GatedAttentionSpec) or other.kv_from is not None:
                    raise ConfigError(f"{where}mixer.kv_from", f"names layer {source}, which has no keys and values of its own")
                theirs, mine = other.mixer, mixer
                if (theirs.kv_heads, theirs.dim, theirs.vdim, theirs.position) != (mine.kv_heads, mine.dim, mine.vdim, mine.position):
                    raise ConfigError(f"{where}mixer.kv_from", f"names layer {source}, whose key/value heads, sizes or "
                                                               f"rotation differ from this layer's")
            layers.append(FikudraLayer(mixer, cls._feed_forward(entry, where, width), source, entry))
        scale, bigram = 1.0, None
        if cfg.get("embedding") is not None:
            section = _section(cfg, "embedding", "")
            if section.get("scale") is not None:
                scale = _number(section, "scale", "embedding.")
            if section.get("bigram") is not None:
                b = _section(section, "bigram", "embedding.")
                bw = "embedding.bigram."
                bigram = (_count(b, "buckets", bw), _count(b, "mul_prev", bw, 0), _count(b, "mul_cur", bw, 0))
        streams = req_int(cfg, "streams") if cfg.get("streams") is not None else None
        if streams is not None and streams > 8:
            raise ConfigError("streams", f"must be at most 8, got {streams}")
        positions = cfg.get("max_positions")
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers), embedding_scale=scale, bigram=bigram,
                   streams=streams, max_positions=req_int(cfg, "max_positions") if positions is not None else 1 << 20,
                   eos_token_id=eos_token_ids(model_dir, cfg))

    def to_dict(self) -> dict:
        """config.json contents that :meth:`from_dict` reads back to an equal configuration."""
        embedding = {"scale": self.embedding_scale}
        if self.bigram is not None:
            embedding["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": embedding, "layers": [layer.raw for layer in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
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
        norm = RMSNormSpec(self.width, self.eps, bare=True, offset=1.0)
        layers = tuple(
            LayerSpec(prefix=f"l{i}", mixer=layer.mixer, feed_forward=layer.feed_forward,
                      mixer_norm=norm, feed_forward_norm=norm if layer.feed_forward is not None else None,
                      arrangement="streams", mixer_prefix="mix", feed_forward_prefix="mlp",
                      mixer_norm_prefix="norm1", feed_forward_norm_prefix="norm2",
                      streams=self.streams or 0, mixer_streams_prefix="hc1", feed_forward_streams_prefix="hc2")
            for i, layer in enumerate(self.layers))
        buckets, mul_prev, mul_cur = self.bigram or (0, 0, 0)
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=self.max_positions, layers=layers, final_norm=norm, tie_embeddings=False,
            schedule=tuple(ScheduleEntry(i, cache_of=layer.kv_from) for i, layer in enumerate(self.layers)),
            embedding_name="embed", final_norm_prefix="final.norm", head_name="head",
            eos_token_ids=self.eos_token_id,
            embedding=HashedBigramEmbeddingSpec(vocab=self.vocab, hidden=self.width, scale=self.embedding_scale,
                                                buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur, table_name="bigram"),
            streams=self.streams or 1, ignored_prefixes=(), ignored_containing=())
