"""Architecture-neutral description of a decoder: what the parts are and how they are arranged.

A model is data: a tuple of :class:`LayerSpec` (which mixer, which feed-forward, which norms, under
which tensor-name prefixes) and a *schedule*, the order in which layers run.  A schedule entry may
name a layer that an earlier entry already named (the layer's weights run twice, each run with a
cache of its own) or read the cache that an earlier entry wrote (``cache_of``).  Every part spec
carries its own sizes and constants; nothing below this file knows which architecture it serves.

The reference keeps the same split between a layer's parts and their constants
(``Layer{input_layernorm, attention, post_attention_layernorm, mlp}``,
crates/mrun-engine/src/models/qwen3.rs:16-21; ``AttentionConfig``,
crates/mrun-engine/src/models/common.rs:50-64) and a per-layer kind list that drives the state
layout (crates/mrun-engine/src/models/registry.rs:208-247).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, ClassVar, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part expects in the checkpoint.

    ``init`` tells the random-weights mode how to fill it: ``"normal"`` (matrices and tables),
    ``"norm"`` (scale vectors: ones, or ones plus noise).  An ``optional`` tensor is bound when
    the checkpoint has it and is neither missed nor made by the random-weights mode otherwise
    (the reference takes a linear layer's ``.bias`` that way, crates/mrun-engine/src/load.rs:281).
    """

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False


# --------------------------------------------------------------------------- norms

@dataclass(frozen=True)
class RMSNormSpec:
    """``bare``: the checkpoint names the scale vector by the norm's own name, without a
    ``.weight`` after it."""

    kind: ClassVar[str] = "rmsnorm"
    size: int
    eps: float
    bare: bool = False
    # the checkpoint holds one number for all coordinates (a tensor without dimensions)
    scalar: bool = False
    # the checkpoint stores the scale vector minus this number (weights kept around zero: 1.0)
    offset: float = 0.0


@dataclass(frozen=True)
class LayerNormSpec:
    """Layer norm with a weight and no bias: (x - mean) / sqrt(variance + eps) * w, the variance
    the mean of the squared deviations.  ``bare`` as for :class:`RMSNormSpec`."""

    kind: ClassVar[str] = "layernorm"
    size: int
    eps: float
    bare: bool = False


# --------------------------------------------------------------------------- position encodings

@dataclass(frozen=True)
class RotarySpec:
    """Rotary positions, half-split pairing: feature j pairs with j + rotary_dim/2."""

    kind: ClassVar[str] = "rotary"
    head_dim: int
    rotary_dim: int
    theta: float


@dataclass(frozen=True)
class ScaledRotarySpec:
    """Rotary positions over the first ``dims`` features of a vector, with a choice of pairing
    (``"interleaved"``: feature 2i with 2i + 1; ``"half"``: i with i + dims/2) and an optional
    band-wise stretch of the frequencies (``scaling`` = (factor, original, fast, slow)).

    Pair i has the frequency f_i = base^(-2i/dims).  With a stretch: d(t) = dims * ln(original /
    (2 pi t)) / (2 ln base) is the (fractional) pair that makes t turns over ``original``
    positions; lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1), r_i = clamp((i - lo)
    / max(hi - lo, 0.001), 0, 1); the frequency becomes f_i / factor * r_i + f_i * (1 - r_i), and
    cos and sin are both multiplied by 0.1 * ln(factor) + 1.  ``linear_factor`` divides every
    frequency (positions stretched evenly), before any band-wise stretch."""

    kind: ClassVar[str] = "rotary_scaled"
    dims: int
    base: float
    pairing: str = "interleaved"
    scaling: Optional[Tuple[float, float, float, float]] = None
    linear_factor: Optional[float] = None


# --------------------------------------------------------------------------- mixers

@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache.

    ``window`` = None: a token sees every earlier key.  ``window`` = W: it sees the last W keys,
    itself included.
    """

    kind: ClassVar[str] = "attention"
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    softmax_scale: float
    qk_norm: Optional[RMSNormSpec] = None
    position: Optional[Any] = None
    window: Optional[int] = None


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are up-projections of one cached latent per token.

    Per token: the query goes through a latent of ``q_rank`` features (RMS-normed), then up to
    ``heads`` heads of ``dim`` plain and ``rot_dim`` rotated features (``q_rank`` = 0: one
    projection ``q`` straight from the input, no latent and no norm).  One down-projection gives
    the key/value latent of ``kv_rank`` features (RMS-normed) and ``rot_dim`` more that are the
    rotated key part all heads share.  A head's plain key is an up-projection of the latent, its
    value (``vdim`` features) another; the score is (plain . plain + rotated . rotated) *
    ``softmax_scale``.  The cache holds the latent and the shared rotated part only.  ``window``
    = W: a token sees the last W keys, itself included."""

    kind: ClassVar[str] = "latent_attention"
    hidden: int
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    softmax_scale: float
    eps: float
    position: Optional[Any] = None
    window: Optional[int] = None


@dataclass(frozen=True)
class DifferentialAttentionSpec:
    """Softmax attention with two maps a head: the query has ``heads * 2 * dim`` rows and the key
    ``kv_heads * 2 * dim``, head by head as [map 1, map 2]; both maps weigh the same values
    (``vdim`` a kv head).  With a1, a2 the maps' outputs and lambda = exp(lq1 . lk1) - exp(lq2 .
    lk2) + ``diff`` (one number a layer, from four vectors of ``dim`` entries): o = a1 - lambda *
    a2, divided by its root mean square over the head's ``vdim`` values (``eps`` inside the
    root, no weight) and multiplied by 1 - ``diff``.  ``position`` rotates the first features of
    every map of every q and k head."""

    kind: ClassVar[str] = "differential_attention"
    hidden: int
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    softmax_scale: float
    diff: float
    eps: float
    position: Optional[Any] = None
    window: Optional[int] = None


@dataclass(frozen=True)
class GatedAttentionSpec:
    """Grouped-query softmax attention whose keys (``dim`` a head) and values (``vdim`` a head)
    may differ in size, with these options.  ``qk_norm`` = ``"projection"``: q and k are each
    divided by the root mean square over the whole projection (all heads together, ``eps`` inside
    the root) and multiplied by a weight of that size, before the rotation; ``"head"``: every head
    is divided by its own root mean square over ``dim`` and multiplied by a weight of ``dim``
    entries that the heads share; None: no norm.
    ``sink``: the softmax has one more term of score 0 and no value, p_j = exp(s_j) / (1 + sum
    exp(s)).  ``head_gate``: head h's output is multiplied by sigmoid(g x)_h, one projection row a
    head.  ``own_kv`` False: the layer has no key and value projections and reads the pages of
    another schedule entry (``ScheduleEntry.cache_of``), with queries, gate and output of its
    own.  ``values`` = ``"keys"``: there is no value projection and the values are the keys as
    they come out of their projection, before norm and rotation (``vdim`` = ``dim``).  Which keys a
    token at position i sees: all up to itself; with ``window`` = W the last W, itself included;
    with ``chunk`` = C those of its own chunk, floor(j / C) = floor(i / C), chunks counted from
    position 0 of the sequence."""

    kind: ClassVar[str] = "gated_attention"
    hidden: int
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    softmax_scale: float
    eps: float
    qk_norm: Optional[str] = "projection"
    sink: bool = True
    head_gate: bool = True
    own_kv: bool = True
    position: Optional[Any] = None
    window: Optional[int] = None
    chunk: Optional[int] = None
    values: str = "projection"


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention with a decay per head and key channel and a state of fixed size: q
    (times dim^-1/2), k (``heads`` x ``dim``) and v (``heads`` x ``vdim``) are projections; the
    decay is sigmoid(a2 (a1 x) + bias)^(1 / ``tau``), a low-rank projection of inner size
    ``rank``.  Per head S_t = diag(decay_t) S_(t-1) + k_t v_t^T (the decay multiplies the rows
    that belong to key channels), o_t = S_t^T q_t.  Every head's o is RMS-normed over ``vdim``
    with a weight the heads share, the heads together are multiplied by SiLU of a gate
    projection and projected out."""

    kind: ClassVar[str] = "gated_linear_attention"
    hidden: int
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int
    eps: float


@dataclass(frozen=True)
class DecayAttentionSpec:
    """Linear attention with one decay a head and a state of fixed size: q, k (``heads`` x
    ``dim``) and v (``heads`` x ``vdim``) pass SiLU; S_t = decay_h * S_(t-1) + k_t v_t^T, o_t =
    S_t^T q_t.  The heads' outputs together are RMS-normed with a weight, multiplied by the
    sigmoid of a gate projection and projected out."""

    kind: ClassVar[str] = "decay_attention"
    hidden: int
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    eps: float


@dataclass(frozen=True)
class ChannelDeltaSpec:
    """Gated delta rule with a decay per head and key channel.  q, k (``kv_heads`` x ``dim``) and
    v (``heads`` x ``vdim``) pass a causal convolution of ``conv`` taps per channel and SiLU; q
    and k become unit vectors per head (1e-6 inside the root), q times dim^-1/2.  beta =
    sigmoid(b x); g = exp(-exp(A_log_h) * softplus(a2 (a1 x) + dt_bias)) per head and key
    channel.  Per head: S <- g * S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Each
    head's o is RMS-normed over ``vdim`` with a weight shared by the heads and multiplied by
    sigmoid(g2 (g1 x)).  ``decay_rank`` and ``gate_rank`` are the inner sizes of the two
    low-rank projections."""

    kind: ClassVar[str] = "channel_delta"
    hidden: int
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int
    eps: float


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side that read the same input: the result is ``share`` times the sum of
    their outputs, each first divided by its root mean square over the model width (``eps``
    inside the root) and multiplied by a weight of its own, ``<left_prefix>.<out_name>`` and
    ``<right_prefix>.<out_name>``.  The two may keep a cache each, at most one of them paged."""

    kind: ClassVar[str] = "parallel"
    hidden: int
    left: Any
    right: Any
    eps: float
    share: float = 0.5
    left_prefix: str = "left"
    right_prefix: str = "right"
    out_name: str = "out"


# --------------------------------------------------------------------------- feed-forwards

@dataclass(frozen=True)
class GatedMLPSpec:
    """``down(act(gate(x)) * up(x))``; ``activation`` names the gate's function."""

    kind: ClassVar[str] = "gated_mlp"
    hidden: int
    intermediate: int
    activation: str = "silu"
    # the checkpoint's names of the gate, up and down matrices under the part's prefix; a name
    # that ends in ``.weight`` may have a ``.bias`` beside it
    tensor_names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


@dataclass(frozen=True)
class ClampedGatedMLPSpec:
    """A dense gated feed-forward with clamped branches: g = min(gate x, limit), u = clamp(up x,
    -limit, limit), y = g * sigmoid(alpha * g) * (u + 1), output down y.  ``biases``: every
    projection has a bias ``<name>.b``."""

    kind: ClassVar[str] = "clamped_gated_mlp"
    hidden: int
    intermediate: int
    limit: float
    alpha: float = 1.702
    biases: bool = True


@dataclass(frozen=True)
class RoutedMLPSpec:
    """A mixture of ``experts`` small feed-forwards ``down(act(up(x)))`` without biases, of which
    each token takes the ``top`` with the largest router scores, plus an optional shared expert
    of the same form that every token takes.  ``score``: ``"softmax"`` over all experts or
    ``"sigmoid"`` of each logit, in 32-bit; ``renormalize``: whether the chosen scores are divided
    by their sum before they weigh the experts' outputs."""

    kind: ClassVar[str] = "routed_mlp"
    hidden: int
    experts: int
    top: int
    expert_ff: int
    shared_ff: int = 0
    activation: str = "relu2"
    score: str = "softmax"
    renormalize: bool = False


@dataclass(frozen=True)
class GroupedRoutedMLPSpec:
    """A mixture of ``experts`` gated feed-forwards ``down(act(gate x) * up x)`` without biases,
    chosen by a router whose scores are sigmoid(router x) in 32-bit.  The experts form ``groups``
    equal groups of neighbours; a group's score is the sum of its ``group_top`` largest scores and
    only experts of the ``keep_groups`` best groups can be chosen (``groups`` = 1: no limit).
    Each token takes the ``top`` allowed experts with the largest scores; their weights are the
    scores divided by their sum (+ 1e-20) times ``route_scale``.  ``shared_ff`` > 0: one more
    expert of that size runs for every token, weighed by sigmoid(sg x) (one number a token) when
    ``shared_gate``, else by 1.  ``score`` = ``"logit"`` (without groups): the router's logits
    themselves are ranked, and the chosen experts weigh the softmax over the chosen logits only.
    ``router_bias``: the router has a bias ``router.b`` added to its logits."""

    kind: ClassVar[str] = "grouped_routed_mlp"
    hidden: int
    experts: int
    top: int
    expert_ff: int
    groups: int = 1
    keep_groups: int = 1
    group_top: int = 2
    route_scale: float = 1.0
    shared_ff: int = 0
    shared_gate: bool = True
    activation: str = "silu"
    score: str = "sigmoid"
    router_bias: bool = False


@dataclass(frozen=True)
class TableRoutedMLPSpec:
    """A mixture of ``experts`` gated feed-forwards without a router: row ``token id`` of an
    integer table [``vocab``, ``top``] names the token's experts, each weighing 1 / ``top``.
    Expert: g = min(gate x, limit), u = clamp(up x, -limit, limit), y = g * sigmoid(alpha * g) *
    (u + 1), output down y."""

    kind: ClassVar[str] = "table_routed_mlp"
    hidden: int
    vocab: int
    experts: int
    top: int
    expert_ff: int
    limit: float
    alpha: float = 1.702


# --------------------------------------------------------------------------- transforms

@dataclass(frozen=True)
class SoftCapSpec:
    """x -> cap * tanh(x / cap)."""

    kind: ClassVar[str] = "soft_cap"
    cap: float


@dataclass(frozen=True)
class ScaleSpec:
    """x -> factor * x."""

    kind: ClassVar[str] = "scale"
    factor: float


@dataclass(frozen=True)
class HashedBigramEmbeddingSpec:
    """Token embedding times ``scale`` plus a row of a second table chosen by the token and the
    one before it: row (previous * ``mul_prev`` + token * ``mul_cur``) mod ``buckets``, and row
    ``buckets`` (the table's last) for a sequence's first token.  ``buckets`` = 0: no second table.
    The previous token is per-request state."""

    kind: ClassVar[str] = "hashed_bigram_embedding"
    vocab: int
    hidden: int
    scale: float = 1.0
    buckets: int = 0
    mul_prev: int = 0
    mul_cur: int = 0
    table_name: str = "bigram"


# --------------------------------------------------------------------------- layers and model

@dataclass(frozen=True)
class LayerSpec:
    """One block: norm → mixer → residual → norm → feed-forward → residual (``pre_norm``).  The
    ``sandwich`` arrangement also norms each branch's output (``*_post_norm``) and multiplies it
    by ``residual_scale`` before the sum; its ``feed_forward`` may be None (a layer of a mixer
    only)."""

    prefix: str
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    feed_forward_norm: Any
    arrangement: str = "pre_norm"
    mixer_prefix: str = "self_attn"
    feed_forward_prefix: str = "mlp"
    mixer_norm_prefix: str = "input_layernorm"
    feed_forward_norm_prefix: str = "post_attention_layernorm"
    mixer_post_norm: Any = None
    feed_forward_post_norm: Any = None
    mixer_post_norm_prefix: str = "post_mixer_norm"
    feed_forward_post_norm_prefix: str = "post_feed_forward_norm"
    residual_scale: float = 1.0
    # the ``streams`` arrangement: how many residual streams a token has (0: the layer's
    # checkpoint has no stream coefficients and the streams reduce to the plain residual sum),
    # the prefixes of the two sublayers' coefficients (``.in`` [S], ``.out`` [S], ``.mix`` [S, S]
    # indexed [from, to]), and the taps of the causal convolution whose output is added to the
    # mixer's input (0: none; its weight is ``<prefix>.<input_conv_name>`` [hidden, taps])
    streams: int = 0
    mixer_streams_prefix: str = "hc1"
    feed_forward_streams_prefix: str = "hc2"
    input_conv_taps: int = 0
    input_conv_name: str = "canon1"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_of`` = index of an *earlier schedule entry* whose cache this
    run reads instead of owning one (it then writes nothing into it)."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    final_norm: Any
    tie_embeddings: bool
    schedule: Tuple[ScheduleEntry, ...] = ()
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm"
    head_name: str = "lm_head.weight"
    eos_token_ids: Tuple[int, ...] = ()
    # optional transform specs (kinds of the ``TRANSFORMS`` registry; a spec that binds tensors
    # carries their ``prefix``): applied to the 32-bit stream right after the embedding, and to
    # the float32 logits of the wanted rows
    embedding_transform: Any = None
    logits_transform: Any = None
    # an embedding part (kinds of the ``EMBEDDINGS`` registry) in place of the plain table
    # lookup; it binds ``embedding_name`` itself and may keep per-request state
    embedding: Any = None
    # residual streams a token (layers of the ``streams`` arrangement); 1: the plain residual row
    streams: int = 1
    # tensors that may be present in a checkpoint and are dropped unread: the vision tower, heads
    # for multi-token prediction and rotary frequency tables
    # (crates/mrun-engine/src/load.rs:168-173, crates/mrun-engine/src/models/qwen3.rs:107)
    ignored_suffixes: Tuple[str, ...] = ()
    ignored_prefixes: Tuple[str, ...] = ("vision_tower", "model.visual")
    ignored_containing: Tuple[str, ...] = ("mtp.", "rotary_emb.inv_freq")
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    def ignores(self, name: str) -> bool:
        """Whether a checkpoint tensor of this name is left unread."""
        return (name.startswith(tuple(self.ignored_prefixes)) or name.endswith(tuple(self.ignored_suffixes))
                or any(part in name for part in self.ignored_containing))

    def run_order(self) -> Tuple[ScheduleEntry, ...]:
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i) for i in range(len(self.layers)))

    def validate(self) -> None:
        order = self.run_order()
        for at, entry in enumerate(order):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {at} names layer {entry.layer}, "
                                 f"the model has {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < at:
                    raise ValueError(f"schedule entry {at} reads the cache of entry "
                                     f"{entry.cache_of}, which does not run before it")
                if order[entry.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {at} reads the cache of entry "
                                     f"{entry.cache_of}, which owns none")
