"""Descriptions of the parts a model is put together from.

A model is described by data only: a :class:`ModelPlan` holds one :class:`LayerSpec` per
layer (each naming its mixer, feed-forward and norms with all their sizes and constants)
and a schedule, the list of layer executions in running order.  Nothing in here computes;
``parts`` turns specs into objects that do.

A new kind of part is a new frozen dataclass deriving from :class:`PartSpec`, registered
with its implementation in ``parts.registry``; nothing in this file has to change for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built, with the offending key in the message."""


@dataclass(frozen=True)
class PartSpec:
    """Base of all part descriptions.  Concrete specs are frozen dataclasses."""


# ------------------------------------------------------------------ norms

@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    """y = x * rsqrt(mean(x^2) + eps) * weight  (pico-engine src/pico_engine/kernels.py:19-23)."""
    size: int
    eps: float
    weight: str                      # tensor name
    one_plus: bool = False           # the stored vector lies around zero and the norm multiplies by 1 + it


@dataclass(frozen=True)
class LayerNormSpec(PartSpec):
    """y = (x - mean) / sqrt(var + eps) * weight + bias, var the mean of the squared deviations."""
    size: int
    eps: float
    weight: str                      # tensor names
    bias: str


# ------------------------------------------------------------------ position encodings

@dataclass(frozen=True)
class RotaryHalfSpec(PartSpec):
    """Rotate-half rotary encoding: element j pairs with j + head_dim/2, angle
    pos * theta^(-2j/head_dim)  (pico-engine src/pico_engine/model.py:75-79, kernels.py:42-47)."""
    head_dim: int
    theta: float


@dataclass(frozen=True)
class NoPositionSpec(PartSpec):
    """Queries and keys are used as projected."""


@dataclass(frozen=True)
class RotaryPairsSpec(PartSpec):
    """Rotary encoding of neighbouring entries: (2i, 2i+1) of the first ``dims`` entries of a head are turned by the
    angle pos * base^(-2i/dims) / factor (``factor`` > 1 stretches positions linearly); the other entries of the
    head stay as they are."""
    head_dim: int
    dims: int
    base: float
    factor: float = 1.0


@dataclass(frozen=True)
class RotaryHalvesSpec(PartSpec):
    """Rotary encoding of the first ``dims`` entries of a head in the layout of halves: entry i < dims/2 pairs with entry i + dims/2,
    the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * f_i, f_i = base^(-2i/dims); the other
    entries of the head stay as they are.  ``stretch`` = (factor, original, fast, slow) lengthens the slow turns: with
    where(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), dims - 1)
    and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is f_i / factor * ramp_i + f_i * (1 - ramp_i), and cos
    and sin are multiplied by ``magnitude_slope`` * ln(factor) + 1."""
    head_dim: int
    dims: int
    base: float
    stretch: Optional[Tuple[float, float, float, float]] = None
    magnitude_slope: float = 0.1


@dataclass(frozen=True)
class SinusoidAddSpec(PartSpec):
    """A position vector added to the embedding: entry 2i of position p is sin(p * base^(-2i/size)),
    entry 2i+1 the cosine of the same angle.  It has no tensors."""
    size: int
    base: float = 10000.0


# ------------------------------------------------------------------ what a sublayer reads

@dataclass(frozen=True)
class CausalConvAddSpec(PartSpec):
    """h_t + sum_j w[:, j] * h_(t - taps + 1 + j) on every channel, zeros before a sequence's start
    (a short causal convolution over time whose result is added to its own input).  ``weight`` names a
    [size, taps] tensor.  The last ``taps - 1`` inputs of a sequence are state that the cache keeps."""
    size: int
    taps: int
    weight: str


# ------------------------------------------------------------------ mixers

@dataclass(frozen=True)
class GQAAttentionSpec(PartSpec):
    """Softmax attention with grouped key/value heads over the key/value cache
    (pico-engine src/pico_engine/model.py:175-213).

    ``window`` None: every earlier key is visible; an integer w: query p sees key j iff
    0 <= p - j < w.  Tensor names are ``prefix + name + ".weight"/".bias"``.
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    qkv_bias: bool
    window: Optional[int]
    scale: float
    position: PartSpec
    prefix: str
    q_name: str = "q_proj"
    k_name: str = "k_proj"
    v_name: str = "v_proj"
    o_name: str = "o_proj"


@dataclass(frozen=True)
class HeadMixAttentionSpec(PartSpec):
    """Softmax attention with grouped key/value heads whose softmax weights are mixed across heads before they
    meet the values: weight_h(i, j) <- sum_g mix[h, g] * weight_g(i, j); head h applies its mixed weights to
    the values of its own key/value head.  Options, each absent when its tensor name is None:
    ``qk_norm`` (RMS norm of every query and key head over ``head_dim`` with one weight vector shared by the
    heads, eps ``norm_eps``), ``sink`` (one learned logit a head that joins the softmax denominator and has no
    value), ``head_mix`` ([n_heads, n_heads]; None: the weights stay as they are).  Keys and values may have
    different head sizes.  ``window`` as in :class:`GQAAttentionSpec`.  Tensor names are ``prefix + name`` for
    weights and ``prefix + name + bias_suffix`` for biases."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    v_head_dim: int
    qkv_bias: bool
    window: Optional[int]
    scale: float
    position: PartSpec
    prefix: str
    norm_eps: float = 1e-6
    q_norm: Optional[str] = None
    k_norm: Optional[str] = None
    sink: Optional[str] = None
    head_mix: Optional[str] = None
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    bias_suffix: str = ".b"


@dataclass(frozen=True)
class MinGRUSpec(PartSpec):
    """A gated recurrence whose gates read the current token only: z = sigmoid(W_z h + b_z), u = W_x h + b_x,
    c = u + 1/2 where u >= 0 and sigmoid(u) elsewhere, S_t = (1 - z) S_(t-1) + z c element by element from
    S = 0, output W_o (S_t * silu(W_g h)).  ``width`` is the size of the state."""
    hidden: int
    width: int
    prefix: str
    z_name: str = "z"
    x_name: str = "x"
    g_name: str = "g"
    o_name: str = "o"
    bias_suffix: str = ".b"


@dataclass(frozen=True)
class GatedAttentionSpec(PartSpec):
    """Softmax attention with grouped key/value heads whose concatenated heads are multiplied by a gate of the
    mixer's own input before the output projection: o <- o * sigmoid(W_g h) (``gate`` None: no gate).  ``position``
    acts on queries and keys; with ``qk_unit_norm`` every query and key head is then divided by its root mean square
    (eps ``norm_eps``, no weight).  Keys and values may have different head sizes; ``window`` as in
    :class:`GQAAttentionSpec`, and with ``keep_first`` = f the first f keys of a sequence stay visible behind the window
    (key j is seen from i iff j <= i and (i - j < window or j < f)).  ``distance_slopes`` (one number a head, or None):
    slope_h * (i - j) is taken off the score of query i and key j before the softmax.  ``bias``: the four projections
    have bias vectors (``name + bias_suffix``).  ``own_kv`` False: the mixer has no key and value projections and reads
    the keys and values another schedule entry wrote (``ScheduleEntry.cache_of``).  ``fixed_sink`` = z: one more place of score z
    that carries no value joins every softmax denominator (z = 0: p_j = exp(s_j) / (1 + sum exp(s_j))).  ``value_blend``: the mixers
    of a model that name the same ``value_blend_key`` share values: the "source" (the first of them in the schedule) uses and caches
    its own values and shows them to the others; a "reader" uses and caches (1 - l) v + l v_source, v_source the source's values of the
    same token and l its own stored number ``prefix + value_blend``.  ``position`` may also be a :class:`RotaryHalvesSpec`.
    Tensor names are ``prefix + name``."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    v_head_dim: int
    window: Optional[int]
    scale: float
    position: PartSpec
    prefix: str
    qk_unit_norm: bool = False
    norm_eps: float = 1e-6
    gate: Optional[str] = "g"
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    keep_first: int = 0
    distance_slopes: Optional[Tuple[float, ...]] = None
    bias: bool = False
    bias_suffix: str = ".b"
    own_kv: bool = True
    cache_span: Optional[Tuple[Optional[int], int]] = None   # (window, keep_first) the cache keeps where other entries that read it see further; None: this mixer's own
    fixed_sink: Optional[float] = None
    value_blend: Optional[str] = None                        # tensor name (behind the prefix) of a reader's blending number
    value_blend_role: Optional[str] = None                   # "source", "reader" or None (values are the mixer's own business)
    value_blend_key: str = "values"


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """Softmax attention whose keys and values are projections of one low-rank row per position.  q = W_q h, laid out head
    by head as [``head_dim`` plain | ``rot_dim`` rotated] entries.  W_dkv h has ``kv_rank`` + ``rot_dim`` entries: the first
    ``kv_rank``, RMS-normed (eps ``norm_eps``, plain weight ``dkv_norm``), are the latent row c; the others are one rotated key
    part that all heads share.  Head h's plain key is W_uk,h c and its value W_uv,h c; score = (q_plain . k_plain + q_rot . k_rot)
    * ``scale``; every earlier key is visible, or with ``window`` = w key j from query i iff 0 <= i - j < w.  With ``q_rank`` the
    queries pass a low-rank row of their own: q = W_uq (rmsnorm(W_dq h) * ``dq_norm``) instead of W_q h.  ``position`` (a
    :class:`RotaryPairsSpec` or :class:`RotaryHalvesSpec` over ``rot_dim`` entries, without stretch) turns q_rot and k_rot.  Head h's output is multiplied by sigmoid((W_g h)_h), one number a head (``gate`` None: no gate), then W_o.
    The cache keeps c and the rotated key part, nothing else.  Tensor names are ``prefix + name``."""
    hidden: int
    n_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    kv_rank: int
    scale: float
    position: PartSpec
    prefix: str
    norm_eps: float = 1e-6
    gate: Optional[str] = "g"
    q_name: str = "q"
    dkv_name: str = "dkv"
    dkv_norm: str = "dkv.norm"
    uk_name: str = "uk"
    uv_name: str = "uv"
    o_name: str = "o"
    window: Optional[int] = None
    q_rank: Optional[int] = None
    dq_name: str = "dq"
    dq_norm: str = "dq.norm"
    uq_name: str = "uq"


@dataclass(frozen=True)
class StateSpaceSpec(PartSpec):
    """A selective state-space mixer with a scalar decay a head.  W_in h = [z | x | B | C | dt] with z, x of ``n_heads`` *
    ``head_dim``, B and C of ``n_groups`` * ``state`` and dt of ``n_heads`` entries.  x, B and C pass a causal convolution
    of ``taps`` taps a channel (weight [channels, taps], the last column the current token's, bias ``conv_name + bias_suffix``)
    and silu.  dt <- softplus(dt + dt_bias).  Head h (group h // (n_heads / n_groups)):
    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T  (S [state, head_dim] float32, zero at a sequence's start),
    y_t = S_t^T C_t + D_h x_t.  y * silu(z) is RMS-normed in ``norm_groups`` equal runs (eps ``norm_eps``) times ``norm_name``,
    then W_o.  The state and the last ``taps`` - 1 inputs of the convolution are kept per sequence."""
    hidden: int
    n_heads: int
    head_dim: int
    state: int
    n_groups: int
    taps: int
    norm_groups: int
    prefix: str
    norm_eps: float = 1e-6
    in_name: str = "in"
    conv_name: str = "conv"
    bias_suffix: str = ".b"
    dt_bias_name: str = "dt_bias"
    a_log_name: str = "A_log"
    d_name: str = "D"
    norm_name: str = "norm"
    o_name: str = "o"


@dataclass(frozen=True)
class LinearAttentionSpec(PartSpec):
    """Attention without a softmax, as a recurrence over a matrix state per head:
    S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, S [head_dim, v_head_dim] float32, zero at a sequence's start.

    The decay a_t is either fixed, one number per head (``head_decay``), or learned per key channel and token:
    a = sigmoid(W_2 (W_1 h) + b)^(1/decay_tau) with the low-rank pair ``decay_names`` = (W_1, W_2, b) of rank
    ``decay_rank``.  ``qk_activation`` / ``v_activation`` ("none" or "silu") act on the projections, queries are
    multiplied by ``q_scale``.  The output is normed (RMS, eps ``norm_eps``, plain weight ``norm_name``) over all heads
    together (``norm_over`` "heads": weight of n_heads * v_head_dim) or head by head (``"head"``: one weight of
    v_head_dim for all heads), multiplied by ``gate_activation`` ("sigmoid" or "silu") of W_g h, and projected by W_o."""
    hidden: int
    n_heads: int
    head_dim: int
    v_head_dim: int
    prefix: str
    head_decay: Optional[Tuple[float, ...]] = None
    decay_names: Optional[Tuple[str, str, str]] = None
    decay_rank: int = 0
    decay_tau: float = 1.0
    qk_activation: str = "none"
    v_activation: str = "none"
    q_scale: float = 1.0
    norm_over: str = "heads"
    norm_eps: float = 1e-6
    norm_name: str = "norm"
    gate_activation: str = "sigmoid"
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    g_name: str = "g"
    o_name: str = "o"


@dataclass(frozen=True)
class BranchSumSpec(PartSpec):
    """Several mixers side by side on the same input: the result is ``weight`` * sum_i rmsnorm(branch_i(h)) * w_i, each
    branch's output normed over the model width (eps ``norm_eps``) with its own plain weight ``out_norms[i]``.  At most
    one branch may keep keys and values; the branches' states lie one behind the other."""
    hidden: int
    branches: Tuple[PartSpec, ...]
    out_norms: Tuple[str, ...]
    norm_eps: float
    weight: float = 0.5


# ------------------------------------------------------------------ feed-forwards

@dataclass(frozen=True)
class SwiGLUSpec(PartSpec):
    """down(silu(gate(x)) * up(x)), no biases  (pico-engine src/pico_engine/model.py:222-235)."""
    hidden: int
    intermediate: int
    prefix: str
    gate_name: str = "gate_proj"
    up_name: str = "up_proj"
    down_name: str = "down_proj"


@dataclass(frozen=True)
class DenseMLPSpec(PartSpec):
    """down(act(up(x))), no biases.  ``activation``: "relu2" (the square of relu), "gelu_tanh" or "silu"."""
    hidden: int
    intermediate: int
    prefix: str
    activation: str = "relu2"
    up_name: str = "up"
    down_name: str = "down"


@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """down(act(gate(x)) * up(x)), no biases; ``activation`` "gelu_tanh" or "silu"; or "clamped_sigmoid": with g = min(gate(x), ``limit``)
    and u = clamp(up(x), -``limit``, ``limit``) the hidden units are g * sigmoid(``alpha`` * g) * (u + 1).  Tensor names are ``prefix + name``."""
    hidden: int
    intermediate: int
    prefix: str
    activation: str = "silu"
    limit: Optional[float] = None
    alpha: float = 1.702
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"


@dataclass(frozen=True)
class MixtureSpec(PartSpec):
    """``n_experts`` gated feed-forwards (``prefix + expert_name.format(e) + "." + gate/up/down``) of which a token uses
    the ``top_k`` with the largest router logits (``prefix + router_name`` [n_experts, hidden], float32), weighted by the
    softmax over the chosen logits alone.  ``shared_intermediate`` not None: one more expert (``prefix + shared_name``)
    runs for every token and is added, multiplied by sigmoid(w_sg . h) (``shared_gate_name`` [1, hidden]; None: added as it is).
    ``gated`` False: an expert is down(act(up(x))) and has no gate matrix (``activation`` then also takes "relu2").
    ``scores`` "softmax_all": the weights are the chosen experts' entries of the softmax over all experts, not renormalised
    ("softmax_chosen": the softmax over the chosen logits alone); either way they are multiplied by ``route_scale``.
    ``scores`` "sigmoid": a score is the sigmoid of the logit; the choice reads score + ``correction_name`` (a stored vector [n_experts];
    None: the score alone), first among ``n_groups`` equal runs of neighbouring experts (a run counts the sum of its ``group_best``
    largest; only the ``keep_groups`` best runs stay), then the ``top_k`` largest of what stays; the weights are the chosen experts'
    plain scores, not renormalised, times ``route_scale``."""
    hidden: int
    n_experts: int
    top_k: int
    intermediate: int
    prefix: str
    activation: str = "silu"
    shared_intermediate: Optional[int] = None
    router_name: str = "router"
    expert_name: str = "e{}"
    shared_name: str = "shared"
    shared_gate_name: Optional[str] = "shared.sg"
    gated: bool = True
    scores: str = "softmax_chosen"
    route_scale: float = 1.0
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"
    correction_name: Optional[str] = None
    n_groups: int = 1
    keep_groups: int = 1
    group_best: int = 2


# ------------------------------------------------------------------ layers and the model

@dataclass(frozen=True)
class LayerSpec:
    """One block: which parts it has and how they are arranged around the residual stream.

    ``arrangement`` names an entry of ``parts.registry.ARRANGEMENTS``; "pre_norm" is
    x += mixer(norm(x)); x += ffn(norm(x))  (pico-engine src/pico_engine/model.py:167-237); "parallel" is
    x += mixer(norm1(x)) + ffn(norm2(x)), both halves reading the same x; "post_norm" is
    x += scale1 * norm1(mixer(x)); x += scale2 * norm2(ffn(x)): the sublayers read the stream as it is and the norms
    act on their outputs (``mixer_scale`` / ``feed_forward_scale`` name the scale vectors; None: no scale); "sandwich" is
    x += out_norm1(mixer(norm1(x))); x += out_norm2(ffn(norm2(x))) with a norm before and one after each sublayer
    (``mixer_out_norm`` / ``feed_forward_out_norm``).
    Every part is optional: a block without a feed-forward is a mixer-only block (pico-engine's
    recurrent layers are such, src/pico_engine/model.py:389-406), one without a mixer a feed-forward-only
    block, and a half without a norm takes the residual stream as it is.
    """
    mixer: Optional[PartSpec]
    mixer_norm: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    arrangement: str = "pre_norm"
    mixer_input: Optional[PartSpec] = None           # applied to norm(x) before the mixer reads it (a CausalConvAddSpec)
    feed_forward_input: Optional[PartSpec] = None    # the same for the feed-forward
    residual_scale: float = 1.0                      # x += residual_scale * sublayer(norm(x))
    mixer_scale: Optional[str] = None                # "post_norm": tensor [hidden] the normed output of the mixer is multiplied by
    feed_forward_scale: Optional[str] = None         # the same for the feed-forward
    mixer_out_norm: Optional[PartSpec] = None        # "sandwich": the norm of the mixer's output before it is added
    feed_forward_out_norm: Optional[PartSpec] = None  # the same for the feed-forward


@dataclass(frozen=True)
class BigramTableSpec(PartSpec):
    """Added to the embedded token: row (previous * mul_prev + current * mul_cur) mod buckets of ``table`` [buckets + 1,
    hidden]; a sequence's first token takes row ``buckets``.  The previous token is kept per sequence."""
    hidden: int
    buckets: int
    mul_prev: int
    mul_cur: int
    table: str = "bigram"


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  Each entry owns a cache of its own unless ``cache_of``
    names an earlier entry of the schedule, whose cache it then reads without writing."""
    layer: int
    cache_of: Optional[int] = None
    add_embedding: bool = False                      # before this execution, the embedded tokens are added to the stream again
    add_vector: Optional[Tuple[str, int]] = None     # before this execution (and after the line above), row r of tensor "name" is added: (name, r)


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: str                                   # tensor name of the [vocab, hidden] table
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: Optional[str]                              # tensor name of [vocab, hidden]; None: tied to the embedding
    max_positions: int
    stop_token_ids: Tuple[int, ...] = ()
    ignorable_tensors: Tuple[str, ...] = field(default_factory=tuple)   # names a checkpoint may carry unused
    embedding_position: Optional[PartSpec] = None    # added to the embedding by position (a SinusoidAddSpec); None: nothing
    logit_softcap: Optional[float] = None            # logits <- cap * tanh(logits / cap); None: logits as projected
    stream_vectors: Tuple[Tuple[str, int], ...] = ()  # (tensor name, rows): [rows, hidden] tensors whose rows schedule entries add to the stream
    embedding_pairs: Optional[PartSpec] = None       # added to the embedding by (previous token, token) (a BigramTableSpec); None: nothing
    embedding_scale: float = 1.0                     # the embedded token is multiplied by this (the head reads the table as stored)

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if self.embedding_scale != 1.0 and self.embedding_pairs is not None:
            raise ConfigError("an embedding that reads pairs of tokens takes no scale")
        for e, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"schedule[{e}] names layer {entry.layer}, but there are {len(self.layers)} layers")
            if entry.add_vector is not None:
                rows = dict(self.stream_vectors).get(entry.add_vector[0])
                if rows is None or not 0 <= entry.add_vector[1] < rows:
                    raise ConfigError(f"schedule[{e}].add_vector={entry.add_vector} names no row of stream_vectors")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < e:
                    raise ConfigError(f"schedule[{e}].cache_of={entry.cache_of} must name an earlier entry")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule[{e}].cache_of={entry.cache_of} names an entry that owns no cache")
