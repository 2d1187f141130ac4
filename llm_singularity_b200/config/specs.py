"""Typed descriptions of a model, one dataclass per kind of part.

An architecture's configuration (read from its own config.json keys) is
translated once into a :class:`ModelSpec`: a list of blocks, each naming its
mixer, feed-forward, norms and position encoding with every size and constant
as a field, plus the order in which the blocks run.  The parts are built from
these specs and never see the architecture's configuration, so no part knows
which model it is in, and two layers of one model may use different parts.

The reference has a single generic ``ModelConfig`` (models/include/models/
model_interface.h:11-23) and hard-wires one layer shape; the spec layer is
what replaces the ``-DMODEL=llama`` compile-time switch (CMakeLists.txt:12,27).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """Base of all part descriptions; ``kind`` selects the implementing class."""

    kind: str = field(init=False, default="")


# --------------------------------------------------------------------------- norms
@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    """``x / sqrt(mean(x^2) + eps) * w``.  ``unit_offset``: the stored weight is the distance from
    one, ``w = 1 + stored``."""

    size: int = 0
    eps: float = 1e-5
    unit_offset: bool = False
    kind: str = field(init=False, default="rmsnorm")


@dataclass(frozen=True)
class GroupRMSNormSpec(PartSpec):
    """RMS norm in ``groups`` equal consecutive parts of the vector, each with its own mean of
    squares, and one weight over the whole vector; one group is the plain RMS norm."""

    size: int = 0
    eps: float = 1e-5
    groups: int = 1
    kind: str = field(init=False, default="group_rmsnorm")


@dataclass(frozen=True)
class LayerNormSpec(PartSpec):
    """``(x - mean) / sqrt(var + eps) * w + b`` with ``var`` the mean of the squared deviations: a
    centred norm with a weight and a bias."""

    size: int = 0
    eps: float = 1e-5
    kind: str = field(init=False, default="layernorm")


# ---------------------------------------------------------------- position encodings
@dataclass(frozen=True)
class Llama3RopeScaling:
    """Frequency-dependent stretching of the rotary wavelengths ("llama3")."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotary position encoding.  ``pairing`` "half" rotates dims (i, i + rotary_dim/2) together,
    "adjacent" rotates dims (2i, 2i + 1); pair i turns by ``pos * theta^(-2i / rotary_dim)``."""

    head_dim: int = 0
    rotary_dim: int = 0           # leading dims of each head that rotate
    theta: float = 10000.0
    scaling: Optional[Llama3RopeScaling] = None
    pairing: str = "half"
    kind: str = field(init=False, default="rotary")


@dataclass(frozen=True)
class NoPositionSpec(PartSpec):
    kind: str = field(init=False, default="none")


# --------------------------------------------------------------------------- mixers
@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Causal softmax attention with grouped keys/values over a paged cache."""

    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0            # multiplies q.k before the softmax
    window: Optional[int] = None  # keys further back than this many are not seen
    position: PartSpec = field(default_factory=NoPositionSpec)
    # score modifiers (this architecture has neither): cap * tanh(s / cap) on the scaled scores, and
    # a linear position bias -slope[h] * distance with the usual geometric slopes over the heads
    logit_softcap: Optional[float] = None
    linear_bias: bool = False
    kind: str = field(init=False, default="attention")


@dataclass(frozen=True)
class LinearRecurrenceSpec(PartSpec):
    """Linear attention with a matrix state per head: ``S <- diag(a) S + b v^T``, ``o = S^T q``.

    ``gate`` says where a and b come from.  "fixed_decay": a is one constant per head (``decay``)
    and b is a key projection; "forget": a is a forget gate per channel with a learnt floor,
    ``a = floor + (1 - floor) * sigmoid(W_f x + bias)``, and ``b = 1 - a`` (no key).  The
    activations of the query, key and value projections, how the output is normed (over all heads
    together, "all", or each head by itself with one weight of head size, "per_head") and whether a
    sigmoid gate projection multiplies it are fields, so that relatives of the two shipped kinds
    (``lightning`` and ``hgrn2``) are other settings of the same part."""

    hidden_size: int = 0
    num_heads: int = 0
    key_dim: int = 0              # per head: channels of q (and of k or the forget gate)
    value_dim: int = 0            # per head
    gate: str = "fixed_decay"
    decay: Tuple[float, ...] = ()
    q_activation: str = "silu"
    k_activation: str = "silu"
    v_activation: str = "none"
    out_norm: str = "all"
    out_gate: bool = False
    eps: float = 1e-5
    kind: str = field(init=False, default="linear_recurrence")


@dataclass(frozen=True)
class KVAttentionSpec(PartSpec):
    """Softmax attention with grouped keys/values over a paged cache whose keys (``key_dim``, shared
    with the queries) and values (``value_dim``) have sizes of their own.  What may stand between the
    projections and the scores, each optional: biases on q, k and v (``qkv_bias``); an RMS norm per
    head of q and of k with one weight of head size each (``qk_norm``, ``eps``), before the rotation;
    a query temperature, ``q *= 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)`` (``temp_every``
    0: none); a rotation (``position``).  A query sees the keys not after it that lie within
    ``window`` positions (None: all) and in its own chunk of ``chunk`` positions counted from the
    start of the sequence (None: no chunks).  ``out_gate``: the heads' outputs are multiplied by
    sigmoid(W_g x) before the output projection; with ``gate_per_head`` W_g has one row per head and
    the gate is one number per head.  ``qk_norm_span`` "all": the norm of q (and of k) is one RMS
    norm over all heads at once, before they are split, with a weight as long as the projection.
    ``v_unit_norm``: each value head is divided by its root mean square (``eps``, no weight) and
    cached so.  ``sink``: one is added to the softmax's denominator, a place with score 0 and no
    value, so that a row's weights may sum to less than one.  ``logit_softcap``: a scaled score s
    becomes ``cap * tanh(s / cap)``.  ``linear_bias``: head h's score for a key d positions back then
    loses ``2^(-8 (h + 1) / heads) * d``.  ``value_mix``: layers of one model that name the same
    ``value_mix_key`` share values within a token; the "source" layer (the first of them) caches its
    values as they are and lends them to the others for the step, a "mixed" layer caches
    ``(1 - lambda) v + lambda v_source`` with its own learnt number ``vmix``."""

    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    scale: float = 0.0
    window: Optional[int] = None
    chunk: Optional[int] = None
    logit_softcap: Optional[float] = None
    linear_bias: bool = False
    value_mix: Optional[str] = None
    value_mix_key: str = "v_first"
    qkv_bias: bool = False
    qk_norm: bool = False
    eps: float = 1e-5
    temp_coef: float = 0.0
    temp_every: int = 0
    out_gate: bool = False
    position: PartSpec = field(default_factory=NoPositionSpec)
    qk_norm_span: str = "head"
    v_unit_norm: bool = False
    sink: bool = False
    gate_per_head: bool = False
    kind: str = field(init=False, default="kv_attention")


@dataclass(frozen=True)
class MatrixMemorySpec(PartSpec):
    """A matrix memory per head with an exponential input gate (the mLSTM cell).  With q scaled by
    ``key_dim^-1/2``, log gates ``i = cap tanh((W_i x + b_i) / cap)`` and ``f = logsigmoid(cap
    tanh((W_f x + b_f) / cap))`` per head, and a running maximum m that starts at 0:

        m_t = max(f + m_(t-1), i)
        S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T        n_t likewise with k alone
        o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

    Each head's o is brought to unit rms (``eps``), the heads are concatenated and multiplied by one
    weight over all of them and by sigmoid(W_g x) (``out_gate``), then projected by W_o."""

    hidden_size: int = 0
    num_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    gate_cap: float = 15.0
    out_gate: bool = True
    eps: float = 1e-5
    kind: str = field(init=False, default="matrix_memory")


@dataclass(frozen=True)
class GatedDeltaSpec(PartSpec):
    """A delta-rule memory with one fade and one write strength per head and token (the gated delta
    rule).  q and k have ``num_key_heads`` heads of ``key_dim`` (value head h reads key head
    ``h // (num_heads / num_key_heads)``), v has ``num_heads`` heads of ``value_dim``.  Each of q, k, v
    passes a causal convolution over time per channel (``conv_taps`` taps, zeros before the start)
    and silu; q and k become unit vectors per head (``x / sqrt(sum x^2 + unit_eps)``), q also times
    ``key_dim^-1/2``.  ``beta = sigmoid(W_b x)``, ``g = exp(-exp(A_log) * softplus(W_a x + dt_bias))``;

        S <- g S;  e = beta (v - S^T k);  S <- S + k e^T;  o = S^T q

    Each head's o is divided by its root mean square (``eps``), times one weight of ``value_dim``
    shared by the heads, times silu(W_g x), then projected by W_o."""

    hidden_size: int = 0
    num_heads: int = 0
    num_key_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    conv_taps: int = 1
    eps: float = 1e-5
    unit_eps: float = 1e-6
    kind: str = field(init=False, default="gated_delta")


@dataclass(frozen=True)
class ChannelDeltaSpec(PartSpec):
    """A delta-rule memory with a decay and a removal rate per key channel (the generalized delta
    rule).  r, k and v have ``num_heads`` heads of ``key_dim``.  With the unit key
    ``u = k / sqrt(sum k^2 + unit_eps)``, the decay ``w = exp(-decay_rate * sigmoid(W_w2 tanh(W_w1 x)
    + w0))`` (a projection through ``decay_rank`` hidden values) and ``a = sigmoid(W_a x + a_bias)``:

        S <- diag(w) S - (a * u) (u^T S) + k v^T   (both terms read the state the token found)
        o = S^T r

    Each head's o is divided by its root mean square (``eps``), the heads are concatenated, times
    one weight over all of them, times sigmoid(W_g x), then projected by W_o."""

    hidden_size: int = 0
    num_heads: int = 0
    key_dim: int = 0
    decay_rank: int = 0
    decay_rate: float = 0.6065306597126334          # e^(-1/2)
    eps: float = 1e-5
    unit_eps: float = 1e-6
    kind: str = field(init=False, default="channel_delta")


@dataclass(frozen=True)
class ParallelMixerSpec(PartSpec):
    """Mixers side by side on one input.  ``combine`` "normed_mean": each branch's result is
    RMS-normed over the model width with a weight of its own (``eps``), and the mean of those is
    the mixer's result; "weighted_sum": the results are added with the fixed factors ``scales``, no
    norm and no parameters.  ``names`` are the branches' names in parameter paths."""

    hidden_size: int = 0
    branches: Tuple[PartSpec, ...] = ()
    names: Tuple[str, ...] = ()
    eps: float = 1e-5
    combine: str = "normed_mean"
    scales: Tuple[float, ...] = ()
    kind: str = field(init=False, default="parallel")


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """Causal softmax attention whose keys and values are made per head from one cached latent
    vector per token, plus one rotated key part that all heads share.  Queries come through a
    normed latent of their own.  ``reads_only``: the layer has no latent projection and reads
    the cache another layer of the same shape writes.  ``gate_per_head``: head h's output is
    multiplied by ``sigmoid(W_g x)_h``, W_g with one row per head."""

    hidden_size: int = 0
    num_heads: int = 0
    plain_dim: int = 0            # per head: query/key dims without rotation
    rot_dim: int = 0              # query/key dims that carry the position
    value_dim: int = 0            # per head
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    eps: float = 1e-5
    reads_only: bool = False
    position: PartSpec = field(default_factory=NoPositionSpec)
    gate_per_head: bool = False
    kind: str = field(init=False, default="latent_attention")


@dataclass(frozen=True)
class RGLRUSpec(PartSpec):
    """A recurrent block with a real-gated linear recurrent unit.  Two branches of ``width``:
    ``y = gelu_tanh(W_y x + b_y)`` and ``u = conv(W_x x + b_x)``, a causal convolution per channel over
    ``conv_taps`` tokens with a bias.  u is cut into ``blocks`` equal parts; in part b
    ``r = sigmoid(R_b u_b + b_r)`` and ``i = sigmoid(I_b u_b + b_i)`` with square matrices R_b, I_b.  Then

        a = exp(-rate * r * softplus(lam));   S <- a S + sqrt(1 - a^2) * i * u;   out = W_o (S * y)

    with S zero when a sequence begins, one number per channel, 32-bit."""

    hidden_size: int = 0
    width: int = 0
    blocks: int = 1
    conv_taps: int = 1
    rate: float = 8.0
    kind: str = field(init=False, default="rglru")


# -------------------------------------------------------------------- feed-forwards
@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """down( act(gate(x)) * up(x) ), dense, no bias.  ``activation`` "capped_glu" with ``limit`` L is
    ``min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1)`` for gate g and up u."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    limit: float = 0.0
    kind: str = field(init=False, default="gated_mlp")


@dataclass(frozen=True)
class DenseMLPSpec(PartSpec):
    """down( act(up(x)) ), dense, no gate and no bias.  ``activation`` "bent_square" is a two-branch
    activation with two learnt numbers p and q stored with the layer: ``softplus(p) z^2 + z/2`` for
    z > 0 and ``(1/2 + softplus(q)) (e^z - 1 - z) + z/2`` for z <= 0; "silu", "gelu_tanh" and "none"
    need no parameter."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "bent_square"
    kind: str = field(init=False, default="dense_mlp")


@dataclass(frozen=True)
class MoESpec(PartSpec):
    """Routed gated experts, no bias: ``sum over the chosen e of down_e(act(gate_e u) * up_e u)``.

    Router logits are 32-bit; ``score`` turns them into scores ("sigmoid", or "softmax" over all
    experts); the ``top`` largest are chosen; ``renormalize`` divides the chosen scores by their
    sum.  ``weight_on`` says what a score multiplies: the expert's "input" (``u = s x``) or its
    "output".  ``choice_bias``: a learnt number per expert is added to the scores for the choice only
    (the weights are the scores without it).  The chosen scores are divided by their sum +
    ``renorm_eps`` and multiplied by ``weight_scale``.  ``limit`` belongs to the activation
    "capped_glu" (see ``GatedMLPSpec``).  ``shared``: a gated feed-forward that every token passes
    besides its chosen experts; its result is added."""

    hidden_size: int = 0
    expert_size: int = 0
    num_experts: int = 0
    top: int = 1
    activation: str = "silu"
    score: str = "sigmoid"
    renormalize: bool = False
    weight_on: str = "input"
    choice_bias: bool = False
    weight_scale: float = 1.0
    renorm_eps: float = 0.0
    limit: float = 0.0
    shared: Optional[GatedMLPSpec] = None
    kind: str = field(init=False, default="moe")


@dataclass(frozen=True)
class TokenSideSpec(PartSpec):
    """A second, narrow embedding of the token that enters a block after its feed-forward:
    ``x += unit(proj(act(gate x) * e)) * w`` with ``e`` this block's ``dim`` columns (from
    ``offset``) of a table held beside the embedding, and ``unit`` the division by the root
    mean square."""

    hidden_size: int = 0
    dim: int = 0
    offset: int = 0
    activation: str = "gelu_tanh"
    eps: float = 1e-5
    kind: str = field(init=False, default="token_side")


# --------------------------------------------------------------------------- blocks
@dataclass(frozen=True)
class BlockSpec(PartSpec):
    """x += mixer(norm1(x)); x += ffn(norm2(x))   (the "pre_norm" arrangement).  ``ffn`` None: the
    block has its first sublayer only."""

    mixer: PartSpec = None
    ffn: Optional[PartSpec] = None
    mixer_norm: PartSpec = None
    ffn_norm: Optional[PartSpec] = None
    kind: str = field(init=False, default="pre_norm")


@dataclass(frozen=True)
class PostNormBlockSpec(PartSpec):
    """x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ffn(x))   (the "post_norm" arrangement:
    the sublayers read the stream itself, the norm follows the sum).  ``ffn`` None: no second
    step.  ``gated_residual``: each sublayer's result is multiplied by ``sigmoid(W x + b)`` of the
    sublayer's input before the sum.  ``side``: a per-token input added last."""

    mixer: PartSpec = None
    ffn: Optional[PartSpec] = None
    mixer_norm: PartSpec = None
    ffn_norm: Optional[PartSpec] = None
    alpha: float = 1.0
    gated_residual: bool = False
    hidden_size: int = 0
    side: Optional[TokenSideSpec] = None
    kind: str = field(init=False, default="post_norm")


@dataclass(frozen=True)
class SandwichBlockSpec(PartSpec):
    """x += mult * post1(mixer(norm1(x))); x += mult * post2(ffn(norm2(x)))   (the "sandwich_norm"
    arrangement: a norm in front of and behind every sublayer).  ``ffn`` None: no second step."""

    mixer: PartSpec = None
    ffn: Optional[PartSpec] = None
    mixer_norm: PartSpec = None
    mixer_post_norm: PartSpec = None
    ffn_norm: Optional[PartSpec] = None
    ffn_post_norm: Optional[PartSpec] = None
    residual_mult: float = 1.0
    kind: str = field(init=False, default="sandwich_norm")


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``block`` indexes ``ModelSpec.blocks``; a block may be named more than once.
    ``cache`` is the id of the cache (pages or state) the mixer uses in this
    call, ``writes_cache`` says whether the call appends this step's tokens to
    it or only reads what an earlier call of the same step wrote (a layer that
    reads another layer's keys and values).
    """

    block: int
    cache: int
    writes_cache: bool = True
    # row of the model's step vectors (``ModelSpec.step_vectors`` rows of model width) that is added
    # to the stream right before this call: the number of the pass a looped stretch begins here
    step: Optional[int] = None


# ---------------------------------------------------------------------------- model
@dataclass(frozen=True)
class EmbeddingSpec(PartSpec):
    vocab_size: int = 0
    hidden_size: int = 0
    side_size: int = 0            # columns of a second table of per-token inputs for the blocks (0: none)
    scale: float = 1.0            # multiplies the looked-up row on its way into the stream
    # a second table of ``pair_buckets`` + 1 rows, added: row (previous token * pair_mul_prev + token *
    # pair_mul_cur) mod pair_buckets, the last row for a sequence's first token (0 buckets: no such table)
    pair_buckets: int = 0
    pair_mul_prev: int = 0
    pair_mul_cur: int = 0
    kind: str = field(init=False, default="embedding")


@dataclass(frozen=True)
class HeadSpec(PartSpec):
    """Final norm followed by the projection to the vocabulary."""

    vocab_size: int = 0
    hidden_size: int = 0
    tied: bool = False            # reuse the embedding table as the projection
    norm: PartSpec = None
    logit_softcap: Optional[float] = None     # logits <- cap * tanh(logits / cap)
    kind: str = field(init=False, default="lm_head")


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    embedding: EmbeddingSpec
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    head: HeadSpec
    # checkpoint tensor name -> (owner path, local parameter name); owner paths are
    # "embedding", "head", "head.norm", "blocks.<i>.mixer", "blocks.<i>.ffn",
    # "blocks.<i>.mixer_norm", "blocks.<i>.ffn_norm", "steps".
    tensor_names: Tuple[Tuple[str, Tuple[str, str]], ...]
    # names that may be present in a checkpoint and are skipped without complaint
    ignorable: Tuple[str, ...] = ()
    stop_token_ids: Tuple[int, ...] = ()
    max_position_embeddings: int = 0
    step_vectors: int = 0         # rows of the table of vectors that run-order entries add to the stream

    @property
    def num_caches(self) -> int:
        return 1 + max((c.cache for c in self.order), default=-1)
