"""
Architecture-neutral description of a decoder: what the engine builds a model from.

An architecture's typed configuration (for instance `LlamaConfig`) is turned by its registered
builder into a `ModelSpec`: a list of block definitions (each naming a mixer, a feed-forward, its
norms and an arrangement, every size and constant as a field) and a run list that says in which
order the blocks execute and which cache entry each execution uses.  Nothing below this file knows
which architecture it serves.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """Base of every part description. `kind` selects the implementation in the part registry."""

    kind: str = field(init=False, default="")


@dataclass(frozen=True)
class Llama3Scaling:
    """Frequency rescaling of llama3-type rotary embeddings (reference: model/llama.py:107-128)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotate-half rotary position encoding applied to queries and keys."""

    kind: str = field(init=False, default="rotary")
    head_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    scaling: Llama3Scaling | None = None


@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    kind: str = field(init=False, default="rmsnorm")
    size: int = 0
    eps: float = 1e-6


@dataclass(frozen=True)
class StreamRMSNormSpec(PartSpec):
    """
    RMS norm beside a residual stream that is kept in float32 whatever the activation dtype.  The
    weight that multiplies is `weight_offset` + the stored tensor (1.0: a weight stored around zero);
    `weight_name` is the tensor's name behind the part's prefix ("" where the prefix is the name).
    """

    kind: str = field(init=False, default="rmsnorm_stream")
    size: int = 0
    eps: float = 1e-6
    weight_offset: float = 0.0
    weight_name: str = "weight"


@dataclass(frozen=True)
class YarnScaling:
    """
    YaRN rescaling of rotary frequencies.  With turns(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(turns(fast)), 0), hi = min(ceil(turns(slow)), dims - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i becomes
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by 0.1 ln(factor) + 1.
    """

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class InlineRotarySpec(PartSpec):
    """
    Rotate-half rotation over the first `dims` channels of a head, channel i paired with i + dims/2,
    angle = position * base^(-2i/dims), computed in float32 inside the kernels (no position table,
    so no longest position).  `yarn` rescales the frequencies and magnifies cos and sin; `bands` rescales
    them by wavelength (short waves kept, long ones divided by the factor, a blend in between); at most one
    of the two.
    """

    kind: str = field(init=False, default="rotary_inline")
    dims: int = 0
    base: float = 10000.0
    yarn: YarnScaling | None = None
    bands: Llama3Scaling | None = None


@dataclass(frozen=True)
class LinearRecurrenceSpec(PartSpec):
    """
    Linear attention as a recurrence over a matrix state per request and head:
    S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; each head's o is RMS-normed over its value
    channels, gated by silu of a projection, and projected out.

    `decay`: "head" (one constant per head, `head_decays`) or "channel_logits" (per key channel,
    a = sigmoid(z)^(1/tau) with z a low-rank projection of the input plus a bias).
    """

    kind: str = field(init=False, default="linear_recurrence")
    hidden_size: int = 0
    num_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    q_scale: float = 1.0                 # multiplies q (after rotation)
    k_scale: float = 1.0                 # multiplies k (after rotation)
    decay: str = "head"
    head_decays: tuple[float, ...] = ()
    decay_rank: int = 0                  # inner size of the low-rank decay projection
    tau: float = 1.0
    position: PartSpec | None = None     # rotation of q and k
    out_norm_weight: bool = True         # the norm of o has a weight (shared by the heads)
    out_norm_eps: float = 1e-6


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """
    Softmax attention whose per-head keys and values are up-projections of one cached latent per
    token; queries go through a normed latent of their own (`q_rank` 0: they are a projection of the input,
    tensor `q`); one rotated key part is shared by the heads (`rot_dim` 0: none, and no `position`);
    `output_gate`: the concatenated heads are multiplied by sigmoid(W_g h) before the output projection.
    """

    kind: str = field(init=False, default="latent_attention")
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0                    # unrotated query/key channels a head
    rot_dim: int = 0                     # rotated query/key channels a head
    value_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    window: int = 0                      # 0: every earlier key; w > 0: the last w keys, the query's own included
    norm_eps: float = 1e-6
    position: PartSpec | None = None
    output_gate: bool = False


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Causal grouped-query attention over a paged key/value cache."""

    kind: str = field(init=False, default="attention")
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0            # multiplies q.k before the softmax
    window: int = 0               # 0: every earlier key; w > 0: the last w keys, the query's own included
    position: PartSpec | None = None


@dataclass(frozen=True)
class SinusoidSpec(PartSpec):
    """
    A position vector added to the token embedding as it starts the residual stream: with
    angle_i = position * base^(-2i/size), entry 2i is sin(angle_i) and entry 2i + 1 cos(angle_i).
    Angles are computed in float32 inside the kernel that gathers the embedding rows (no table).
    """

    kind: str = field(init=False, default="sinusoid")
    size: int = 0
    base: float = 10000.0


@dataclass(frozen=True)
class MinGRUSpec(PartSpec):
    """
    Element-wise gated recurrence whose gates read the current token only (a minGRU), `width` channels:
    z = sigmoid(W_z h + b_z), u = W_x h + b_x, c = u + 1/2 where u >= 0 and sigmoid(u) below,
    S_t = (1 - z) S_(t-1) + z c, y = W_o (S_t * silu(W_g h)).  The state (float32, one number a channel
    and request) starts at zero.  `bias`: the tensors `z.b` and `x.b` exist.
    """

    kind: str = field(init=False, default="mingru")
    hidden_size: int = 0
    width: int = 0
    bias: bool = True


@dataclass(frozen=True)
class StreamLayerNormSpec(PartSpec):
    """
    Layer norm with a weight and no bias, (x - mean) / sqrt(mean((x - mean)^2) + eps) * w, beside a
    residual stream kept in float32.  `weight_name` is the tensor's name behind the part's prefix.
    """

    kind: str = field(init=False, default="layernorm_stream")
    size: int = 0
    eps: float = 1e-6
    weight_offset: float = 0.0
    weight_name: str = "weight"


@dataclass(frozen=True)
class GatedAttentionSpec(PartSpec):
    """
    Causal grouped-query softmax attention whose keys and values may differ in head size, with
    optional biases on q, k, v (tensor name + ".b"), an optional RMS norm of q and of k over the whole
    projection (all heads at once, plain weights `q.norm`, `k.norm`) before the rotation, and an
    optional output gate sigmoid(W_g h) on the concatenated heads before the output projection.

    Further options, each off by default: `qk_norm_scope` "head" norms every head of q and of k by
    itself with one weight of head_dim elements shared by the heads; `q_temperature_every` > 0
    multiplies q by 1 + q_temperature_coef * ln(floor((position + 1) / every) + 1);
    `distance_slope_exponent` c > 0 takes slope_h * (i - j) off the score of query i and key j,
    slope_h = 2^(-c (h + 1) / num_heads); `head_bias` adds the number `pb`[h] to every score of head h;
    `weights` "sigmoid" makes a visible key's weight sigmoid(score) without any normalisation over
    the keys; `output_gate_scope` "head" gates with one number a head (`g` is [num_heads, hidden]);
    `chunk` n > 0 lets query i see key j only if floor(i / n) = floor(j / n), positions counted from the
    request's first token; `softcap` c > 0 turns the scaled product into c tanh(q . k * scale / c).
    """

    kind: str = field(init=False, default="gated_attention")
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    scale: float = 0.0
    window: int = 0
    bias: bool = False
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    output_gate: bool = False
    position: PartSpec | None = None
    qk_norm_scope: str = "projection"    # "projection": one norm over all heads' channels; "head": one a head
    q_temperature_coef: float = 0.0
    q_temperature_every: int = 0         # 0: no query temperature
    distance_slope_exponent: float = 0.0  # 0: no distance penalty
    head_bias: bool = False
    weights: str = "softmax"             # "softmax" over the visible keys, or "sigmoid" of each score
    output_gate_scope: str = "channel"   # "channel": a gate a value channel; "head": one a head
    chunk: int = 0                       # 0: no chunks
    softcap: float = 0.0                 # 0: scores are not capped


@dataclass(frozen=True)
class DifferentialAttentionSpec(PartSpec):
    """
    Grouped-query attention whose heads each hold `maps` = 2 score maps over the same values: q has
    num_heads * 2 * head_dim rows and k num_kv_heads * 2 * head_dim, head by head as [map 1 | map 2]; each map is
    a softmax attention of its own (rotation, score scale, `softcap`, `window` and `chunk` as in
    `GatedAttentionSpec`), and a head's output is
        (a_1 - lambda a_2) / sqrt(mean((a_1 - lambda a_2)^2) + norm_eps) * (1 - difference)
    over its value_dim channels (no weight), lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + difference, one number
    for the layer from four tensors of head_dim elements.  `bias`: q, k and v have biases (name + ".b").
    """

    kind: str = field(init=False, default="differential_attention")
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    scale: float = 0.0
    window: int = 0
    chunk: int = 0
    softcap: float = 0.0
    difference: float = 0.0
    norm_eps: float = 1e-6
    bias: bool = False
    position: PartSpec | None = None


@dataclass(frozen=True)
class GatedDeltaRuleSpec(PartSpec):
    """
    Gated delta rule over a matrix state per request and value head:
    S <- diag(a_t) S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t.
    q, k (`num_kv_heads` heads) and v (`num_heads` heads) pass a short causal convolution of
    `conv_taps` taps and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)),
    q also times `q_scale`; beta = sigmoid(W_b h); a = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias))
    per head and key channel; each head's o is RMS-normed (weight shared by the heads) and multiplied
    by sigmoid(W_g2 W_g1 h).  The inner sizes of the two low-rank projections are the checkpoint's
    (`decay_rank`, `gate_rank` only serve to draw random weights).
    """

    kind: str = field(init=False, default="gated_delta_rule")
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    conv_taps: int = 1
    q_scale: float = 1.0
    unit_eps: float = 1e-6
    out_norm_eps: float = 1e-6
    decay_rank: int = 0
    gate_rank: int = 0


@dataclass(frozen=True)
class MatrixLSTMSpec(PartSpec):
    """
    Matrix memory with exponential gating (mLSTM): per head a log input gate i = cap tanh((W_i h + b_i) / cap),
    a log forget gate f = log_sigmoid(cap tanh((W_f h + b_f) / cap)), a running maximum m_t = max(f + m_(t-1), i)
    that starts at 0, S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T, n_t likewise with k alone,
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + denominator_eps); each head's o is RMS-normed, the heads
    concatenated, multiplied by a weight over all heads and by sigmoid(W_g h).
    """

    kind: str = field(init=False, default="mlstm")
    hidden_size: int = 0
    num_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    q_scale: float = 1.0
    gate_cap: float = 15.0
    denominator_eps: float = 1e-6
    out_norm_eps: float = 1e-6


@dataclass(frozen=True)
class ParallelMixerSpec(PartSpec):
    """
    Mixers side by side on one input: sum_b scale_b * mixer_b(h).  `branches` holds (mixer description,
    prefix of its tensors behind the mixer's own prefix, scale).  At most one branch keeps keys and values.
    """

    kind: str = field(init=False, default="parallel")
    branches: tuple[tuple[PartSpec, str, float], ...] = ()


@dataclass(frozen=True)
class PlainMLPSpec(PartSpec):
    """
    Ungated feed-forward down(act(up(x))); `activation` "relu2" is the square of relu; "xielu" is
    softplus(p) z^2 + z/2 for z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2 for z <= 0 with the
    two numbers p, q of the tensor `param_name`.
    """

    kind: str = field(init=False, default="plain_mlp")
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "relu2"
    tensor_names: tuple[str, str] = ("up", "down")
    param_name: str | None = None        # the activation's own numbers, where it has some


@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    kind: str = field(init=False, default="gated_mlp")
    hidden_size: int = 0
    intermediate_size: int = 0
    # "silu": silu(g) * u; "relu": relu(g) * u;
    # "clamped_swish": g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit);
    # "gelu_tanh": g/2 (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) u
    activation: str = "silu"
    limit: float = 0.0
    alpha: float = 1.0
    tensor_names: tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


@dataclass(frozen=True)
class RoutedExpertsSpec(PartSpec):
    """
    `num_experts` gated feed-forward layers of which each token uses the `top` with the largest router
    logits (float32, with a bias), weighted by the softmax over the chosen logits; an optional shared
    expert runs for every token and is added.  `expert` describes one expert (its tensors live under
    `expert_prefix` with the expert's index in place of "{}").
    """

    kind: str = field(init=False, default="routed_experts")
    hidden_size: int = 0
    num_experts: int = 0
    top: int = 1
    expert: GatedMLPSpec | PlainMLPSpec | None = None
    shared: GatedMLPSpec | None = None
    expert_prefix: str = "e{}."
    shared_prefix: str = "shared."
    router_name: str = "router"
    router_bias_name: str | None = "router.b"
    # "softmax_chosen": softmax over the chosen logits; "sigmoid": each chosen expert's sigmoid(logit), not renormalised;
    # "softmax_all": scores are the softmax over ALL router outputs; the choice is made by score + `correction_name`
    # (a tensor, optional) among the experts of the `group_keep` best of `group_count` groups of neighbours (a group's
    # rank is its largest choice score); the weights are the chosen scores (without the correction) divided by
    # their sum + `share_eps`, times `weight_scale`
    scoring: str = "softmax_chosen"
    # "output": the weight multiplies the expert's output; "input": its input (experts without a gate only)
    weight_on: str = "output"
    correction_name: str | None = None
    group_count: int = 1
    group_keep: int = 1
    weight_scale: float = 1.0
    share_eps: float = 0.0
    # the router's last `identity_experts` outputs stand for experts without tensors whose output is their input
    identity_experts: int = 0


@dataclass(frozen=True)
class BlockSpec:
    """
    One layer definition: its parts, how they are wired, and the checkpoint prefix its tensors
    live under.  `arrangement` picks the wiring (the registry of arrangements); "pre_norm" is
    x + mixer(norm(x)) followed by x + ffn(norm(x)) with the adds deferred into the next norm;
    "sandwich_norm" norms each sublayer's output as well, x + norm_b(mixer(norm(x))), around a
    float32 residual stream; "pre_norm_stream" is "pre_norm" around a float32 residual stream.
    """

    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec | None    # None (arrangements that allow it): the block has no feed-forward
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec | None
    prefix: str                      # e.g. "model.layers.3."
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."
    # arrangements that also norm each sublayer's output ("sandwich_norm")
    mixer_post_norm: PartSpec | None = None
    feed_forward_post_norm: PartSpec | None = None
    mixer_post_norm_prefix: str = ""
    feed_forward_post_norm_prefix: str = ""


@dataclass(frozen=True)
class RunEntry:
    """
    One execution of a block.  `block` indexes `ModelSpec.blocks` (the same block may be named by
    several entries: shared weights).  `cache_entry` is the cache/state entry this execution uses;
    entries that share a `cache_entry` share keys and values, and only the one with `writes_cache`
    stores into it (the others read what it stored in the same step).
    """

    block: int
    cache_entry: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: tuple[BlockSpec, ...]
    run: tuple[RunEntry, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_prefix: str
    lm_head_name: str | None         # None: tied to the embedding
    max_positions: int
    eos_token_id: int
    optional_tensors: tuple[str, ...] = ()     # names a checkpoint may carry that the model does not read
    ignored_suffixes: tuple[str, ...] = ()     # tensors whose names end so are skipped (buffers the model recomputes)
    extras: dict[str, Any] = field(default_factory=dict, compare=False)
    embedding_scale: float = 1.0               # multiplies the embedding rows as they start the stream (not the tied head)
    embedding_position: PartSpec | None = None  # a position vector added to the scaled embedding rows (`SinusoidSpec`)
    embedding_norm: PartSpec | None = None     # a norm of the embedding rows before they start the stream (a stream norm's spec)
    embedding_norm_prefix: str = ""            # where its tensors live
    logit_scale: float = 1.0                   # multiplies the logits
    logit_softcap: float = 0.0                 # c > 0: logits <- c tanh(logits / c), after the scale

    @property
    def num_cache_entries(self) -> int:
        return 1 + max((e.cache_entry for e in self.run), default=-1)
