"""Typed descriptions of a model: what each layer is made of and in which order layers run.

A ``ModelConfig`` is plain data. It never holds tensors and never knows how a part is
computed; the parts registry (``glassbox_b200.parts``) turns each spec into a part.
Every spec class carries a ``kind`` string, which is the key under which its part class is
registered, so a new mixer / feed-forward / norm / position encoding is a new spec dataclass
plus a new registered part class: nothing in this file changes.

Glassbox reads its sizes off one flat ``Config`` struct inside ``forward``
(crates/glassbox-core/src/model.rs:7-55, 216-226); here the same numbers are split up and
handed to the part that uses them, layer by layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model; the message names the key."""


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the first ``rotary_dim`` channels of each head.

    ``pairing`` "half" rotates channel i with channel i + rotary_dim/2 (the Hugging Face
    weight layout, crates/glassbox-core/src/model.rs:110 with interleaved=false); "interleaved" rotates channel 2i
    with channel 2i + 1, at the angle position * theta^(-2i / rotary_dim) formed in float32 on the device.
    """
    theta: float
    rotary_dim: int
    max_position: int
    pairing: str = "half"
    #: None, or a ``RopeRescaleSpec``: the frequencies are stretched for contexts longer than the trained one
    rescale: Any = None
    kind: str = "rope"


@dataclass(frozen=True)
class RopeRescaleSpec:
    """Stretching of a rotation's frequencies by wavelength: with dim(t) = rotary_dim * ln(``original`` / (2 pi t)) /
    (2 ln theta), lo = max(floor(dim(``fast``)), 0), hi = min(ceil(dim(``slow``)), rotary_dim - 1) and ramp_i =
    clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i becomes f_i / ``factor`` * ramp_i + f_i * (1 - ramp_i): pairs
    that turn more than ``fast`` times within the ``original`` context keep their frequency, pairs that turn less than
    ``slow`` times are slowed by ``factor``, the ones between are blended. Sine and cosine carry the factor
    ``magnitude_slope`` * ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float
    magnitude_slope: float = 0.1


@dataclass(frozen=True)
class NoPositionSpec:
    kind: str = "none"


@dataclass(frozen=True)
class RmsNormSpec:
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class UnitOffsetRmsNormSpec:
    """RMSNorm whose stored weight lies around zero: the gain is 1 + weight."""
    eps: float
    kind: str = "rmsnorm_unit_offset"


@dataclass(frozen=True)
class LayerNormSpec:
    """Layer norm with a weight and (``bias`` True) a bias: (x - mean) / sqrt(var + eps) * w + b, var the mean of the
    squared deviations."""
    eps: float
    bias: bool = True
    kind: str = "layernorm"


@dataclass(frozen=True)
class GqaAttentionSpec:
    """Causal grouped-query attention over a paged key/value cache.

    ``window`` None means every earlier key is visible; an integer w means a query at
    position p sees keys p-w+1 .. p. ``scale`` multiplies the scores before softmax.
    """
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: Any
    window: Optional[int] = None
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention over a compressed cache: per token one latent of ``latent_dim`` numbers (RMS-normed with a plain
    gain, ``latent_eps``), from which each head's unrotated key (``nope_dim``) and value (``value_dim``) are linear
    maps, and one rotated key part of ``rope_dim`` numbers shared by all heads. A head's query is [nope_dim unrotated |
    rope_dim rotated]. ``sink`` adds a learned logit per head to the softmax denominator. ``kv_source`` None: the layer
    projects and stores its own latent; otherwise it has no such projection and reads the cache of the layer it names
    (the schedule says which cache layer that is)."""
    num_heads: int
    nope_dim: int
    rope_dim: int
    value_dim: int
    latent_dim: int
    scale: float
    position: Any
    latent_eps: float
    sink: bool = True
    kv_source: Optional[int] = None
    window: Optional[int] = None
    kind: str = "latent_attention"


@dataclass(frozen=True)
class ChannelDeltaSpec:
    """A gated delta-rule mixer with a fixed-size state per head: S [key_dim, value_dim] decays per key channel, is
    corrected towards the token's value along its key, and is read with the query. Queries and keys have
    ``num_kv_heads`` heads shared by groups of value heads; q, k, v pass a causal convolution of ``conv_taps`` taps and
    SiLU; the decay and the output gate come through low-rank maps (``decay_rank``, ``gate_rank``); the read-out is
    RMS-normed per head (``norm_eps``) and gated."""
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    decay_rank: int
    gate_rank: int
    norm_eps: float
    kind: str = "channel_delta"


@dataclass(frozen=True)
class SigmoidAttentionSpec:
    """Causal grouped-query attention whose weights are not a softmax: a visible key weighs sigmoid(q.k * scale + b_head),
    on its own, with a learned number ``b_head`` per query head (``head_bias``). Queries and keys have ``head_dim``
    channels and are RMS-normed per head (``qk_norm_eps``; None: no norm; one gain for all query heads, one for all key
    heads) before ``position`` rotates them; values have ``value_dim`` channels. ``window`` as in ``GqaAttentionSpec``."""
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    position: Any
    window: Optional[int] = None
    qk_norm_eps: Optional[float] = None
    head_bias: bool = True
    kind: str = "sigmoid_attention"


@dataclass(frozen=True)
class SinkAttentionSpec:
    """Causal grouped-query softmax attention without a rotation, whose positions enter through a bias on the distance:
    score(i, j) = q_i . k_j * ``scale`` - r1_h * ln(1 + r2_h * (i - j)) with two learned numbers per query head
    (``distance_bias``). With ``sink`` the softmax's denominator also holds exp(sink_h), a learned logit per head that has no
    key and no value. Queries and keys have ``head_dim`` channels and are RMS-normed per head (``qk_norm_eps``; None: no
    norm; one gain for all query heads, one for all key heads); values have ``value_dim`` channels. ``value_mix``:
    "none"; "source": this layer's values are kept for the step, for later layers to mix in; "mixed": the values become
    (1 - lambda) v + lambda v_source (lambda a learned scalar, v_source the source layer's values of the same token) before
    they are cached. ``output_gate``: head h's output is multiplied by sigmoid(w_gate_h . x), one number per head and
    token, from the same input as the projections. ``window`` as in ``GqaAttentionSpec``."""
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    window: Optional[int] = None
    qk_norm_eps: Optional[float] = None
    distance_bias: bool = True
    sink: bool = True
    value_mix: str = "none"
    output_gate: bool = True
    kind: str = "sink_attention"


@dataclass(frozen=True)
class TalkingAttentionSpec:
    """Causal grouped-query softmax attention whose heads exchange their weights: after the softmax the weights of query
    head h become sum_g ``talk``[h, g] * weight_g (a learned [heads, heads] matrix), and head h applies them to the values
    of its own key/value head. Scores are q . k * ``scale``, then (``softcap`` not None) softcap * tanh(score / softcap).
    ``unit_sink`` adds one to the softmax's denominator: a key of score 0 that has no value and whose share is not mixed.
    ``bias``: q, k and v carry biases, added in the projection. ``position`` rotates the leading channels of queries and
    keys. ``window`` as in ``GqaAttentionSpec``. ``talk`` False leaves the weights as they are."""
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    position: Any
    softcap: Optional[float] = None
    unit_sink: bool = True
    bias: bool = True
    talk: bool = True
    window: Optional[int] = None
    kind: str = "talking_attention"


@dataclass(frozen=True)
class DecayLinearAttentionSpec:
    """Linear attention with one fixed decay per head: q = silu(W_q h), k = silu(W_k h) (heads x head_dim), v = silu(W_v h)
    (heads x value_dim); per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with a float32 state S [head_dim,
    value_dim] per request. The heads' read-outs are RMS-normed together (``norm_eps``, a gain per channel), times
    sigmoid(W_g h), and projected."""
    num_heads: int
    head_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    norm_eps: float
    kind: str = "decay_linear_attention"


@dataclass(frozen=True)
class HeadDeltaSpec:
    """A gated delta-rule mixer with ONE decay per head and token: as ``ChannelDeltaSpec`` (state, convolutions, unit
    vectors, beta, read-out norm per head), but g = exp(-exp(A_log_h) * softplus(w_a_h . x + dt_bias_h)) is one number per
    head, decay and output gate are plain projections of the input, and the gate is silu (``gate`` "silu") or a sigmoid."""
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    gate: str = "silu"
    kind: str = "head_delta"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side that read the same input: the output is ``left_scale`` * left + ``right_scale`` * right.
    Either may keep keys in pages, a state per request, or both."""
    left: Any
    right: Any
    left_scale: float = 1.0
    right_scale: float = 1.0
    kind: str = "parallel"


@dataclass(frozen=True)
class MinGruSpec:
    """minGRU: per channel S_t = (1 - z_t) S_(t-1) + z_t c_t with the gate z_t = sigmoid(W_z h + b_z) and the candidate c_t
    from u = W_x h + b_x (u + 1/2 where u >= 0, sigmoid(u) elsewhere), both functions of the current token alone; the
    output is W_o (S_t * silu(W_g h)). ``width`` channels; the state is float32 and starts at zero."""
    width: int
    kind: str = "mingru"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of ``num_experts`` squared-ReLU feed-forwards of ``expert_size`` hidden units, of which a token uses
    ``top_k``. Scores are sigmoid(router logits) (float32); the choice is made by score + a stored correction
    (``correction`` True), the weights are the chosen scores times ``route_scale``, not renormalised. With ``num_groups``
    > 1 the experts form that many equal runs of neighbours, a run scores the sum of its two best choice scores, and only
    experts of the ``keep_groups`` best runs can be chosen. ``shared_size`` > 0 adds one expert of that size that every
    token uses, times sigmoid(w_gate . h) when ``shared_gate`` is True."""
    num_experts: int
    top_k: int
    expert_size: int
    route_scale: float = 1.0
    num_groups: int = 1
    keep_groups: int = 1
    correction: bool = True
    shared_size: int = 0
    shared_gate: bool = True
    #: "sigmoid": as above. "softmax_chosen": the choice is made by the logits themselves (plus ``router_bias``, a stored
    #: number per expert that is part of the logit) and the weights are the softmax over the chosen logits alone
    scoring: str = "sigmoid"
    router_bias: bool = False
    #: "relu2": W_down relu(W_up h)^2. "clamped_glu": the expert has a gate and an up matrix and computes
    #: W_down (g * sigmoid(``glu_slope`` g) * (u + 1)) with g = min(W_gate h, ``limit``), u = clamp(W_up h, -limit, limit)
    activation: str = "relu2"
    limit: float = 0.0
    glu_slope: float = 1.702
    kind: str = "routed_experts"


@dataclass(frozen=True)
class SquaredReluSpec:
    """Dense feed-forward without a gate: down(relu(up(x))^2)."""
    intermediate_size: int
    kind: str = "relu2"


@dataclass(frozen=True)
class ClampedGluSpec:
    """Dense gated feed-forward with clamped branches and biases: g = min(W_gate x + b_gate, ``limit``),
    u = clamp(W_up x + b_up, -limit, limit), output W_down (g * sigmoid(``slope`` g) * (u + 1)) + b_down. ``bias`` False
    leaves the three biases out."""
    intermediate_size: int
    limit: float
    slope: float = 1.702
    bias: bool = True
    kind: str = "clamped_glu"


@dataclass(frozen=True)
class SwiGluSpec:
    """Dense gated feed-forward: down(silu(gate(x)) * up(x))."""
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class GeluGluSpec:
    """Dense gated feed-forward whose gate passes the tanh form of GELU: down(gelu_tanh(gate(x)) * up(x)) with
    gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))."""
    intermediate_size: int
    kind: str = "gelu_glu"


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token embedding: the float32 residual row of a token is its row of the table, as it is
    (crates/glassbox-core/src/model.rs:228-231). Another kind (a scaled table, a learned position added to it) is
    another registered "embedding" part."""
    kind: str = "embedding"


@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    """Token embedding times a constant: the residual row of a token is its row of the table times ``scale``."""
    scale: float
    kind: str = "scaled_embedding"


@dataclass(frozen=True)
class PositionalEmbeddingSpec:
    """Token embedding plus a learned vector per position: the residual row of a token at position p is its row of the
    table plus row p of a second table of ``max_position`` rows (neither scaled), summed in float32."""
    max_position: int
    kind: str = "positional_embedding"


@dataclass(frozen=True)
class ScaledLmHeadSpec:
    """Output head whose logits carry a constant factor: logits = (hidden states times the head matrix) * ``scale``."""
    scale: float
    kind: str = "scaled_lm_head"


@dataclass(frozen=True)
class LmHeadSpec:
    """Output head: float32 logits = hidden states times the head matrix, no bias, no cap
    (crates/glassbox-core/src/model.rs:359-361). Another kind is another registered "head" part."""
    kind: str = "lm_head"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer and a feed-forward, each behind its norm.

    ``arrangement`` names how they are wired around the residual stream; "pre_norm" is
    x += mixer(norm(x)); x += ffn(norm(x)) (crates/glassbox-core/src/model.rs:251-348).
    """
    mixer: Any
    ffn: Any
    mixer_norm: Any
    ffn_norm: Any
    arrangement: str = "pre_norm"
    #: "sandwich_norm" also norms each branch's output before it joins the residual: x += post(mixer(norm(x))),
    #: x += post(ffn(norm(x))); there ``ffn`` may be None (a layer without a feed-forward)
    mixer_post_norm: Any = None
    ffn_post_norm: Any = None
    #: "branch_norm" norms each branch on the way out only: x += post(mixer(x)), x += post(ffn(x)); the branches read the
    #: residual itself (rounded to the activation dtype); ``mixer_norm`` and ``ffn_norm`` are None, ``ffn`` may be None
    #: "hyper_connections": the residual is ``streams`` rows per token; each branch reads a learned mix of them through
    #: its norm and its output comes back into all of them through a learned matrix (``ModelConfig.residual_streams`` says
    #: the same number for the whole model); ``ffn`` may be None
    streams: int = 0
    #: "hyper_connections" with ``learned_streams`` False has no stream tensors: it reads the plain sum, every stream
    #: keeps itself and takes the branch's output once (with one stream this is the plain residual)
    learned_streams: bool = True
    #: every branch's output is multiplied by this before it joins the residual (arrangement "hyper_connections")
    branch_scale: float = 1.0
    #: taps of a causal convolution over time, per channel, on what the mixer reads: h <- h + conv(h), with the last
    #: taps - 1 inputs kept per request (arrangement "hyper_connections"); 0: none
    mixer_input_conv: int = 0


@dataclass(frozen=True)
class RunSpec:
    """One entry of the execution order.

    ``layer`` indexes ``ModelConfig.layers`` (a layer may be named by several entries and
    then runs several times with the same weights). ``cache`` is the cache layer this run
    reads; with ``writes_cache`` False the run writes nothing of its own and reads what an
    earlier run of this step (or of earlier steps) put into that cache layer.
    """
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position: int
    tie_word_embeddings: bool
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[RunSpec, ...]
    final_norm: Any
    raw: dict = field(default_factory=dict, compare=False, hash=False)
    embedding: Any = EmbeddingSpec()
    head: Any = LmHeadSpec()
    #: 0: one residual row per token. s >= 1: the residual is s rows per token, all equal to the embedding's output at
    #: the start and summed in front of the final norm; every layer then has the arrangement "hyper_connections"
    residual_streams: int = 0

    @property
    def num_cache_layers(self) -> int:
        return 1 + max((r.cache for r in self.schedule), default=-1)

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i, layer in enumerate(self.layers):
            if (layer.arrangement == "hyper_connections") != (self.residual_streams > 0) or \
                    (self.residual_streams > 0 and layer.streams != self.residual_streams):
                raise ConfigError(f"layer {i}: a model with {self.residual_streams} residual streams needs every layer wired "
                                  "for exactly that many (arrangement 'hyper_connections'), and no other model has such layers")
        writers = {}
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"schedule[{i}] names layer {run.layer}, but there are {len(self.layers)} layers")
            if run.cache < 0:
                raise ConfigError(f"schedule[{i}] has a negative cache layer")
            if run.writes_cache:
                if run.cache in writers:
                    raise ConfigError(
                        f"schedule[{i}] and schedule[{writers[run.cache]}] both write cache layer {run.cache}")
                writers[run.cache] = i
            elif run.cache not in writers:
                raise ConfigError(f"schedule[{i}] reads cache layer {run.cache} before any run has written it")
        for c in range(self.num_cache_layers):
            if c not in writers:
                raise ConfigError(f"cache layer {c} is never written")
