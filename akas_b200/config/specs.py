"""Architecture-neutral descriptions of a decoder: what the engine builds from.

An architecture's typed configuration (for instance ``Lfm2Config``) turns itself
into a ``ModelSpec``. The model builder, the cache manager and the weight loader
read only the spec: every size and constant that a part needs is a field here,
chosen layer by layer, so one model may hold different mixers and feed-forwards
in different layers. The order in which layers run is data too (``ModelSpec.schedule``).

A spec of a part is a frozen dataclass with a ``kind`` string; the registries in
``akas_b200.parts.registry`` map that string to the class that implements it.
Parts defined outside this package use ``PartSpec`` directly (kind + free-form
``options``) or their own dataclass with a ``kind`` attribute.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part that this package does not know: its kind and whatever it needs."""

    kind: str
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * (w, or 1 + w when zero_centered)."""

    size: int
    eps: float
    zero_centered: bool = False
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class DynamicTanhSpec:
    """y = tanh(alpha * x) * w + b: a norm that takes no mean and no variance. alpha is one learned number, w and b
    are vectors of ``size``; in the checkpoint alpha and b stand beside the weight as ``<name>.alpha`` and ``<name>.b``."""

    size: int
    kind: str = "dynamic_tanh"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary encoding of the first ``rotary_dim`` channels of each head: channel i turns with channel
    i + rotary / 2 (rotate-half), or, ``interleaved``, channel 2i with channel 2i + 1; the angle of pair i at
    position p is p * theta^(-2i / rotary) either way."""

    head_dim: int
    theta: float
    rotary_dim: Optional[int] = None  # None: the whole head
    kind: str = "rope"
    interleaved: bool = False  # only the general attention kernels take it
    # Long waves slowed, as (factor, low, high, original): with wavelength l = 2 pi / f, a pair keeps its rate f where
    # l < original / high, turns at f / factor where l > original / low, and in between at (1 - s) f / factor + s f with
    # s = (original / l - low) / (high - low). None: every pair keeps its rate.
    scaling: Optional[Tuple[float, float, float, float]] = None
    # Every pair's rate divided by this number (positions stretched evenly). None: rates as they are.
    linear_factor: Optional[float] = None
    # Rates blended by the pair's index, as (factor, original, fast, slow): with
    # d(t) = rotary * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(d(fast)), 0),
    # hi = min(ceil(d(slow)), rotary - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at
    # r_i f_i / factor + (1 - r_i) f_i.
    blend: Optional[Tuple[float, float, float, float]] = None
    amplitude: float = 1.0  # cosine and sine are both multiplied by this number

    @property
    def rotary(self) -> int:
        return self.head_dim if self.rotary_dim is None else self.rotary_dim


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged key/value cache."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qk_norm: Optional[Any] = None  # a norm spec of size head_dim, applied per head before the position encoding
    position: Optional[Any] = None  # a position-encoding spec, or None
    window: Optional[int] = None  # None: every earlier key; w: the last w keys, the query's own included
    scale: Optional[float] = None  # None: head_dim ** -0.5
    kind: str = "attention"
    names: Mapping[str, str] = field(default_factory=dict)  # local parameter name -> name in the checkpoint
    # Options that LFM2 leaves at their defaults. Any of them sends the layer to the general attention kernels.
    v_head_dim: Optional[int] = None  # size of a value head; None: head_dim
    softcap: Optional[float] = None  # score <- cap * tanh(score / cap), after the scale
    distance_bias: bool = False  # score <- score - r1_h * ln(1 + r2_h * (i - j)); r1, r2 are two tensors [heads]
    keep_first: int = 0  # with a window: the first keep_first positions of a request stay visible behind it
    # one more term in the softmax's denominator, without a key or a value: True: exp(0); "learned": exp(sink_h) with
    # a tensor [heads] of logits, which the scale does not touch
    sink: Any = False
    # "head": head h's output times sigmoid(W_g x)_h, W_g [heads, hidden], x the mixer's input; "channel": the
    # concatenated heads times sigmoid(W_g x) element by element, W_g [heads * value_dim, hidden]
    gate: Optional[str] = None
    # The values are the keys as projected (before QK-norm and the position encoding): there is no value matrix, and
    # the value heads have the keys' size.
    values_are_keys: bool = False
    bias: bool = False  # q, k and v have biases (``<name>.b`` beside each matrix), added to the projections in float32
    # False: the layer has no key and value projections; it reads the cache of another layer (the run order names
    # whose), which holds that layer's keys after their rotation and its values, with queries and a mask of its own.
    own_kv: bool = True

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim

    @property
    def general(self) -> bool:
        """Whether the layer needs what only the general attention kernels compute."""
        return bool(self.v_head_dim not in (None, self.head_dim) or self.softcap or self.distance_bias or self.keep_first
                    or self.sink or self.gate or self.values_are_keys or getattr(self.position, "interleaved", False)
                    or self.bias or not self.own_kv)


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose queries, keys and values are projections of low-rank latents; only the key/value latent and one
    rotated key part per token are kept.

    c_q = RMSnorm(W_dq x) [q_rank]; q = W_uq c_q, per head [head_dim plain channels, rope_dim rotated]. W_dkv x has
    kv_rank + rope_dim rows: the first kv_rank, RMS-normed, are the latent c; the last rope_dim, rotated (not normed),
    are a key part that all heads share. Per head the plain key is W_uk c and the value W_uv c;
    score = (q_plain . k_plain + q_rot . k_rot) * scale. ``window``: position i sees j with 0 <= i - j < window
    (None: every earlier key). ``sink``: as for ``AttentionSpec``. ``gate="channel"``: the concatenated heads times
    sigmoid(W_g x), element by element, before the output product; ``gate="head"``: head h's output times
    sigmoid(W_g x)_h with W_g [heads, hidden]. ``q_rank`` None: the queries are one projection of the input,
    q = W_q x (a tensor ``q``), with no latent and no norm of their own."""

    hidden_size: int
    num_heads: int
    head_dim: int
    rope_dim: int
    v_head_dim: int
    q_rank: Optional[int]
    kv_rank: int
    norm_eps: float
    scale: float
    position: Optional[Any] = None  # the rotation of the rope_dim part (a ``RopeSpec`` whose head is that part)
    window: Optional[int] = None
    sink: Any = False
    gate: Optional[str] = None
    kind: str = "latent_attention"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class ShortConvSpec:
    """LFM2's gated causal depthwise convolution with a state of kernel_size-1 rows."""

    hidden_size: int
    kernel_size: int
    bias: bool = False
    kind: str = "short_conv"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class SwiGLUSpec:
    """silu(x W1^T) * (x W3^T), then W2."""

    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class GatedMLPSpec:
    """W_down (act(W_gate x + b_gate) * (W_up x + b_up)) + b_down with ``activation`` one of "gelu_tanh"
    (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))) and "silu"; ``bias``: the three projections have biases
    (``<name>.b``), else none has."""

    hidden_size: int
    intermediate_size: int
    activation: str = "gelu_tanh"
    bias: bool = False
    kind: str = "gated_mlp"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class MLPSpec:
    """W_down act(W_up x) without a gate; ``activation`` one of "relu2" (the square of max(z, 0)), "gelu_tanh", "silu"."""

    hidden_size: int
    intermediate_size: int
    activation: str = "relu2"
    kind: str = "mlp"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention with a decay per key channel: S <- diag(alpha) S + k v^T, o = S^T q, per head.

    alpha = sigmoid(W_a2 (W_a1 x) + b)^(1 / tau) through a low-rank pair of matrices; q is scaled by
    ``key_dim ** -0.5``; each head's o is RMS-normed over ``value_dim`` (plain weight shared by the heads) and the
    concatenated heads are multiplied by silu(W_g x) before the output product."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay_rank: int
    tau: float
    norm_eps: float
    kind: str = "gated_linear_attention"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class DecayedLinearAttentionSpec:
    """Linear attention with one constant decay per head: S <- decay_h S + k v^T, o = S^T (q_scale q), per head.

    q, k [heads x key_dim] and v [heads x value_dim] pass ``activation`` ("silu" or None) after their products. The
    read-out is RMS-normed, over all heads together when ``whole_norm`` (weight [heads * value_dim]), else per head
    (weight [value_dim] shared by the heads; ``norm_weight`` False: the division alone, no tensor), and multiplied by
    ``gate_activation`` ("sigmoid" or "silu") of W_g x before the output product. The state is float32 and starts at
    zero."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    norm_eps: float
    activation: Optional[str] = "silu"
    whole_norm: bool = True
    gate_activation: str = "sigmoid"
    q_scale: float = 1.0
    norm_weight: bool = True
    kind: str = "decayed_linear_attention"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side that read the same input; the result is the sum of ``scale_i * mixer_i(x)``.

    ``branches``: (prefix of the branch's tensors inside the mixer, the branch's spec, its scale). Each branch keeps
    the cache its kind needs. The branches' input matrices are stacked into one product and so are their output
    matrices (the scales ride on the activations), so the branches cost two products together."""

    hidden_size: int
    branches: Tuple[Tuple[str, Any, float], ...]
    kind: str = "parallel_mixer"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of SwiGLU experts W_down (silu(W_gate x) * (W_up x)), ``top`` per token.

    The router has ``num_experts + num_identity`` outputs; the last ``num_identity`` are experts without tensors
    that return their input. Scores are a softmax over all outputs (float32); the choice goes by score plus a
    learned correction, among the outputs of the ``keep_groups`` best of ``groups`` equal groups of neighbours (a
    group's score is its largest choice score); the weights are the chosen outputs' plain scores over their sum.

    Options: ``scoring="sigmoid"``: every output's score is the sigmoid of its logit; ``correction`` False: no
    correction tensor, the choice goes by the plain scores; ``renormalize`` False: the weights are the chosen
    scores as they are; ``weight_on="input"``: the weight multiplies the expert's input, the result is
    sum expert(w x), where otherwise it is sum w expert(x); ``shared_size`` F_s: one more expert of that hidden size
    (tensors ``shared.{gate,up,down}``) that every token passes, added to the sum, and with ``shared_gate`` times
    sigmoid(W_sg x), one number per token (``shared.sg`` [1, hidden])."""

    hidden_size: int
    intermediate_size: int
    num_experts: int
    num_identity: int
    top: int
    groups: int = 1
    keep_groups: int = 1
    scoring: str = "softmax"
    correction: bool = True
    renormalize: bool = True
    weight_on: str = "output"
    shared_size: Optional[int] = None
    shared_gate: bool = False
    kind: str = "routed_experts"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, per head.

    q and k (``num_kv_heads`` heads of ``key_dim``, shared by groups of value heads) and v pass a causal depthwise
    convolution of ``conv_kernel`` taps and silu; q and k are then made unit vectors (``unit_eps`` under the root), q
    times ``key_dim ** -0.5``. beta = sigmoid(W_b x); g = exp(-exp(A_log) * softplus(W_a x + dt_bias)), one per head.
    Each head's o is divided by its root mean square over ``value_dim``, times a weight shared by the heads, times
    silu(W_g x)."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_kernel: int
    norm_eps: float
    unit_eps: float = 1e-6
    kind: str = "gated_delta"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class PolyNormMLPSpec:
    """W_down act(W_up x), act(z) = a N(z) + b N(z^2) + c N(z^3) + e with N the division of a token's row by its
    root mean square (``eps`` under the root) and a, b, c, e four learned numbers."""

    hidden_size: int
    intermediate_size: int
    eps: float
    kind: str = "polynorm_mlp"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One block: which parts it holds, how they are arranged, and where its weights are.

    ``mixer_prefix`` and ``ffn_prefix`` are prepended to the parts' local parameter
    names (``"model.layers.3.self_attn."``); the two norms name their weight whole.
    """

    mixer: Any
    ffn: Any  # None: the layer has no feed-forward (and no norm for it)
    mixer_norm: Any
    ffn_norm: Any
    mixer_prefix: str
    ffn_prefix: str
    mixer_norm_name: str
    ffn_norm_name: Optional[str]
    arrangement: str = "pre_norm"
    # What the "sandwich" arrangement adds: a second norm behind each sublayer, on its result, before the sum:
    # h += mixer_post_norm(mixer(mixer_norm(h))); h += ffn_post_norm(ffn(ffn_norm(h))).
    mixer_post_norm: Any = None
    ffn_post_norm: Any = None
    mixer_post_norm_name: Optional[str] = None
    ffn_post_norm_name: Optional[str] = None
    # What the "parallel" arrangement adds: h += residual_multiplier * (mixer_scale * mixer(n) + ffn_scale * ffn(n))
    # with ONE norm n = mixer_norm(h) that both sublayers read; the two scales are tensors [hidden] (None: ones).
    residual_multiplier: float = 1.0
    mixer_scale_name: Optional[str] = None
    ffn_scale_name: Optional[str] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One call in the run order: layer ``layer`` runs with cache ``cache``.

    ``cache`` names a cache by the index of the schedule entry that owns it; by
    default an entry owns its own cache. An entry whose ``cache`` is another
    entry's index reads that entry's cache and writes nothing into it (the mixer
    is told ``write=False``). Naming a layer in two entries runs its weights twice,
    each time with the cache of its own entry. ``add_embedding``: before the layer runs, the embedding's output (the
    stream as it was in front of the first entry) is added to the stream once more.
    """

    layer: int
    cache: Optional[int] = None
    add_embedding: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    final_norm: Any
    embedding_name: str
    final_norm_name: str
    head_name: Optional[str]  # None: the head is always the embedding
    head_optional: bool = False  # the head tensor may be absent; the embedding is the head then
    schedule: Tuple[ScheduleEntry, ...] = ()
    max_context: int = 128000
    # What some architectures do at the decoder's two ends (LFM2 does none of it): the embedding's rows times a
    # constant; the logits times a constant; then cap * tanh(logits / cap).
    embedding_multiplier: Optional[float] = None
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    # Learned absolute positions: row p of this tensor [max_context, hidden] is added to the embedding of the token at
    # position p (after the multiplier). And a norm of the sum before the first block.
    position_table_name: Optional[str] = None
    embedding_norm: Any = None
    embedding_norm_name: Optional[str] = None

    def run_order(self) -> Tuple[ScheduleEntry, ...]:
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i) for i in range(len(self.layers)))
