"""Typed descriptions of a decoder: what each layer is made of and in which order layers run.

These dataclasses are the only thing the engine knows about a model.  An
architecture's config class (for instance ``Qwen3Config``) turns its own
``config.json`` keys into a ``ModelSpec``; the parts, the cache and the step
function are built from the spec and never ask which architecture it came from.

Every spec carries a ``kind`` string.  ``starter_b200.parts.registry`` maps a
kind to the class that implements it, so a new mixer, feed-forward, norm or
position encoding is a new spec dataclass plus one registry entry.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    """Root-mean-square norm ``x / sqrt(mean(x^2) + eps) * gain``.  ``unit_offset`` false: the stored
    weight is the gain; true: the weight is stored around zero and the gain is ``1 + weight``.  ``gain_32bit``: the
    gain is held in float32 on the device however it is stored (for kernels that norm a float32 stream)."""

    size: int
    eps: float
    kind: str = "rmsnorm"
    unit_offset: bool = False
    gain_32bit: bool = False


@dataclass(frozen=True)
class LayerNormSpec:
    """Layer norm with a gain and no bias: ``(x - mean) / sqrt(mean((x - mean)^2) + eps) * gain``."""

    size: int
    eps: float
    kind: str = "layernorm"


@dataclass(frozen=True)
class DynamicTanhSpec:
    """Dynamic Tanh in a norm's place: ``tanh(alpha * x) * weight + bias`` with a scalar ``alpha``; it
    takes no statistics of the row."""

    size: int
    kind: str = "dynamic_tanh"


@dataclass(frozen=True)
class RopeSpec:
    """Half-split rotary position encoding over the whole head."""

    head_dim: int
    theta: float
    kind: str = "rope"


@dataclass(frozen=True)
class InterleavedRopeSpec:
    """Rotary positions that turn entry ``2i`` with entry ``2i + 1`` of the first ``dims`` entries of a
    vector by the angle ``position * base ** (-2i / dims)``; entries from ``dims`` on pass unchanged."""

    dims: int
    base: float
    kind: str = "rope_interleaved"


@dataclass(frozen=True)
class PartialRopeSpec:
    """Rotary positions that turn entry ``i`` with entry ``i + dims / 2`` of the first ``dims`` entries of a
    vector by the angle ``position * base ** (-2i / dims)``; entries from ``dims`` on pass unchanged."""

    dims: int
    base: float
    kind: str = "rope_partial"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a key/value cache.

    ``window`` is ``None`` for attention over all keys, or the number of most
    recent keys (the query's own included) a query may see.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qk_norm: bool
    qk_norm_eps: float
    position: Optional[RopeSpec]
    window: Optional[int] = None
    kind: str = "attention"


@dataclass(frozen=True)
class QueryTemperatureSpec:
    """Queries at position ``p`` are multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``."""

    coef: float
    every: int


@dataclass(frozen=True)
class DifferentialAttentionSpec:
    """Causal grouped-query attention with two softmax maps per head over the same values.

    A query head has two query vectors of ``head_dim`` each and a key/value head two key vectors and
    one value vector of ``value_dim``; the head's output is ``a1 - lambda * a2`` with ``lambda =
    exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init`` (four learnt vectors of ``head_dim``), divided by
    its root mean square over ``value_dim`` (``norm_eps`` inside the root, no gain) and multiplied by
    ``1 - lambda_init``.  ``bias``: q, k, v and the output projection have biases.  ``gated``: the
    concatenated heads are multiplied by ``sigmoid(g(x))`` before the output projection.
    ``own_kv`` false: the layer has no key and value projections and attends over the cache entry
    another layer fills (the run order says which).  No rotation; ``q_temperature`` or None.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    lambda_init: float
    norm_eps: float
    q_temperature: Optional[QueryTemperatureSpec] = None
    bias: bool = True
    gated: bool = True
    own_kv: bool = True
    window: Optional[int] = None
    position: Optional[RopeSpec] = None
    kind: str = "differential_attention"


@dataclass(frozen=True)
class SinkAttentionSpec:
    """Causal grouped-query attention without rotation, whose positions enter through the scores and the
    mask.  Each of the four is optional:

    ``distance_penalty``: ``r1_h * ln(1 + r2_h * (i - j))`` is taken off the scaled score of query ``i`` and
    key ``j`` (two learnt numbers per head).  ``chunk``: a query sees only the keys of its own chunk of
    that many positions, chunks counted from position 0 of the sequence; ``window``: only the most recent
    that many keys, its own included.  ``sink``: the softmax's denominator holds one more term
    ``exp(sink_h)`` (a learnt number per head) that has no value.  ``head_gate``: a head's output is
    multiplied by ``sigmoid(g_h . x)``, one learnt vector per head, read from the mixer's own input.
    Keys have ``head_dim`` entries, values ``value_dim``.

    ``fixed_sink`` (a number; needs ``sink`` false): the extra term is ``exp(fixed_sink)`` for every head and the
    layer has no sink tensor.  ``position`` (an ``InterleavedRopeSpec``): queries and keys are turned by their
    positions before they are scored.  ``values_from_keys``: the layer has no value projection; a key/value head's
    value is its key as projected, before any rotation (``value_dim`` = ``head_dim``)."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    distance_penalty: bool = True
    sink: bool = True
    head_gate: bool = True
    chunk: Optional[int] = None
    window: Optional[int] = None
    position: Optional[object] = None
    fixed_sink: Optional[float] = None
    values_from_keys: bool = False
    kind: str = "sink_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are up-projections of one cached low-rank latent per token.

    Queries: ``W_uq`` of the RMS-normed ``q_rank`` latent ``W_dq h``; a head's query has ``head_dim`` plain
    and ``rot_dim`` rotated entries.  Keys and values: ``W_dkv h`` gives ``kv_rank`` entries, RMS-normed
    into the latent ``c``, and ``rot_dim`` more, rotated, that all heads share as the rotated key part; a
    head's plain key is ``W_uk c``, its value ``W_uv c`` (``value_dim`` entries).  The cache holds ``c``
    and the rotated part.  ``window``: a query sees itself and the ``window - 1`` tokens before it (None:
    all).  ``own_kv`` false: no ``W_dkv``; the layer reads the cache entry of another layer (the run order
    says which) with its own ``W_uk`` and ``W_uv``.  The inner norms have plain gains."""

    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    norm_eps: float
    #: how the rotated parts turn: ``InterleavedRopeSpec`` (entry 2i with 2i + 1) or ``PartialRopeSpec``
    #: (entry i with i + dims / 2)
    position: Optional[object]
    window: Optional[int] = None
    own_kv: bool = True
    kind: str = "latent_attention"


@dataclass(frozen=True)
class WkvSpec:
    """A linear recurrence with a ``head_dim x head_dim`` state per head (the time mixing of the RWKV
    family): receptance, key, value, gate and decay each read their own mix of the token's input and the
    previous token's; the decay of a key channel is ``exp(-exp(w2 tanh(w1 mix) + w0))`` with a low-rank
    ``w1``/``w2`` of ``decay_rank``; the current token's ``k v^T`` enters its own output through a bonus
    vector; each head's output is divided by its root mean square (``norm_eps``), scaled by a gain and by
    ``silu`` of the gate."""

    hidden_size: int
    num_heads: int
    head_dim: int
    decay_rank: int
    norm_eps: float
    kind: str = "wkv"


@dataclass(frozen=True)
class GatedLinearRecurrenceSpec:
    """Two branches of ``width`` channels: ``y = gelu_tanh(W_y h + b_y)`` and ``u = conv(W_x h + b_x)``, a causal
    convolution per channel over ``conv`` taps with a bias.  ``u`` in ``blocks`` equal parts, each with two square
    matrices and biases: ``r = sigmoid(ra u + b)``, ``i = sigmoid(ri u + b)``; per channel ``a = exp(-decay_scale * r *
    softplus(lam))`` and the state ``S <- a S + sqrt(1 - a^2) i u`` from zero, every token alike; the output is
    ``W_o (S * y)``.  The state and the convolution's last ``conv - 1`` inputs are kept per sequence in 32-bit."""

    hidden_size: int
    width: int
    blocks: int
    conv: int
    decay_scale: float = 8.0
    kind: str = "gated_linear_recurrence"


@dataclass(frozen=True)
class StateSpaceSpec:
    """A selective state-space recurrence with a ``state x head_dim`` matrix per head.  One projection gives ``[z |
    x | B | C | dt]`` (``inner = heads * head_dim`` gate entries, as many inputs, ``groups * state`` entries each of B
    and C, a step per head); x, B and C pass a causal convolution per channel (``conv`` taps, bias) and silu; ``dt <-
    softplus(dt + dt_bias)``; per head (its group: ``head / (heads / groups)``) ``S <- exp(-exp(A_log) dt) S + dt B
    x^T``, ``y = S^T C + D x``; ``y * silu(z)`` is RMS-normed in ``norm_groups`` equal parts with a gain, then the
    output projection.  State and convolution inputs are kept per sequence in 32-bit."""

    hidden_size: int
    num_heads: int
    head_dim: int
    state: int
    groups: int
    conv: int
    norm_groups: int
    norm_eps: float
    kind: str = "state_space"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule with a ``head_dim x value_dim`` matrix per head.  Queries and keys have ``num_kv_heads``
    heads (value head ``h`` reads ``h / (num_heads / num_kv_heads)``); q, k and v each pass a causal convolution per
    channel (``conv`` taps, no bias) and silu; q and k are made unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``),
    q times ``head_dim ** -0.5``; ``beta = sigmoid(W_b h)``, ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))`` per
    head; per token ``S <- g S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``; each head's ``o`` is
    RMS-normed with a gain of ``value_dim`` entries shared by the heads and multiplied by ``silu(W_g h)``, then the
    output projection."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    conv: int
    norm_eps: float
    kind: str = "gated_delta"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side that read the same input: the result is half the sum of their outputs, each first
    RMS-normed over the model width with a plain gain of its own."""

    hidden_size: int
    left: object
    right: object
    norm_eps: float
    kind: str = "parallel"

    @property
    def position(self):
        """The position spec of the side that has one (the model builds the tables from it)."""
        return getattr(self.left, "position", None) or getattr(self.right, "position", None)


@dataclass(frozen=True)
class BiasedFeedForwardSpec:
    """Dense feed-forward with biases on both projections: ``down(act(up(x) + b_up)) + b_down``;
    ``activation`` ``"relu2"`` is the square of relu.  ``bias`` false: no biases, ``down(act(up(x)))``."""

    hidden_size: int
    intermediate_size: int
    activation: str = "relu2"
    bias: bool = True
    kind: str = "dense_biased"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of ``experts`` small feed-forwards without biases, of which a token uses the ``top`` with
    the largest router logits (``router(x)``, plus a bias when ``router_bias``, in 32-bit).

    ``scoring`` ``"softmax_top"``: the weights are the softmax over the chosen logits alone;
    ``"sigmoid_normalised"``: the chosen experts' ``sigmoid(logit)`` divided by their sum (+ 1e-20), times
    ``weight_scale``.  ``expert`` ``"gated_clamped"``: ``down(g * sigmoid(1.702 g) * (u + 1))`` with ``g =
    min(gate(x), limit)``, ``u = clamp(up(x), -limit, limit)``; ``"relu2"``: ``down(relu(up(x))^2)``, no gate
    and no limit; ``"gated_silu"``: ``down(silu(gate(x)) * up(x))``, no limit.

    ``scoring`` ``"softmax_all"``: the scores are the softmax over ALL router outputs; the choice goes by
    ``score + correction`` (a stored vector, ``correction`` true) among the experts of the ``group_keep`` of
    ``group_count`` equal groups of neighbouring experts whose largest such number is largest (``group_count`` 1:
    among all); the weights are the chosen experts' plain scores over their sum (+ 1e-20), times ``weight_scale``.

    ``identity_experts``: the router has that many outputs more than there are experts; one of those, chosen,
    stands for an expert that hands its input on (times its weight) and has no tensors.  Groups are formed over
    experts and identity experts together.  ``shared_size`` > 0: a gated expert of that inner size (``"gated_silu"``
    form) runs for every token and is added times ``sigmoid(sg . x)``, one learnt vector."""

    hidden_size: int
    intermediate_size: int
    experts: int
    top: int
    limit: float = 0.0
    expert: str = "gated_clamped"
    scoring: str = "softmax_top"
    weight_scale: float = 1.0
    router_bias: bool = True
    correction: bool = False
    group_count: int = 1
    group_keep: int = 1
    identity_experts: int = 0
    shared_size: int = 0
    kind: str = "routed_experts"


@dataclass(frozen=True)
class ClampedGatedFeedForwardSpec:
    """Dense gated feed-forward with clamps: ``down(g * sigmoid(1.702 g) * (u + 1))`` with ``g = min(gate(x),
    limit)`` and ``u = clamp(up(x), -limit, limit)``; no biases."""

    hidden_size: int
    intermediate_size: int
    limit: float
    kind: str = "gated_clamped"


@dataclass(frozen=True)
class DepthAverageSpec:
    """How a layer stands in a float32 residual stream that is joined over depth: its sublayers' outputs
    enter the stream times ``multiplier``, and behind the layer the stream becomes the weighted sum of the
    embedding output and of all ``levels - 1`` layer results so far (``levels`` learnt weights, the
    embedding's first)."""

    levels: int
    multiplier: float = 1.0
    kind: str = "depth_average"


@dataclass(frozen=True)
class HyperConnectionSpec:
    """How one sublayer reads from and writes to ``streams`` residual streams: ``in`` and ``out``
    vectors of that length and a ``[from, to]`` mixing matrix."""

    streams: int
    kind: str = "hyper"


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    """Dense gated feed-forward: ``down(act(gate(x)) * up(x))``."""

    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    kind: str = "gated_dense"


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: named part specs and the arrangement that puts them together.

    ``parts`` maps a part's name inside the layer to its spec.  Which names there are and to which
    family each belongs (mixer, feed_forward, norm ...) is the arrangement's business: the pre-norm
    block wants ``mixer``, ``feed_forward``, ``norm1`` and ``norm2``; an arrangement with a third norm,
    without a feed-forward or with two mixers names its own.  ``names`` maps each part's logical
    parameter name (``"mixer.q"``, ``"norm1.weight"`` ...) to the tensor name in the checkpoint.
    """

    parts: dict
    names: dict
    arrangement: str = "prenorm"

    def __getattr__(self, name):
        # layer.mixer, layer.norm1 ...: the spec of the part of that name
        parts = object.__getattribute__(self, "parts")
        if name in parts:
            return parts[name]
        raise AttributeError(f"this layer has no part named {name!r} (it has: {', '.join(parts)})")


def hyper_layer(mixer, feed_forward, norm1, norm2, connection, names) -> LayerSpec:
    """The pre-norm layer over several residual streams; ``feed_forward`` (and ``norm2``) None: the
    layer is its mixer alone."""
    if feed_forward is None:
        return LayerSpec({"mixer": mixer, "norm1": norm1, "connection1": connection}, names, "hyper_mixer_only")
    return LayerSpec({"mixer": mixer, "feed_forward": feed_forward, "norm1": norm1, "norm2": norm2,
                      "connection1": connection, "connection2": connection}, names, "hyper_prenorm")


def sandwich_layer(mixer, feed_forward, norm, names) -> LayerSpec:
    """A layer with a norm in front of and behind each sublayer, around a float32 residual stream:
    ``x + norm1b(mixer(norm1(x)))``, then ``+ norm2b(feed_forward(norm2(.)))``; ``feed_forward`` None: the
    layer is its mixer alone."""
    if feed_forward is None:
        return LayerSpec({"mixer": mixer, "norm1": norm, "norm1b": norm}, names, "sandwich_mixer_only")
    return LayerSpec({"mixer": mixer, "feed_forward": feed_forward, "norm1": norm, "norm1b": norm,
                      "norm2": norm, "norm2b": norm}, names, "sandwich")


def depth_layer(mixer, feed_forward, norm1, norm2, connection, names) -> LayerSpec:
    """A pre-norm layer in a stream joined over depth (see ``DepthAverageSpec``); ``feed_forward`` (and
    ``norm2``) None: the layer is its mixer alone."""
    if feed_forward is None:
        return LayerSpec({"mixer": mixer, "norm1": norm1, "connection": connection}, names, "depth_mixer_only")
    return LayerSpec({"mixer": mixer, "feed_forward": feed_forward, "norm1": norm1, "norm2": norm2,
                      "connection": connection}, names, "depth_prenorm")


def prenorm_layer(mixer, feed_forward, norm1, norm2, names, arrangement: str = "prenorm") -> LayerSpec:
    """The layer of the pre-norm block: ``x + mixer(norm1(x))``, then ``+ feed_forward(norm2(.))``."""
    return LayerSpec({"mixer": mixer, "feed_forward": feed_forward, "norm1": norm1, "norm2": norm2},
                     names, arrangement)


def prenorm32_layer(mixer, feed_forward, norm1, norm2, names) -> LayerSpec:
    """The pre-norm layer around a residual stream that is a 32-bit sum: ``x + mixer(norm1(x))``, then ``+
    feed_forward(norm2(.))``; ``feed_forward`` (and ``norm2``) None: the layer is its mixer alone."""
    if feed_forward is None:
        return LayerSpec({"mixer": mixer, "norm1": norm1}, names, "prenorm32_mixer_only")
    return LayerSpec({"mixer": mixer, "feed_forward": feed_forward, "norm1": norm1, "norm2": norm2}, names, "prenorm32")


@dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named by several
    entries; its weights are then shared).  ``cache`` names the cache entry the
    mixer uses; entries that share a number share keys and values.  An entry with
    ``writes_cache=False`` only reads the cache another entry filled.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, run order, final norm and output head."""

    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple
    schedule: tuple
    final_norm: object
    tie_embeddings: bool
    embed_name: str
    final_norm_name: str
    lm_head_name: str
    max_position: int = 0
    extra: dict = field(default_factory=dict)
    #: how many residual streams a token has (1: the single stream of the working type; more: float32
    #: streams that the layers' hyper-connections read and write, summed before the final norm)
    streams: int = 1
    #: the parameters of the final norm by logical name -> checkpoint name (None: its one ``weight``
    #: under ``final_norm_name``)
    final_norm_names: Optional[dict] = None
    #: checkpoint tensors that may be there and are not read
    ignored_tensors: tuple = ()
    #: what a token's embedding is multiplied by (models whose residual stream is float32)
    embedding_scale: float = 1.0
    #: None, or the constant ``c`` of ``logits <- c * tanh(logits / c)``
    logit_softcap: Optional[float] = None

    def cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)


def default_schedule(num_layers: int) -> tuple:
    """Each layer once, in order, each with a cache entry of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(num_layers))
