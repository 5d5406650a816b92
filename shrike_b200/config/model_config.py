"""Typed model configuration.

A `ModelConfig` is what an architecture's `parse_config` makes of the keys of its
own `config.json`: the widths, and for every layer a `LayerSpec` that names the
parts the layer is put together from (mixer, feed-forward, norm, position
encoding) with their sizes and constants.  The order in which layers run is data
too (`order`, a list of `LayerRun`).  Nothing here knows a model by name; no size
appears in code outside the values read from `config.json`.

Reference: Azimml/shrike reads a flat set of keys into `QwenConfig`
(shrike/models/qwen.py:23-49); the per-layer specs are this engine's own design so
that another architecture can choose other parts layer by layer.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


@dataclass(frozen=True)
class PartSpec:
    """Base of all part specifications: `kind` selects the implementation."""

    kind: str = field(init=False, default="")


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotate-half rotary position encoding (shrike/models/qwen.py:77-101)."""

    head_dim: int
    theta: float
    kind: str = field(init=False, default="rotary")


@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    """Root-mean-square norm with a plain weight (shrike/models/qwen.py:64-74)."""

    width: int
    eps: float
    offset: float = 0.0   # added to the stored weight: a design that keeps its weights around zero has 1.0 here
    kind: str = field(init=False, default="rmsnorm")


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Grouped-query softmax attention over a paged key/value cache.

    `window` is the number of most recent keys a query sees (None: all of them).
    `scale` multiplies the scores before the softmax.
    """

    width: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qkv_bias: bool
    out_bias: bool
    window: int | None
    position: PartSpec | None
    kind: str = field(init=False, default="attention")

    def __post_init__(self):
        if self.num_heads % self.num_kv_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_heads} is not a multiple of "
                f"num_key_value_heads={self.num_kv_heads}"
            )
        if self.window is not None and self.window < 1:
            raise ConfigError(f"attention window must be >= 1, got {self.window}")


@dataclass(frozen=True)
class LayerNormSpec(PartSpec):
    """Layer norm: (x - mean) / sqrt(var + eps) * weight (+ bias), var the mean squared deviation."""

    width: int
    eps: float
    bias: bool = True
    kind: str = field(init=False, default="layernorm")


@dataclass(frozen=True)
class SharedKeyValueAttentionSpec(PartSpec):
    """Grouped-query softmax attention whose values are its keys: k = Wk x is stored twice, as
    projected (the values) and normed (the keys); there is no value projection and no rotation.

    `qk_norm`: q and k are each divided by their root mean square over the WHOLE projection (all
    heads at once) and scaled by a weight of that size.  `q_temperature` (coef, every): the query
    at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).  `softcap`: a score
    s becomes softcap * tanh(s / softcap).  `slope_decay` d: head h (of H) takes
    2^(-d (h + 1) / H) * (query position - key position) off its scores.  `window`: a query sees
    only the `window` latest keys, itself included.  Each of these may be None (left out).
    """

    width: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    eps: float
    qk_norm: bool = True
    q_temperature: tuple | None = None
    softcap: float | None = None
    slope_decay: float | None = None
    window: int | None = None
    kind: str = field(init=False, default="shared_kv_attention")

    def __post_init__(self):
        if self.num_heads % self.num_kv_heads:
            raise ConfigError(f"heads={self.num_heads} is not a multiple of kv_heads={self.num_kv_heads}")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"attention window must be >= 1, got {self.window}")
        if self.softcap is not None and not self.softcap > 0:
            raise ConfigError(f"softcap must be positive, got {self.softcap}")
        if self.q_temperature is not None and self.q_temperature[1] < 1:
            raise ConfigError(f"the query temperature's period must be >= 1, got {self.q_temperature[1]}")


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """Causal softmax attention over a cached low-rank latent, without positions.

    c = RMS(Wdkv x) * weight is all that is cached (`latent_rank` numbers a token); head h's keys
    and values are Wuk_h c and Wuv_h c.  `own_latent` False: the layer has no Wdkv and attends over
    the latent another layer cached (the run order says whose).  `gated`: head h's output is
    multiplied by sigmoid(Wg x)_h.
    """

    width: int
    num_heads: int
    head_dim: int
    value_dim: int
    latent_rank: int
    scale: float
    eps: float
    own_latent: bool = True
    gated: bool = True
    kind: str = field(init=False, default="latent_attention")


@dataclass(frozen=True)
class DynamicTanhSpec(PartSpec):
    """A norm without statistics: tanh(alpha x) * weight + bias, alpha one learned number."""

    width: int
    kind: str = field(init=False, default="dynamic_tanh")


@dataclass(frozen=True)
class GatedHeadAttentionSpec(PartSpec):
    """Grouped-query softmax attention over a paged key/value cache with, each optional:

    `qkv_bias` / `out_bias`; `qk_norm`: q and k divided by their root mean square PER HEAD and scaled
    by one weight of the head's size that all heads share (before rotation); `rotary` (dims, base):
    the first `dims` dimensions of each head rotate, dimension i with i + dims/2, by
    position * base^(-2i/dims), the rest pass; `window`: a query sees the `window` latest keys;
    `chunk`: a query at position p sees key j <= p only if floor(p / chunk) = floor(j / chunk), runs
    counted from position 0 of the sequence; `head_gate`: head h's output times sigmoid(Wg x)_h.
    Keys have `head_dim` elements, values `value_dim`.  `rotation` (a `PairRotationSpec`, instead of
    `rotary`): the same rotation with the pairing, and the stretch of the frequencies, that it names.
    `sink`: every head has one learned number whose exponential is added to the softmax's denominator;
    that share of the weight goes to nothing, and the number enters as it is, without `scale`.
    """

    width: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    eps: float
    qkv_bias: bool = False
    out_bias: bool = False
    qk_norm: bool = False
    rotary: tuple | None = None
    window: int | None = None
    chunk: int | None = None
    head_gate: bool = False
    rotation: PartSpec | None = None
    sink: bool = False
    # `qk_norm` "whole" (instead of True, the norm per head): q and k are each divided by the root mean square of
    # their WHOLE projection, all heads at once, and scaled by a weight of the projection's size
    # `conv` T: a causal convolution of T taps over time on every channel of q, k and v, right behind the
    # projection (bias included) and before norm and rotation; the T - 1 latest projected values are state
    conv: int | None = None
    # `value_norm`: every value head is divided by its own root mean square (no weight) before it is cached
    value_norm: bool = False
    # `softcap` c: a score s becomes c tanh(s / c)
    softcap: float | None = None
    # `keep_first` n (with a window): the sequence's first n keys stay visible to every later query
    keep_first: int = 0
    # `own_kv` False: the layer has no key and value projections and attends over the keys and values another
    # layer cached (the run order says whose)
    own_kv: bool = True
    kind: str = field(init=False, default="gated_head_attention")

    def __post_init__(self):
        if self.num_heads % self.num_kv_heads:
            raise ConfigError(f"heads={self.num_heads} is not a multiple of kv_heads={self.num_kv_heads}")
        if self.window is not None and self.chunk is not None:
            raise ConfigError("an attention layer has a window or a chunk, not both")
        if self.qk_norm not in (False, True, "whole"):
            raise ConfigError(f"qk_norm {self.qk_norm!r}; known: False, True (per head), 'whole'")
        if self.conv is not None and not 1 <= self.conv <= 32:
            raise ConfigError(f"a short convolution has 1 to 32 taps, got {self.conv}")
        if self.conv is not None and not self.own_kv:
            raise ConfigError("a layer that reads another layer's keys and values has no convolution state of its own")
        if self.softcap is not None and not self.softcap > 0:
            raise ConfigError(f"softcap must be positive, got {self.softcap}")
        if self.keep_first < 0 or (self.keep_first and self.window is None):
            raise ConfigError("keep_first goes with a window and is not negative")
        if self.rotary is not None and self.rotation is not None:
            raise ConfigError("an attention layer has `rotary` or `rotation`, not both")
        if self.rotation is not None and self.rotation.dims > self.head_dim:
            raise ConfigError(f"rotation over {self.rotation.dims} dimensions of a head of {self.head_dim}")
        for name in ("window", "chunk"):
            if getattr(self, name) is not None and getattr(self, name) < 1:
                raise ConfigError(f"attention {name} must be >= 1, got {getattr(self, name)}")
        if self.rotary is not None:
            dims = self.rotary[0]
            if isinstance(dims, bool) or not isinstance(dims, int) or dims < 2 or dims % 2 or dims > self.head_dim:
                raise ConfigError(f"rotary dims must be even and at most the head size {self.head_dim}, got {dims!r}")


@dataclass(frozen=True)
class PairRotationSpec(PartSpec):
    """A rotation by position of the first `dims` dimensions of a vector: pair i of dims/2 turns by
    position * f_i, f_i = base^(-2i/dims).  `pairing`: "halves" pairs dimension i with i + dims/2,
    "neighbours" pairs 2i with 2i + 1.  `stretch` (factor, original, fast, slow), the YaRN rule: with
    d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)),
    dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i becomes f_i / factor * r_i +
    f_i (1 - r_i), and cos and sin are both multiplied by 0.1 ln(factor) + 1."""

    dims: int
    base: float
    pairing: str = "halves"
    stretch: tuple | None = None
    divide: float | None = None   # linear scaling: every f_i is divided by this
    kind: str = field(init=False, default="pair_rotation")

    def __post_init__(self):
        if isinstance(self.dims, bool) or not isinstance(self.dims, int) or self.dims < 2 or self.dims % 2:
            raise ConfigError(f"a rotation needs an even number of dimensions, got {self.dims!r}")
        if self.pairing not in ("halves", "neighbours"):
            raise ConfigError(f"rotation pairing {self.pairing!r}; known: halves, neighbours")
        if not self.base > 1:
            raise ConfigError(f"a rotation's base must exceed 1, got {self.base}")
        if self.stretch is not None and (len(self.stretch) != 4 or not self.stretch[0] > 0):
            raise ConfigError("a rotation's stretch is (factor, original, fast, slow) with a positive factor")
        if self.divide is not None and not self.divide > 0:
            raise ConfigError(f"a rotation's frequencies are divided by a positive number, got {self.divide}")


@dataclass(frozen=True)
class RotaryLatentAttentionSpec(PartSpec):
    """Softmax attention over a cached low-rank latent with a rotated key part that all heads share.

    Per token the cache holds c = RMS(first `latent_rank` rows of Wdkv x) * weight and the last
    `rotary_dim` rows of Wdkv x, rotated by position (`rotation`, over all `rotary_dim` dimensions).
    Head h's query is [head_dim plain | rotary_dim rotated]; its score with token j is
    scale * (q_plain . Wuk_h c_j + q_rotated . r_j), its value Wuv_h c_j.  `window`: a query sees the
    `window` latest keys, itself included (None: all).  `gate`: "element" multiplies the heads' outputs,
    side by side, by sigmoid(Wg x) element by element; None: no gate.
    """

    width: int
    num_heads: int
    head_dim: int
    rotary_dim: int
    value_dim: int
    latent_rank: int
    scale: float
    eps: float
    rotation: PartSpec
    window: int | None = None
    gate: str | None = "element"
    kind: str = field(init=False, default="rotary_latent_attention")

    def __post_init__(self):
        if self.rotation.dims != self.rotary_dim:
            raise ConfigError(f"the rotated part has {self.rotary_dim} dimensions but its rotation {self.rotation.dims}")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"attention window must be >= 1, got {self.window}")
        if self.gate not in (None, "element"):
            raise ConfigError(f"latent attention gate {self.gate!r}; known: element")


@dataclass(frozen=True)
class DecayLinearAttentionSpec(PartSpec):
    """Linear attention with a fixed decay per head: q = act(Wq x), k = act(Wk x), v = act(Wv x);
    S_t = decay_h S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t (no scale).  The heads' outputs, side by
    side, are divided by their common root mean square, scaled by a weight, multiplied by
    sigmoid(Wg x) and projected.  `decays`: one number in (0, 1] per head.  State and recurrence are 32-bit."""

    width: int
    num_heads: int
    head_dim: int
    value_dim: int
    decays: tuple
    eps: float
    activation: str = "silu"
    kind: str = field(init=False, default="decay_linear_attention")

    def __post_init__(self):
        if len(self.decays) != self.num_heads:
            raise ConfigError(f"{len(self.decays)} decays for {self.num_heads} heads")
        if any(isinstance(d, bool) or not isinstance(d, (int, float)) or not 0 < d <= 1 for d in self.decays):
            raise ConfigError(f"every decay lies in (0, 1], got {list(self.decays)}")
        if self.activation != "silu":
            raise ConfigError(f"linear attention activation {self.activation!r}; known: silu")


@dataclass(frozen=True)
class GatedLinearRecurrenceSpec(PartSpec):
    """A linear recurrence with one gate for both ends (the HGRN2 cell): what a state row keeps, f, fixes what it takes in, 1 - f.  Per head, with
    q = silu(Wq x) (dim), v = Wv x (vdim) and the gate f = lower + (1 - lower) * sigmoid(Wf x + b) per channel of q:

        S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T  from S = 0;   o_t = S_t^T q_t   (no key, no scale)

    Every head's output is divided by its root mean square and scaled by one weight of the head's size that all
    heads share; the heads side by side are projected.  `lower_bound`: the model holds `lower` (one number a gate
    channel); without it the bound is 0.  Gates, state and recurrence are 32-bit."""

    width: int
    num_heads: int
    head_dim: int
    value_dim: int
    eps: float
    lower_bound: bool = True
    kind: str = field(init=False, default="gated_linear_recurrence")


@dataclass(frozen=True)
class HyperConnectionSpec(PartSpec):
    """How a sublayer's result y joins a residual of `streams` streams x_1 .. x_S, and how the sublayer reads them:
    u = sum_s in[s] x_s is what the sublayer's norm sees; afterwards, all streams at once from the old ones,
    x_t <- sum_s mix[s, t] x_s + out[t] * (scale * y), `scale` a learned vector over the width (`layer_scale`; else 1).
    `learned` False: one stream's worth of constants (in = out = mix = 1), the ordinary residual sum."""

    width: int
    streams: int = 1
    layer_scale: bool = False
    learned: bool = True
    kind: str = field(init=False, default="hyper_connection")

    def __post_init__(self):
        if not 1 <= self.streams <= 8:
            raise ConfigError(f"a residual has 1 to 8 streams, got {self.streams}")
        if not self.learned and self.streams != 1:
            raise ConfigError("several residual streams need learned connections")


@dataclass(frozen=True)
class ResidualStreamsSpec(PartSpec):
    """The residual as `streams` copies of the embedding's output that the layers' connections mix; what the final
    norm sees is their sum."""

    width: int
    streams: int
    kind: str = field(init=False, default="residual_streams")


@dataclass(frozen=True)
class MatrixMemorySpec(PartSpec):
    """A recurrent mixer whose state is a matrix per head (the mLSTM cell of xLSTM), with an
    exponential input gate, a sigmoid forget gate (both soft-capped at `gate_cap` before their
    nonlinearity) and a running maximum that keeps the exponentials in range:

        m_t = max(f_t + m_(t-1), i_t);  S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T
        z_t likewise with k_t alone;  o_t = S_t^T q_t / (max(|z_t . q_t|, exp(-m_t)) + `denominator_floor`)

    q is scaled by head_dim^(-1/2).  Each head's output is divided by its root mean square, the heads
    are scaled by one weight, gated by sigmoid(Wg x) and projected.  `m_0` is the running maximum a
    sequence starts with; state and gates are 32-bit.
    """

    width: int
    num_heads: int
    head_dim: int
    value_dim: int
    gate_cap: float
    eps: float
    denominator_floor: float = 1e-6
    initial_max: float = 0.0
    kind: str = field(init=False, default="matrix_memory")

    def __post_init__(self):
        if not self.gate_cap > 0:
            raise ConfigError(f"gate_cap must be positive, got {self.gate_cap}")


@dataclass(frozen=True)
class ParallelMixerSpec(PartSpec):
    """Several mixers that read the same input; their outputs are added with a scale each.
    `branches`: (name, spec, scale); a branch's tensors are named `<name>.<its own names>`."""

    width: int
    branches: tuple
    kind: str = field(init=False, default="parallel_mixer")

    def __post_init__(self):
        if not self.branches:
            raise ConfigError("a parallel mixer needs at least one branch")


@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """Dense gated feed-forward: down(act(gate(x)) * up(x)) (shrike/models/qwen.py:128-136)."""

    width: int
    intermediate: int
    activation: str
    # for the activation "clamped_swish": g <- min(g, limit), u <- clamp(u, -limit, limit), then
    # g * sigmoid(1.702 g) * (u + 1)
    limit: float | None = None
    kind: str = field(init=False, default="gated_mlp")


@dataclass(frozen=True)
class RoutedExpertsSpec(PartSpec):
    """A mixture of gated feed-forward experts: router logits in 32-bit, softmax over all experts,
    the `top` largest, their scores divided by the sum of those (+ `renorm_eps`); the output is the
    weighted sum of the chosen experts' down(act(gate x) * (up x)).  `shared_intermediate` (None: no
    shared expert): one more expert of that size that every token uses, times sigmoid(w_sg . x)
    when `shared_gate`."""

    width: int
    experts: int
    top: int
    intermediate: int
    activation: str = "silu"
    shared_intermediate: int | None = None
    shared_gate: bool = True
    renorm_eps: float = 1e-20
    # `scoring` "sigmoid": an expert's score is the sigmoid of its own logit; `renormalise` False: the chosen experts
    # keep their scores as weights; `weight_on` "input": an expert runs on weight * x instead of its output being
    # multiplied, sum_e expert_e(w_e x)
    scoring: str = "softmax"
    renormalise: bool = True
    weight_on: str = "output"
    kind: str = field(init=False, default="routed_experts")

    def __post_init__(self):
        if not 1 <= self.top <= self.experts:
            raise ConfigError(f"router: top={self.top} must lie in 1..experts={self.experts}")
        if self.scoring not in ("softmax", "sigmoid"):
            raise ConfigError(f"router scoring {self.scoring!r}; known: softmax, sigmoid")
        if self.weight_on not in ("output", "input"):
            raise ConfigError(f"an expert's weight sits on its output or its input, got {self.weight_on!r}")


@dataclass(frozen=True)
class TokenEmbeddingSpec(PartSpec):
    """One table row per token id, copied into the residual (shrike/models/qwen.py:161)."""

    vocab: int
    width: int
    scale: float = 1.0   # every row is multiplied by this as it enters the residual stream
    kind: str = field(init=False, default="token_embedding")


@dataclass(frozen=True)
class TokenPositionEmbeddingSpec(PartSpec):
    """A table row per token id plus a learned vector per position (not scaled), summed in 32-bit."""

    vocab: int
    width: int
    max_positions: int
    kind: str = field(init=False, default="token_position_embedding")


@dataclass(frozen=True)
class PassEntrySpec(PartSpec):
    """Entering pass t over a run of repeated layers: the embedding's output is added to the residual
    again (`add_embedding`, every pass but the first) and then a learned vector `step[t]`.  `mix`: instead
    of that sum, every pass (the first too) replaces the residual x by Win [x ; e], e the embedding's
    output and Win a [width, 2 width] matrix, before `step[t]` is added."""

    width: int
    passes: int
    add_embedding: bool = True
    mix: bool = False
    kind: str = field(init=False, default="pass_entry")


@dataclass(frozen=True)
class LMHeadSpec(PartSpec):
    """Normed hidden rows times a [vocab, width] matrix, which may be the embedding's table
    (shrike/models/qwen.py:192,211-212)."""

    width: int
    vocab: int
    tied: bool = False
    scale: float = 1.0   # every logit is multiplied by this
    kind: str = field(init=False, default="lm_head")


STANDARD_ROLES = (
    ("mixer", "mixer"),
    ("mixer_norm", "norm"),
    ("feed_forward", "feed_forward"),
    ("feed_forward_norm", "norm"),
)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which parts, and how they are arranged (`block`).

    The four named parts are what a pre-norm block takes.  A block that arranges more parts
    (norms after its branches, a third branch) lists them in `extra` as (role, category, spec);
    the block class is built with every role as a keyword and the architecture names the
    tensors of every role.
    """

    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec | None
    feed_forward_norm: PartSpec | None
    block: str = "pre_norm"
    extra: tuple = ()

    def roles(self):
        """(role, category, spec) of every part of the layer; a part the layer leaves out (None, where
        its block allows that: a layer without a feed-forward) is not listed."""
        for role, category in STANDARD_ROLES:
            if getattr(self, role) is not None:
                yield role, category, getattr(self, role)
        yield from self.extra


@dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    `layer` indexes `ModelConfig.layers` (weights); `cache` is the id of the cache
    (pages or state) this run uses.  A run with `writes_cache=False` reads the cache
    that an earlier run with the same `cache` id wrote in this step.
    """

    layer: int
    cache: int
    writes_cache: bool = True
    # a number t: before this run the model's pass entry (`ModelConfig.pass_entry`) is applied for pass t
    enter: int | None = None


@dataclass
class ModelConfig:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: list[LayerSpec]
    order: list[LayerRun]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: list[int]
    dtype: str  # "bfloat16" | "float32": what config.json asks for
    raw: dict[str, Any] = field(default_factory=dict, repr=False)
    # how token ids become the residual and how normed rows become logits: parts like the others,
    # chosen by `kind`.  None: one table, and a plain (or tied) matrix, from the sizes above.
    embedding: PartSpec | None = None
    head: PartSpec | None = None
    # what happens to the residual when a run opens a pass over repeated layers (`LayerRun.enter`)
    pass_entry: PartSpec | None = None
    # a residual that is not one row a token (several streams): made from the embedding's output before the first
    # layer, turned into the final norm's input after the last
    residual: PartSpec | None = None

    def __post_init__(self):
        if self.embedding is None:
            self.embedding = TokenEmbeddingSpec(vocab=self.vocab_size, width=self.hidden_size)
        if self.head is None:
            self.head = LMHeadSpec(width=self.hidden_size, vocab=self.vocab_size, tied=self.tie_word_embeddings)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @property
    def num_caches(self) -> int:
        return 1 + max(run.cache for run in self.order) if self.order else 0

    def validate(self) -> None:
        writers: dict[int, int] = {}
        for index, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"run {index} names layer {run.layer}, model has {len(self.layers)}")
            if run.enter is not None and self.pass_entry is None:
                raise ConfigError(f"run {index} opens pass {run.enter} but the model has no pass entry")
            if run.writes_cache:
                if run.cache in writers:
                    raise ConfigError(
                        f"runs {writers[run.cache]} and {index} both write cache {run.cache}"
                    )
                writers[run.cache] = index
            elif run.cache not in writers:
                raise ConfigError(f"run {index} reads cache {run.cache} before any run wrote it")


DTYPE_NAMES = {
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
    "float": "float32",
}


def normalise_dtype(name: str) -> str:
    try:
        return DTYPE_NAMES[str(name).replace("torch.", "")]
    except KeyError:
        raise ConfigError(
            f"dtype {name!r} is not served; this engine runs bfloat16 or float32"
        ) from None


def require(raw: dict, key: str, kind=None):
    """A key that config.json must hold; a clear error when it does not."""
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks the key {key!r}")
    value = raw[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int) or value < 1):
        raise ConfigError(f"config.json: {key} must be a positive integer, got {value!r}")
    if kind is float and (isinstance(value, bool) or not isinstance(value, (int, float))):
        raise ConfigError(f"config.json: {key} must be a number, got {value!r}")
    return value


def read_config_json(model_dir: str | Path) -> dict:
    """The raw dictionary; missing file is a FileNotFoundError with a hint
    (shrike/models/qwen.py:25-31)."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(
            f"no config.json under {str(model_dir)!r}; point --model (or SHRIKE_B200_MODEL_DIR) at "
            "a folder with config.json and *.safetensors, or write one with "
            "`python -m shrike_b200.weights.random_init`"
        )
    return json.loads(path.read_text())
