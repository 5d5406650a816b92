"""Setotar: a small decoder whose layers are listed one by one in config.json, on a residual of several streams.

    x_1 .. x_S = embed[token]                                   (`streams` S; without the key: one residual)
    a sublayer with its connection (in, out, mix) and layer scale ls:
        u = sum_s in[s] x_s;  y = ls * sublayer(N(u));  x_t <- sum_s mix[s, t] x_s + out[t] y
    every layer: the mixer, then the feed-forward when the layer has one;  N(x) = x / sqrt(mean(x^2) + eps) * w
    logits = head . N_final(sum_s x_s)

`layers[i]` gives `type` (which mixer), `mixer` (its sizes and constants) and `mlp` (null: none).

  parallel   two mixers that read the same input, added as left_scale * left + right_scale * right:
             `left`  grouped-query softmax attention (heads / kv_heads / dim / vdim) with biases on q, k and v, a
                     causal convolution of `conv` taps over time behind each projection, `rot` {dims, base,
                     scaling}: a rotation of each head's first dims (dimension i with i + dims/2), every value head
                     over its root mean square, `scale`, `softcap`, `mask` {size, keep_first}: a window of keys
                     that keeps the sequence's first keys visible;
             `right` a gated linear recurrence (heads / dim / vdim), see `parts/gated_recurrence.py`.
  attention  grouped-query softmax attention without biases, q and k each over the root mean square of the whole
             projection times a weight of that size, `rot`, `scale`, every key up to the query's own; `kv_from` j:
             the layer has no keys and values of its own and attends over those layer j cached.

`rot.scaling` {factor} alone divides every frequency by factor; {factor, original, fast, slow} is the stretch of
`PairRotationSpec`.  Feed-forward: `kind` moe (`router` {experts, top}, `expert` {ff}: SiLU-gated experts, an
expert's score the sigmoid of its router logit, the `top` largest chosen, their scores, as they are, multiplying the
experts' INPUT).  Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.ls1`, `l<i>.ls2`,
`l<i>.hc1.{in,out,mix}`, `l<i>.hc2.*`, `final.norm`, `head`.
"""

from __future__ import annotations

from ..config.model_config import (
    ConfigError,
    GatedHeadAttentionSpec,
    GatedLinearRecurrenceSpec,
    HyperConnectionSpec,
    LayerRun,
    LayerSpec,
    LMHeadSpec,
    ModelConfig,
    PairRotationSpec,
    ParallelMixerSpec,
    ResidualStreamsSpec,
    RMSNormSpec,
    RoutedExpertsSpec,
    TokenEmbeddingSpec,
    normalise_dtype,
    require,
)
from ..config.registry import Architecture, TensorNames, register_architecture
from .vupitar import _need, _sub

DEFAULT_MAX_POSITIONS = 1 << 20   # the design has no position table: nothing bounds a sequence but the pool


def _rotation(raw: dict | None, where: str) -> PairRotationSpec | None:
    if raw is None:
        return None
    scaling = raw.get("scaling")
    stretch = divide = None
    if scaling is not None:
        if "original" in scaling:
            stretch = tuple(float(_need(scaling, key, float, where + ".scaling")) for key in ("factor", "original", "fast", "slow"))
        else:
            divide = float(_need(scaling, "factor", float, where + ".scaling"))
    return PairRotationSpec(dims=_need(raw, "dims", int, where), base=float(_need(raw, "base", float, where)),
                            pairing="halves", stretch=stretch, divide=divide)


def _value_dim(raw: dict, dim: int) -> int:
    return raw["vdim"] if raw.get("vdim") is not None else dim


def _left(raw: dict, width: int, eps: float, where: str) -> GatedHeadAttentionSpec:
    dim = _need(raw, "dim", int, where)
    mask = raw.get("mask")
    return GatedHeadAttentionSpec(
        width=width, num_heads=_need(raw, "heads", int, where), num_kv_heads=_need(raw, "kv_heads", int, where),
        head_dim=dim, value_dim=_value_dim(raw, dim), scale=float(_need(raw, "scale", float, where)), eps=eps,
        qkv_bias=True, rotation=_rotation(raw.get("rot"), where + ".rot"),
        window=None if mask is None or mask.get("size") is None else _need(mask, "size", int, where + ".mask"),
        keep_first=0 if mask is None or mask.get("size") is None else int(mask.get("keep_first") or 0),
        conv=None if raw.get("conv") is None else _need(raw, "conv", int, where),
        value_norm=True,
        softcap=None if raw.get("softcap") is None else float(_need(raw, "softcap", float, where)),
    )


def _right(raw: dict, width: int, eps: float, where: str) -> GatedLinearRecurrenceSpec:
    dim = _need(raw, "dim", int, where)
    return GatedLinearRecurrenceSpec(width=width, num_heads=_need(raw, "heads", int, where), head_dim=dim,
                                     value_dim=_value_dim(raw, dim), eps=eps, lower_bound=True)


def _attention(raw: dict, width: int, eps: float, where: str) -> GatedHeadAttentionSpec:
    dim = _need(raw, "dim", int, where)
    return GatedHeadAttentionSpec(
        width=width, num_heads=_need(raw, "heads", int, where), num_kv_heads=_need(raw, "kv_heads", int, where),
        head_dim=dim, value_dim=_value_dim(raw, dim), scale=float(_need(raw, "scale", float, where)), eps=eps,
        qk_norm="whole", rotation=_rotation(raw.get("rot"), where + ".rot"), own_kv=raw.get("kv_from") is None,
    )


def _feed_forward(mlp: dict, width: int, where: str) -> RoutedExpertsSpec:
    kind = mlp.get("kind", "moe")
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind={kind!r}; known: moe")
    router = _sub(mlp, "router", where)
    return RoutedExpertsSpec(
        width=width, experts=_need(router, "experts", int, where + ".router"), top=_need(router, "top", int, where + ".router"),
        intermediate=_need(_sub(mlp, "expert", where), "ff", int, where + ".expert"), activation="silu",
        scoring="sigmoid", renormalise=False, weight_on="input",
    )


def parse_setotar(raw: dict) -> ModelConfig:
    width = require(raw, "width", int)
    vocab = require(raw, "vocab", int)
    listed = require(raw, "layers")
    if not isinstance(listed, list) or not listed:
        raise ConfigError("config.json: `layers` must be a non-empty list")
    eps = float(require(require(raw, "norm"), "eps", float))
    streams = raw.get("streams")
    if streams is not None:
        streams = require(raw, "streams", int)
    norm = RMSNormSpec(width=width, eps=eps)
    join = HyperConnectionSpec(width=width, streams=streams or 1, layer_scale=True, learned=streams is not None)
    layers, order = [], []
    for index, layer in enumerate(listed):
        where = f"layers[{index}]"
        kind = layer.get("type")
        mixer = _sub(layer, "mixer", where)
        run = LayerRun(layer=index, cache=index)
        if kind == "parallel":
            spec = ParallelMixerSpec(width=width, branches=(
                ("left", _left(_sub(mixer, "left", where + ".mixer"), width, eps, where + ".mixer.left"),
                 float(_need(mixer, "left_scale", float, where + ".mixer"))),
                ("right", _right(_sub(mixer, "right", where + ".mixer"), width, eps, where + ".mixer.right"),
                 float(_need(mixer, "right_scale", float, where + ".mixer"))),
            ))
        elif kind == "attention":
            spec = _attention(mixer, width, eps, where + ".mixer")
            source = mixer.get("kv_from")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < index:
                    raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier layer, got {source!r}")
                if listed[source].get("type") != "attention" or listed[source]["mixer"].get("kv_from") is not None:
                    raise ConfigError(f"config.json: {where}.mixer.kv_from={source}: that layer has no keys and values of its own kind")
                run = LayerRun(layer=index, cache=source, writes_cache=False)
        else:
            raise ConfigError(f"config.json: {where}.type={kind!r}; known: attention, parallel")
        mlp = layer.get("mlp")
        ffn = None if mlp is None else _feed_forward(mlp, width, where + ".mlp")
        extra = [("mixer_join", "join", join)] + ([("feed_forward_join", "join", join)] if ffn is not None else [])
        layers.append(LayerSpec(mixer=spec, mixer_norm=norm, feed_forward=ffn,
                                feed_forward_norm=norm if ffn is not None else None, block="hyper", extra=tuple(extra)))
        order.append(run)
    eos = raw.get("eos_token_id")
    return ModelConfig(
        architecture="Setotar",
        hidden_size=width,
        vocab_size=vocab,
        layers=layers,
        order=order,
        final_norm=norm,
        tie_word_embeddings=False,
        max_position_embeddings=int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS),
        eos_token_ids=list(eos) if isinstance(eos, list) else ([] if eos is None else [int(eos)]),
        dtype=normalise_dtype(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
        raw=dict(raw),
        embedding=TokenEmbeddingSpec(vocab=vocab, width=width),
        head=LMHeadSpec(width=width, vocab=vocab, tied=False),
        residual=ResidualStreamsSpec(width=width, streams=streams or 1),
    )


_ROLE_PREFIX = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2",
                "mixer_join": "", "feed_forward_join": ""}
_ATTENTION = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o", "q_proj.bias": "q.b",
              "k_proj.bias": "k.b", "v_proj.bias": "v.b", "q_norm.weight": "q.norm", "k_norm.weight": "k.norm",
              "q_conv.weight": "q.conv", "k_conv.weight": "k.conv", "v_conv.weight": "v.conv"}
_RIGHT = {"q_proj.weight": "q", "forget_gate.weight": "f", "forget_gate.bias": "f.b", "lower": "lower", "v_proj.weight": "v",
          "norm.weight": "norm", "o_proj.weight": "o"}
_PROJECTIONS = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}
_JOIN = {"in": "in", "out": "out", "mix": "mix"}


def _local(role: str, local: str) -> str:
    """A part's own parameter name -> the last piece of the tensor's name in a Setotar file."""
    if role in ("mixer_norm", "feed_forward_norm", "final_norm"):
        return {"weight": ""}[local]
    if role == "mixer":
        branch, _, rest = local.partition(".")
        if branch in ("left", "right"):
            return f"{branch}." + (_ATTENTION if branch == "left" else _RIGHT)[rest]
        return _ATTENTION[local]
    if role == "feed_forward":
        if local == "router.weight":
            return "router"
        prefix, _, rest = local.rpartition(".")          # experts.<e>.gate_proj, then "weight"
        owner, _, projection = prefix.rpartition(".")
        return f"e{owner.split('.')[1]}.{_PROJECTIONS[projection + '.' + rest]}"
    if role in ("mixer_join", "feed_forward_join"):
        number = "1" if role == "mixer_join" else "2"
        return f"ls{number}" if local == "scale" else f"hc{number}.{_JOIN[local]}"
    raise KeyError((role, local))


def setotar_tensor_names(config: ModelConfig) -> TensorNames:
    return TensorNames(
        embedding="embed",
        final_norm_prefix="final.norm",
        lm_head="head",
        layer_part=lambda layer, role: f"l{layer}.{_ROLE_PREFIX[role]}",
        embedding_prefix="",
        head_prefix="head.",
        pass_entry_prefix="",
        local_name=_local,
    )


SETOTAR = register_architecture(
    Architecture(name="Setotar", parse_config=parse_setotar, tensor_names=setotar_tensor_names)
)
