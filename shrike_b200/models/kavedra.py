"""Kavedra: a small decoder whose layers are listed one by one in config.json, each with one of three
mixers, with a stretch of layers that runs several times.

    e = embed[token]
    layers `loop.start` .. `loop.stop` - 1 run `loop.times` times in a row with the same weights and a
    cache or state of their own each pass, then the rest follow.  Entering pass t (the first too):
    x <- Win [x ; e] with `loop.in` ([width, 2 width]), then x += loop.step[t].
    every layer:  x += mixer(N1(x));  x += ff(N2(x)),  N(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
    logits = logit_scale * head . N_final(x)

`layers[i]` gives `type` (which mixer), `mixer` (its sizes and constants) and `mlp` (null: none).

  lightning         linear attention with a decay per head (`heads` / `dim` / `vdim` / `decay`), see
                    `parts/linear_attention.py`
  attention         grouped-query softmax attention (`heads` / `kv_heads` / `dim` / `vdim`) with biases on
                    q, k and v, `rot` {dims, base}: neighbouring dimensions of each head's first dims
                    rotate, `scale`, every key up to the query's own, and a learned sink per head in the
                    softmax's denominator
  latent_attention  attention over a cached latent of `kv_rank` numbers and one rotated key part of
                    `rot_dim` that all heads share (`heads` / `dim` / `rot_dim` / `vdim`), `rot` {dims,
                    base, scaling {factor, original, fast, slow}}, `scale`, `mask` {size}: a window of keys,
                    and a sigmoid gate element by element on the heads' outputs; see
                    `parts/latent_attention.py`

Feed-forward: `kind` dense, down(silu(gate x) * up x).  Tensor names: `embed`, `loop.in`, `loop.step`,
`l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""

from __future__ import annotations

from ..config.model_config import (
    ConfigError,
    DecayLinearAttentionSpec,
    GatedHeadAttentionSpec,
    GatedMLPSpec,
    LayerSpec,
    LMHeadSpec,
    ModelConfig,
    PairRotationSpec,
    PassEntrySpec,
    RMSNormSpec,
    RotaryLatentAttentionSpec,
    TokenEmbeddingSpec,
    normalise_dtype,
    require,
)
from ..config.registry import Architecture, TensorNames, register_architecture
from .vupitar import _need, _sub, run_order

NORM_OFFSET = 1.0   # a norm's stored weight is its distance from one
DEFAULT_MAX_POSITIONS = 1 << 20   # the design has no position table: nothing bounds a sequence but the pool


def _rotation(raw: dict, where: str) -> PairRotationSpec:
    stretch = raw.get("scaling")
    if stretch is not None:
        stretch = tuple(float(_need(stretch, key, float, where + ".scaling")) for key in ("factor", "original", "fast", "slow"))
    return PairRotationSpec(dims=_need(raw, "dims", int, where), base=float(_need(raw, "base", float, where)),
                            pairing="neighbours", stretch=stretch)


def _value_dim(raw: dict, dim: int) -> int:
    return raw["vdim"] if raw.get("vdim") is not None else dim


def _lightning(raw: dict, width: int, eps: float, where: str) -> DecayLinearAttentionSpec:
    dim = _need(raw, "dim", int, where)
    decays = raw.get("decay")
    if not isinstance(decays, list):
        raise ConfigError(f"config.json: {where}.decay must list one number per head")
    return DecayLinearAttentionSpec(width=width, num_heads=_need(raw, "heads", int, where), head_dim=dim,
                                    value_dim=_value_dim(raw, dim), decays=tuple(decays), eps=eps)


def _attention(raw: dict, width: int, eps: float, where: str) -> GatedHeadAttentionSpec:
    dim = _need(raw, "dim", int, where)
    rot, mask = raw.get("rot"), raw.get("mask")
    return GatedHeadAttentionSpec(
        width=width, num_heads=_need(raw, "heads", int, where), num_kv_heads=_need(raw, "kv_heads", int, where),
        head_dim=dim, value_dim=_value_dim(raw, dim), scale=float(_need(raw, "scale", float, where)), eps=eps,
        qkv_bias=True, rotation=None if rot is None else _rotation(rot, where + ".rot"),
        window=None if mask is None else _need(mask, "size", int, where + ".mask"), sink=True)


def _latent(raw: dict, width: int, eps: float, where: str) -> RotaryLatentAttentionSpec:
    dim = _need(raw, "dim", int, where)
    mask = raw.get("mask")
    return RotaryLatentAttentionSpec(
        width=width, num_heads=_need(raw, "heads", int, where), head_dim=dim, rotary_dim=_need(raw, "rot_dim", int, where),
        value_dim=_value_dim(raw, dim), latent_rank=_need(raw, "kv_rank", int, where),
        scale=float(_need(raw, "scale", float, where)), eps=eps, rotation=_rotation(_sub(raw, "rot", where), where + ".rot"),
        window=None if mask is None else _need(mask, "size", int, where + ".mask"), gate="element")


_MIXERS = {"lightning": _lightning, "attention": _attention, "latent_attention": _latent}


def parse_kavedra(raw: dict) -> ModelConfig:
    width = require(raw, "width", int)
    vocab = require(raw, "vocab", int)
    listed = require(raw, "layers")
    if not isinstance(listed, list) or not listed:
        raise ConfigError("config.json: `layers` must be a non-empty list")
    eps = float(require(require(raw, "norm"), "eps", float))
    norm = RMSNormSpec(width=width, eps=eps, offset=NORM_OFFSET)
    layers = []
    for index, layer in enumerate(listed):
        where = f"layers[{index}]"
        kind = layer.get("type")
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: {where}.type={kind!r}; known: " + ", ".join(sorted(_MIXERS)))
        mixer = _MIXERS[kind](_sub(layer, "mixer", where), width, eps, where + ".mixer")
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None:
            if mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json: {where}.mlp.kind={mlp.get('kind')!r}; known: dense")
            ffn = GatedMLPSpec(width=width, intermediate=_need(mlp, "ff", int, where + ".mlp"), activation="silu")
        layers.append(LayerSpec(mixer=mixer, mixer_norm=norm, feed_forward=ffn,
                                feed_forward_norm=norm if ffn is not None else None, block="pre_norm"))
    loop = raw.get("loop")
    eos = raw.get("eos_token_id")
    return ModelConfig(
        architecture="Kavedra",
        hidden_size=width,
        vocab_size=vocab,
        layers=layers,
        order=run_order(len(layers), loop),
        final_norm=norm,
        tie_word_embeddings=False,
        max_position_embeddings=int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS),
        eos_token_ids=list(eos) if isinstance(eos, list) else ([] if eos is None else [int(eos)]),
        dtype=normalise_dtype(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
        raw=dict(raw),
        embedding=TokenEmbeddingSpec(vocab=vocab, width=width),
        head=LMHeadSpec(width=width, vocab=vocab, tied=False, scale=float(raw.get("logit_scale", 1.0))),
        pass_entry=None if loop is None else PassEntrySpec(width=width, passes=require(loop, "times", int),
                                                           add_embedding=False, mix=True),
    )


_ROLE_PREFIX = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2"}
_MIXER = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o", "q_proj.bias": "q.b",
          "k_proj.bias": "k.b", "v_proj.bias": "v.b", "sink": "sink", "gate.weight": "g", "norm.weight": "norm",
          "kv_down.weight": "dkv", "kv_norm.weight": "dkv.norm", "k_up.weight": "uk", "v_up.weight": "uv"}
_FEED_FORWARD = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}


def _local(role: str, local: str) -> str:
    """A part's own parameter name -> the last piece of the tensor's name in a Kavedra file."""
    if role in ("mixer_norm", "feed_forward_norm", "final_norm"):
        return {"weight": ""}[local]
    if role == "mixer":
        return _MIXER[local]
    if role == "feed_forward":
        return _FEED_FORWARD[local]
    if role == "pass_entry":
        return {"step": "loop.step", "in": "loop.in"}[local]
    raise KeyError((role, local))


def kavedra_tensor_names(config: ModelConfig) -> TensorNames:
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


KAVEDRA = register_architecture(
    Architecture(name="Kavedra", parse_config=parse_kavedra, tensor_names=kavedra_tensor_names)
)
