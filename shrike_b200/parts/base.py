"""What a part is, and the registries that map a spec's `kind` to its class.

A layer is put together from four kinds of part, chosen by the configuration layer
by layer: a mixer (attention here), a feed-forward, a norm and a position encoding,
arranged by a block.  A part is built from its spec alone; it never learns which
model it is in.  Azimml/shrike hard-wires these as nn.Modules
(shrike/models/qwen.py:64-150) and injects only the attention backend
(qwen.py:52-61); the split into registered parts is this engine's design.

Interfaces (duck-typed; `parameters` and `cache_needs` are static so that weights can
be checked and the cache sized before anything is put on the device):

  every part class
      parameters(spec) -> {local name: ParamSpec}
      __init__(spec, tensors: {local name: Tensor}, ops, runtime)
  norm
      add_norm(resid_f32[N,W], delta | None) -> normed[N,W]
          resid += delta (32-bit), then the normalised rows in the activation dtype;
          delta is [N,W], or a stack [P,N,W] of partial sums that the kernel adds in order
          (what `ops.linear(..., allow_partials=True)` may return)
      gather_norm(resid_f32, delta, rows_i32[R]) -> normed[R,W]   (only the wanted rows)
  position encoding
      rotary_table() -> float32 [D/2] inverse frequencies, when the mixer's fused
          kernel can apply it; else None and
      apply(q[N,H,D], k[N,Hkv,D], positions_i32[N]) rotates in place
  mixer
      cache_needs(spec) -> [KVNeed | StateNeed]
      forward(x[N,W], ctx: StepContext, run: LayerRun) -> delta[N,W]
  feed-forward
      forward(x[N,W], ctx) -> delta[N,W]
  block
      __init__(**parts by role)   ("mixer", "mixer_norm", "feed_forward", "feed_forward_norm"
          and whatever further roles the layer's spec lists in `extra`)
      forward(resid_f32, delta, ctx, run) -> (resid_f32, delta)
          `delta` is a sum not yet added to the residual; the next norm adds it.
  embedding
      forward(ctx) -> resid_f32[N,W]   the residual stream of the step's tokens.  A token id of
          -1 - r stands for `ctx.previous_tokens[r]` (what the step before drew in its row r).
      `table`: the [vocab, W] tensor a tied head may share, or None
  pass entry (a model whose run order repeats layers may have one; `LayerRun.enter` = t calls it)
      before_embedding(ctx)            may put a float32 buffer into ctx.carried["embedding_copy"]; an embedding
                                       that fills it says so with ctx.carried["embedding_copied"] = True
      begin(resid_f32, ctx)            right after the embedding: keeps what later passes need of it
      forward(resid_f32, delta, ctx, t) -> (resid_f32, delta)   what entering pass t does to the residual
  join (a block that lists one per sublayer, roles "mixer_join" and "feed_forward_join")
      read_norm(streams_f32[N,S*W], pending | None, norm) -> normed[N,W]
          the pending sublayer result joins the streams, then the next sublayer's input is formed and normed
  residual (a model whose residual is several streams a token; `ModelConfig.residual`)
      begin(resid_f32[N,W], ctx) -> streams_f32[N,S*W]       right after the embedding
      finish(streams, pending, rows_i32[R], norm) -> normed[R,W]   the final norm's input on the wanted rows
  head
      forward(hidden[R,W]) -> float32 logits [R, vocab]   (hidden: the final norm's output on the
          wanted rows); built with tensors {"weight": ...}, the embedding's table when tied

A part may declare the class attribute `capture_safe = True`.  It then promises that forward()
launches the same kernels with the same sizes for the same batch shape, whatever the positions,
slots and pages of the step (so a recorded launch sequence can be replayed), and that it leaves
rows alone whose cache slot and state slot are -1: the step function pads batches of single
tokens with such rows up to a few fixed sizes.  A model is treated so only if all its parts say so.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ParamSpec:
    """A tensor a part expects: its shape and how random weights fill it.

    init: "matrix" | "table" (N(0, 0.02)), "bias" (N(0, 0.02)), "norm" (1 + N(0, 0.1)),
    "around_zero" (N(0, 0.1)), "sink" (N(0, 1)), "mix" ([W, 2 W]: identity | 0, plus N(0, 0.02)),
    "conv" (N(0, 0.4)), "unit_interval" (sigmoid of N(0, 1)), "stream_mix" ([S, S]: identity plus N(0, 0.15)).
    """

    shape: tuple[int, ...]
    init: str


@dataclass(frozen=True)
class KVNeed:
    """Keys and values in pages: `window` None keeps all, else the last `window`.  `planes` 2: a key
    and a value tensor; 1: one tensor a token (a latent that serves as both), at half the memory.
    `chunk`: queries see only the keys of their own run of `chunk` positions (runs counted from
    position 0), so the pages of earlier runs are given back as the request moves on."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    planes: int = 2
    chunk: int | None = None
    # with a window: a sequence's first `keep_first` keys stay visible to every later query, so the pages that hold
    # them are never given back
    keep_first: int = 0


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, one slot per live request.  `name` "": the run's one state,
    `storage.state[cache id]`; a mixer that needs a second state beside it (the last inputs of a short
    convolution, say) names it, and finds it at `storage.state[(cache id, name)]`."""

    shape: tuple[int, ...]
    dtype: str = "float32"
    name: str = ""


class PendingSum:
    """Branch outputs that are not yet added to the residual: `terms`, a list of (tensor, scale), each
    tensor float32 [N, W] or a K-split stack [P, N, W].  A block whose branches run side by side hands
    one on as its `delta`; a norm that takes it adds every term in the kernel that norms the sum."""

    __slots__ = ("terms",)

    def __init__(self, terms=()):
        self.terms = list(terms)

    @staticmethod
    def of(delta, scale: float = 1.0) -> list:
        """The terms of a delta in any of its forms (None, a tensor, a PendingSum), each times `scale`."""
        if delta is None:
            return []
        if isinstance(delta, PendingSum):
            return [(tensor, s * scale) for tensor, s in delta.terms]
        return [(delta, scale)]


MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
NORMS: dict[str, type] = {}
POSITIONS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}
EMBEDDINGS: dict[str, type] = {}
HEADS: dict[str, type] = {}
PASS_ENTRIES: dict[str, type] = {}
JOINS: dict[str, type] = {}       # how a sublayer's result joins the residual (a layer lists them as further roles)
RESIDUALS: dict[str, type] = {}   # a residual that is not one row a token (`ModelConfig.residual`)

_CATEGORIES = {
    "embedding": EMBEDDINGS,
    "head": HEADS,
    "pass_entry": PASS_ENTRIES,
    "join": JOINS,
    "residual": RESIDUALS,
    "mixer": MIXERS,
    "feed_forward": FEED_FORWARDS,
    "norm": NORMS,
    "position": POSITIONS,
    "block": BLOCKS,
}


def register_part(category: str, kind: str, cls: type) -> type:
    """Adds a part class; `category` is one of mixer, feed_forward, norm, position, block,
    embedding, head, pass_entry, join, residual."""
    _CATEGORIES[category][kind] = cls
    return cls


def part_class(category: str, kind: str) -> type:
    table = _CATEGORIES[category]
    if kind not in table:
        raise KeyError(f"no {category} of kind {kind!r} is registered; known: {sorted(table)}")
    return table[kind]
