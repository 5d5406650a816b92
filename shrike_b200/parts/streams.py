"""A residual of several streams (hyper-connections), and the block that runs a pre-norm layer on it.

Instead of one residual row a token there are S of them, x_1 .. x_S, all equal to the embedding's output
before the first layer.  A sublayer (mixer or feed-forward) owns a `HyperConnection`: weights `in` (S), `out` (S),
`mix` (S x S, indexed [from, to]) and, when the design has one, a layer scale over the width.  It reads
u = sum_s in[s] x_s, runs on the norm of u, and its result y joins the streams, all at once from the old ones,

    x_t <- sum_s mix[s, t] x_s + out[t] * (scale * y).

With one stream and in = out = mix = 1 this is the ordinary residual sum, x <- x + scale * y, which is how a
model of the same design without streams runs (`learned=False`).  What the final norm sees is the sum of the
streams.

How it runs here: the streams are one float32 array [N, S, W].  A sublayer's result is never added by a kernel
of its own: it travels on as a `PendingJoin` (the result's terms, K-split stacks included, and the connection
that owns it), and the NEXT sublayer's norm kernel (`stream_norm`) joins it, forms that sublayer's input and
norms it in one pass over the row.  The last pending result is joined by the final norm's kernel, on the wanted
rows only.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, PendingSum, register_part


class PendingJoin:
    """A sublayer result that has not joined the streams yet: its terms and the connection it joins through."""

    __slots__ = ("terms", "join")

    def __init__(self, terms, join):
        self.terms, self.join = terms, join


class HyperConnection:
    capture_safe = True
    MAX_TERMS = 4   # pending sums one launch of the kernel takes

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        params = {}
        if spec.learned:
            params["in"] = ParamSpec((spec.streams,), "norm")
            params["out"] = ParamSpec((spec.streams,), "norm")
            params["mix"] = ParamSpec((spec.streams, spec.streams), "stream_mix")
        if spec.layer_scale:
            params["scale"] = ParamSpec((spec.width,), "norm")
        return params

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        count = spec.streams
        if spec.learned:
            self.in_w = tensors["in"].to(torch.float32).contiguous()
            self.out_w = tensors["out"].to(torch.float32).contiguous()
            self.mix = tensors["mix"].to(torch.float32).contiguous()
        else:
            self.in_w = torch.ones(count, dtype=torch.float32, device=runtime.device)
            self.out_w = torch.ones(count, dtype=torch.float32, device=runtime.device)
            self.mix = torch.eye(count, dtype=torch.float32, device=runtime.device).contiguous()
        self.scale = tensors["scale"].to(torch.float32).contiguous() if spec.layer_scale else None

    def joining(self):
        return (self.mix, self.out_w, self.scale)

    def flush(self, streams, pending):
        """A pending result of more terms than one launch of the kernel takes is summed into one term first."""
        terms = pending.terms
        if len(terms) <= self.MAX_TERMS:
            return pending
        first, scale = terms[0]
        total = (first if first.dim() == 2 else first.sum(0)) * scale
        for tensor, scale in terms[1:]:
            total = total + (tensor if tensor.dim() == 2 else tensor.sum(0)) * scale
        return PendingJoin([(total.contiguous(), 1.0)], pending.join)

    def read_norm(self, streams, pending, norm, out_name="normed"):
        """The pending result joins the streams; then this sublayer's input, normed by `norm` (an RMS norm)."""
        rt = self.runtime
        n = streams.shape[0]
        shaped = streams.view(n, self.spec.streams, self.spec.width)
        out = rt.buffer(out_name, (n, self.spec.width), rt.act_dtype)
        if pending is not None:
            pending = pending.join.flush(streams, pending)
        self.ops.stream_norm(shaped, None if pending is None else pending.terms,
                             None if pending is None else pending.join.joining(), self.in_w, norm.weight, norm.spec.eps, out)
        return out


class ResidualStreams:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime

    def begin(self, resid, ctx):
        """Every stream starts as the embedding's output."""
        n, width = resid.shape
        streams = self.runtime.buffer("streams", (n, self.spec.streams * width), torch.float32)
        streams.view(n, self.spec.streams, width).copy_(resid.unsqueeze(1).expand(n, self.spec.streams, width))
        return streams

    def finish(self, streams, pending, rows, norm, out_name="normed_rows"):
        """The final norm of the streams' sum, on the wanted rows; the last pending result joins on the way."""
        rt = self.runtime
        n = streams.shape[0]
        shaped = streams.view(n, self.spec.streams, self.spec.width)
        out = rt.buffer(out_name, (rows.shape[0], self.spec.width), rt.act_dtype)
        if pending is not None:
            pending = pending.join.flush(streams, pending)
        self.ops.stream_norm(shaped, None if pending is None else pending.terms,
                             None if pending is None else pending.join.joining(), None, norm.weight, norm.spec.eps, out,
                             rows=rows)
        return out

    def summed(self, streams, pending, out):
        """The sum of the streams (float32 [N, W]) with the pending result joined; the streams are rewritten."""
        n = streams.shape[0]
        shaped = streams.view(n, self.spec.streams, self.spec.width)
        self.ops.stream_norm(shaped, None if pending is None else pending.terms,
                             None if pending is None else pending.join.joining(), None, None, 0.0, None, sum_out=out)
        return out


class HyperBlock:
    """A pre-norm layer on a residual of several streams: each sublayer reads the streams through its connection
    and its result joins them through it; the feed-forward may be absent."""

    capture_safe = True

    def __init__(self, mixer, mixer_norm, mixer_join, feed_forward=None, feed_forward_norm=None, feed_forward_join=None):
        if (feed_forward is None) != (feed_forward_norm is None) or (feed_forward is None) != (feed_forward_join is None):
            raise ValueError("a feed-forward, its norm and its connection come together")
        self.mixer, self.mixer_norm, self.mixer_join = mixer, mixer_norm, mixer_join
        self.feed_forward, self.feed_forward_norm, self.feed_forward_join = feed_forward, feed_forward_norm, feed_forward_join

    def forward(self, resid, delta, ctx, run):
        if delta is not None and not isinstance(delta, PendingJoin):
            raise NotImplementedError("a block on residual streams takes a pending result that names its connection")
        hidden = self.mixer_join.read_norm(resid, delta, self.mixer_norm)
        pending = PendingJoin(PendingSum.of(self.mixer.forward(hidden, ctx, run)), self.mixer_join)
        if self.feed_forward is None:
            return resid, pending
        hidden = self.feed_forward_join.read_norm(resid, pending, self.feed_forward_norm)
        return resid, PendingJoin(PendingSum.of(self.feed_forward.forward(hidden, ctx)), self.feed_forward_join)


register_part("join", "hyper_connection", HyperConnection)
register_part("residual", "residual_streams", ResidualStreams)
register_part("block", "hyper", HyperBlock)
