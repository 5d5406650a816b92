"""Residual blocks.

`ParallelBlock`: both branches read the same residual, x += mixer(norm1(x)) + ff(norm2(x)).  The two
norms come from one pass over the row where the norm part offers that (`add_norm_pair`), and the
branch outputs stay pending (a `PendingSum`): the next norm kernel adds them, so the sum costs no pass.

`BranchNormBlock`: the norm sits on a branch's OUTPUT, x += norm(mixer(x)); x += norm(ffn(x)), and both
branches read x itself; the feed-forward may be absent.  The residual sum is 32-bit; a 16-bit engine
gets the rounded residual a branch reads from the kernel that made the sum.

`PreNormBlock`: pre-norm residual block: x += mixer(norm(x)); x += ffn(norm(x))
(shrike/models/qwen.py:147-150); the feed-forward may be absent.  The residual `resid` is float32; a branch output
is handed on as `delta` and added by the next norm kernel.

When the kernels offer a native issue of whole layers (`ops.layer_program()`) and the four parts
are ones it serves, the layer's launches are issued by one native call instead of part by part:
the same kernels with the same arguments in the same order, without the interpreter between them."""

from __future__ import annotations

from .base import PendingSum, register_part


class PreNormBlock:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    def __init__(self, mixer, mixer_norm, feed_forward=None, feed_forward_norm=None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.feed_forward = feed_forward
        self.feed_forward_norm = feed_forward_norm
        self._program = None
        self._asked = False
        self._native_constants: dict = {}   # what the native issue keeps per run of this layer

    def _native(self):
        if not self._asked:
            self._asked = True
            offer = getattr(getattr(self.mixer, "ops", None), "layer_program", None)
            program = offer() if offer is not None and self.feed_forward is not None else None
            if program is not None and program.serves(self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm):
                self._program = program
        return self._program

    def prepare(self) -> None:
        """Called once when the model is built: settles how the layer is issued, so that what that
        takes (the native library's set-up) does not fall into a request's first step."""
        self._native()

    def forward(self, resid, delta, ctx, run):
        program = self._native()
        if program is not None and getattr(program.ops, "native_layers", False):
            return resid, program.run(self._native_constants, self.mixer, self.mixer_norm, self.feed_forward,
                                      self.feed_forward_norm, resid, delta, ctx, run)
        hidden = self.mixer_norm.add_norm(resid, delta)
        delta = self.mixer.forward(hidden, ctx, run)
        if self.feed_forward is None:   # a layer of a mixer alone
            return resid, delta
        hidden = self.feed_forward_norm.add_norm(resid, delta)
        delta = self.feed_forward.forward(hidden, ctx)
        return resid, delta


class BranchNormBlock:
    capture_safe = True

    def __init__(self, mixer, mixer_norm, feed_forward=None, feed_forward_norm=None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.feed_forward = feed_forward
        self.feed_forward_norm = feed_forward_norm

    def forward(self, resid, delta, ctx, run):
        if delta is not None:
            raise NotImplementedError("a branch-norm block takes a residual with nothing pending")
        # the block before (if of this kind) left the residual in the activation type with its last sum
        held = ctx.carried.pop("residual_cast", None)
        hidden = held[1] if held is not None and held[0] is resid else self.mixer_norm.norm_add(resid, None)
        hidden = self.mixer_norm.norm_add(resid, self.mixer.forward(hidden, ctx, run))
        if self.feed_forward is not None:
            hidden = self.feed_forward_norm.norm_add(resid, self.feed_forward.forward(hidden, ctx))
        ctx.carried["residual_cast"] = (resid, hidden)
        return resid, None


class ParallelBlock:
    capture_safe = True

    def __init__(self, mixer, mixer_norm, feed_forward=None, feed_forward_norm=None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.feed_forward = feed_forward
        self.feed_forward_norm = feed_forward_norm

    def forward(self, resid, delta, ctx, run):
        if self.feed_forward is None:
            hidden = self.mixer_norm.add_norm(resid, delta)
            return resid, PendingSum(PendingSum.of(self.mixer.forward(hidden, ctx, run)))
        pair = getattr(self.mixer_norm, "add_norm_pair", None)
        if pair is not None:
            for_mixer, for_ffn = pair(resid, delta, self.feed_forward_norm)
        else:
            for_mixer = self.mixer_norm.add_norm(resid, delta, "normed")
            for_ffn = self.feed_forward_norm.add_norm(resid, None, "normed_b")
        mixed = self.mixer.forward(for_mixer, ctx, run)
        fed = self.feed_forward.forward(for_ffn, ctx)
        return resid, PendingSum(PendingSum.of(mixed) + PendingSum.of(fed))


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "branch_norm", BranchNormBlock)
