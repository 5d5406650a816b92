"""Token embedding and output head: how ids enter the residual stream and how it leaves as logits.

The embedding copies one table row per token into the float32 residual
(shrike/models/qwen.py:161); the head multiplies the final norm's output at the wanted
rows by a [vocab, width] matrix, the embedding's own table when the model ties them
(qwen.py:192,211-212), into float32 logits.  Both are parts like the others, chosen by the
`kind` of `ModelConfig.embedding` and `ModelConfig.head`: an architecture that scales its
embedding, adds a learned position table or caps its logits registers a part of its own
instead of changing the model class.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, PendingSum, register_part


class TokenEmbedding:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab, spec.width), "table")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.table = tensors["weight"]

    def forward(self, ctx) -> torch.Tensor:
        resid = self.runtime.buffer("resid", (ctx.num_tokens, self.spec.width), torch.float32)
        keep = ctx.carried.get("embedding_copy")   # a pass entry may ask for a second copy of what leaves here
        scale = getattr(self.spec, "scale", 1.0)
        if keep is None and scale == 1.0:
            self.ops.embed(ctx.token_ids, self.table, resid, ctx.previous_tokens)
        else:
            self.ops.embed(ctx.token_ids, self.table, resid, ctx.previous_tokens, scale=scale, keep=keep)
            if keep is not None:
                ctx.carried["embedding_copied"] = True
        return resid


class PassEntry:
    """What entering pass t over a run of repeated layers does to the residual: the embedding's output is
    added again (every pass but the first) and the learned vector step[t], in 32-bit, in the kernel that
    also adds whatever branch outputs are still pending.  With `mix`, the residual x is instead replaced
    by Win [x ; e] + step[t] in every pass, the first included (e: the embedding's output)."""

    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        params = {"step": ParamSpec((spec.passes, spec.width), "bias")}
        if getattr(spec, "mix", False):
            params["in"] = ParamSpec((spec.width, 2 * spec.width), "mix")
        return params

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.step = tensors["step"].to(torch.float32).contiguous()
        self.mix = bool(getattr(spec, "mix", False))
        self.w_in = tensors["in"].contiguous() if self.mix else None
        self._kept = None

    def before_embedding(self, ctx) -> None:
        self._kept = None
        if self.mix or (self.spec.add_embedding and self.spec.passes > 1):
            self._kept = self.runtime.buffer("embedding_out", (ctx.num_tokens, self.spec.width), torch.float32)
            ctx.carried["embedding_copy"] = self._kept

    def begin(self, resid, ctx) -> None:
        if self._kept is not None and not ctx.carried.get("embedding_copied"):
            self._kept.copy_(resid)   # an embedding part that does not write the copy itself

    def forward(self, resid, delta, ctx, number: int):
        if not 0 <= number < self.spec.passes:
            raise ValueError(f"pass {number} of {self.spec.passes}")
        terms = PendingSum.of(delta)
        if self.mix:
            # x <- Win [x ; e] + step[t]: the pending sums are added, the residual and the kept embedding are laid
            # side by side in the engine's type by one kernel, and the product's 32-bit result, which reads
            # that copy only, overwrites the residual
            rt = self.runtime
            both = rt.buffer("pass_both", (resid.shape[0], 2 * self.spec.width), rt.act_dtype)
            self.ops.concat_cast(resid, terms, self._kept, both)
            self.ops.linear(both, self.w_in, resid, bias=self.step[number])
            return resid, None
        if number > 0 and self._kept is not None:
            terms.append((self._kept, 1.0))
        while len(terms) > 4:
            self.ops.tanh_norm(resid, terms[:4])
            terms = terms[4:]
        self.ops.tanh_norm(resid, terms, row_add=self.step[number])
        return resid, None


class TokenPositionEmbedding:
    """Token row plus the learned vector of the token's position, summed in 32-bit."""

    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab, spec.width), "table"),
                "positions": ParamSpec((spec.max_positions, spec.width), "table")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.table = tensors["weight"]
        self.position_table = tensors["positions"].to(self.table.dtype).contiguous()

    def forward(self, ctx) -> torch.Tensor:
        resid = self.runtime.buffer("resid", (ctx.num_tokens, self.spec.width), torch.float32)
        self.ops.embed(ctx.token_ids, self.table, resid, ctx.previous_tokens,
                       position_table=self.position_table, positions=ctx.positions)
        return resid


class LMHead:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab, spec.width), "matrix")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.weight = tensors["weight"]

    def forward(self, hidden) -> torch.Tensor:
        logits = self.runtime.buffer("logits", (hidden.shape[0], self.spec.vocab), torch.float32)
        if hidden.shape[0]:
            self.ops.linear(hidden, self.weight, logits)
            scale = float(getattr(self.spec, "scale", 1.0))
            if scale != 1.0:
                logits.mul_(scale)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "token_position_embedding", TokenPositionEmbedding)
register_part("head", "lm_head", LMHead)
register_part("pass_entry", "pass_entry", PassEntry)
