"""A linear recurrence with one gate for both ends (the HGRN2 cell): what a state row keeps, f, fixes what it takes in, 1 - f.

Per head, with q = silu(Wq x) (dim numbers), v = Wv x (vdim numbers) and a gate per channel of q,
f = lower + (1 - lower) * sigmoid(Wf x + b):

    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T      (S = 0 before a sequence's first token)
    o_t = S_t^T q_t                                 (no key of its own, no scale)

Every head's o is divided by its root mean square and scaled by one weight of the head's size, the heads side
by side are projected.  S of every head is the request's state: one float32 slot `[heads, dim * vdim (rounded up
to four)]`, zeroed by the step function when the request is opened, read and left updated by the scan kernel
however the prompt is cut.  A single token takes one update of S.  A long portion is cut into runs of tokens that
walk side by side: every run first from a zero state (which also gives the product of its gates), then the
runs' states are carried in order, then every run walks again from the state it starts from; the same numbers up
to the order of a few sums.  The three projections are one matrix product; activations, gates, the state and the
norm are 32-bit.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, StateNeed, register_part
from .matrix_memory import padded_rows


class GatedLinearRecurrence:
    capture_safe = True   # it reads the batch's metadata on the device only and leaves rows alone whose state slot is -1

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        qk, v = spec.num_heads * spec.head_dim, spec.num_heads * spec.value_dim
        params = {
            "q_proj.weight": ParamSpec((qk, spec.width), "matrix"),
            "forget_gate.weight": ParamSpec((qk, spec.width), "matrix"),
            "forget_gate.bias": ParamSpec((qk,), "bias"),
            "v_proj.weight": ParamSpec((v, spec.width), "matrix"),
            "o_proj.weight": ParamSpec((spec.width, v), "matrix"),
            "norm.weight": ParamSpec((spec.value_dim,), "norm"),
        }
        if spec.lower_bound:
            params["lower"] = ParamSpec((qk,), "unit_interval")
        return params

    @staticmethod
    def state_shape(spec) -> tuple:
        return (spec.num_heads, -(-spec.head_dim * spec.value_dim // 4) * 4)   # every head starts on a 16-byte border

    @staticmethod
    def cache_needs(spec) -> list:
        return [StateNeed(GatedLinearRecurrence.state_shape(spec), "float32")]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        rows = [tensors.pop(name) for name in ("q_proj.weight", "forget_gate.weight", "v_proj.weight")]
        self.w_fused = padded_rows(torch.cat(rows))
        self.total = self.w_fused.shape[0]
        self.gate_bias = tensors.pop("forget_gate.bias").to(torch.float32).contiguous()
        self.lower = tensors.pop("lower").to(torch.float32).contiguous() if spec.lower_bound else None
        self.norm_weight = tensors.pop("norm.weight").to(torch.float32).contiguous()
        self.w_o = tensors.pop("o_proj.weight").contiguous()
        self.out_width = spec.num_heads * spec.value_dim

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        if not run.writes_cache:
            raise NotImplementedError("a recurrence owns its state: no run can read another run's")
        n = x.shape[0]
        fused = rt.buffer("memory_in", (n, self.total), torch.float32)
        fused = ops.linear(x, self.w_fused, fused, allow_partials=True)
        scanned = rt.buffer("memory_num", (n, self.out_width), torch.float32)
        ops.gated_scan(fused, self.gate_bias, self.lower, ctx.storage.state[run.cache], ctx.q_start, ctx.state_slot, scanned,
                       ctx.num_seqs, spec.num_heads, spec.head_dim, spec.value_dim, q_lens=ctx.q_lens)
        out = rt.buffer("memory_out", (n, self.out_width), rt.act_dtype)
        ops.head_rms(scanned, self.norm_weight, spec.eps, out, spec.num_heads)
        delta = rt.buffer("memory_delta", (n, spec.width), torch.float32)
        return ops.linear(out, self.w_o, delta, allow_partials=True)


register_part("mixer", "gated_linear_recurrence", GatedLinearRecurrence)
