"""Linear attention with a fixed decay per head.

Per head, with q = silu(Wq x), k = silu(Wk x), v = silu(Wv x):

    S_t = d S_(t-1) + k_t v_t^T      (S = 0 before a sequence's first token; d the head's decay, 0 < d <= 1)
    o_t = S_t^T q_t                   (no scale)

The heads' outputs, side by side, are divided by their common root mean square, scaled by one
weight of that length, multiplied by sigmoid(Wg x) and projected.  S of every head is the request's
state: one float32 slot `[heads, dim * vdim (rounded up to four)]`, zeroed by the step function when
the request is opened, read and left updated by the scan kernel however the prompt is cut.  Over a
portion of several tokens the recurrence is evaluated as products over runs of tokens,

    o_t = d^(t-a+1) S_a^T q_t + sum_(a <= j <= t) d^(t-j) (q_t . k_j) v_j,

which is the same sum in another order; a single token takes one update of S.  The four projections
are one matrix product; activations, decays, their powers and the state are 32-bit.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, StateNeed, register_part
from .matrix_memory import padded_rows


class DecayLinearAttention:
    capture_safe = True   # it reads the batch's metadata on the device only and skips rows whose state slot is -1

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        qk, v = spec.num_heads * spec.head_dim, spec.num_heads * spec.value_dim
        return {
            "q_proj.weight": ParamSpec((qk, spec.width), "matrix"),
            "k_proj.weight": ParamSpec((qk, spec.width), "matrix"),
            "v_proj.weight": ParamSpec((v, spec.width), "matrix"),
            "gate.weight": ParamSpec((v, spec.width), "matrix"),
            "o_proj.weight": ParamSpec((spec.width, v), "matrix"),
            "norm.weight": ParamSpec((v,), "norm"),
        }

    @staticmethod
    def state_shape(spec) -> tuple:
        return (spec.num_heads, -(-spec.head_dim * spec.value_dim // 4) * 4)   # every head starts on a 16-byte border

    @staticmethod
    def cache_needs(spec) -> list:
        return [StateNeed(DecayLinearAttention.state_shape(spec), "float32")]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        rows = [tensors.pop(name) for name in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate.weight")]
        self.w_fused = padded_rows(torch.cat(rows))
        self.total = self.w_fused.shape[0]
        self.norm_weight = tensors.pop("norm.weight").to(torch.float32).contiguous()
        self.w_o = tensors.pop("o_proj.weight").contiguous()
        self.out_width = spec.num_heads * spec.value_dim
        self.gate_at = 2 * spec.num_heads * spec.head_dim + self.out_width   # the gate's first column of the fused product
        self.decays = torch.tensor([float(d) for d in spec.decays], dtype=torch.float64).to(torch.float32).to(runtime.device)

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        if not run.writes_cache:
            raise NotImplementedError("linear attention owns its state: no run can read another run's")
        n = x.shape[0]
        fused = rt.buffer("memory_in", (n, self.total), torch.float32)
        fused = ops.linear(x, self.w_fused, fused, allow_partials=True)
        scanned = rt.buffer("memory_num", (n, self.out_width), torch.float32)
        ops.decay_scan(fused, self.decays, ctx.storage.state[run.cache], ctx.q_start, ctx.state_slot, scanned,
                       ctx.num_seqs, spec.num_heads, spec.head_dim, spec.value_dim, longest=ctx.max_q_len)
        out = rt.buffer("memory_out", (n, self.out_width), rt.act_dtype)
        ops.norm_gate(scanned, fused, self.gate_at, self.norm_weight, spec.eps, out)
        delta = rt.buffer("memory_delta", (n, spec.width), torch.float32)
        return ops.linear(out, self.w_o, delta, allow_partials=True)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
