"""Causal softmax attention over a cached low-rank latent.

Per token only the latent c = RMS(Wdkv x) * weight is cached (`latent_rank` numbers, one plane of
pages).  Head h's keys and values are k = Wuk_h c and v = Wuv_h c, its score scale * q_h.k.  Neither
k nor v is ever formed for a cached token: the key projection is moved to the query and the value
projection to the output,

    (Wq_h x) . (Wuk_h c_j) = (Wuk_h^T Wq_h x) . c_j      Wo_h sum_j p_j Wuv_h c_j = (Wo_h Wuv_h) sum_j p_j c_j,

so the layer is attention with ONE key/value head of size `latent_rank` whose keys and values are
the same cached rows, and it runs on the engine's paged attention kernels as they are.  The two
products of matrices are formed once, when the weights are loaded (in float32, then kept in the
engine's type): the query projection becomes [heads * rank, width] and the output projection
[width, heads * rank].  With rank = 2 * dim that is twice the weights and products of the two
projections, about 1 % of a layer's; in exchange a step has no per-head products at all.  A layer
without a latent of its own reads the pages another layer's run wrote (the run order names the
cache) with its own Wuk, Wuv, queries and output.  An optional gate multiplies head h's output by
sigmoid(Wg x)_h; it is applied to the attended latent, which the output projection takes linearly.
Query, latent and gate come from one fused product.
"""

from __future__ import annotations

import torch

from .attention import padded_head
from .base import KVNeed, ParamSpec, register_part
from .matrix_memory import padded_rows


class LatentAttention:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        q_out = spec.num_heads * spec.head_dim
        v_out = spec.num_heads * spec.value_dim
        params = {"q_proj.weight": ParamSpec((q_out, spec.width), "matrix")}
        if spec.own_latent:
            params["kv_down.weight"] = ParamSpec((spec.latent_rank, spec.width), "matrix")
            params["kv_norm.weight"] = ParamSpec((spec.latent_rank,), "norm")
        params["k_up.weight"] = ParamSpec((q_out, spec.latent_rank), "matrix")
        params["v_up.weight"] = ParamSpec((v_out, spec.latent_rank), "matrix")
        if spec.gated:
            params["gate.weight"] = ParamSpec((spec.num_heads, spec.width), "matrix")
        params["o_proj.weight"] = ParamSpec((spec.width, v_out), "matrix")
        return params

    @staticmethod
    def cache_needs(spec) -> list:
        return [KVNeed(1, padded_head(spec.latent_rank), None, planes=1)]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        heads, dim, vdim, rank = spec.num_heads, spec.head_dim, spec.value_dim, spec.latent_rank
        self.padded = padded_head(rank)
        ops.check_head_dim(self.padded)
        k_up = tensors.pop("k_up.weight").float().view(heads, dim, rank)
        v_up = tensors.pop("v_up.weight").float().view(heads, vdim, rank)
        w_q = tensors.pop("q_proj.weight")
        w_o = tensors.pop("o_proj.weight")
        kept = w_q.dtype
        # queries straight into the latent space: rows [h * padded + r] = sum_d Wuk[h, d, r] Wq[h * dim + d, :]
        absorbed = torch.zeros(heads, self.padded, spec.width, dtype=torch.float32, device=w_q.device)
        absorbed[:, :rank] = torch.einsum("hdr,hdw->hrw", k_up, w_q.float().view(heads, dim, spec.width))
        rows = [absorbed.view(heads * self.padded, spec.width).to(kept)]
        # the attended latent straight to the residual's width: columns [h * padded + r] = Wo[:, h, :] Wuv[h, :, r]
        expanded = torch.zeros(spec.width, heads, self.padded, dtype=torch.float32, device=w_o.device)
        expanded[:, :, :rank] = torch.einsum("whv,hvr->whr", w_o.float().view(spec.width, heads, vdim), v_up)
        self.w_o = expanded.view(spec.width, heads * self.padded).to(kept).contiguous()
        del absorbed, expanded
        self.latent_weight = None
        if spec.own_latent:
            rows.append(tensors.pop("kv_down.weight"))
            self.latent_weight = tensors.pop("kv_norm.weight").to(torch.float32).contiguous()
        if spec.gated:
            rows.append(tensors.pop("gate.weight"))
        used = sum(block.shape[0] for block in rows)
        if used % 16:   # the library's fast product kernels want a row count they can tile: zero rows fill it up
            rows.append(w_q.new_zeros(16 - used % 16, spec.width))
        self.w_in = torch.cat(rows).contiguous()
        self.q_width = heads * self.padded
        self.in_width = self.w_in.shape[0]

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        heads, padded = spec.num_heads, self.padded
        n = x.shape[0]
        fused = rt.buffer("qkv", (n, self.in_width), torch.float32)
        fused = ops.linear(x, self.w_in, fused, allow_partials=True)
        group, latents, _ = ctx.storage.keys_values(run.cache)
        view = ctx.groups[group]
        q = rt.buffer("q", (n, self.q_width), rt.act_dtype)
        gate = rt.buffer("head_gate", (n, heads), torch.float32) if spec.gated else None
        writes = spec.own_latent and run.writes_cache
        ops.latent_store(fused, self.latent_weight, spec.eps, q, latents if writes else None, view.slot_mapping, gate,
                         self.q_width, spec.latent_rank if spec.own_latent else 0, padded, heads if spec.gated else 0)
        attended = rt.buffer("attn_out", (n, self.q_width), rt.act_dtype)
        ops.paged_attention(
            q, latents, latents, view.block_table, ctx.q_start, ctx.ctx_len, ctx.seq_of_token,
            heads, 1, padded, spec.scale, None, attended,
            max_q_len=ctx.max_q_len, max_ctx_len=ctx.max_ctx_len, min_q_len=ctx.min_q_len, q_lens=ctx.q_lens,
        )
        if spec.gated:
            ops.head_scale(attended, gate, heads, padded)
        delta = rt.buffer("mixer_delta", (n, spec.width), torch.float32)
        return ops.linear(attended, self.w_o, delta, allow_partials=True)


register_part("mixer", "latent_attention", LatentAttention)


class RotaryLatentAttention:
    """Latent attention whose keys have a rotated part that all heads share (`RotaryLatentAttentionSpec`).

    A token's page row is [c | r | 0]: the normed latent, the rotated shared key part, zeros up to the
    next multiple of 16.  It serves as key AND value of one key/value head on the paged attention
    kernels: head h's query row is [Wuk_h^T q_plain | rotated q part | 0], whose dot product with the
    page row is q_plain . (Wuk_h c) + q_rotated . r, and the attended row's first `latent_rank` numbers
    are sum_j p_j c_j, from which Wuv_h makes the head's output (a product per head; the columns
    that met r meet zeros in Wuv).  Wuk_h^T Wq_h is formed once when the weights are loaded (in
    float64, then kept in the engine's type).  The gate multiplies the heads' outputs element by
    element, which is why Wuv is not folded into the output projection here.  Query, latent, shared key
    part and gate come from one fused product; the pairing of the rotation is a reordering of the rows
    of the query's and the key part's projections, made at load, the factor on cos and sin goes to the
    kernel that rotates.
    """

    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        q_out = spec.num_heads * (spec.head_dim + spec.rotary_dim)
        v_out = spec.num_heads * spec.value_dim
        params = {
            "q_proj.weight": ParamSpec((q_out, spec.width), "matrix"),
            "kv_down.weight": ParamSpec((spec.latent_rank + spec.rotary_dim, spec.width), "matrix"),
            "kv_norm.weight": ParamSpec((spec.latent_rank,), "norm"),
            "k_up.weight": ParamSpec((spec.num_heads * spec.head_dim, spec.latent_rank), "matrix"),
            "v_up.weight": ParamSpec((v_out, spec.latent_rank), "matrix"),
            "o_proj.weight": ParamSpec((spec.width, v_out), "matrix"),
        }
        if spec.gate == "element":
            params["gate.weight"] = ParamSpec((v_out, spec.width), "matrix")
        return params

    @staticmethod
    def cache_needs(spec) -> list:
        return [KVNeed(1, padded_head(spec.latent_rank + spec.rotary_dim), spec.window, planes=1)]

    def __init__(self, spec, tensors, ops, runtime):
        from .rotary import PairRotation

        self.spec, self.ops, self.runtime = spec, ops, runtime
        heads, dim, rot, vdim, rank = spec.num_heads, spec.head_dim, spec.rotary_dim, spec.value_dim, spec.latent_rank
        self.padded = padded_head(rank + rot)
        ops.check_head_dim(self.padded)
        self.rotation = PairRotation(spec.rotation, runtime.device)
        w_q = tensors.pop("q_proj.weight")
        kept = w_q.dtype
        per_head = w_q.view(heads, dim + rot, spec.width)
        k_up = tensors.pop("k_up.weight").double().view(heads, dim, rank)
        # rows [h, r] = sum_d Wuk[h, d, r] Wq[h, d, :]: the query goes straight into the latent's space
        absorbed = torch.einsum("hdr,hdw->hrw", k_up, per_head[:, :dim].double()).to(kept)
        turned = self.rotation.arrange_rows(per_head[:, dim:].reshape(heads * rot, spec.width), heads, rot, fold_gain=False)
        rows = [torch.cat([absorbed, turned.view(heads, rot, spec.width)], dim=1).reshape(heads * (rank + rot), spec.width)]
        down = tensors.pop("kv_down.weight")
        rows += [down[:rank], self.rotation.arrange_rows(down[rank:], 1, rot, fold_gain=False)]
        self.gated = spec.gate == "element"
        if self.gated:
            rows.append(tensors.pop("gate.weight"))
        self.w_in = padded_rows(torch.cat(rows))
        self.in_width = self.w_in.shape[0]
        self.q_width = heads * (rank + rot)
        self.gate_at = self.q_width + rank + rot
        self.latent_weight = tensors.pop("kv_norm.weight").to(torch.float32).contiguous()
        # [heads, vdim, padded]: what follows the latent in an attended row meets zeros
        v_up = tensors.pop("v_up.weight").view(heads, vdim, rank)
        wide = v_up.new_zeros(heads, vdim, self.padded)
        wide[:, :, :rank] = v_up
        self.w_up = wide.contiguous()
        self.w_o = tensors.pop("o_proj.weight").contiguous()
        self.out_width = heads * vdim

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        heads, padded = spec.num_heads, self.padded
        n = x.shape[0]
        fused = rt.buffer("qkv", (n, self.in_width), torch.float32)
        fused = ops.linear(x, self.w_in, fused, allow_partials=True)
        group, latents, _ = ctx.storage.keys_values(run.cache)
        view = ctx.groups[group]
        q = rt.buffer("q", (n, heads * padded), rt.act_dtype)
        ops.latent_rope_store(fused, self.latent_weight, spec.eps, ctx.positions, self.rotation.inv_freq, self.rotation.gain,
                              q, latents if run.writes_cache else None, view.slot_mapping, heads, spec.latent_rank,
                              spec.rotary_dim, padded)
        attended = rt.buffer("attn_out", (n, heads * padded), rt.act_dtype)
        ops.paged_attention(
            q, latents, latents, view.block_table, ctx.q_start, ctx.ctx_len, ctx.seq_of_token,
            heads, 1, padded, spec.scale, spec.window, attended,
            max_q_len=ctx.max_q_len, max_ctx_len=ctx.max_ctx_len, min_q_len=ctx.min_q_len, q_lens=ctx.q_lens,
        )
        raised = rt.buffer("latent_up", (n, self.out_width), torch.float32)
        ops.head_linear(attended, self.w_up, raised, heads)
        out = rt.buffer("latent_gated", (n, self.out_width), rt.act_dtype)
        ops.norm_gate(raised, fused if self.gated else None, self.gate_at, None, spec.eps, out)
        delta = rt.buffer("mixer_delta", (n, spec.width), torch.float32)
        return ops.linear(out, self.w_o, delta, allow_partials=True)


register_part("mixer", "rotary_latent_attention", RotaryLatentAttention)
