"""Grouped-query attention over the paged cache.

The formulas are Azimml/shrike's: q/k/v projections with optional bias, heads as
consecutive column blocks (shrike/models/qwen.py:111-122), position encoding on q
and k (qwen.py:123), new keys and values stored before attention reads
(shrike/engine/model_runner.py:69-70), q head i on kv head i // G, scores * scale,
a query at position p sees keys <= p (model_runner.py:129-150), softmax and PV in
32-bit, then the output projection (qwen.py:125).  The three projections are one
matrix product here (rows of Wq, Wk, Wv stacked at load), bias and rotation are
applied to its 32-bit result and rounded once, and one kernel serves single tokens
and portions alike.  Optional `window`: a query sees only the `window` latest keys.

`SharedKeyValueAttention` is the same attention for a design whose values are its keys: one q|k
projection, no value projection and no rotation; queries and keys normed over the whole projection,
a query temperature that grows with the logarithm of the position, scores soft-capped and biased
by distance, a key window.  Each of these is a parameter of its spec.

`GatedHeadAttention` adds, each as an option of its spec: a norm of q and k per head, a rotation of
part of each head (in either pairing, with stretched or divided frequencies), chunks of positions in
place of a window, keys and values of different sizes, a sigmoid gate per head on the output, a learned
sink per head in the softmax's denominator, a norm of q and k over the whole projection, a short causal
convolution over time behind the projections (its last inputs are per-request state), a unit norm of every
value head, a soft cap on the scores, a window that keeps the sequence's first keys visible, and keys and
values read from another layer's cache.
"""

from __future__ import annotations

import torch

from .base import KVNeed, ParamSpec, StateNeed, part_class, register_part
from .rotary import PairRotation


class PagedAttention:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        q_out = spec.num_heads * spec.head_dim
        kv_out = spec.num_kv_heads * spec.head_dim
        params = {
            "q_proj.weight": ParamSpec((q_out, spec.width), "matrix"),
            "k_proj.weight": ParamSpec((kv_out, spec.width), "matrix"),
            "v_proj.weight": ParamSpec((kv_out, spec.width), "matrix"),
            "o_proj.weight": ParamSpec((spec.width, q_out), "matrix"),
        }
        if spec.qkv_bias:
            params["q_proj.bias"] = ParamSpec((q_out,), "bias")
            params["k_proj.bias"] = ParamSpec((kv_out,), "bias")
            params["v_proj.bias"] = ParamSpec((kv_out,), "bias")
        if spec.out_bias:
            params["o_proj.bias"] = ParamSpec((spec.width,), "bias")
        return params

    @staticmethod
    def cache_needs(spec) -> list:
        return [KVNeed(spec.num_kv_heads, spec.head_dim, spec.window)]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec = spec
        self.ops = ops
        self.runtime = runtime
        ops.check_head_dim(spec.head_dim)
        self.w_qkv = torch.cat(
            [tensors.pop("q_proj.weight"), tensors.pop("k_proj.weight"), tensors.pop("v_proj.weight")]
        ).contiguous()
        self.w_o = tensors.pop("o_proj.weight").contiguous()
        self.b_qkv = None
        if spec.qkv_bias:
            self.b_qkv = torch.cat(
                [tensors.pop("q_proj.bias"), tensors.pop("k_proj.bias"), tensors.pop("v_proj.bias")]
            ).to(torch.float32).contiguous()
        self.b_o = tensors.pop("o_proj.bias").to(torch.float32).contiguous() if spec.out_bias else None
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, ops, runtime)
        self.q_width = spec.num_heads * spec.head_dim
        self.qkv_width = (spec.num_heads + 2 * spec.num_kv_heads) * spec.head_dim

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        n = x.shape[0]
        qkv = rt.buffer("qkv", (n, self.qkv_width), torch.float32)
        qkv = ops.linear(x, self.w_qkv, qkv, allow_partials=True)
        group, keys, values = ctx.storage.keys_values(run.cache)
        view = ctx.groups[group]
        q = rt.buffer("q", (n, self.q_width), rt.act_dtype)
        table = self.position.rotary_table() if self.position is not None else None
        fused = self.position is None or table is not None
        if fused:
            ops.rope_kv_write(
                qkv, self.b_qkv, ctx.positions, table, q,
                keys if run.writes_cache else None, values if run.writes_cache else None,
                view.slot_mapping, spec.num_heads, spec.num_kv_heads, spec.head_dim,
            )
        else:  # a position encoding with no table: rotate q and k with its own code, then store
            kv_width = spec.num_kv_heads * spec.head_dim
            k_new = rt.buffer("k_new", (n, kv_width), rt.act_dtype)
            v_new = rt.buffer("v_new", (n, kv_width), rt.act_dtype)
            ops.rope_kv_write(
                qkv, self.b_qkv, ctx.positions, None, q, None, None, view.slot_mapping,
                spec.num_heads, spec.num_kv_heads, spec.head_dim, k_out=k_new, v_out=v_new,
            )
            self.position.apply(
                q.view(n, spec.num_heads, spec.head_dim),
                k_new.view(n, spec.num_kv_heads, spec.head_dim),
                ctx.positions,
            )
            if run.writes_cache:
                ops.kv_write(k_new, v_new, keys, values, view.slot_mapping)
        attn = rt.buffer("attn_out", (n, self.q_width), rt.act_dtype)
        ops.paged_attention(
            q, keys, values, view.block_table, ctx.q_start, ctx.ctx_len, ctx.seq_of_token,
            spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.scale, spec.window, attn,
            max_q_len=ctx.max_q_len, max_ctx_len=ctx.max_ctx_len, min_q_len=ctx.min_q_len, q_lens=ctx.q_lens,
        )
        delta = rt.buffer("mixer_delta", (n, spec.width), torch.float32)
        return ops.linear(attn, self.w_o, delta, bias=self.b_o, allow_partials=True)


def padded_head(dim: int) -> int:
    """The head size the attention kernels are built for: the next multiple of 16."""
    return -(-dim // 16) * 16


class SharedKeyValueAttention:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        q_out = spec.num_heads * spec.head_dim
        k_out = spec.num_kv_heads * spec.head_dim
        params = {
            "q_proj.weight": ParamSpec((q_out, spec.width), "matrix"),
            "k_proj.weight": ParamSpec((k_out, spec.width), "matrix"),
            "o_proj.weight": ParamSpec((spec.width, q_out), "matrix"),
        }
        if spec.qk_norm:
            params["q_norm.weight"] = ParamSpec((q_out,), "norm")
            params["k_norm.weight"] = ParamSpec((k_out,), "norm")
        return params

    @staticmethod
    def cache_needs(spec) -> list:
        return [KVNeed(spec.num_kv_heads, padded_head(spec.head_dim), spec.window)]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.padded = padded_head(spec.head_dim)
        ops.check_head_dim(self.padded)
        self.w_qk = torch.cat([tensors.pop("q_proj.weight"), tensors.pop("k_proj.weight")]).contiguous()
        w_o = tensors.pop("o_proj.weight")
        if self.padded != spec.head_dim:   # the kernels' heads are wider: the added columns meet zeros
            wide = w_o.new_zeros(spec.width, spec.num_heads, self.padded)
            wide[:, :, : spec.head_dim] = w_o.view(spec.width, spec.num_heads, spec.head_dim)
            w_o = wide.view(spec.width, spec.num_heads * self.padded)
        self.w_o = w_o.contiguous()
        self.q_weight = self.k_weight = None
        if spec.qk_norm:
            self.q_weight = tensors.pop("q_norm.weight").to(torch.float32).contiguous()
            self.k_weight = tensors.pop("k_norm.weight").to(torch.float32).contiguous()
        self.slopes = None
        if spec.slope_decay is not None:
            slopes = [2.0 ** (-spec.slope_decay * (head + 1) / spec.num_heads) for head in range(spec.num_heads)]
            self.slopes = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.qk_width = (spec.num_heads + spec.num_kv_heads) * spec.head_dim
        self.out_width = spec.num_heads * self.padded

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        n = x.shape[0]
        qk = rt.buffer("qkv", (n, self.qk_width), torch.float32)
        qk = ops.linear(x, self.w_qk, qk, allow_partials=True)
        group, keys, values = ctx.storage.keys_values(run.cache)
        view = ctx.groups[group]
        q = rt.buffer("q", (n, self.out_width), rt.act_dtype)
        ops.qk_norm_store(
            qk, self.q_weight, self.k_weight, spec.eps, ctx.positions, spec.q_temperature, q,
            keys if run.writes_cache else None, values if run.writes_cache else None, view.slot_mapping,
            spec.num_heads, spec.num_kv_heads, spec.head_dim, self.padded,
        )
        attn = rt.buffer("attn_out", (n, self.out_width), rt.act_dtype)
        ops.paged_attention(
            q, keys, values, view.block_table, ctx.q_start, ctx.ctx_len, ctx.seq_of_token,
            spec.num_heads, spec.num_kv_heads, self.padded, spec.scale, spec.window, attn,
            max_q_len=ctx.max_q_len, max_ctx_len=ctx.max_ctx_len, min_q_len=ctx.min_q_len, q_lens=ctx.q_lens,
            softcap=spec.softcap, slopes=self.slopes,
        )
        delta = rt.buffer("mixer_delta", (n, spec.width), torch.float32)
        return ops.linear(attn, self.w_o, delta, allow_partials=True)


class GatedHeadAttention:
    """Grouped-query attention with the options of `GatedHeadAttentionSpec`: biases, a root-mean-square
    norm of q and k per head with one weight for all heads, a rotation of each head's first
    dimensions, a window or chunks of positions, an output gate per head.  q, k, v and the gate are
    one matrix product; one kernel turns its 32-bit result into queries and cache rows; the paged
    attention kernels run as they are (a chunk is handed to them as a negative window).  Keys and
    values share the pages' head size, the next multiple of 16 above the larger of the two; the
    columns so added meet zeros in q, the pages and `o_proj`."""

    capture_safe = True

    @staticmethod
    def _own_kv(spec) -> bool:
        return getattr(spec, "own_kv", True)

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        q_out, k_out, v_out = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.num_kv_heads * spec.value_dim
        own = GatedHeadAttention._own_kv(spec)
        whole = spec.qk_norm == "whole"
        params = {"q_proj.weight": ParamSpec((q_out, spec.width), "matrix")}
        if own:
            params["k_proj.weight"] = ParamSpec((k_out, spec.width), "matrix")
            params["v_proj.weight"] = ParamSpec((v_out, spec.width), "matrix")
        params["o_proj.weight"] = ParamSpec((spec.width, spec.num_heads * spec.value_dim), "matrix")
        if spec.qkv_bias:
            params["q_proj.bias"] = ParamSpec((q_out,), "bias")
            if own:
                params["k_proj.bias"] = ParamSpec((k_out,), "bias")
                params["v_proj.bias"] = ParamSpec((v_out,), "bias")
        if spec.out_bias:
            params["o_proj.bias"] = ParamSpec((spec.width,), "bias")
        if spec.qk_norm:
            params["q_norm.weight"] = ParamSpec((q_out if whole else spec.head_dim,), "norm")
            if own:
                params["k_norm.weight"] = ParamSpec((k_out if whole else spec.head_dim,), "norm")
        if getattr(spec, "conv", None):
            params["q_conv.weight"] = ParamSpec((q_out, spec.conv), "conv")
            params["k_conv.weight"] = ParamSpec((k_out, spec.conv), "conv")
            params["v_conv.weight"] = ParamSpec((v_out, spec.conv), "conv")
        if spec.head_gate:
            params["gate.weight"] = ParamSpec((spec.num_heads, spec.width), "matrix")
        if getattr(spec, "sink", False):
            params["sink"] = ParamSpec((spec.num_heads,), "sink")
        return params

    @staticmethod
    def cache_needs(spec) -> list:
        needs = [KVNeed(spec.num_kv_heads, padded_head(max(spec.head_dim, spec.value_dim)), spec.window, chunk=spec.chunk,
                        keep_first=getattr(spec, "keep_first", 0) if spec.window is not None else 0)]
        taps = getattr(spec, "conv", None)
        if taps and taps > 1:   # the last projected q, k and v of the request, the newest last
            channels = spec.num_heads * spec.head_dim + spec.num_kv_heads * (spec.head_dim + spec.value_dim)
            needs.append(StateNeed((taps - 1, channels), "float32", name="conv"))
        return needs

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.padded = padded_head(max(spec.head_dim, spec.value_dim))
        ops.check_head_dim(self.padded)
        self.own_kv = self._own_kv(spec)
        self.whole_norm = spec.qk_norm == "whole"
        projections = (("q_proj", spec.num_heads), ("k_proj", spec.num_kv_heads)) if self.own_kv else (("q_proj", spec.num_heads),)
        rotation = None
        if getattr(spec, "rotation", None) is not None:
            # the kernel pairs dimension i with i + dims/2: another pairing, and a factor on cos and sin,
            # become a reordering and a scaling of the q and k rows (weights and biases alike)
            rotation = PairRotation(spec.rotation, runtime.device)
            reordered = rotation.order != list(range(spec.rotation.dims))
            if (spec.qk_norm or getattr(spec, "conv", None)) and reordered:
                raise NotImplementedError("a q/k norm weight or a convolution with neighbours paired: those are not reordered")
            if not spec.qk_norm:   # with a norm between projection and rotation the factor goes into the norm's weight
                for name, heads in projections:
                    for kind in ("weight", "bias") if spec.qkv_bias else ("weight",):
                        tensors[f"{name}.{kind}"] = rotation.arrange_rows(tensors[f"{name}.{kind}"], heads, spec.head_dim)
        rows = [tensors.pop("q_proj.weight")]
        if self.own_kv:
            rows += [tensors.pop("k_proj.weight"), tensors.pop("v_proj.weight")]
        self.channels = sum(r.shape[0] for r in rows)   # what a convolution runs over: q, k and v
        if spec.head_gate:
            rows.append(tensors.pop("gate.weight").to(rows[0].dtype))
        extra = -sum(r.shape[0] for r in rows) % 16   # rows of zeros: output rows of a whole number of 64 bytes
        if extra:
            rows.append(rows[0].new_zeros(extra, spec.width))
        self.w_fused = torch.cat(rows).contiguous()
        self.total = self.w_fused.shape[0]
        self.bias = None
        if spec.qkv_bias:
            bias = torch.zeros(self.total, dtype=torch.float32, device=self.w_fused.device)   # the gate has none
            given = [tensors.pop("q_proj.bias")] + ([tensors.pop("k_proj.bias"), tensors.pop("v_proj.bias")] if self.own_kv else [])
            given = torch.cat(given)
            bias[: given.numel()] = given.to(torch.float32)
            self.bias = bias
        self.taps = None
        if getattr(spec, "conv", None):
            self.taps = torch.cat([tensors.pop(f"{name}_conv.weight") for name in ("q", "k", "v")]).to(torch.float32).contiguous()
            # a convolution of one tap keeps nothing: an empty state of the right shape stands in
            self.no_state = torch.zeros((1, 0, self.channels), dtype=torch.float32, device=self.taps.device)
        w_o = tensors.pop("o_proj.weight")
        if self.padded != spec.value_dim:   # the kernels' heads are wider: the added columns meet zeros
            wide = w_o.new_zeros(spec.width, spec.num_heads, self.padded)
            wide[:, :, : spec.value_dim] = w_o.view(spec.width, spec.num_heads, spec.value_dim)
            w_o = wide.view(spec.width, spec.num_heads * self.padded)
        self.w_o = w_o.contiguous()
        self.b_o = tensors.pop("o_proj.bias").to(torch.float32).contiguous() if spec.out_bias else None
        self.q_weight = self.k_weight = None
        if spec.qk_norm:
            self.q_weight = tensors.pop("q_norm.weight").to(torch.float32).contiguous()
            self.k_weight = tensors.pop("k_norm.weight").to(torch.float32).contiguous() if self.own_kv else None
            if rotation is not None and rotation.gain != 1.0:
                # the factor on cos and sin: a rotation is linear, so the rotated dimensions' norm weights carry it
                def with_gain(weight, heads):
                    shaped = weight.view(heads if self.whole_norm else 1, spec.head_dim).clone()
                    shaped[:, : spec.rotation.dims] *= rotation.gain
                    return shaped.reshape(-1).contiguous()
                self.q_weight = with_gain(self.q_weight, spec.num_heads)
                if self.k_weight is not None:
                    self.k_weight = with_gain(self.k_weight, spec.num_kv_heads)
        self.inv_freq, self.rot = None, 0
        if spec.rotary is not None:
            dims, base = spec.rotary
            table = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
            self.inv_freq, self.rot = table.to(torch.float32).to(runtime.device), int(dims)
        if rotation is not None:
            self.inv_freq, self.rot = rotation.inv_freq, int(spec.rotation.dims)
        self.sinks = tensors.pop("sink").to(torch.float32).contiguous() if getattr(spec, "sink", False) else None
        self.out_width = spec.num_heads * self.padded

    def forward(self, x, ctx, run):
        spec, rt, ops = self.spec, self.runtime, self.ops
        if run.writes_cache != self.own_kv:
            raise ValueError("a layer with key and value projections writes its cache; one without reads another's")
        n = x.shape[0]
        fused = rt.buffer("qkv", (n, self.total), torch.float32)
        fused = ops.linear(x, self.w_fused, fused, allow_partials=True)
        bias = self.bias
        if self.taps is not None:
            # the convolution over time runs on the projected values, bias included; the T - 1 before this portion
            # are the request's state
            mixed = rt.buffer("qkv_conv", (n, self.total), torch.float32)
            ops.short_conv(fused, bias, self.taps, ctx.storage.state[(run.cache, "conv")] if self.taps.shape[1] > 1 else self.no_state,
                           ctx.q_start, ctx.state_slot, ctx.seq_of_token, mixed, ctx.num_seqs, self.channels)
            fused, bias = mixed, None
        group, keys, values = ctx.storage.keys_values(run.cache)
        view = ctx.groups[group]
        q = rt.buffer("q", (n, self.out_width), rt.act_dtype)
        gate = rt.buffer("head_gate", (n, spec.num_heads), torch.float32) if spec.head_gate else None
        ops.head_prep(
            fused, bias, ctx.positions, self.inv_freq, self.rot, self.q_weight, self.k_weight, spec.eps, q,
            keys if run.writes_cache else None, values if run.writes_cache else None, view.slot_mapping, gate,
            spec.num_heads, spec.num_kv_heads if self.own_kv else 0, spec.head_dim, spec.value_dim, self.padded,
            **({"whole_norm": True} if self.whole_norm else {}),
            **({"value_norm": True} if getattr(spec, "value_norm", False) else {}),
        )
        attn = rt.buffer("attn_out", (n, self.out_width), rt.act_dtype)
        ops.paged_attention(
            q, keys, values, view.block_table, ctx.q_start, ctx.ctx_len, ctx.seq_of_token,
            spec.num_heads, spec.num_kv_heads, self.padded, spec.scale, spec.window, attn,
            max_q_len=ctx.max_q_len, max_ctx_len=ctx.max_ctx_len, min_q_len=ctx.min_q_len, q_lens=ctx.q_lens,
            **({"chunk": spec.chunk} if spec.chunk is not None else {}),
            **({"sinks": self.sinks} if self.sinks is not None else {}),
            **({"softcap": spec.softcap} if getattr(spec, "softcap", None) else {}),
            **({"keep_first": spec.keep_first} if getattr(spec, "keep_first", 0) else {}),
        )
        if gate is not None:
            ops.head_scale(attn, gate, spec.num_heads, self.padded)
        delta = rt.buffer("mixer_delta", (n, spec.width), torch.float32)
        return ops.linear(attn, self.w_o, delta, bias=self.b_o, allow_partials=True)


register_part("mixer", "attention", PagedAttention)
register_part("mixer", "gated_head_attention", GatedHeadAttention)
register_part("mixer", "shared_kv_attention", SharedKeyValueAttention)
