"""A stand-in for the CUDA kernels, for tests that run without a GPU.

It has the interface of `shrike_b200.ops.cuda_ops.CudaOps` and the same meaning for
every argument, written with plain torch on the CPU, one loop at a time.  Host
logic (batch metadata, block tables, slots, the scheduler, the engine loop) can so
be driven end to end here; the kernels themselves are tested on the GPU.  Nothing
in the package imports this file.
"""

from __future__ import annotations

import math

import torch

from shrike_b200.sampling.rng import gumbel_noise_host


class EmulatedOps:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype
        self.launches = 0

    def check_head_dim(self, head_dim):
        if head_dim % 16 or not 16 <= head_dim <= 1024:
            raise ValueError(f"head size {head_dim} is not served")

    def embed(self, ids, table, out, previous=None, position_table=None, positions=None, scale=1.0, keep=None):
        ids = ids.long()
        if previous is not None and (ids < 0).any():
            ids = torch.where(ids < 0, previous.long()[(-1 - ids).clamp(min=0, max=previous.numel() - 1)], ids)
        out.copy_(table[ids].float() * scale)
        if position_table is not None:
            out.add_(position_table[positions.long()].float())
        if keep is not None:
            keep.copy_(out)

    def tanh_norm(self, resid, terms=(), row_add=None, rows=None, norms=()):
        x = resid if rows is None else resid[rows.long()]
        for tensor, scale in terms:
            summed = tensor.float().sum(0) if tensor.dim() == 3 else tensor.float()
            x = x + scale * (summed if rows is None else summed[rows.long()])
        if row_add is not None:
            x = x + row_add
        if rows is None and (terms or row_add is not None):
            resid.copy_(x)
        for alpha, weight, bias, out in norms:
            out.copy_((torch.tanh(alpha * x) * weight + bias).to(out.dtype))

    def head_prep(self, fused, bias, positions, inv_freq, rot, q_weight, k_weight, eps, q_out, keys, values, slots,
                  gate_out, num_heads, num_kv_heads, dim, vdim, padded, whole_norm=False, value_norm=False):
        if fused.dim() == 3:
            fused = fused.sum(0)
        n = fused.shape[0]
        x = fused.float() if bias is None else fused.float() + bias
        q_cols, k_cols, v_cols = num_heads * dim, num_kv_heads * dim, num_kv_heads * vdim
        q = x[:, :q_cols].view(n, num_heads, dim)
        k = x[:, q_cols: q_cols + k_cols].view(n, num_kv_heads, dim)
        v = x[:, q_cols + k_cols: q_cols + k_cols + v_cols].view(n, num_kv_heads, vdim)
        if whole_norm:   # over the whole projection, one weight a column
            if q_weight is not None:
                q = (q / torch.sqrt(q.pow(2).mean((-2, -1), keepdim=True) + eps)) * q_weight.view(num_heads, dim)
            if k_weight is not None and num_kv_heads:
                k = (k / torch.sqrt(k.pow(2).mean((-2, -1), keepdim=True) + eps)) * k_weight.view(num_kv_heads, dim)
        else:
            if q_weight is not None:
                q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight
            if k_weight is not None:
                k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight
        if value_norm and num_kv_heads:
            v = v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        if inv_freq is not None and rot:
            half = rot // 2
            angle = positions.float()[:, None] * inv_freq[None, :]
            cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]

            def turn(t):
                a, b = t[..., :half], t[..., half:rot]
                return torch.cat([a * cos - b * sin, b * cos + a * sin, t[..., rot:]], -1)

            q, k = turn(q), turn(k)

        def pad(t, heads, size):
            wide = torch.zeros(n, heads, padded)
            wide[:, :, :size] = t
            return wide.view(n, -1)

        q_out.copy_(pad(q, num_heads, dim).to(q_out.dtype))
        if gate_out is not None:
            gate_out.copy_(torch.sigmoid(x[:, q_cols + k_cols + v_cols: q_cols + k_cols + v_cols + num_heads]))
        if keys is not None:
            stored = slots.long() >= 0
            self.kv_write(pad(k, num_kv_heads, dim)[stored], pad(v, num_kv_heads, vdim)[stored], keys, values, slots[stored])

    def matrix_memory(self, fused, gate_bias, state, q_start, state_slot, numerator, denominator, weight, eps, out,
                      num_seqs, num_heads, dim, vdim, cap, floor, longest=0):
        if fused.dim() == 3:
            fused = fused.sum(0)
        x = fused.float()
        H, D, Dv = num_heads, dim, vdim
        out.zero_()
        for s in range(num_seqs):
            slot = int(state_slot[s])
            if slot < 0:
                continue
            held = state[slot]
            S = held[:, : D * Dv].reshape(H, D, Dv).clone()
            z = held[:, D * Dv: D * Dv + D].clone()
            m = held[:, D * Dv + D].clone()
            for t in range(int(q_start[s]), int(q_start[s + 1])):
                row = x[t]
                q = row[: H * D].view(H, D) * D ** -0.5
                k = row[H * D: 2 * H * D].view(H, D)
                v = row[2 * H * D: 2 * H * D + H * Dv].view(H, Dv)
                g = row[2 * H * D + H * Dv: 2 * H * D + 2 * H * Dv]
                gates = row[2 * H * D + 2 * H * Dv: 2 * H * D + 2 * H * Dv + 2 * H] + gate_bias
                a = cap * torch.tanh(gates[:H] / cap)
                f = torch.nn.functional.logsigmoid(cap * torch.tanh(gates[H:] / cap))
                m_new = torch.maximum(f + m, a)
                keep, take = torch.exp(f + m - m_new), torch.exp(a - m_new)
                S = keep[:, None, None] * S + take[:, None, None] * k[:, :, None] * v[:, None, :]
                z = keep[:, None] * z + take[:, None] * k
                m = m_new
                o = torch.einsum("hdv,hd->hv", S, q) / (torch.maximum((z * q).sum(-1).abs(), torch.exp(-m)) + floor)[:, None]
                o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps)
                out[t] = (o.reshape(-1) * weight * torch.sigmoid(g)).to(out.dtype)
            held[:, : D * Dv] = S.reshape(H, -1)
            held[:, D * Dv: D * Dv + D] = z
            held[:, D * Dv + D] = m

    def route_top(self, x, router, shared_gate, weights, top, renorm_eps, scoring="softmax", renormalise=True):
        logits = x.float() @ router.T
        scores = torch.sigmoid(logits) if scoring == "sigmoid" else torch.softmax(logits, -1)
        _, chosen = torch.topk(logits, top, -1)   # the logits order the experts as either score does
        best = scores.gather(1, chosen)
        weights.zero_()
        weights[:, : router.shape[0]].scatter_(1, chosen, best / (best.sum(-1, keepdim=True) + renorm_eps) if renormalise else best)
        if weights.shape[1] > router.shape[0]:
            weights[:, -1] = 1.0 if shared_gate is None else torch.sigmoid(x.float() @ shared_gate)

    def act_mul_blocks(self, gate_up, weights, out, experts, each, activation="silu", limit=None, weight_on="output"):
        inter = out.shape[1]
        column = torch.arange(inter)
        block = torch.where(column < experts * each, column // each, torch.full_like(column, experts))
        plain = torch.empty(out.shape, dtype=torch.float32)
        if weight_on == "input":   # the weight reaches gate and up alike
            share = weights[:, block]
            self.act_mul((gate_up.float() * torch.cat([share, share], -1)).to(gate_up.dtype), plain, 0, activation, limit)
            out.copy_(plain.to(out.dtype))
            return
        self.act_mul(gate_up, plain, 0, activation, limit)
        out.copy_((plain * weights[:, block]).to(out.dtype))

    @staticmethod
    def _norm(x, weight, bias, eps, layer_norm):
        if layer_norm:
            x = x - x.mean(-1, keepdim=True)
        y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight
        return y if bias is None else y + bias

    def norm_add(self, resid, branch, weight, bias, eps, out, layer_norm=True):
        if branch is not None:
            summed = branch.float().sum(0) if branch.dim() == 3 else branch.float()
            resid.add_(self._norm(summed, weight, bias, eps, layer_norm))
        if out is not None:
            out.copy_(resid.to(out.dtype))

    def gather_norm(self, resid, rows, weight, bias, eps, out, layer_norm=True):
        out.copy_(self._norm(resid[rows.long()], weight, bias, eps, layer_norm).to(out.dtype))

    def qk_norm_store(self, qk, q_weight, k_weight, eps, positions, temperature, q_out, keys, values, slots,
                      num_heads, num_kv_heads, dim, padded):
        if qk.dim() == 3:
            qk = qk.sum(0)
        n = qk.shape[0]
        q, k = qk[:, : num_heads * dim].float(), qk[:, num_heads * dim:].float()
        v = k
        if q_weight is not None:
            q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight
        if k_weight is not None:
            k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight
        if temperature is not None:
            coef, every = temperature
            steps = torch.div(positions.long() + 1, every, rounding_mode="floor") + 1
            q = q * (1.0 + coef * torch.log(steps.float()))[:, None]

        def pad(t, heads):
            wide = torch.zeros(n, heads, padded)
            wide[:, :, :dim] = t.view(n, heads, dim)
            return wide

        q_out.copy_(pad(q, num_heads).view(n, -1).to(q_out.dtype))
        if keys is not None:
            self.kv_write(pad(k, num_kv_heads).view(n, -1), pad(v, num_kv_heads).view(n, -1), keys, values, slots)

    def latent_store(self, fused, latent_weight, eps, q_out, latents, slots, gate_out, q_width, rank, padded, gates):
        if fused.dim() == 3:
            fused = fused.sum(0)
        n = fused.shape[0]
        q_out.copy_(fused[:, :q_width].to(q_out.dtype))
        if gates:
            gate_out.copy_(torch.sigmoid(fused[:, q_width + rank: q_width + rank + gates].float()))
        if rank and latents is not None:
            c = fused[:, q_width: q_width + rank].float()
            c = c / torch.sqrt(c.pow(2).mean(-1, keepdim=True) + eps) * latent_weight
            wide = torch.zeros(n, padded)
            wide[:, :rank] = c
            flat = latents.view(-1, latents.shape[-2] * latents.shape[-1])
            flat[slots.long()] = wide.to(flat.dtype)

    def concat_cast(self, resid, terms, other, out):
        for tensor, scale in terms:
            resid.add_(scale * (tensor.float().sum(0) if tensor.dim() == 3 else tensor.float()))
        width = resid.shape[1]
        out[:, :width] = resid.to(out.dtype)
        out[:, width:] = other.to(out.dtype)

    def decay_scan(self, fused, decays, state, q_start, state_slot, out, num_seqs, num_heads, dim, vdim, longest=0):
        if fused.dim() == 3:
            fused = fused.sum(0)
        x = fused.float()
        qk, vw = num_heads * dim, num_heads * vdim
        act = lambda z: z * torch.sigmoid(z)  # noqa: E731
        q, k = act(x[:, :qk]).view(-1, num_heads, dim), act(x[:, qk:2 * qk]).view(-1, num_heads, dim)
        v = act(x[:, 2 * qk:2 * qk + vw]).view(-1, num_heads, vdim)
        for s in range(num_seqs):
            slot = int(state_slot[s])
            if slot < 0:
                continue
            held = state[slot][:, : dim * vdim].reshape(num_heads, dim, vdim).clone()
            for t in range(int(q_start[s]), int(q_start[s + 1])):
                held = decays.view(-1, 1, 1) * held + k[t, :, :, None] * v[t, :, None, :]
                out[t] = torch.einsum("hdv,hd->hv", held, q[t]).reshape(-1)
            state[slot][:, : dim * vdim] = held.reshape(num_heads, -1)

    def norm_gate(self, x, gate_source, gate_at, weight, eps, out):
        y = x.float()
        if weight is not None:
            y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * weight
        if gate_source is not None:
            if gate_source.dim() == 3:
                gate_source = gate_source.sum(0)
            y = y * torch.sigmoid(gate_source[:, gate_at: gate_at + y.shape[1]].float())
        out.copy_(y.to(out.dtype))

    def latent_rope_store(self, fused, latent_weight, eps, positions, inv_freq, gain, q_out, latents, slots, heads, rank,
                          rot, padded):
        if fused.dim() == 3:
            fused = fused.sum(0)
        n, x = fused.shape[0], fused.float()
        angle = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = angle.cos() * gain, angle.sin() * gain

        def turn(t):   # [..., rot], dimension i with i + rot/2
            a, b = t[..., : rot // 2], t[..., rot // 2:]
            shape = (n,) + (1,) * (t.dim() - 2) + (rot // 2,)
            return torch.cat([a * cos.view(shape) - b * sin.view(shape), b * cos.view(shape) + a * sin.view(shape)], -1)

        q = x[:, : heads * (rank + rot)].view(n, heads, rank + rot)
        wide = torch.zeros(n, heads, padded)
        wide[..., :rank] = q[..., :rank]
        wide[..., rank: rank + rot] = turn(q[..., rank:])
        q_out.copy_(wide.view(n, -1).to(q_out.dtype))
        if latents is not None:
            at = heads * (rank + rot)
            c = x[:, at: at + rank]
            row = torch.zeros(n, padded)
            row[:, :rank] = c / torch.sqrt(c.pow(2).mean(-1, keepdim=True) + eps) * latent_weight
            row[:, rank: rank + rot] = turn(x[:, at + rank: at + rank + rot])
            flat = latents.view(-1, latents.shape[-2] * latents.shape[-1])
            keep = slots.long() >= 0
            flat[slots.long()[keep]] = row[keep].to(flat.dtype)

    def head_linear(self, x, w, out, heads):
        n = x.shape[0]
        out.copy_(torch.einsum("nhp,hvp->nhv", x.float().view(n, heads, -1), w.float()).reshape(n, -1).to(out.dtype))

    def head_scale(self, x, gate, heads, dim):
        n = x.shape[0]
        x.copy_((x.float().view(n, heads, dim) * gate[:, :, None]).view(n, -1).to(x.dtype))

    def add_rmsnorm(self, resid, delta, weight, eps, out):
        if delta is not None:
            resid.add_(delta.float().sum(0) if delta.dim() == 3 else delta.float())
        var = resid.pow(2).mean(-1, keepdim=True)
        out.copy_((resid * torch.rsqrt(var + eps) * weight).to(out.dtype))

    def gather_add_rmsnorm(self, resid, delta, rows, weight, eps, out):
        x = resid[rows.long()]
        if delta is not None:
            summed = delta.float().sum(0) if delta.dim() == 3 else delta.float()
            x = x + summed[rows.long()]
        var = x.pow(2).mean(-1, keepdim=True)
        out.copy_((x * torch.rsqrt(var + eps) * weight).to(out.dtype))

    def linear(self, x, w, out, bias=None, allow_partials=False):
        y = x.float() @ w.float().T
        if bias is not None:
            y = y + bias
        out.copy_(y.to(out.dtype))
        if allow_partials and out.dtype == torch.float32 and x.shape[0] <= 4:
            # as the K-split tensor-core product does for few tokens: a stack whose sum is the result
            return torch.stack([0.5 * out, 0.25 * out, 0.25 * out])
        return out

    def rope_kv_write(self, qkv, bias, positions, inv_freq, q_out, keys, values, slots,
                      num_heads, num_kv_heads, head_dim, k_out=None, v_out=None):
        if qkv.dim() == 3:
            qkv = qkv.sum(0)
        n = qkv.shape[0]
        x = qkv.float()
        if bias is not None:
            x = x + bias
        qw, kw = num_heads * head_dim, num_kv_heads * head_dim
        q = x[:, :qw].view(n, num_heads, head_dim)
        k = x[:, qw:qw + kw].view(n, num_kv_heads, head_dim)
        v = x[:, qw + kw:].view(n, num_kv_heads, head_dim)
        if inv_freq is not None:
            angle = positions.float()[:, None] * inv_freq[None, :]
            cos = torch.cat([angle.cos(), angle.cos()], -1)[:, None]
            sin = torch.cat([angle.sin(), angle.sin()], -1)[:, None]

            def rot(t):
                a, b = t.chunk(2, -1)
                return t * cos + torch.cat([-b, a], -1) * sin

            q, k = rot(q), rot(k)
        q_out.copy_(q.reshape(n, -1).to(q_out.dtype))
        if k_out is not None:
            k_out.copy_(k.reshape(n, -1).to(k_out.dtype))
            v_out.copy_(v.reshape(n, -1).to(v_out.dtype))
        if keys is not None:
            self.kv_write(k.reshape(n, -1), v.reshape(n, -1), keys, values, slots)

    def kv_write(self, k_new, v_new, keys, values, slots):
        n = k_new.shape[0]
        flat_k = keys.view(-1, keys.shape[-2], keys.shape[-1])
        flat_v = values.view(-1, values.shape[-2], values.shape[-1])
        flat_k[slots.long()] = k_new.view(n, *flat_k.shape[1:]).to(flat_k.dtype)
        flat_v[slots.long()] = v_new.view(n, *flat_v.shape[1:]).to(flat_v.dtype)

    def paged_attention(self, q, keys, values, block_table, q_start, ctx_len, seq_of_token,
                        num_heads, num_kv_heads, head_dim, scale, window, out,
                        max_q_len=0, max_ctx_len=0, min_q_len=0, q_lens=None, softcap=None, slopes=None, chunk=None,
                        sinks=None, keep_first=0):
        page = keys.shape[1]
        group = num_heads // num_kv_heads
        n = q.shape[0]
        for token in range(n):
            s = int(seq_of_token[token])
            t = token - int(q_start[s])
            q_len = int(q_start[s + 1]) - int(q_start[s])
            last = int(ctx_len[s]) - q_len + t
            first = 0 if not window else max(0, last - window + 1)
            if chunk:
                first = last // chunk * chunk
            idx = torch.arange(first, last + 1)
            if window and keep_first:   # the sequence's first keys stay visible behind the window
                idx = torch.cat([torch.arange(0, min(keep_first, first)), idx])
            pages = block_table[s].long()[idx // page]
            assert (pages >= 0).all(), "attention read a page that was given back"
            k = keys[pages, idx % page].float()  # [c, Hkv, D]
            v = values[pages, idx % page].float()
            qt = q[token].float().view(num_kv_heads, group, head_dim)
            scores = torch.einsum("kgd,ckd->kgc", qt, k) * scale
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            if slopes is not None:
                scores = scores - slopes.view(num_kv_heads, group, 1) * (last - idx).float()
            if sinks is not None:   # one more term in the denominator, without a key or a value
                both = torch.cat([scores, sinks.float().view(num_kv_heads, group, 1)], dim=-1)
                probs = both.softmax(-1)[..., :-1]
            else:
                probs = scores.softmax(-1)
            o = torch.einsum("kgc,ckd->kgd", probs, v)
            out[token] = o.reshape(-1).to(out.dtype)

    def stream_norm(self, streams, pending, join, in_weights, norm_weight, eps, out, rows=None, sum_out=None):
        x = streams if rows is None else streams[rows.long()]
        if join is not None:
            mix, out_w, layer_scale = join
            y = 0.0
            for tensor, scale in pending or []:
                summed = tensor.float().sum(0) if tensor.dim() == 3 else tensor.float()
                y = y + scale * (summed if rows is None else summed[rows.long()])
            if layer_scale is not None:
                y = y * layer_scale
            x = torch.einsum("st,nsw->ntw", mix, x) + out_w[None, :, None] * y[:, None, :]
            if rows is None:
                streams.copy_(x)
        u = x.sum(1) if in_weights is None else torch.einsum("s,nsw->nw", in_weights, x)
        if sum_out is not None:
            sum_out.copy_(u)
        if out is not None and norm_weight is not None:
            out.copy_((u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + eps) * norm_weight).to(out.dtype))

    def short_conv(self, fused, bias, taps, state, q_start, state_slot, seq_of_token, out, num_seqs, channels):
        if fused.dim() == 3:
            fused = fused.sum(0)
        u = fused.float() if bias is None else fused.float() + bias
        out.copy_(u)
        count = taps.shape[1]
        for s in range(num_seqs):
            a, b, slot = int(q_start[s]), int(q_start[s + 1]), int(state_slot[s])
            before = state[slot] if slot >= 0 and count > 1 else torch.zeros(count - 1, channels)
            joined = torch.cat([before, u[a:b, :channels]])
            mixed = torch.zeros(b - a, channels)
            for j in range(count):
                mixed += joined[j: j + b - a] * taps[:, j]
            out[a:b, :channels] = mixed
            if slot >= 0 and count > 1:
                state[slot] = joined[-(count - 1):]

    def gated_scan(self, fused, f_bias, lower, state, q_start, state_slot, out, num_seqs, num_heads, dim, vdim, q_lens=None):
        if fused.dim() == 3:
            fused = fused.sum(0)
        x = fused.float()
        H, D, Dv = num_heads, dim, vdim
        out.zero_()
        for s in range(num_seqs):
            slot = int(state_slot[s])
            if slot < 0:
                continue
            S = state[slot][:, : D * Dv].reshape(H, D, Dv).clone()
            for t in range(int(q_start[s]), int(q_start[s + 1])):
                zq, zf = x[t, : H * D], x[t, H * D: 2 * H * D]
                v = x[t, 2 * H * D: 2 * H * D + H * Dv].view(H, Dv)
                gate = torch.sigmoid(zf if f_bias is None else zf + f_bias)
                low = lower if lower is not None else torch.zeros_like(gate)
                f = (low + (1.0 - low) * gate).view(H, D)
                q = (zq * torch.sigmoid(zq)).view(H, D)
                S = f[:, :, None] * S + (1.0 - f)[:, :, None] * v[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
            state[slot][:, : D * Dv] = S.reshape(H, -1)

    def head_rms(self, x, weight, eps, out, heads):
        shaped = x.float().view(x.shape[0], heads, -1)
        normed = shaped / torch.sqrt(shaped.pow(2).mean(-1, keepdim=True) + eps)
        if weight is not None:
            normed = normed * weight
        out.copy_(normed.reshape(x.shape).to(out.dtype))

    def silu_mul(self, gate_up, out):
        self.act_mul(gate_up, out)

    def act_mul(self, gate_up, out, block=0, activation="silu", limit=None):
        assert block == 0
        inter = out.shape[1]
        g = gate_up[:, :inter].float()
        u = gate_up[:, inter:].float()
        if activation == "clamped_swish":
            g = g.clamp(max=limit)
            act, u = g * torch.sigmoid(1.702 * g), u.clamp(-limit, limit) + 1.0
        elif activation == "gelu_tanh":
            act = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
        else:
            act = g * torch.sigmoid(g)
        out.copy_((act * u).to(out.dtype))

    def sample(self, logits, temperature, top_p, seeds, out):
        for row in range(logits.shape[0]):
            temp = float(temperature[row])
            if temp == 0.0:
                out[row] = int(torch.argmax(logits[row]))
                continue
            scaled = logits[row].double() / temp
            probs = torch.softmax(scaled, -1)
            p = float(top_p[row])
            keep = torch.ones_like(probs, dtype=torch.bool)
            if p < 1.0:
                sorted_probs, order = probs.sort(descending=True)
                before = sorted_probs.cumsum(-1) - sorted_probs
                keep = torch.zeros_like(keep)
                keep[order] = before < p
            noise = torch.from_numpy(gumbel_noise_host(int(seeds[row]), logits.shape[1])).double()
            score = torch.where(keep, scaled + noise, torch.full_like(scaled, -math.inf))
            out[row] = int(torch.argmax(score))
