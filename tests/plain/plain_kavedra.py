"""Plain, slow, whole-sequence implementation of the Kavedra decoder.

One function per mechanism, written from the design's equations; no cache, no batching, no code
shared with the `shrike_b200` package.  It reads the raw `config.json` dictionary and a
name -> tensor dictionary itself.

The design in this file's notation (x: residual stream [n, W], p: position from 0, e: embed[token]):

  passes     : layers start .. stop - 1 run `times` times (same weights, fresh memory each pass), then the
               rest once.  Entering pass t (t = 0 too): x <- Win [x ; e], then x <- x + step[t].
  layer      : x <- x + mixer(N1(x));  x <- x + ff(N2(x)) when the layer has a feed-forward
  N(x)       = x / sqrt(mean(x^2) + eps) * (1 + w)
  rotation   : inside the first R dimensions of a vector, (x[2i], x[2i+1]) turns by the angle p * f_i,
               f_i = base^(-2i/R); with stretched frequencies, f_i <- f_i / factor * r_i + f_i (1 - r_i), r_i a
               ramp over i between two borders, and cos and sin are both multiplied by 0.1 ln(factor) + 1
  lightning  : q = silu(Wq h), k = silu(Wk h), v = silu(Wv h) per head; S_t = d_head S_(t-1) + k_t v_t^T, S_0 = 0;
               o_t = S_t^T q_t; all heads side by side over their common root mean square, times weight, times
               sigmoid(Wg h); Wo
  attention  : q, k, v = W h + b; rotation of q and k; s_ij = scale q_i.k_j, j <= i; weights
               exp(s_ij) / (sum_j exp(s_ij) + exp(sink_head)); query head a reads key/value head a // (H / G); Wo
  latent     : q = Wq h, per head [D plain | R turned]; Wdkv h = [c' (rank) | r (R)], c = c' over its root mean
               square times weight; keys per head [Wuk c | turned r], values Wuv c; j sees i - window < j <= i;
               softmax; heads side by side times sigmoid(Wg h) element by element; Wo
  ff         : Wd (silu(Wg h) * (Wu h))
  logits     = logit_scale * head N_final(x)

`rounding=True` rounds to bfloat16 where a bfloat16 engine may (products' outputs and activations);
norms, scores, softmax, the recurrence, the residual sum and positions stay in the working precision.
"""

from __future__ import annotations

import math

import torch


def _r(x: torch.Tensor, on: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype) if on else x


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_norm(x, weights, name, eps):
    """The layers' norm: the stored weight lies around zero and one is added to it."""
    return unit_rms(x, eps) * (1.0 + weights[name].to(x.dtype))


def frequencies(rot: dict, dtype) -> tuple[torch.Tensor, float]:
    """(angle per position of each pair, the factor on cos and sin) of a rotation's settings."""
    dims, base = rot["dims"], rot["base"]
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    stretch = rot.get("scaling")
    gain = 1.0
    if stretch:
        def border(turns):   # the (fractional) pair index whose wavelength makes `turns` turns over `original` positions
            return dims * math.log(stretch["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(border(stretch["fast"])), 0)
        hi = min(math.ceil(border(stretch["slow"])), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freq[i] = freq[i] / stretch["factor"] * ramp + freq[i] * (1.0 - ramp)
        gain = 0.1 * math.log(stretch["factor"]) + 1.0
    return torch.tensor(freq, dtype=dtype), gain


def turn_pairs(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [n, H, D]: neighbouring dimensions (2i, 2i + 1) of the first rot.dims turn; the rest pass."""
    dims = rot["dims"]
    freq, gain = frequencies(rot, x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    cos, sin = (torch.cos(angle) * gain)[:, None, :], (torch.sin(angle) * gain)[:, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def decayed_recurrence(q, k, v, decay, state=None):
    """q, k [n, H, D], v [n, H, V], decay [H]: S <- decay S + k v^T token by token from `state` ([H, D, V]; None:
    zeros), o = S^T q.  Returns (o [n, H, V], the state after the last token)."""
    n, heads, dim = q.shape
    state = torch.zeros(heads, dim, v.shape[-1], dtype=q.dtype) if state is None else state.clone()
    out = torch.zeros(n, heads, v.shape[-1], dtype=q.dtype)
    for t in range(n):
        state = decay[:, None, None] * state + k[t, :, :, None] * v[t, :, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    return out, state


def lightning(h, weights, prefix, spec, eps, rounding, states_out=None) -> torch.Tensor:
    n, dtype = h.shape[0], h.dtype
    heads, dim, vdim = spec["heads"], spec["dim"], spec["vdim"]
    w = lambda name: weights[f"{prefix}.{name}"].to(dtype)  # noqa: E731
    q = _r(silu(h @ w("q").T), rounding).view(n, heads, dim)
    k = _r(silu(h @ w("k").T), rounding).view(n, heads, dim)
    v = _r(silu(h @ w("v").T), rounding).view(n, heads, vdim)
    out, state = decayed_recurrence(q, k, v, torch.tensor(spec["decay"], dtype=dtype))
    if states_out is not None:
        states_out.append(state)
    flat = unit_rms(out.reshape(n, heads * vdim), eps) * w("norm")
    gated = flat * torch.sigmoid(h @ w("g").T)
    return _r(gated, rounding) @ w("o").T


def attend(q, k, v, scale, sinks=None, window=None, first_position=0) -> torch.Tensor:
    """q [m, H, D] are the queries of positions first_position .. first_position + m - 1, k [ctx, G, D] and
    v [ctx, G, V] the keys and values of positions 0 .. ctx - 1.  Query head a reads key/value head a // (H / G);
    position i sees j <= i, with a window only i - window < j.  `sinks` [H]: exp(sink) is one more term of the
    softmax's denominator.  Returns [m, H, V]."""
    m, heads, _ = q.shape
    share = heads // k.shape[1]
    at = first_position + torch.arange(m)
    distance = at[:, None] - torch.arange(k.shape[0])[None, :]
    seen = distance >= 0
    if window is not None:
        seen = seen & (distance < window)
    out = torch.zeros(m, heads, v.shape[-1], dtype=q.dtype)
    for a in range(heads):
        scores = ((q[:, a] @ k[:, a // share].T) * scale).masked_fill(~seen, -math.inf)
        if sinks is None:
            weight = torch.softmax(scores, dim=-1)
        else:
            top = torch.maximum(scores.max(-1, keepdim=True).values, sinks[a])
            weight = torch.exp(scores - top)
            weight = weight / (weight.sum(-1, keepdim=True) + torch.exp(sinks[a] - top))
        out[:, a] = weight @ v[:, a // share]
    return out


def sink_attention(h, weights, prefix, spec, rounding) -> torch.Tensor:
    n, dtype = h.shape[0], h.dtype
    heads, groups, dim, vdim = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    w = lambda name: weights[f"{prefix}.{name}"].to(dtype)  # noqa: E731
    positions = torch.arange(n)
    q = _r(h @ w("q").T + w("q.b"), rounding).view(n, heads, dim)
    k = _r(h @ w("k").T + w("k.b"), rounding).view(n, groups, dim)
    v = _r(h @ w("v").T + w("v.b"), rounding).view(n, groups, vdim)
    q, k = _r(turn_pairs(q, positions, spec["rot"]), rounding), _r(turn_pairs(k, positions, spec["rot"]), rounding)
    out = attend(q, k, v, spec["scale"], sinks=w("sink"))
    return _r(out.reshape(n, heads * vdim), rounding) @ w("o").T


def latent_attention(h, weights, prefix, spec, eps, rounding) -> torch.Tensor:
    n, dtype = h.shape[0], h.dtype
    heads, dim, turned, vdim, rank = spec["heads"], spec["dim"], spec["rot_dim"], spec["vdim"], spec["kv_rank"]
    w = lambda name: weights[f"{prefix}.{name}"].to(dtype)  # noqa: E731
    positions = torch.arange(n)
    q = _r(h @ w("q").T, rounding).view(n, heads, dim + turned)
    down = h @ w("dkv").T
    latent = _r(unit_rms(down[:, :rank], eps) * w("dkv.norm"), rounding)
    shared = _r(turn_pairs(_r(down[:, None, rank:], rounding), positions, spec["rot"]), rounding)[:, 0]   # [n, turned]
    q_turned = _r(turn_pairs(q[..., dim:], positions, spec["rot"]), rounding)
    keys = _r(latent @ w("uk").T, rounding).view(n, heads, dim)
    values = _r(latent @ w("uv").T, rounding).view(n, heads, vdim)
    # per head the key is [Wuk c | the shared turned part]
    full_q = torch.cat([q[..., :dim], q_turned], dim=-1)
    full_k = torch.cat([keys, shared[:, None, :].expand(n, heads, turned)], dim=-1)
    window = spec["mask"]["size"] if spec.get("mask") is not None else None   # the latest keys, the query's own included
    out = attend(full_q, full_k, values, spec["scale"], window=window)
    gated = out.reshape(n, heads * vdim) * torch.sigmoid(h @ w("g").T)
    return _r(gated, rounding) @ w("o").T


def feed_forward(h, weights, prefix, spec, rounding) -> torch.Tensor:
    if spec.get("kind", "dense") != "dense":
        raise ValueError(spec["kind"])
    w = lambda name: weights[f"{prefix}.{name}"].to(h.dtype)  # noqa: E731
    return _r(silu(h @ w("gate").T) * (h @ w("up").T), rounding) @ w("down").T


def mixer(h, weights, prefix, kind, spec, eps, rounding) -> torch.Tensor:
    if kind == "lightning":
        return lightning(h, weights, prefix, spec, eps, rounding)
    if kind == "attention":
        return sink_attention(h, weights, prefix, spec, rounding)
    if kind == "latent_attention":
        return latent_attention(h, weights, prefix, spec, eps, rounding)
    raise ValueError(kind)


def layer(x, weights, index: int, spec, eps, rounding) -> torch.Tensor:
    name = f"l{index}"
    x = x + mixer(_r(offset_norm(x, weights, name + ".norm1", eps), rounding), weights, name + ".mix", spec["type"],
                  spec["mixer"], eps, rounding)
    if spec.get("mlp") is not None:
        x = x + feed_forward(_r(offset_norm(x, weights, name + ".norm2", eps), rounding), weights, name + ".mlp", spec["mlp"], rounding)
    return x


def run_order(raw: dict):
    """(layer, pass number or None when the layer's run does not open a pass)."""
    count = len(raw["layers"])
    loop = raw.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, t if i == loop["start"] else None))
    return order + [(i, None) for i in range(loop["stop"], count)]


def enter_pass(x, e, weights, number: int, rounding) -> torch.Tensor:
    both = torch.cat([_r(x, rounding), _r(e, rounding)], dim=-1)
    return both @ weights["loop.in"].to(x.dtype).T + weights["loop.step"].to(x.dtype)[number]


def forward(raw: dict, weights: dict, tokens, dtype=torch.float64, rounding: bool = False, layers_out=None) -> torch.Tensor:
    """Logits [n, vocab] of one whole sequence.  `layers_out`, a list, receives the residual after every run."""
    eps = raw["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    e = weights["embed"].to(dtype)[ids]
    x = e.clone()
    for index, opens in run_order(raw):
        if opens is not None:
            x = enter_pass(x, e, weights, opens, rounding)
        x = layer(x, weights, index, raw["layers"][index], eps, rounding)
        if layers_out is not None:
            layers_out.append(x.clone())
    hidden = _r(offset_norm(x, weights, "final.norm", eps), rounding)
    return hidden @ weights["head"].to(dtype).T * raw.get("logit_scale", 1.0)


def greedy_continue(raw: dict, weights: dict, prompt, count: int, dtype=torch.float64):
    """`count` greedy tokens after `prompt`, each from a whole-sequence pass, and the gap between
    the two largest logits at each step."""
    tokens, margins = list(prompt), []
    for _ in range(count):
        logits = forward(raw, weights, tokens, dtype=dtype)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        tokens.append(int(torch.argmax(logits)))
    return tokens[len(prompt):], margins
