"""Plain, slow, whole-sequence implementation of the Setotar decoder.

One function per mechanism, written from the design's equations; no cache, no batching, no code
shared with the `shrike_b200` package.  It reads the raw `config.json` dictionary and a
name -> tensor dictionary itself.

The design in this file's notation (x_1 .. x_S: the residual streams [n, W], p: position from 0):

  streams    : every stream starts as embed[token].  A sublayer (mixer or feed-forward) with its tensors
               in (S), out (S), mix (S x S, [from, to]) and the layer scale ls (W):
               u = sum_s in[s] x_s;  y = ls * sublayer(N(u));  x_t <- sum_s mix[s, t] x_s + out[t] y
               (all new streams from the old ones).  Without `streams`: x <- x + ls * sublayer(N(x)).
               At the end x = sum_s x_s.
  N(x)       = x / sqrt(mean(x^2) + eps) * w
  rotation   : inside the first R dimensions of a head, (x[i], x[i + R/2]) turns by the angle p * f_i,
               f_i = base^(-2i/R); `scaling` {factor} alone divides every f_i by factor; with {factor, original,
               fast, slow} f_i <- f_i / factor * r_i + f_i (1 - r_i), r_i a ramp over i between two borders, and
               cos and sin are both multiplied by 0.1 ln(factor) + 1
  parallel   : left_scale * left(h) + right_scale * right(h)
    left     : q, k, v = W h + b; a causal convolution over time on every channel of each
               (c_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start); rotation of q and k; every
               value head over its root mean square; s_ij = cap tanh(scale q_i.k_j / cap); i sees j <= i with
               i - j < size or j < keep_first; softmax; query head a reads key/value head a // (H / G); Wo
    right    : q = silu(Wq h), f = l + (1 - l) sigmoid(Wf h + b), v = Wv h per head;
               S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, S_0 = 0; o_t = S_t^T q_t; every head's o over its root
               mean square times one weight of the head's size; Wo
  attention  : q, k, v = W h; q and k each over the root mean square of the WHOLE projection times a weight
               of that size; rotation; s_ij = scale q_i.k_j, j <= i; softmax; Wo.  `kv_from` j: the layer has
               no keys and values of its own and reads those of layer j (rotated keys, values).
  ff         : z = Wr h; s = sigmoid(z); the `top` largest s are chosen; out = sum over the chosen e of
               Wd_e (silu(Wg_e (s_e h)) * (Wu_e (s_e h)))
  logits     = head N_final(x)

`rounding=True` rounds to bfloat16 where a bfloat16 engine may (products' inputs and outputs);
norms, scores, softmax, the recurrence, gates, routers, the residual sums and positions stay in the working
precision.
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


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight.to(x.dtype)


def frequencies(rot: dict) -> tuple[list, float]:
    """(angle per position of each pair, the factor on cos and sin) of a rotation's settings."""
    dims, base = rot["dims"], rot["base"]
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    gain = 1.0
    if scaling and "original" in scaling:
        factor = scaling["factor"]

        def border(turns):
            return dims * math.log(scaling["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(border(scaling["fast"])), 0)
        hi = min(math.ceil(border(scaling["slow"])), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freq[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp)
        gain = 0.1 * math.log(factor) + 1.0
    elif scaling:
        freq = [f / scaling["factor"] for f in freq]
    return freq, gain


def rotate_halves(x: torch.Tensor, rot: dict | None) -> torch.Tensor:
    """x [n, heads, size]: the first rot.dims dimensions of every head turn, dimension i with i + dims/2."""
    if not rot:
        return x
    dims = rot["dims"]
    freq, gain = frequencies(rot)
    half = dims // 2
    positions = torch.arange(x.shape[0], dtype=x.dtype)
    angle = positions[:, None] * torch.tensor(freq, dtype=x.dtype)[None, :]
    cos, sin = (torch.cos(angle) * gain)[:, None, :], (torch.sin(angle) * gain)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def short_convolution(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [n, channels], taps [channels, T]: c_t = sum_j taps[:, j] u_(t - T + 1 + j), zeros before the start."""
    count = taps.shape[1]
    padded = torch.cat([u.new_zeros(count - 1, u.shape[1]), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(count):
        out = out + padded[j: j + u.shape[0]] * taps[:, j].to(u.dtype)[None, :]
    return out


def visible(n: int, size: int | None, keep_first: int) -> torch.Tensor:
    """[n, n] True where query i sees key j."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def softmax_attention(q, k, v, scale, seen, softcap=None):
    """q [n, H, D], k [n, G, D], v [n, G, Dv] -> [n, H * Dv]."""
    n, heads, _ = q.shape
    group = heads // k.shape[1]
    outs = []
    for a in range(heads):
        s = (q[:, a] @ k[:, a // group].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~seen, float("-inf"))
        outs.append(torch.softmax(s, dim=-1) @ v[:, a // group])
    return torch.cat(outs, dim=-1)


def left_keys_values(h, weights, prefix, spec, eps, rounding):
    """(rotated keys [n, G, D], normed values [n, G, Dv]) of a `left` mixer."""
    dtype = h.dtype
    g, dim, vdim = spec["kv_heads"], spec["dim"], spec.get("vdim") or spec["dim"]
    k = h @ weights[prefix + "k"].to(dtype).T + weights[prefix + "k.b"].to(dtype)
    v = h @ weights[prefix + "v"].to(dtype).T + weights[prefix + "v.b"].to(dtype)
    if spec.get("conv"):
        k = short_convolution(k, weights[prefix + "k.conv"])
        v = short_convolution(v, weights[prefix + "v.conv"])
    k = rotate_halves(k.view(-1, g, dim), spec.get("rot"))
    v = unit_rms(v.view(-1, g, vdim), eps)
    return _r(k, rounding), _r(v, rounding)


def left_mixer(h, weights, prefix, spec, eps, rounding):
    dtype = h.dtype
    heads, dim = spec["heads"], spec["dim"]
    q = h @ weights[prefix + "q"].to(dtype).T + weights[prefix + "q.b"].to(dtype)
    if spec.get("conv"):
        q = short_convolution(q, weights[prefix + "q.conv"])
    q = _r(rotate_halves(q.view(-1, heads, dim), spec.get("rot")), rounding)
    k, v = left_keys_values(h, weights, prefix, spec, eps, rounding)
    mask = spec.get("mask") or {}
    seen = visible(h.shape[0], mask.get("size"), mask.get("keep_first", 0))
    out = _r(softmax_attention(q, k, v, spec["scale"], seen, spec.get("softcap")), rounding)
    return out @ weights[prefix + "o"].to(dtype).T


def gated_recurrence(q, f, v):
    """q, f [n, D], v [n, Dv]: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T from S = 0; returns o_t = S_t^T q_t [n, Dv]."""
    state = q.new_zeros(q.shape[1], v.shape[1])
    outs = []
    for t in range(q.shape[0]):
        state = f[t][:, None] * state + (1.0 - f[t])[:, None] * v[t][None, :]
        outs.append(state.T @ q[t])
    return torch.stack(outs)


def right_mixer(h, weights, prefix, spec, eps, rounding):
    dtype = h.dtype
    heads, dim, vdim = spec["heads"], spec["dim"], spec.get("vdim") or spec["dim"]
    q = silu(h @ weights[prefix + "q"].to(dtype).T).view(-1, heads, dim)
    lower = weights[prefix + "lower"].to(dtype)
    gate = torch.sigmoid(h @ weights[prefix + "f"].to(dtype).T + weights[prefix + "f.b"].to(dtype))
    f = (lower + (1.0 - lower) * gate).view(-1, heads, dim)
    v = (h @ weights[prefix + "v"].to(dtype).T).view(-1, heads, vdim)
    outs = [rms_norm(gated_recurrence(q[:, a], f[:, a], v[:, a]), weights[prefix + "norm"], eps) for a in range(heads)]
    return _r(torch.cat(outs, dim=-1), rounding) @ weights[prefix + "o"].to(dtype).T


def parallel_mixer(h, weights, prefix, spec, eps, rounding):
    left = left_mixer(h, weights, prefix + "left.", spec["left"], eps, rounding)
    right = right_mixer(h, weights, prefix + "right.", spec["right"], eps, rounding)
    return spec["left_scale"] * left + spec["right_scale"] * right


def attention_keys_values(h, weights, prefix, spec, eps, rounding):
    dtype = h.dtype
    g, dim, vdim = spec["kv_heads"], spec["dim"], spec.get("vdim") or spec["dim"]
    k = rms_norm(h @ weights[prefix + "k"].to(dtype).T, weights[prefix + "k.norm"], eps)
    k = rotate_halves(k.view(-1, g, dim), spec.get("rot"))
    v = (h @ weights[prefix + "v"].to(dtype).T).view(-1, g, vdim)
    return _r(k, rounding), _r(v, rounding)


def attention_mixer(h, weights, prefix, spec, eps, rounding, keys_values):
    dtype = h.dtype
    heads, dim = spec["heads"], spec["dim"]
    q = rms_norm(h @ weights[prefix + "q"].to(dtype).T, weights[prefix + "q.norm"], eps)
    q = _r(rotate_halves(q.view(-1, heads, dim), spec.get("rot")), rounding)
    k, v = keys_values
    seen = visible(h.shape[0], None, 0)
    out = _r(softmax_attention(q, k, v, spec["scale"], seen), rounding)
    return out @ weights[prefix + "o"].to(dtype).T


def routed_experts(h, weights, prefix, spec, rounding, margins=None):
    """Sigmoid router; the chosen experts' scores multiply their INPUT.  `margins`, a list, receives for every token
    the gap between the last chosen score and the first one left out."""
    dtype = h.dtype
    experts, top = spec["router"]["experts"], spec["router"]["top"]
    scores = torch.sigmoid(h @ weights[prefix + "router"].to(dtype).T)
    ranked = torch.sort(scores, dim=-1, descending=True, stable=True)
    if margins is not None and top < experts:
        margins.extend((ranked.values[:, top - 1] - ranked.values[:, top]).tolist())
    out = h.new_zeros(h.shape[0], weights[prefix + "e0.down"].shape[0])
    for e in range(experts):
        chosen = (ranked.indices[:, :top] == e).any(dim=-1)
        if not bool(chosen.any()):
            continue
        fed = _r(h[chosen] * scores[chosen, e][:, None], rounding)
        gate = _r(fed @ weights[f"{prefix}e{e}.gate"].to(dtype).T, rounding)
        up = _r(fed @ weights[f"{prefix}e{e}.up"].to(dtype).T, rounding)
        out[chosen] = out[chosen] + _r(silu(gate) * up, rounding) @ weights[f"{prefix}e{e}.down"].to(dtype).T
    return out


def join(streams, y, weights, name, layer_scale):
    """What a sublayer's result y does to the residual streams (or to the one residual)."""
    y = y * layer_scale.to(y.dtype)
    if name + ".mix" not in weights:
        return [streams[0] + y]
    mix, out = weights[name + ".mix"].to(y.dtype), weights[name + ".out"].to(y.dtype)
    count = len(streams)
    return [sum(mix[s, t] * streams[s] for s in range(count)) + out[t] * y for t in range(count)]


def read(streams, weights, name):
    if name + ".in" not in weights:
        return streams[0]
    weight = weights[name + ".in"].to(streams[0].dtype)
    return sum(weight[s] * streams[s] for s in range(len(streams)))


def forward(raw: dict, weights: dict, tokens, dtype=torch.float64, rounding: bool = False, layers_out=None,
            margins=None) -> torch.Tensor:
    """Logits [n, vocab] of one whole sequence.  `layers_out`, a list, receives the summed streams after every layer."""
    eps = raw["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    e = weights["embed"].to(dtype)[ids]
    streams = [e.clone() for _ in range(raw.get("streams") or 1)]
    held = {}   # layer -> its keys and values, for a later layer that reads them
    for index, listed in enumerate(raw["layers"]):
        name, spec = f"l{index}.", listed["mixer"]
        h = _r(rms_norm(read(streams, weights, name + "hc1"), weights[name + "norm1"], eps), rounding)
        if listed["type"] == "parallel":
            y = parallel_mixer(h, weights, name + "mix.", spec, eps, rounding)
        elif listed["type"] == "attention":
            source = spec.get("kv_from")
            if source is None:
                held[index] = attention_keys_values(h, weights, name + "mix.", spec, eps, rounding)
                source = index
            y = attention_mixer(h, weights, name + "mix.", spec, eps, rounding, held[source])
        else:
            raise ValueError(listed["type"])
        streams = join(streams, y, weights, name + "hc1", weights[name + "ls1"])
        if listed.get("mlp") is not None:
            h = _r(rms_norm(read(streams, weights, name + "hc2"), weights[name + "norm2"], eps), rounding)
            y = routed_experts(h, weights, name + "mlp.", listed["mlp"], rounding, margins)
            streams = join(streams, y, weights, name + "hc2", weights[name + "ls2"])
        if layers_out is not None:
            layers_out.append(sum(streams).clone())
    hidden = _r(rms_norm(sum(streams), weights["final.norm"], eps), rounding)
    return hidden @ weights["head"].to(dtype).T


def greedy_continue(raw: dict, weights: dict, prompt, count: int, dtype=torch.float64):
    """`count` greedy tokens after `prompt`, each from a whole-sequence pass, and the gap between
    the two largest logits at each step."""
    tokens, gaps = list(prompt), []
    for _ in range(count):
        logits = forward(raw, weights, tokens, dtype=dtype)[-1]
        top = torch.topk(logits, 2).values
        gaps.append(float(top[0] - top[1]))
        tokens.append(int(torch.argmax(logits)))
    return tokens[len(prompt):], gaps
