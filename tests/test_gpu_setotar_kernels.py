"""Each kernel of the Setotar design alone, against plain torch in float64: the stream norm (pending K-split
stacks, layer scale, gathered rows, one to eight streams, widths that are no multiple of four), the short
convolution across cuts of a sequence and on slots with neighbours, head preparation with the norm over the whole
projection and the value norm, attention behind a window that keeps the first keys (planted keys just inside and
outside both), the gated recurrence walked whole, in portions, in runs of tokens, and with padding rows, the
per-head norm, and the router and activation in their sigmoid / weight-on-input forms."""

import numpy as np
import pytest
import torch

from tests.gpu_common import cuda_ops

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def close(got, want, tol, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    assert torch.isfinite(got).all(), what
    err = float((got - want).abs().max()) / max(1.0, float(want.abs().max()))
    assert err <= tol, f"{what}: {err:.3e} > {tol:.1e}"


def tolerance(dtype):
    return 3e-6 if dtype == torch.float32 else 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,count,width,partials", [(5, 2, 256, 1), (70, 3, 96, 3), (3, 1, 50, 2), (9, 8, 36, 1), (2, 4, 8192, 2)])
def test_stream_norm_joins_reads_and_norms(dtype, n, count, width, partials):
    ops = cuda_ops(dtype)
    g = torch.Generator().manual_seed(n * 7 + count)
    streams = torch.randn(n, count, width, generator=g)
    terms = [(torch.randn(partials, n, width, generator=g) if partials > 1 else torch.randn(n, width, generator=g), 1.2),
             (torch.randn(n, width, generator=g), 0.9)]
    mix, out_w, in_w = torch.randn(count, count, generator=g), torch.randn(count, generator=g), torch.randn(count, generator=g)
    scale, weight = torch.randn(width, generator=g), 1 + 0.1 * torch.randn(width, generator=g)
    y = sum(s * (t.double().sum(0) if t.dim() == 3 else t.double()) for t, s in terms) * scale.double()
    joined = torch.einsum("st,nsw->ntw", mix.double(), streams.double()) + out_w.double()[None, :, None] * y[:, None, :]
    u = torch.einsum("s,nsw->nw", in_w.double(), joined)
    want = u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + 1e-5) * weight.double()
    dev = lambda t: t.cuda().contiguous()
    x = dev(streams)
    out = torch.empty(n, width, dtype=dtype, device="cuda")
    ops.stream_norm(x, [(dev(t), s) for t, s in terms], (dev(mix), dev(out_w), dev(scale)), dev(in_w), dev(weight), 1e-5, out)
    close(out, want, tolerance(dtype), "normed input")
    close(x, joined, 3e-6, "streams after the join")
    # nothing pending: the streams stay, the sum of the streams on gathered rows
    rows = torch.tensor([n - 1, 0], dtype=torch.int32, device="cuda")
    gathered = torch.empty(2, width, dtype=dtype, device="cuda")
    before = x.clone()
    ops.stream_norm(x, None, None, None, dev(weight), 1e-5, gathered, rows=rows)
    total = joined.sum(1)[[n - 1, 0]]
    close(gathered, total / torch.sqrt(total.pow(2).mean(-1, keepdim=True) + 1e-5) * weight.double(), tolerance(dtype), "gathered")
    assert torch.equal(x, before)
    # pending on gathered rows: joined on the way, the streams untouched
    ops.stream_norm(x, [(dev(terms[1][0]), 0.5)], (dev(mix), dev(out_w), None), None, dev(weight), 1e-5, gathered, rows=rows)
    again = torch.einsum("st,nsw->ntw", mix.double(), joined) + out_w.double()[None, :, None] * (0.5 * terms[1][0].double())[:, None, :]
    total = again.sum(1)[[n - 1, 0]]
    close(gathered, total / torch.sqrt(total.pow(2).mean(-1, keepdim=True) + 1e-5) * weight.double(), tolerance(dtype), "gathered with a join")
    assert torch.equal(x, before)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("channels,extra,partials", [(40, 8, 1), (130, 0, 3)])
def test_short_convolution_across_cuts_and_slots(taps, channels, extra, partials):
    ops = cuda_ops(torch.float32)
    g = torch.Generator().manual_seed(taps)
    lengths = [23, 1, 9]
    total = channels + extra
    whole = [torch.randn(n, total, generator=g) for n in lengths]
    bias = torch.randn(total, generator=g)
    weights = torch.randn(channels, taps, generator=g)

    def plain(u):
        u = u.double() + bias.double()
        padded = torch.cat([torch.zeros(taps - 1, channels, dtype=torch.float64), u[:, :channels]])
        mixed = sum(padded[j: j + u.shape[0]] * weights[:, j].double() for j in range(taps))
        return torch.cat([mixed, u[:, channels:]], -1)

    want = [plain(u) for u in whole]
    state = torch.full((5, max(taps - 1, 0), channels), 7.0, device="cuda")
    slots = [3, 0, 4]
    state[slots] = 0.0
    got = [[] for _ in lengths]
    fed = [0, 0, 0]
    for cut in ([2, 1, 4], [1, 0, 5], [5, 0, 0], [15, 0, 0]):   # portions of unequal length, a request left out
        live = [i for i, c in enumerate(cut) if c]
        rows = torch.cat([whole[i][fed[i]: fed[i] + cut[i]] for i in live])
        fused = rows.cuda()
        if partials > 1:
            noise = torch.randn(partials - 1, *rows.shape, generator=g)
            fused = torch.cat([(rows - noise.sum(0))[None], noise]).cuda().contiguous()
        starts = np.cumsum([0] + [cut[i] for i in live]).astype(np.int32)
        out = torch.empty(rows.shape, device="cuda")
        seq_of = torch.tensor(sum([[k] * cut[i] for k, i in enumerate(live)], []), dtype=torch.int32, device="cuda")
        ops.short_conv(fused, bias.cuda(), weights.cuda().contiguous(), state, torch.tensor(starts, device="cuda"),
                       torch.tensor([slots[i] for i in live], dtype=torch.int32, device="cuda"), seq_of, out, len(live), channels)
        for k, i in enumerate(live):
            got[i].append(out[starts[k]: starts[k + 1]].cpu())
            fed[i] += cut[i]
    for i in range(3):
        close(torch.cat(got[i]), want[i][: fed[i]], 2e-5 if partials > 1 else 3e-6, f"sequence {i}")
    if taps > 1:
        assert float(state[1].min()) == 7.0 and float(state[2].min()) == 7.0   # the neighbours' slots stay


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot", [(4, 2, 16, 8, 8), (3, 3, 24, 40, 0), (2, 0, 32, 32, 32), (5, 1, 6, 10, 2)])
def test_head_preparation_with_whole_and_value_norms(dtype, heads, kv_heads, dim, vdim, rot):
    ops = cuda_ops(dtype)
    g = torch.Generator().manual_seed(heads + dim)
    n, padded = 7, -(-max(dim, vdim) // 16) * 16
    total = -(-(heads * dim + kv_heads * (dim + vdim)) // 16) * 16
    fused = torch.randn(2, n, total, generator=g)
    x = fused.double().sum(0)
    q_w, k_w = 1 + 0.1 * torch.randn(heads * dim, generator=g), 1 + 0.1 * torch.randn(max(kv_heads, 1) * dim, generator=g)
    positions = torch.tensor([0, 1, 5, 17, 100, 1000, 3], dtype=torch.int32)
    inv_freq = torch.tensor([10.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)])
    q = x[:, : heads * dim]
    q = (q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + 1e-5) * q_w.double()).view(n, heads, dim)
    k = x[:, heads * dim: (heads + kv_heads) * dim]
    if kv_heads:
        k = (k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + 1e-5) * k_w.double()[: kv_heads * dim]).view(n, kv_heads, dim)
        v = x[:, (heads + kv_heads) * dim: (heads + kv_heads) * dim + kv_heads * vdim].view(n, kv_heads, vdim)
        v = v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)

    def turn(t):
        if not rot:
            return t
        angle = positions.double()[:, None] * inv_freq.double()[None, :]
        cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
        a, b = t[..., : rot // 2], t[..., rot // 2: rot]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, t[..., rot:]], -1)

    q_out = torch.empty(n, heads * padded, dtype=dtype, device="cuda")
    keys = torch.full((4, 4, max(kv_heads, 1), padded), float("nan"), dtype=dtype, device="cuda")
    values = keys.clone()
    slots = torch.tensor([3, 0, 7, -1, 15, 8, 9], dtype=torch.int32, device="cuda")
    ops.head_prep(fused.cuda(), None, positions.cuda(), inv_freq.cuda() if rot else None, rot, q_w.cuda(),
                  k_w.cuda()[: kv_heads * dim] if kv_heads else None, 1e-5, q_out, keys if kv_heads else None,
                  values if kv_heads else None, slots, None, heads, kv_heads, dim, vdim, padded, whole_norm=True, value_norm=True)
    tol = 1e-4 if dtype == torch.float32 else 1e-2   # angles are float32(position) * frequency: 1e-4 radians at position 1000
    close(q_out.view(n, heads, padded)[..., :dim], turn(q), tol, "queries")
    assert float(q_out.view(n, heads, padded)[..., dim:].abs().sum()) == 0
    if kv_heads:
        stored = [i for i in range(n) if int(slots[i]) >= 0]
        at = slots[stored].long()
        close(keys.view(16, kv_heads, padded)[at][..., :dim], turn(k)[stored], tol, "keys")
        close(values.view(16, kv_heads, padded)[at][..., :vdim], v[stored], tol, "values")


def paged(ops, q, k, v, page, window, keep, scale, softcap, lengths, new, dtype):
    """q [sum new, H, D], k/v per sequence [len, G, D]: runs the paged attention on a shuffled pool."""
    heads, D = q.shape[1], q.shape[2]
    G = k[0].shape[1]
    blocks = [-(-n // page) for n in lengths]
    order = torch.randperm(sum(blocks) + 3, generator=torch.Generator().manual_seed(1)).tolist()
    keys = torch.full((sum(blocks) + 3, page, G, D), float("nan"), dtype=dtype, device="cuda")
    values = keys.clone()
    width = max(blocks)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for s, n in enumerate(lengths):
        for b in range(blocks[s]):
            pid = order.pop()
            table[s, b] = pid
            rows = slice(b * page, min((b + 1) * page, n))
            keys[pid, : rows.stop - rows.start] = k[s][rows].to(dtype).cuda()
            values[pid, : rows.stop - rows.start] = v[s][rows].to(dtype).cuda()
            if rows.stop - rows.start < page:
                keys[pid, rows.stop - rows.start:] = 0
                values[pid, rows.stop - rows.start:] = 0
    q_start = torch.tensor(np.cumsum([0] + new), dtype=torch.int32, device="cuda")
    seq_of = torch.tensor(sum([[s] * c for s, c in enumerate(new)], []), dtype=torch.int32, device="cuda")
    out = torch.empty(q.shape[0], heads * D, dtype=dtype, device="cuda")
    ops.paged_attention(q.reshape(q.shape[0], -1).to(dtype).cuda().contiguous(), keys, values, table.cuda(), q_start,
                        torch.tensor(lengths, dtype=torch.int32, device="cuda"), seq_of, heads, G, D, scale, window, out,
                        max_q_len=max(new), max_ctx_len=max(lengths), min_q_len=min(new), q_lens=list(new), softcap=softcap, keep_first=keep)
    return out.view(q.shape[0], heads, D)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,page,window,keep", [(64, 16, 140, 5), (128, 16, 33, 20), (32, 8, 1, 1), (64, 32, 5, 70), (16, 16, 300, 3)])
def test_attention_behind_a_window_that_keeps_the_first_keys(dtype, D, page, window, keep):
    """Portions beside single tokens; one key is made to stand far above the rest just inside the window, just outside it,
    the last kept key and the first one not kept, in turn."""
    ops = cuda_ops(dtype)
    g = torch.Generator().manual_seed(D + window)
    heads, G, scale, cap = 4, 2, 0.3, 6.0
    lengths, new = [window + keep + 45, 700, 3], [1, 130, 3]
    for lag in (window - 1, window, None, None):
        k = [0.3 * torch.randn(n, G, D, generator=g) for n in lengths]
        v = [torch.randn(n, G, D, generator=g) for n in lengths]
        q = 0.3 * torch.randn(sum(new), heads, D, generator=g)
        if dtype == torch.bfloat16:
            k, v, q = [t.bfloat16().float() for t in k], [t.bfloat16().float() for t in v], q.bfloat16().float()
        spot = lengths[0] - 1 - lag if lag is not None else (keep - 1 if g.initial_seed() % 2 else keep)
        if lag is None:
            g.manual_seed(g.initial_seed() + 1)
        k[0][spot] = 4.0 * q[0, ::2] / q[0, ::2].norm(dim=-1, keepdim=True)   # the lone query's heads point at it
        v[0][spot] = 5.0
        want = []
        for s, n in enumerate(lengths):
            for t in range(new[s]):
                p = n - new[s] + t
                seen = [j for j in range(p + 1) if p - j < window or j < keep]
                row = q[sum(new[:s]) + t].double()
                scores = torch.einsum("hd,jhd->hj", row, k[s][seen].double().repeat_interleave(heads // G, 1)) * scale
                scores = cap * torch.tanh(scores / cap)
                want.append(torch.einsum("hj,jhd->hd", scores.softmax(-1), v[s][seen].double().repeat_interleave(heads // G, 1)))
        got = paged(ops, q, k, v, page, window, keep, scale, cap, lengths, new, dtype)
        close(got, torch.stack(want), 2e-5 if dtype == torch.float32 else 2e-2, f"lag {lag} spot {spot}")


def plain_scan(zq, zf, v, bias, lower, state):
    """One sequence, float64: returns the outputs and the state it leaves."""
    H, D = lower.shape
    outs = []
    for t in range(zq.shape[0]):
        q = zq[t].view(H, D) * torch.sigmoid(zq[t].view(H, D))
        f = lower + (1 - lower) * torch.sigmoid(zf[t].view(H, D) + bias)
        state = f[:, :, None] * state + (1 - f)[:, :, None] * v[t].view(H, 1, -1)
        outs.append(torch.einsum("hdv,hd->hv", state, q).reshape(-1))
    return torch.stack(outs), state


@pytest.mark.parametrize("heads,dim,vdim", [(4, 32, 64), (1, 72, 24), (3, 8, 100), (2, 130, 8), (2, 4, 4)])
def test_gated_recurrence_whole_in_portions_in_runs_and_with_padding(heads, dim, vdim):
    ops = cuda_ops(torch.float32)
    g = torch.Generator().manual_seed(heads * dim)
    lengths = [450, 1, 37]
    total = -(-heads * (2 * dim + vdim) // 16) * 16
    fused = [torch.randn(n, total, generator=g) for n in lengths]
    for u in fused:
        u[:, heads * dim: 2 * heads * dim] *= 3.0   # gates that open and close
    bias, lower = torch.randn(heads, dim, generator=g), torch.rand(heads, dim, generator=g) * 0.9
    size = -(-dim * vdim // 4) * 4
    want = []
    for u in fused:
        x = u.double()
        out, _ = plain_scan(x[:, : heads * dim], x[:, heads * dim: 2 * heads * dim], x[:, 2 * heads * dim: 2 * heads * dim + heads * vdim],
                            bias.double(), lower.double(), torch.zeros(heads, dim, vdim, dtype=torch.float64))
        want.append(out)
    for cuts in ([[450, 1, 37]], [[200, 1, 0], [250, 0, 37]], [[1, 1, 30], [2, 0, 1], [447, 0, 6]], [[7, 1, 37]] + [[1, 0, 0]] * 9 + [[434, 0, 0]]):
        state = torch.full((6, heads, size), 5.0, device="cuda")
        slots = [4, 1, 2]
        state[slots] = 0.0
        got, fed = [[] for _ in lengths], [0, 0, 0]
        for cut in cuts:
            live = [i for i, c in enumerate(cut) if c]
            lens = [cut[i] for i in live] + [1]   # a padding row at the end: state slot -1, nothing kept
            rows = torch.cat([fused[i][fed[i]: fed[i] + cut[i]] for i in live] + [torch.randn(1, total, generator=g)]).cuda()
            starts = np.cumsum([0] + lens).astype(np.int32)
            out = torch.full((rows.shape[0], heads * vdim), float("nan"), device="cuda")
            ops.gated_scan(rows, bias.reshape(-1).cuda(), lower.reshape(-1).cuda(), state, torch.tensor(starts, device="cuda"),
                           torch.tensor([slots[i] for i in live] + [-1], dtype=torch.int32, device="cuda"), out, len(lens), heads, dim, vdim,
                           q_lens=lens)
            assert float(out[-1].abs().sum()) == 0
            for k, i in enumerate(live):
                got[i].append(out[starts[k]: starts[k + 1]].cpu())
                fed[i] += cut[i]
        for i in range(3):
            close(torch.cat(got[i]), want[i], 2e-5, f"cuts {cuts[0]} sequence {i}")
        assert float(state[0].min()) == 5.0 and float(state[3].min()) == 5.0 and float(state[5].min()) == 5.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_norm(dtype):
    ops = cuda_ops(dtype)
    x = torch.randn(9, 5 * 24, generator=torch.Generator().manual_seed(1)) * 3
    weight = 1 + 0.1 * torch.randn(24, generator=torch.Generator().manual_seed(2))
    out = torch.empty(9, 120, dtype=dtype, device="cuda")
    ops.head_rms(x.cuda(), weight.cuda(), 1e-5, out, 5)
    shaped = x.double().view(9, 5, 24)
    close(out, (shaped / torch.sqrt(shaped.pow(2).mean(-1, keepdim=True) + 1e-5) * weight.double()).reshape(9, 120), tolerance(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,each", [(8, 1, 64), (5, 2, 12), (3, 3, 7)])
def test_sigmoid_router_and_weights_on_the_input(dtype, experts, top, each):
    ops = cuda_ops(dtype)
    g = torch.Generator().manual_seed(experts)
    n, width = 11, 96
    x = torch.randn(n, width, generator=g).to(dtype)
    router = torch.randn(experts, width, generator=g) * 0.3
    share = torch.empty(n, experts, device="cuda")
    ops.route_top(x.cuda(), router.cuda(), None, share, top, 0.0, scoring="sigmoid", renormalise=False)
    scores = torch.sigmoid(x.double() @ router.double().T)
    best, chosen = torch.topk(scores, top, -1)
    want = torch.zeros(n, experts, dtype=torch.float64).scatter_(1, chosen, best)
    close(share, want, 1e-5, "expert weights")
    gate_up = torch.randn(n, 2 * experts * each, generator=g).to(dtype)
    out = torch.empty(n, experts * each, dtype=dtype, device="cuda")
    ops.act_mul_blocks(gate_up.cuda(), share, out, experts, each, "silu", weight_on="input")
    w = want.repeat_interleave(each, 1)
    gate, up = gate_up.double()[:, : experts * each] * w, gate_up.double()[:, experts * each:] * w
    close(out, gate * torch.sigmoid(gate) * up, tolerance(dtype), "activation")
