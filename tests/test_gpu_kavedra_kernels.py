"""Each mechanism of the Kavedra parts alone on the GPU, against the plain functions of
`tests/plain/plain_kavedra.py` in float64: the decayed linear attention's scan (whole over runs of
tokens, as a walk, in portions, token by token, several sequences of unequal length, slots that had
other owners, K-split inputs), the norm with a sigmoid gate, the latent's norm, rotation and page
row, neighbouring dimensions rotated through reordered rows, the per-head product, the joined rows of
a pass entry, and paged attention with softmax sinks (single tokens, portions, the tensor-core
kernels with and without key splits, with a window, keys and values in one plane) with keys planted
at a window's edges, at page borders and far back."""

import math

import pytest
import torch

from shrike_b200.config.model_config import PairRotationSpec
from shrike_b200.parts.rotary import PairRotation
from tests.gpu_common import cuda_ops
from tests.plain import plain_kavedra as pk
from tests.test_gpu_sadodra_kernels import close, paged, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}


# ------------------------------------------------------------------ decayed linear attention
def scan_case(heads, dim, vdim, n, seed, decays):
    total = 2 * heads * dim + 2 * heads * vdim + 8          # q | k | v | gate | padding
    fused = rnd(n, total, seed=seed, scale=1.2)
    act = pk.silu(fused.double())
    q = act[:, : heads * dim].view(n, heads, dim)
    k = act[:, heads * dim: 2 * heads * dim].view(n, heads, dim)
    v = act[:, 2 * heads * dim: 2 * heads * dim + heads * vdim].view(n, heads, vdim)
    want, state = pk.decayed_recurrence(q, k, v, torch.tensor(decays, dtype=torch.float64))
    return fused, want.reshape(n, heads * vdim), state


def run_scan(ops, fused, decays, state, slot, cuts, heads, dim, vdim, partials=1, walk=False):
    outs, position = [], 0
    d = torch.tensor(decays, dtype=torch.float32, device=DEV)
    for cut in cuts:
        piece = fused[position: position + cut].contiguous().to(DEV)
        if partials > 1:
            piece = torch.stack([piece * 0.5] + [piece * (0.5 / (partials - 1))] * (partials - 1)).contiguous()
        out = torch.full((cut, heads * vdim), float("nan"), dtype=torch.float32, device=DEV)
        ops.decay_scan(piece, d, state, torch.tensor([0, cut], dtype=torch.int32, device=DEV),
                       torch.tensor([slot], dtype=torch.int32, device=DEV), out, 1, heads, dim, vdim, longest=0 if walk else cut)
        outs.append(out)
        position += cut
    return torch.cat(outs)


@pytest.mark.parametrize("heads,dim,vdim,decays", [
    (2, 64, 48, (0.6, 0.9995)), (3, 16, 24, (0.5, 1.0, 0.93)), (1, 64, 64, (0.97,)), (2, 40, 8, (0.3, 0.8)), (3, 8, 40, (0.9, 0.99, 0.6)),
    (1, 128, 128, (0.995,)), (2, 256, 96, (0.9, 1.0)), (2, 96, 200, (0.99, 0.7)), (1, 1, 1, (0.5,)), (2, 5, 3, (1.0, 0.25)),
    (1, 320, 72, (0.98,)), (1, 520, 64, (0.9,)), (2, 600, 8, (0.99, 1.0))])
def test_decayed_scan_whole_in_portions_and_token_by_token(heads, dim, vdim, decays):
    ops = cuda_ops(torch.float32)
    n = 200
    fused, want, final = scan_case(heads, dim, vdim, n, heads * 100 + dim, decays)
    size = max(1.0, float(want.abs().max()))
    width = -(-dim * vdim // 4) * 4
    state = torch.zeros(3, heads, width, dtype=torch.float32, device=DEV)
    state[1] = float("nan")                           # a neighbour's slot: never read, never written
    # whole (products over runs of 64 tokens), the same as a walk inside one launch, and cut into portions that meet
    # both forms, leave a run part full and bring single tokens in between
    for slot, cuts, partials, walk in ((0, [n], 1, False), (0, [n], 1, True), (2, [1, 2, 7, 64, 3, 1, 1, 100, 21], 3, False),
                                       (2, [33, 31, 65, 71], 1, False)):
        state[slot].zero_()
        got = run_scan(ops, fused, decays, state, slot, cuts, heads, dim, vdim, partials, walk)
        close(got / size, want / size, 2e-5, f"cuts {cuts}")
        held = state[slot, :, : dim * vdim].view(heads, dim, vdim)
        big = max(1.0, float(final.abs().max()))
        close(held / big, final / big, 1e-5, "the state left behind")
    assert torch.isnan(state[1]).all()
    state[0].zero_()                                  # the slot's next owner, token by token
    got = run_scan(ops, fused[:50], decays, state, 0, [1] * 50, heads, dim, vdim)
    close(got / size, want[:50] / size, 2e-5, "token by token")


def test_decayed_scan_over_unequal_sequences_skips_padding():
    """Five sequences in one launch: a long portion, a single token with a state, a padding row (slot -1), a short
    portion and one of exactly a run; each equals itself alone."""
    ops = cuda_ops(torch.float32)
    heads, dim, vdim, decays = 2, 32, 48, (0.9, 0.999)
    lengths = [150, 1, 1, 9, 64]
    slots = [3, 0, -1, 4, 1]
    cases = [scan_case(heads, dim, vdim, n + 10, 40 + i, decays) for i, n in enumerate(lengths)]
    state = torch.zeros(5, heads, dim * vdim, dtype=torch.float32, device=DEV)
    state[2] = float("nan")
    d = torch.tensor(decays, dtype=torch.float32, device=DEV)
    for (fused, _, _), slot in zip(cases, slots):     # every request has ten tokens behind it
        if slot >= 0:
            run_scan(ops, fused[:10], decays, state, slot, [10], heads, dim, vdim)
    rows = torch.cat([fused[10:] for fused, _, _ in cases]).contiguous().to(DEV)
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    out = torch.full((starts[-1], heads * vdim), float("nan"), dtype=torch.float32, device=DEV)
    ops.decay_scan(rows, d, state, torch.tensor(starts, dtype=torch.int32, device=DEV),
                   torch.tensor(slots, dtype=torch.int32, device=DEV), out, len(lengths), heads, dim, vdim, longest=max(lengths))
    assert torch.isnan(state[2]).all(), "a slot nobody named was written"
    for index, ((_, want, final), slot) in enumerate(zip(cases, slots)):
        if slot < 0:
            continue
        size = max(1.0, float(want.abs().max()))
        close(out[starts[index]: starts[index + 1]] / size, want[10:] / size, 2e-5, f"sequence {index}")
        big = max(1.0, float(final.abs().max()))
        close(state[slot].view(heads, dim, vdim) / big, final / big, 1e-5, f"state of sequence {index}")


def test_a_decay_of_one_keeps_a_token_for_ever_and_a_small_one_forgets_it():
    """One large key and value at the first token, the matching query 900 tokens later: the head with decay 1 returns
    the value in full, the head with decay 0.98 a share of 0.98^900 of it, in the chunked form and walking."""
    ops = cuda_ops(torch.float32)
    heads, dim, vdim, n, decays = 2, 16, 8, 901, (1.0, 0.98)
    total = 2 * heads * dim + heads * vdim
    fused = torch.full((n, total), -30.0)                         # silu(-30) is nothing
    for a in range(heads):
        fused[0, heads * dim + a * dim + 3] = 5.0                 # k
        fused[0, 2 * heads * dim + a * vdim: 2 * heads * dim + (a + 1) * vdim] = 7.0   # v
        fused[-1, a * dim + 3] = 4.0                              # q
    amount = float(pk.silu(torch.tensor(5.0, dtype=torch.float64)) * pk.silu(torch.tensor(7.0, dtype=torch.float64))
                   * pk.silu(torch.tensor(4.0, dtype=torch.float64)))
    for walk in (False, True):
        state = torch.zeros(1, heads, dim * vdim, dtype=torch.float32, device=DEV)
        got = run_scan(ops, fused, decays, state, 0, [n], heads, dim, vdim, walk=walk)[-1].view(heads, vdim).double().cpu()
        assert torch.allclose(got[0], torch.full((vdim,), amount, dtype=torch.float64), rtol=1e-5)
        assert torch.allclose(got[1], torch.full((vdim,), amount * 0.98 ** 900, dtype=torch.float64), rtol=2e-3, atol=0)


# ------------------------------------------------------------------ norm and gate
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,partials,normed,gated", [(3, 64, 1, True, True), (5, 72, 3, True, True), (300, 128, 1, False, True),
                                                           (2, 4096, 2, True, False), (70, 1030, 2, True, True), (1, 8, 1, True, True)])
def test_rows_are_normed_and_gated(dtype, n, width, partials, normed, gated):
    ops = cuda_ops(dtype)
    x = rnd(n, width, seed=1, scale=3.0) + 0.5
    gate_at = 24
    source = rnd(partials, n, gate_at + width + 8, seed=2, scale=2.0)
    weight = 1.0 + 0.3 * rnd(width, seed=3)
    want = x.double()
    if normed:
        want = pk.unit_rms(want, 1e-5) * weight.double()
    if gated:
        want = want * torch.sigmoid(source.double().sum(0)[:, gate_at: gate_at + width])
    out = torch.full((n, width), float("nan"), dtype=dtype, device=DEV)
    stack = source.to(DEV) if partials > 1 else source[0].contiguous().to(DEV)
    ops.norm_gate(x.to(DEV), stack if gated else None, gate_at, weight.to(DEV) if normed else None, 1e-5, out)
    close(out, want, 2e-5 if dtype == torch.float32 else 4e-2, "normed and gated rows")


# ------------------------------------------------------------------ rotation
def halves(x, dims, first=0):
    """Neighbouring pairs (2i, 2i + 1) of x[..., first : first + dims] put at (i, i + dims/2), as the loader reorders rows."""
    out = x.clone()
    out[..., first: first + dims // 2] = x[..., first: first + dims: 2]
    out[..., first + dims // 2: first + dims] = x[..., first + 1: first + dims: 2]
    return out


STRETCHES = [None, (8.0, 1024, 32.0, 1.0), (4.0, 64, 8.0, 2.0), (2.0, 4, 1000.0, 0.0001)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rank,rot,partials,stretch", [(4, 80, 32, 1, 1), (3, 40, 8, 3, 2), (2, 12, 2, 1, 3), (1, 20, 4, 2, 0),
                                                             (2, 48, 16, 1, 0), (16, 512, 64, 1, 1)])
def test_latent_is_normed_rotated_and_stored(dtype, heads, rank, rot, partials, stretch):
    ops = cuda_ops(dtype)
    stretch = STRETCHES[stretch]
    raw = {"dims": rot, "base": 5000.0}
    if stretch is not None:
        raw["scaling"] = dict(zip(("factor", "original", "fast", "slow"), stretch))
    rotation = PairRotation(PairRotationSpec(dims=rot, base=5000.0, pairing="neighbours", stretch=stretch), DEV)
    padded = -(-(rank + rot) // 16) * 16
    positions = torch.tensor([0, 1, 7, 300, 1113, 5, 64, 2, 9], dtype=torch.int32)
    n = len(positions)
    used = (heads + 1) * (rank + rot)
    total = used + 24                                           # a gate's columns follow; the kernel leaves them alone
    given = rnd(partials, n, total, seed=3, scale=0.7)           # as the product of the unchanged weights would be
    x = given.double().sum(0)
    per_head = x[:, : heads * (rank + rot)].view(n, heads, rank + rot)
    own = x[:, heads * (rank + rot): used]
    weight = 1.0 + 0.2 * rnd(rank, seed=4)
    want_q = torch.cat([per_head[..., :rank], halves(pk.turn_pairs(per_head[..., rank:], positions, raw), rot)], dim=-1)
    want_c = pk.unit_rms(own[:, :rank], 1e-5) * weight.double()
    want_r = halves(pk.turn_pairs(own[:, None, rank:], positions, raw), rot)[:, 0]
    # the loader reorders the rows of the projections, so the kernel's input has the rotated parts' pairs at (i, i + rot/2)
    fused = given.clone()
    view = fused[..., :used].view(partials, n, heads + 1, rank + rot)
    view[..., rank:] = halves(given[..., :used].view(partials, n, heads + 1, rank + rot)[..., rank:], rot)
    page, pages = 4, 6
    latents = torch.full((pages, page, 1, padded), float("nan"), dtype=dtype, device=DEV)
    slots = torch.tensor([5, 0, 9, 23, 11, 2, 7, 8, -1], dtype=torch.int32)
    q_out = torch.full((n, heads * padded), float("nan"), dtype=dtype, device=DEV)
    stack = fused.to(DEV) if partials > 1 else fused[0].contiguous().to(DEV)
    ops.latent_rope_store(stack, weight.to(DEV), 1e-5, positions.to(DEV), rotation.inv_freq, rotation.gain, q_out, latents,
                          slots.to(DEV), heads, rank, rot, padded)
    # the angle is position * frequency in 32-bit: at position 1113 its rounding alone moves a component by about 1e-4
    tol = 4e-4 if dtype == torch.float32 else 4e-2
    got_q = q_out.view(n, heads, padded)
    close(got_q[:, :, : rank + rot], want_q, tol, "queries")
    assert (got_q[:, :, rank + rot:] == 0).all()
    flat = latents.view(-1, padded)
    for row, slot in enumerate(slots.tolist()):
        if slot >= 0:
            close(flat[slot, :rank], want_c[row], tol, f"latent of token {row}")
            close(flat[slot, rank: rank + rot], want_r[row], tol, f"rotated key part of token {row}")
            assert (flat[slot, rank + rot:] == 0).all()
    assert torch.isnan(flat[1].float()).all(), "a slot nobody named was written"
    # without a cache to write (a run that reads another's pages) the queries are the same
    again = torch.full_like(q_out, float("nan"))
    ops.latent_rope_store(stack, weight.to(DEV), 1e-5, positions.to(DEV), rotation.inv_freq, rotation.gain, again, None,
                          slots.to(DEV), heads, rank, rot, padded)
    assert torch.equal(again, q_out)


# ------------------------------------------------------------------ attention with softmax sinks
def attend_with_sinks(ops, dtype, sequences, page, heads, kv_heads, dim, scale, window, sinks, shared_plane=False):
    case = paged(dtype, sequences, page, kv_heads, dim, shared_plane)
    out = torch.full_like(case["q"], float("nan"))
    ops.paged_attention(case["q"], case["keys"], case["values"], case["table"], case["q_start"], case["ctx_len"], case["seq_of"],
                        heads, kv_heads, dim, scale, window, out, max_q_len=max(case["q_lens"]), max_ctx_len=max(case["ctx_lens"]),
                        min_q_len=min(case["q_lens"]), q_lens=case["q_lens"], sinks=sinks.float().to(DEV))
    ops.check_status()
    want = []
    for q, k, v, q_len in sequences:
        ctx = len(k)
        r = lambda t: t.to(dtype).double()   # noqa: E731  the oracle sees the stored values
        want.append(pk.attend(r(q[ctx - q_len:]), r(k), r(v), scale, sinks.double(), window, first_position=ctx - q_len))
    return out, torch.cat(want).reshape(out.shape)


def random_sequences(lengths, heads, kv_heads, dim, seed, spread=1.5):
    sequences = []
    for s, (ctx, q_len) in enumerate(lengths):
        g = torch.Generator().manual_seed(seed + s)
        sequences.append((torch.randn(ctx, heads, dim, generator=g) * spread, torch.randn(ctx, kv_heads, dim, generator=g),
                          torch.randn(ctx, kv_heads, dim, generator=g), q_len))
    return sequences


def spread_sinks(heads):
    """From a sink that takes nearly all of the weight to one that takes none."""
    return torch.linspace(7.0, -30.0, heads)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,page,window", [(4, 2, 32, 8, None), (3, 3, 48, 5, 37), (8, 1, 64, 16, None), (6, 2, 16, 16, 9),
                                                            (2, 1, 256, 16, 70), (3, 1, 272, 8, None)])
def test_sinks_in_single_tokens_and_portions(dtype, heads, kv_heads, dim, page, window):
    """Every denominator holds exp(sink): single tokens (few and many keys, so split and not), portions beside them, the
    first token of a sequence (one key against the sink), heads wider than the tensor-core kernels take."""
    ops = cuda_ops(dtype)
    sinks = spread_sinks(heads)
    lengths = [(1, 1), (40, 1), (130, 1), (21, 2), (100, 37), (300, 129), (64, 64), (33, 1), (200, 3), (900, 1)]
    sequences = random_sequences(lengths, heads, kv_heads, dim, 150)
    got, want = attend_with_sinks(ops, dtype, sequences, page, heads, kv_heads, dim, dim ** -0.5 * 2, window, sinks)
    close(got, want, TOL[dtype], "attention with sinks")
    without = pk.attend(sequences[4][0][-37:].double(), sequences[4][1].double(), sequences[4][2].double(), dim ** -0.5 * 2, None, window, 63)
    with_sinks = pk.attend(sequences[4][0][-37:].double(), sequences[4][1].double(), sequences[4][2].double(), dim ** -0.5 * 2, sinks.double(), window, 63)
    assert (without - with_sinks).abs().max() > 0.3, "the oracle itself: these sinks matter"
    singles = [(q, k, v, 1) for q, k, v, _ in sequences]     # the single-token kernel alone (other split and cluster shapes)
    got, want = attend_with_sinks(ops, dtype, singles, page, heads, kv_heads, dim, dim ** -0.5 * 2, window, sinks)
    close(got, want, TOL[dtype], "single tokens only")


@pytest.mark.parametrize("tensor_core,splits", [(True, 0), (True, 3), (False, 0)])
@pytest.mark.parametrize("heads,kv_heads,dim,page,window", [(6, 2, 64, 16, 150), (4, 1, 128, 16, None), (2, 2, 128, 8, 300), (3, 3, 64, 32, None)])
def test_sinks_on_the_tensor_core_portions_kernel(heads, kv_heads, dim, page, window, tensor_core, splits):
    """Head sizes 64 and 128 take the tcgen05 kernel for portions: with and without it, and with a query tile's keys
    shared by several CTAs (the sink must count once, not once a CTA), the same weights."""
    ops = cuda_ops(torch.bfloat16)
    ops.tensor_core_attention, ops.portion_splits = tensor_core, splits
    sinks = spread_sinks(heads)
    sequences = random_sequences([(700, 700), (130, 1), (500, 129), (300, 300), (64, 2), (1000, 37)], heads, kv_heads, dim, 170, spread=1.0)
    got, want = attend_with_sinks(ops, torch.bfloat16, sequences, page, heads, kv_heads, dim, dim ** -0.5 * 3, window, sinks)
    close(got, want, TOL[torch.bfloat16], "portions on the tensor cores with sinks")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_sink_above_every_score_leaves_almost_nothing(dtype):
    """A sink far above the scores takes the weight: the outputs shrink by exp(score - sink), and a sink far below
    changes nothing; a planted key far back still gets its share against the sink."""
    ops = cuda_ops(dtype)
    heads, kv_heads, dim, page = 2, 1, 32, 16
    sequences = random_sequences([(600, 1), (600, 40)], heads, kv_heads, dim, 190, spread=0.3)
    for q, k, v, _ in sequences:
        k *= 0.1                    # the other keys' scores stay near 0
        k[7] = 0.0
        k[7, 0, 3] = 4.0
        q[-1] = 0.0
        q[-1, :, 3] = 5.0           # score 20 with key 7, about 0 with the others
        v[7] = 50.0
    sinks = torch.tensor([20.0, -40.0])
    got, want = attend_with_sinks(ops, dtype, sequences, page, heads, kv_heads, dim, 1.0, None, sinks)
    close(got, want, TOL[dtype] * 50, "a planted key against a sink")
    for last in (got[0], got[-1]):
        per_head = last.float().view(heads, dim).mean(-1)
        assert 20 < per_head[0] < 30 and per_head[1] > 45, per_head   # half of the weight with the sink, all of it without


# ------------------------------------------------------------------ the per-head product and the joined rows
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,heads,padded,vdim", [(1, 3, 48, 16), (37, 2, 64, 64), (130, 4, 128, 24), (5, 1, 32, 40)])
def test_every_head_has_its_own_product(dtype, n, heads, padded, vdim):
    ops = cuda_ops(dtype)
    x = rnd(n, heads * padded, seed=1).to(dtype)
    w = (rnd(heads, vdim, padded, seed=2) * 0.3).to(dtype)
    out = torch.full((n, heads * vdim), float("nan"), dtype=torch.float32, device=DEV)
    ops.head_linear(x.to(DEV), w.to(DEV), out, heads)
    want = torch.einsum("nhp,hvp->nhv", x.double().view(n, heads, padded), w.double()).reshape(n, heads * vdim)
    close(out, want, 1e-4 if dtype == torch.float32 else 2e-2, "per-head product")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,terms,partials", [(1, 64, 0, 1), (9, 96, 1, 1), (40, 72, 2, 3), (3, 128, 5, 2)])
def test_pending_sums_are_added_and_the_rows_joined(dtype, n, width, terms, partials):
    ops = cuda_ops(dtype)
    resid, other = rnd(n, width, seed=1), rnd(n, width, seed=2)
    pending, total = [], resid.double().clone()
    for t in range(terms):
        stack = rnd(partials, n, width, seed=10 + t)
        scale = 0.5 + t
        total += scale * stack.double().sum(0)
        pending.append(((stack if partials > 1 else stack[0]).contiguous().to(DEV), scale))
    held = resid.clone().to(DEV)
    out = torch.full((n, 2 * width), float("nan"), dtype=dtype, device=DEV)
    ops.concat_cast(held, pending, other.to(DEV), out)
    close(held, total, 1e-5, "the residual holds the sums")
    close(out[:, :width], total, TOL[dtype], "left half")
    close(out[:, width:], other.double(), TOL[dtype], "right half")
