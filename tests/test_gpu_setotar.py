"""The Setotar decoder on the GPU through the engine's own step function, cache manager and scheduler, against
the plain implementation in float64: every way of cutting (whole; most in one step and the last tokens one by one;
portions of changing size down to two tokens; mixed batches of unequal requests on a poisoned pool), tight pools
whose pages and state slots have several owners, long decoding past a window and many pages, the first tokens,
other page sizes, a request against itself in other company, captured against eager steps, keys just inside and
outside a window and among the kept first keys, a far key among a thousand, a state that keeps its first token,
greedy generation through `LLMEngine` with a preemption, and the replay and command-line programs."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.gpu_common import replay
from tests.helpers import mixed_trace, portions_trace, random_tokens, read_weights, tail_decode_trace, whole_trace
from tests.plain import plain_setotar as ps
from tests.setotar_configs import ASKER, MARK, SETOTAR, make_setotar_folder, planted_pair

pytestmark = pytest.mark.gpu
LENGTHS = {"A": [5, 47, 1, 230, 2, 64, 33], "B": [5, 17, 150, 70, 1, 90, 2], "C": [40, 3, 25, 1, 18], "D": [30, 2, 300, 140],
           "E": [9, 100, 1, 33], "M": [700, 37, 1, 260, 5], "N": [700, 37, 1, 260, 5]}
_cache = {}


def distance(got, want, scale):
    """Per position: the root mean square over the vocabulary of the difference of the logits, each
    with its mean taken off, in units of the logits' own spread."""
    d = got.astype(np.float64) - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / scale


# float32 kernels against float64: rounding alone stays far below this, a key wrongly seen or missed does not.
# bfloat16: three times what rounding alone causes in that request, measured with the plain implementation
# rounding its products' inputs and outputs to bfloat16 (both sides see the weights rounded to bfloat16).
LIMIT_FLOAT32 = 3e-5


def check(got, want, scale, limit, what, margins=None):
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    err = distance(got, want, scale)
    bad = np.nonzero(err > limit)[0]
    if len(bad) and margins is not None:
        # a router whose two best scores lie within rounding of each other may choose otherwise: from the first
        # such token on the request is another one
        close = np.nonzero(margins < 2e-2)[0]
        if len(close) and close[0] <= bad[0]:
            return
    assert not len(bad), f"{what}: position {int(bad[0])} is off by {err.max():.3e} (limit {limit:.1e})"


def rounded_weights(weights):
    return {k: (v.to(torch.bfloat16).float() if v.dim() >= 2 else v) for k, v in weights.items()}


def oracle(raw, weights, tokens, dtype, scale=None):
    """(logits, limit, the router's smallest margin at every position or None) for one request."""
    if dtype == "float32":
        return ps.forward(raw, weights, tokens).numpy(), LIMIT_FLOAT32, None
    weights = rounded_weights(weights)
    margins = []
    want = ps.forward(raw, weights, tokens, margins=margins).numpy()
    rough = ps.forward(raw, weights, tokens, rounding=True).numpy()
    scale = scale or float(np.sqrt(np.var(want, axis=-1).mean()))
    closest = np.array(margins).reshape(-1, len(tokens)).min(0) if margins else None
    return want, max(2e-2, 3.0 * float(distance(rough, want, scale).max())), closest


def reference(key, dtype, tmp_path_factory):
    """folder, requests, {id: logits}, scale, {id: limit}, {id: margins}"""
    if key not in _cache:
        folder = make_setotar_folder(tmp_path_factory.mktemp(f"setotar_{key}"), key)
        weights = read_weights(folder)
        requests = {f"r{i}": random_tokens(SETOTAR[key]["vocab"], n, 300 + i) for i, n in enumerate(LENGTHS[key])}
        want = {ident: ps.forward(SETOTAR[key], weights, tokens).numpy() for ident, tokens in requests.items()}
        scale = float(np.sqrt(np.mean([np.var(w, axis=-1).mean() for w in want.values()])))
        _cache[key] = (folder, requests, want, scale)
    folder, requests, want, scale = _cache[key]
    if dtype == "float32":
        return folder, requests, want, scale, {ident: LIMIT_FLOAT32 for ident in requests}, {ident: None for ident in requests}
    if key + "/bf16" not in _cache:
        weights = read_weights(folder)
        both = {ident: oracle(SETOTAR[key], weights, tokens, dtype, scale) for ident, tokens in requests.items()}
        _cache[key + "/bf16"] = tuple({i: b[n] for i, b in both.items()} for n in range(3))
    want, limits, margins = _cache[key + "/bf16"]
    return folder, requests, want, scale, limits, margins


WAYS = {
    "whole": lambda reqs: whole_trace(reqs),
    "tail": lambda reqs: tail_decode_trace(reqs, 45),
    "portions": lambda reqs: portions_trace(reqs, [7, 2, 5, 3, 2, 15, 16, 17, 2, 31, 33]),
    "long_portions": lambda reqs: portions_trace(reqs, [64, 33, 2, 70, 1]),
    "mixed": lambda reqs: mixed_trace(reqs, seed=3),
    "mixed_other_order": lambda reqs: mixed_trace(dict(reversed(list(reqs.items()))), seed=11),
}


@pytest.mark.parametrize("way", list(WAYS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page", [("A", 16), ("B", 16), ("A", 8), ("B", 24), ("C", 4), ("C", 32), ("D", 16), ("D", 64), ("E", 16)])
def test_replay_matches_plain(tmp_path_factory, key, page, dtype, way):
    folder, requests, want, scale, limits, margins = reference(key, dtype, tmp_path_factory)
    steps = WAYS[way](requests)
    got, session = replay(folder, dtype, steps, poison=way.startswith("mixed"), page_size=page, max_live=4)
    assert session.runner.cache.whole(), "pages or slots were not given back"
    for ident in requests:
        check(got[ident], want[ident], scale, limits[ident], f"{key} page {page} {dtype} {way} {ident}", margins[ident])


@pytest.mark.parametrize("way", ["whole", "tail", "long_portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page", [("M", 16), ("N", 32)])
def test_heads_of_the_tensor_core_kernels_sizes_and_long_prompts(tmp_path_factory, key, page, dtype, way):
    """Heads of 64 and 128 with prompts of several hundred tokens: the tcgen05 portions kernel with the kept keys' split,
    the recurrence's runs, the norm's clusters, the paged single-token kernel."""
    folder, requests, want, scale, limits, margins = reference(key, dtype, tmp_path_factory)
    steps = WAYS[way](requests)
    got, session = replay(folder, dtype, steps, poison=way.startswith("mixed"), page_size=page, max_live=4)
    assert session.runner.cache.whole(), "pages or slots were not given back"
    for ident in requests:
        check(got[ident], want[ident], scale, limits[ident], f"{key} page {page} {dtype} {way} {ident}", margins[ident])


def pages_needed(steps, page):
    held, worst = {}, 0
    for record in steps:
        for entry in record["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        worst = max(worst, sum(-(-n // page) for n in held.values()))
        for ident in record["end"]:
            held.pop(ident, None)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page", [("A", 8), ("B", 16), ("D", 16)])
def test_pages_and_slots_have_several_owners_on_a_tight_pool(tmp_path_factory, key, page, dtype):
    folder, requests, want, scale, limits, margins = reference(key, dtype, tmp_path_factory)
    steps = mixed_trace(requests, seed=5, max_live=3)
    num_pages = pages_needed(steps, page)
    assert num_pages < sum(-(-len(t) // page) for t in requests.values())
    got, session = replay(folder, dtype, steps, num_pages=num_pages, page_size=page, max_live=3, poison=True)
    shared = {pid: owners for pid, owners in session.page_owners.items() if len(owners) > 1}
    assert len({owner for owners in shared.values() for owner in owners}) >= 3
    assert session.runner.cache.whole()
    for ident in requests:
        check(got[ident], want[ident], scale, limits[ident], f"reuse {key} {dtype} {ident}", margins[ident])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "D"])
def test_long_decoding_token_by_token_past_the_window(tmp_path_factory, key, dtype):
    folder, _, _, scale, _, _ = reference(key, dtype, tmp_path_factory)
    tokens = random_tokens(SETOTAR[key]["vocab"], 300, 9)
    want, limit, margins = oracle(SETOTAR[key], read_weights(folder), tokens, dtype, scale)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == 299 else []}
             for i, t in enumerate(tokens)]
    got, session = replay(folder, dtype, steps, page_size=16)
    check(got["x"], want, scale, limit, f"long decode {key} {dtype}", margins)
    assert session.runner.cache.whole()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(tmp_path_factory, key, dtype):
    folder, _, _, scale, _, _ = reference(key, dtype, tmp_path_factory)
    tokens = random_tokens(SETOTAR[key]["vocab"], 4, 77)
    want, limit, margins = oracle(SETOTAR[key], read_weights(folder), tokens, dtype, scale)
    one_by_one = [{"step": i, "entries": [{"id": "f", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(tokens)]
    got, _ = replay(folder, dtype, one_by_one, max_tokens=64)
    check(got["f"], want, scale, limit, "first tokens one by one", margins)
    two_two = [{"step": 0, "entries": [{"id": "f", "tokens": tokens[:2], "want": [0, 1]}], "end": []},
               {"step": 1, "entries": [{"id": "f", "tokens": tokens[2:], "want": [0, 1]}], "end": ["f"]}]
    got, _ = replay(folder, dtype, two_two, max_tokens=64)
    check(got["f"], want, scale, limit, "first tokens two and two", margins)


@pytest.mark.parametrize("key", ["B", "D"])
def test_a_request_in_company_equals_itself_alone(tmp_path_factory, key):
    """float32: the logits of a position change by rounding at most with the cutting and the company."""
    folder, requests, want, scale, _, _ = reference(key, "float32", tmp_path_factory)
    whole, _ = replay(folder, "float32", whole_trace(requests))
    mixed, _ = replay(folder, "float32", mixed_trace(requests, seed=3), poison=True)
    cut, _ = replay(folder, "float32", portions_trace(requests, [2, 9, 2, 33, 64]))
    for ident in requests:
        bound = np.maximum(1e-5, 3.0 * distance(whole[ident], want[ident], scale))
        assert (distance(mixed[ident], whole[ident], scale) <= bound).all()
        assert (distance(cut[ident], whole[ident], scale) <= bound).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_captured_decode_steps_equal_eager_ones(tmp_path_factory, key, dtype):
    """Decode steps are replayed from CUDA graphs; the same trace with graphs off gives the same bits."""
    from shrike_b200.replay import TraceSession

    folder, requests, _, _, _, _ = reference(key, dtype, tmp_path_factory)
    steps = tail_decode_trace({k: v for k, v in list(requests.items())[:3]}, 20)
    results = []
    for graphs in (True, False):
        session = TraceSession(folder, dtype, 512, page_size=16, max_live=4)
        session.runner.use_graphs = graphs
        results.append([session.step(record).copy() for record in steps])
        if graphs:
            assert session.runner.capture_safe and session.runner._graphs, "no decode step was captured"
    for a, b in zip(*results):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,lengths,new", [("A", (5, 17, 33), 8), ("D", (3, 40, 75), 8)])
def test_greedy_generation_through_the_engine(tmp_path_factory, key, lengths, new, dtype):
    from shrike_b200 import SamplingParams
    from shrike_b200.engine.llm_engine import LLMEngine

    folder, _, _, scale, _, _ = reference(key, dtype, tmp_path_factory)
    weights = read_weights(folder)
    if dtype == "bfloat16":
        weights = rounded_weights(weights)
    engine = LLMEngine(str(folder), block_size=8, num_blocks=40, max_tokens_per_step=32, dtype=dtype)
    prompts = [random_tokens(SETOTAR[key]["vocab"], n, 30 + n) for n in lengths]
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    assert engine.block_manager.whole()
    tie = 12 * scale * (LIMIT_FLOAT32 if dtype == "float32" else 4e-2)   # a top-2 gap within the logits' tolerance is a tie
    for prompt, out in zip(prompts, outs):
        want, gaps = ps.greedy_continue(SETOTAR[key], weights, prompt, new)
        for position, (a, b, gap) in enumerate(zip(out, want, gaps)):
            if a != b:
                assert gap < tie or dtype == "bfloat16", f"token {position}: engine {a}, plain {b}, gap {gap}"
                break   # after a tie went the other way the continuations differ


@pytest.mark.parametrize("dtype", ["float32"])
def test_generation_survives_preemption_with_state(tmp_path_factory, dtype):
    """A pool too small for three requests at once: one is preempted (pages and state slots returned) and
    computed again later from zero state; every continuation still equals the plain implementation's."""
    from shrike_b200 import SamplingParams
    from shrike_b200.engine.llm_engine import LLMEngine

    folder, _, _, scale, _, _ = reference("E", dtype, tmp_path_factory)
    weights = read_weights(folder)
    engine = LLMEngine(str(folder), block_size=8, num_blocks=15, max_tokens_per_step=32, dtype=dtype)
    prompts = [random_tokens(SETOTAR["E"]["vocab"], n, 60 + n) for n in (30, 31, 29)]
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=24, ignore_eos=True))
    assert engine.block_manager.whole() and engine.scheduler.num_preemptions >= 1
    tie = 12 * scale * LIMIT_FLOAT32
    for prompt, out in zip(prompts, outs):
        want, gaps = ps.greedy_continue(SETOTAR["E"], weights, prompt, 24)
        for position, (a, b, gap) in enumerate(zip(out, want, gaps)):
            if a != b:
                assert gap < tie, f"token {position}: engine {a}, plain {b}, gap {gap}"
                break


def _one_layer(layer, width=64, vocab=61, **more):
    return dict({"architecture": "Setotar", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "layers": [layer]}, **more)


def sequence_with(count, place, seed):
    """`count` tokens, none of them the planted pair's, but MARK at `place` and ASKER last."""
    tokens = [5 + t % 50 for t in random_tokens(1000, count, seed)]
    tokens[place], tokens[-1] = MARK, ASKER
    return tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,keep,page", [(1, 1, 16), (2, 5, 16), (17, 4, 16), (32, 16, 16), (130, 5, 16), (21, 9, 8), (64, 70, 64), (300, 3, 32)])
def test_keys_at_the_windows_edge_and_among_the_kept_first_decide(tmp_path, window, keep, page, dtype):
    """Attention whose last query finds one marked key above all others: the last logits are the marked token's when
    it sits just inside the window or is the last kept key, and show no trace of it just outside the window or just
    behind the kept keys, in a whole prompt, in portions that start or end at the edge, and decoding token by token."""
    raw = _one_layer({"type": "parallel", "mlp": None, "mixer": {
        "left": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.4, "conv": 3, "softcap": 50.0,
                 "rot": {"dims": 8, "base": 20.0, "scaling": {"factor": 2.0}}, "mask": {"size": window, "keep_first": keep}},
        "right": {"heads": 1, "dim": 8, "vdim": 8}, "left_scale": 1.0, "right_scale": 1.0}}, streams=2)
    folder = make_setotar_folder(tmp_path, f"edge{window}", raw=raw, seed=window, change=planted_pair(raw))
    weights = read_weights(folder)
    count = window + keep + 40
    for place, seen in ((count - window, True), (count - window - 1, False), (keep - 1, True), (keep, False)):
        tokens = sequence_with(count, place, 2)
        without = list(tokens)
        without[place] = 9
        want, limit, _ = oracle(raw, weights, tokens, dtype)
        unmarked, _, _ = oracle(raw, weights, without, dtype)
        scale = float(np.sqrt(np.var(want, axis=-1).mean()))
        moved = distance(want[-1:], unmarked[-1:], scale)[0]
        assert (moved > 0.2) == seen, f"the plain implementation itself: place {place}, moved {moved}"
        ways = (whole_trace({"a": tokens}), portions_trace({"a": tokens}, [place + 1, 2, count]), tail_decode_trace({"a": tokens}, window + 3),
                portions_trace({"a": tokens}, [max(place, 1), 3, count]), portions_trace({"a": tokens}, [count - 2, 2]))
        for steps in ways:
            got, _ = replay(folder, dtype, steps, page_size=page, max_live=1)
            check(got["a"][-1:], want[-1:], scale, limit, f"window {window}, keep {keep}, place {place}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("place", [0, 1, 15, 16, 255, 256, 700])
def test_a_far_key_is_found_among_hundreds(tmp_path, dtype, place):
    """Attention over every key of a thousand on many pages, read by a second layer from the first one's cache too:
    the last query finds the one marked key wherever it lies."""
    attention = {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2, "rot": {"dims": 16, "base": 100.0}}
    raw = _one_layer({"type": "attention", "mlp": None, "mixer": attention})
    raw["layers"].append({"type": "attention", "mlp": None, "mixer": dict(attention, kv_from=0)})
    folder = make_setotar_folder(tmp_path, "far", raw=raw, seed=5, change=planted_pair(raw))
    weights = read_weights(folder)
    tokens = sequence_with(1000, place, 8)
    without = list(tokens)
    without[place] = 9
    want, limit, _ = oracle(raw, weights, tokens, dtype)
    scale = float(np.sqrt(np.var(want, axis=-1).mean()))
    unmarked, _, _ = oracle(raw, weights, without, dtype)
    assert distance(want[-1:], unmarked[-1:], scale)[0] > 0.2
    for steps in (whole_trace({"a": tokens}), tail_decode_trace({"a": tokens}, 40), portions_trace({"a": tokens}, [2, 130, 1, 1, 65, 500])):
        got, _ = replay(folder, dtype, steps, page_size=16, max_live=1)
        check(got["a"], want, scale, limit, f"marked key at {place}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_gate_that_never_forgets_keeps_the_first_token(tmp_path, dtype):
    """A recurrence whose lower bound is all but one in one head: the last token reads the first token's value out of
    the state three hundred tokens later, however the prompt was cut and whoever else is in the batch."""
    raw = _one_layer({"type": "parallel", "mlp": None, "mixer": {
        "left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.3, "mask": {"size": 4, "keep_first": 0}},
        "right": {"heads": 2, "dim": 16, "vdim": 32}, "left_scale": 0.0, "right_scale": 1.0}}, streams=3)

    def change(tensors):
        tensors["l0.mix.right.lower"][:16] = 0.9995
        tensors["l0.mix.right.o"] *= 4.0
        tensors["l0.mix.right.v"] *= 3.0

    folder = make_setotar_folder(tmp_path, "state", raw=raw, seed=11, change=change)
    weights = read_weights(folder)
    tokens = random_tokens(61, 300, 4)
    other = [(tokens[0] + 7) % 61] + tokens[1:]
    (want, limit, _), (want_other, _, _) = oracle(raw, weights, tokens, dtype), oracle(raw, weights, other, dtype)
    scale = float(np.sqrt(np.var(want, axis=-1).mean()))
    if dtype == "float32":   # what such a gate lets in is small: the first token's trace shows at float32's accuracy alone
        assert distance(want[-1:], want_other[-1:], scale)[0] > 20 * limit
    both = {"a": tokens, "b": other}
    for steps in (whole_trace(both), portions_trace(both, [2, 33, 1, 100, 3]), mixed_trace(both, seed=1, max_live=2), tail_decode_trace(both, 70)):
        got, session = replay(folder, dtype, steps, page_size=16, max_live=2)
        check(got["a"], want, scale, limit, "the request itself")
        check(got["b"], want_other, scale, limit, "its neighbour with another first token")


def test_trace_run_program_serves_the_design(tmp_path):
    folder = make_setotar_folder(tmp_path, "A")
    requests = {"a": random_tokens(211, 41, 1), "b": random_tokens(211, 9, 2)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": requests["a"][:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": requests["a"][30:31], "want": []},
                                {"id": "b", "tokens": requests["b"], "want": [8]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": requests["a"][31:], "want": [9]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    program = Path(__file__).resolve().parents[1] / "bin" / "trace_run"
    run = subprocess.run(
        [sys.executable, str(program), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900,
    )
    assert run.returncode == 0, run.stderr[-2000:]
    assert [line for line in run.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    weights = read_weights(folder)
    raw = SETOTAR["A"]
    ref_a, ref_b = ps.forward(raw, weights, requests["a"]).numpy(), ps.forward(raw, weights, requests["b"]).numpy()
    scale = float(np.sqrt(np.var(ref_a, axis=-1).mean()))
    check(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, 211), ref_a[[0, 29]], scale, LIMIT_FLOAT32, "step 0")
    check(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, 211), ref_b[[8]], scale, LIMIT_FLOAT32, "step 1")
    check(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, 211), ref_a[[40]], scale, LIMIT_FLOAT32, "step 2")


def test_command_line_program_serves_the_design(tmp_path):
    """The one-prompt program on a folder: the model class comes from config.json."""
    import os

    bin_dir = Path(__file__).resolve().parents[1] / "bin"
    folder = make_setotar_folder(tmp_path, "A")
    prompt = [7, 200, 41, 41, 2]
    want, gaps = ps.greedy_continue(SETOTAR["A"], read_weights(folder), prompt, 6)
    assert min(gaps) > 1e-4
    done = subprocess.run([sys.executable, str(bin_dir / "shrike_b200_complete"), " ".join(map(str, prompt)), "--model", str(folder),
                           "--max-tokens", "6", "--dtype", "float32", "--num-blocks", "8", "--block-size", "8"],
                          capture_output=True, text=True, timeout=900, env=dict(os.environ, PYTHONUNBUFFERED="1"))
    assert done.returncode == 0, done.stderr[-3000:]
    assert [int(t) for t in done.stdout.split()] == want
