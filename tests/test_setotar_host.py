"""The Setotar design on the CPU: the reader of its config.json, its tensor names, the pools and states a
request holds, and the engine's step function, cache manager and batching driven through the stand-in kernels
against the plain implementation."""

import copy

import numpy as np
import pytest
import torch

from shrike_b200 import models  # noqa: F401
from shrike_b200.cache.manager import CacheManager, KVGroupSpec, pages_in_flight
from shrike_b200.config.model_config import ConfigError
from shrike_b200.config.registry import parse_config
from shrike_b200.replay import TraceSession
from shrike_b200.weights.expected import expected_tensors
from tests.emulated_ops import EmulatedOps
from tests.helpers import collect, mixed_trace, portions_trace, random_tokens, read_weights, tail_decode_trace, whole_trace
from tests.plain import plain_setotar as ps
from tests.setotar_configs import ASKER, MARK, SETOTAR, make_setotar_folder, planted_pair


def test_config_gives_each_layer_its_parts_and_every_run_its_cache():
    config = parse_config(SETOTAR["A"])
    assert [layer.block for layer in config.layers] == ["hyper"] * 4
    assert [(run.layer, run.cache, run.writes_cache) for run in config.order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False)]
    left = config.layers[0].mixer.branches[0][1]
    assert (left.conv, left.window, left.keep_first, left.softcap, left.value_norm, left.qkv_bias) == (4, 21, 3, 5.0, True, True)
    assert left.rotation.divide == 4.0 and left.rotation.stretch is None and left.rotation.pairing == "halves"
    attention = config.layers[1].mixer
    assert attention.qk_norm == "whole" and attention.own_kv and attention.rotation.stretch == (8.0, 32.0, 4.0, 0.5)
    assert not config.layers[3].mixer.own_kv
    experts = config.layers[1].feed_forward
    assert (experts.scoring, experts.renormalise, experts.weight_on, experts.top) == ("sigmoid", False, "input", 2)
    assert config.residual.streams == 2 and config.layers[2].feed_forward is None
    assert parse_config(SETOTAR["C"]).residual.streams == 1 and not parse_config(SETOTAR["C"]).layers[0].extra[0][2].learned


def test_tensor_names_follow_the_layers():
    names = set(expected_tensors(parse_config(SETOTAR["A"])))
    for name in ("embed", "head", "final.norm", "l0.norm1", "l0.ls1", "l0.ls2", "l0.hc1.in", "l0.hc1.out", "l0.hc1.mix", "l0.hc2.mix",
                 "l0.mix.left.q", "l0.mix.left.q.b", "l0.mix.left.q.conv", "l0.mix.left.v.conv", "l0.mix.left.o", "l0.mix.right.f",
                 "l0.mix.right.f.b", "l0.mix.right.lower", "l0.mix.right.norm", "l0.mlp.router", "l0.mlp.e3.down", "l1.mix.q.norm",
                 "l1.mix.k.norm", "l1.mix.v", "l3.mix.q", "l3.mix.q.norm", "l3.mix.o", "l2.ls1", "l2.hc1.in"):
        assert name in names, name
    for name in ("l3.mix.k", "l3.mix.v", "l3.mix.k.norm", "l2.norm2", "l2.ls2", "l2.hc2.in", "l1.mix.q.b", "l0.mlp.e4.gate"):
        assert name not in names, name
    assert not any(".hc" in name for name in expected_tensors(parse_config(SETOTAR["C"])))   # no streams, no connections


@pytest.mark.parametrize("change,text", [
    (lambda raw: raw["layers"][0].update(type="other"), "type"),
    (lambda raw: raw["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda raw: raw["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda raw: raw["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda raw: raw["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda raw: raw.update(streams=9), "streams"),
    (lambda raw: raw.pop("width"), "width"),
])
def test_config_errors_name_the_key(change, text):
    raw = copy.deepcopy(SETOTAR["A"])
    change(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


def test_the_pages_of_kept_keys_are_never_given_back():
    group = KVGroupSpec((0,), 1, 16, window=10, keep_first=6)
    manager = CacheManager([group], page_size=4, num_pages=32, max_slots=2)
    cache = manager.open()
    manager.append(cache, 0, 50)
    manager.advance(cache, 50)   # the next query, at 50, sees keys 41 .. and 0 .. 5
    pages = cache.tables[0].view()
    assert (pages[:2] >= 0).all() and (pages[2:10] < 0).all() and (pages[10:] >= 0).all()
    manager.append(cache, 50, 30)
    manager.advance(cache, 80)
    assert (cache.tables[0].view()[:2] >= 0).all() and int((cache.tables[0].view() < 0).sum()) == 15
    manager.free(cache)
    assert manager.whole()
    assert pages_in_flight(1 << 30, 10, 1, 4, 6) == pages_in_flight(1 << 30, 10, 1, 4) + 2


def run(folder, steps, **options):
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), **options)
    outputs = {}
    for record in steps:
        result = session.step(record)
        if result is not None:
            outputs[record["step"]] = result.copy()
    return collect(steps, outputs), session


LENGTHS = [5, 41, 1, 2, 23]


@pytest.mark.parametrize("key", ["A", "B", "C", "D", "E"])
def test_engine_with_stand_in_kernels_matches_plain(tmp_path, key):
    folder = make_setotar_folder(tmp_path, key)
    weights = read_weights(folder)
    requests = {f"r{i}": random_tokens(SETOTAR[key]["vocab"], n, 200 + i) for i, n in enumerate(LENGTHS)}
    want = {ident: ps.forward(SETOTAR[key], weights, tokens).numpy() for ident, tokens in requests.items()}
    spread = float(np.sqrt(np.mean([np.var(w, axis=-1).mean() for w in want.values()])))
    ways = (whole_trace(requests), tail_decode_trace(requests, 25), portions_trace(requests, [7, 2, 5, 3, 16, 17, 2]),
            mixed_trace(requests, seed=4))
    for steps in ways:
        got, session = run(folder, steps, page_size=8, num_pages=40, max_live=4)
        assert session.runner.cache.whole()
        for ident in requests:
            assert np.abs(got[ident] - want[ident]).max() < 2e-4 * max(1.0, spread), ident   # float32 stand-ins against float64


def test_a_request_holds_pages_a_recurrent_state_and_the_convolutions_last_inputs(tmp_path):
    folder = make_setotar_folder(tmp_path, "A")
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), page_size=4, num_pages=64, max_live=2)
    groups = session.runner.groups
    assert sorted((g.cache_ids, g.head_dim, g.window, g.keep_first, g.num_kv_heads) for g in groups) == [
        ((0,), 16, 21, 3, 2), ((1,), 16, None, 0, 2), ((2,), 32, 130, 20, 1)]
    state = session.runner.storage.state
    assert sorted(state, key=str) == [(0, "conv"), (2, "conv"), 0, 2]
    assert tuple(state[(0, "conv")].shape) == (2, 3, 4 * 16 + 2 * 16 + 2 * 8) and tuple(state[0].shape) == (2, 3, 8 * 16)
    tokens = random_tokens(211, 70, 5)
    session.step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": []}], "end": []})
    table = session.live["a"][0].tables[[g.cache_ids for g in groups].index((0,))].view()
    assert (table[:1] >= 0).all() and (table[1:12] < 0).all() and (table[12:] >= 0).all()   # keys 0 .. 2 kept, 50 .. seen next
    slot = session.live["a"][0].slot
    for key in state:
        assert float(state[key][slot].abs().sum()) > 0 and float(state[key][1 - slot].abs().sum()) == 0
    session.step({"step": 1, "entries": [], "end": ["a"]})
    assert session.runner.cache.whole()
    # the slot's next owner starts from zero state although the kernels left the old one's behind
    session.step({"step": 2, "entries": [{"id": "b", "tokens": tokens[:3], "want": []}], "end": []})
    session.step({"step": 3, "entries": [{"id": "c", "tokens": tokens[:3], "want": []}], "end": []})
    b, c = session.live["b"][0].slot, session.live["c"][0].slot
    assert b != c and all(torch.equal(state[key][b], state[key][c]) for key in state)


def _one_layer(layer, width=32, vocab=61, **more):
    return dict({"architecture": "Setotar", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "layers": [layer]}, **more)


@pytest.mark.parametrize("window,keep", [(1, 1), (5, 2), (17, 4), (40, 9)])
def test_keys_at_the_windows_edge_and_among_the_kept_first_decide(tmp_path, window, keep):
    """The last query finds one marked key above all others: just inside the window and among the kept first keys it
    decides the last logits, just outside either it leaves no trace."""
    raw = _one_layer({"type": "parallel", "mlp": None, "mixer": {
        "left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.4, "conv": 3, "softcap": 50.0,
                 "rot": {"dims": 8, "base": 20.0}, "mask": {"size": window, "keep_first": keep}},
        "right": {"heads": 1, "dim": 8, "vdim": 8}, "left_scale": 1.0, "right_scale": 1.0}}, streams=2)
    folder = make_setotar_folder(tmp_path, f"edge{window}", raw=raw, seed=window, change=planted_pair(raw))
    weights = read_weights(folder)
    count = window + keep + 30
    for place, seen in ((count - window, True), (count - window - 1, False), (keep - 1, True), (keep, False)):
        tokens = [5 + t % 50 for t in random_tokens(1000, count, 2)]
        tokens[place], tokens[-1] = MARK, ASKER
        without = list(tokens)
        without[place] = 9
        want, unmarked = ps.forward(raw, weights, tokens).numpy(), ps.forward(raw, weights, without).numpy()
        spread = float(np.sqrt(np.var(want, axis=-1).mean()))
        moved = float(np.abs(want[-1] - unmarked[-1]).max()) / spread
        assert (moved > 0.2) == seen, f"the plain implementation itself: place {place}, moved {moved}"
        for steps in (whole_trace({"a": tokens}), portions_trace({"a": tokens}, [place + 1, 2, count]), tail_decode_trace({"a": tokens}, window + 3)):
            got, _ = run(folder, steps, page_size=4, num_pages=64, max_live=1)
            assert np.abs(got["a"][-1] - want[-1]).max() < 2e-4 * max(1.0, spread)
