"""Kavedra on the CPU: the configuration reader, the tensor names, the run order with its passes, the
caches (pages behind a window given back, a latent's single plane, one state slot a request and pass),
the rotation's frequencies, and the whole model stepped through the engine's replay session with the
stand-in kernels against the plain implementation: whole, in portions down to two tokens, and mixed on
a tight pool; with weights planted so that a sink, a window's edge or a lost state decides the logits."""

import copy
import math

import numpy as np
import pytest
import torch

import shrike_b200.models  # noqa: F401
from shrike_b200.config import ConfigError, parse_config
from shrike_b200.config.model_config import (
    DecayLinearAttentionSpec,
    GatedHeadAttentionSpec,
    GatedMLPSpec,
    PairRotationSpec,
    RotaryLatentAttentionSpec,
)
from shrike_b200.parts.rotary import PairRotation
from shrike_b200.replay import TraceSession
from shrike_b200.weights.expected import expected_tensors
from tests.emulated_ops import EmulatedOps
from tests.helpers import collect, mixed_trace, portions_trace, random_tokens, read_weights, tail_decode_trace, whole_trace
from tests.kavedra_configs import KAVEDRA, KAVEDRA_A, KAVEDRA_B, KAVEDRA_C, KAVEDRA_D, make_kavedra_folder
from tests.plain import plain_kavedra as pk


def test_config_gives_each_layer_its_mixer_and_every_run_its_cache():
    config = parse_config(KAVEDRA_A)
    assert config.architecture == "Kavedra" and config.num_layers == 3
    assert [(run.layer, run.cache, run.enter) for run in config.order] == [
        (0, 0, None), (1, 1, 0), (2, 2, None), (1, 3, 1), (2, 4, None), (1, 5, 2), (2, 6, None)]
    assert config.pass_entry.passes == 3 and config.pass_entry.mix and config.head.scale == 0.5
    latent, linear, attention = (layer.mixer for layer in config.layers)
    assert isinstance(latent, RotaryLatentAttentionSpec) and isinstance(linear, DecayLinearAttentionSpec)
    assert isinstance(attention, GatedHeadAttentionSpec)
    assert (latent.num_heads, latent.head_dim, latent.rotary_dim, latent.value_dim, latent.latent_rank) == (3, 24, 8, 16, 40)
    assert (latent.window, latent.scale, latent.gate, latent.rotation.stretch) == (21, 0.21, "element", (4.0, 64.0, 8.0, 2.0))
    assert (linear.num_heads, linear.head_dim, linear.value_dim, linear.decays) == (3, 16, 24, (0.5, 1.0, 0.93))
    assert (attention.num_heads, attention.num_kv_heads, attention.head_dim, attention.value_dim) == (6, 2, 16, 32)
    assert attention.sink and attention.qkv_bias and attention.window is None and attention.scale == 0.3
    assert (attention.rotation.dims, attention.rotation.base, attention.rotation.pairing) == (8, 1000.0, "neighbours")
    assert [type(layer.feed_forward) for layer in config.layers] == [GatedMLPSpec, type(None), GatedMLPSpec]
    assert config.layers[1].feed_forward_norm is None and config.layers[0].mixer_norm.offset == 1.0
    plain = parse_config(KAVEDRA_B)
    assert plain.pass_entry is None and [run.enter for run in plain.order] == [None] * 4 and plain.head.scale == 1.0
    assert plain.layers[1].mixer.window is None and plain.layers[1].mixer.rotation.stretch is None
    once = parse_config(KAVEDRA_C)
    assert [(run.layer, run.enter) for run in once.order] == [(0, 0), (1, None), (2, None), (3, None), (4, None)]
    assert [(run.layer, run.cache, run.enter) for run in parse_config(KAVEDRA_D).order] == [
        (0, 0, None), (1, 1, 0), (2, 2, None), (3, 3, None), (1, 4, 1), (2, 5, None), (3, 6, None), (1, 7, 2), (2, 8, None),
        (3, 9, None), (4, 10, None)]


def test_tensor_names_follow_the_layers():
    names = expected_tensors(parse_config(KAVEDRA_A))
    assert {"embed", "loop.in", "loop.step", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.dkv",
            "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down",
            "l1.mix.q", "l1.mix.k", "l1.mix.v", "l1.mix.g", "l1.mix.norm", "l1.mix.o", "l2.mix.q.b", "l2.mix.k.b",
            "l2.mix.v.b", "l2.mix.sink", "l2.mix.o"} <= set(names)
    assert "l1.norm2" not in names and "l1.mlp.gate" not in names and "l0.mix.sink" not in names and "l2.mix.g" not in names
    assert names["loop.in"].shape == (96, 192) and names["loop.step"].shape == (3, 96)
    assert names["l0.mix.q"].shape == (3 * (24 + 8), 96) and names["l0.mix.dkv"].shape == (40 + 8, 96)
    assert names["l0.mix.uk"].shape == (3 * 24, 40) and names["l0.mix.uv"].shape == (3 * 16, 40)
    assert names["l0.mix.g"].shape == (3 * 16, 96) and names["l0.mix.o"].shape == (96, 3 * 16)
    assert names["l1.mix.q"].shape == (3 * 16, 96) and names["l1.mix.v"].shape == (3 * 24, 96) and names["l1.mix.norm"].shape == (72,)
    assert names["l2.mix.k"].shape == (2 * 16, 96) and names["l2.mix.v"].shape == (2 * 32, 96)
    assert names["l2.mix.o"].shape == (96, 6 * 32) and names["l2.mix.sink"].shape == (6,)
    assert "loop.step" not in expected_tensors(parse_config(KAVEDRA_B)) and "loop.in" not in expected_tensors(parse_config(KAVEDRA_B))


@pytest.mark.parametrize("change,text", [
    (lambda raw: raw["layers"][0].update(type="convolution"), "known: attention, latent_attention, lightning"),
    (lambda raw: raw["layers"][2]["mixer"].pop("kv_heads"), "kv_heads"),
    (lambda raw: raw["layers"][2]["mixer"]["rot"].update(dims=18), "rotation over 18"),
    (lambda raw: raw["layers"][2]["mixer"]["rot"].update(dims=7), "even number"),
    (lambda raw: raw["layers"][2]["mixer"].update(kv_heads=4), "multiple"),
    (lambda raw: raw["layers"][1]["mixer"].update(decay=[0.5, 0.5]), "2 decays for 3 heads"),
    (lambda raw: raw["layers"][1]["mixer"].update(decay=[0.5, 1.5, 0.2]), r"\(0, 1\]"),
    (lambda raw: raw["layers"][1]["mixer"].update(decay=0.5), "one number per head"),
    (lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=6), "rotated part has 8"),
    (lambda raw: raw["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda raw: raw["layers"][0]["mixer"].pop("rot"), "lacks `rot`"),
    (lambda raw: raw["layers"][0]["mixer"]["mask"].update(size=0), "size must be a positive integer"),
    (lambda raw: raw["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda raw: raw["layers"][0]["mlp"].update(kind="moe"), "known: dense"),
    (lambda raw: raw["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda raw: raw["loop"].update(stop=4), "loop runs layers"),
    (lambda raw: raw["loop"].pop("times"), "times"),
    (lambda raw: raw.pop("norm"), "norm"),
    (lambda raw: raw.pop("width"), "width"),
])
def test_config_errors_name_the_key(change, text):
    raw = copy.deepcopy(KAVEDRA_A)
    change(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


@pytest.mark.parametrize("dims,base,stretch", [(8, 10000.0, (4.0, 64, 8.0, 2.0)), (32, 40000.0, (8.0, 1024, 32.0, 1.0)),
                                               (2, 10.0, (2.0, 4, 1000.0, 0.0001)), (16, 100.0, None), (4, 50.0, (16.0, 32, 4.0, 1.0)),
                                               (64, 1e6, (40.0, 4096, 32.0, 1.0)), (6, 7.0, (3.0, 16, 1.0, 1.0))])
def test_rotation_frequencies_and_gain(dims, base, stretch):
    """The part's table against the plain reading of the stretch rule, also where a border falls outside the pairs
    or both borders meet."""
    spec = PairRotationSpec(dims=dims, base=base, pairing="neighbours", stretch=stretch)
    rotation = PairRotation(spec, "cpu")
    raw = {"dims": dims, "base": base}
    if stretch is not None:
        raw["scaling"] = dict(zip(("factor", "original", "fast", "slow"), stretch))
    freq, gain = pk.frequencies(raw, torch.float64)
    assert rotation.inv_freq.dtype == torch.float32 and rotation.inv_freq.shape == (dims // 2,)
    assert torch.allclose(rotation.inv_freq.double(), freq, rtol=1e-6, atol=0)
    assert math.isclose(rotation.gain, gain, rel_tol=1e-12)


def run(folder, steps, **options):
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), **options)
    outputs = {}
    for record in steps:
        result = session.step(record)
        if result is not None:
            outputs[record["step"]] = result.copy()
    return collect(steps, outputs), session


LENGTHS = [5, 47, 1, 83, 2, 30]


@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_engine_with_stand_in_kernels_matches_plain(tmp_path, key):
    folder = make_kavedra_folder(tmp_path, key)
    weights = read_weights(folder)
    requests = {f"r{i}": random_tokens(KAVEDRA[key]["vocab"], n, 200 + i) for i, n in enumerate(LENGTHS)}
    want = {ident: pk.forward(KAVEDRA[key], weights, tokens).numpy() for ident, tokens in requests.items()}
    spread = float(np.sqrt(np.mean([np.var(w, axis=-1).mean() for w in want.values()])))
    ways = (whole_trace(requests), tail_decode_trace(requests, 25), portions_trace(requests, [7, 2, 5, 3, 16, 17, 2]),
            mixed_trace(requests, seed=4))
    for steps in ways:
        got, session = run(folder, steps, page_size=8, num_pages=40, max_live=4)
        assert session.runner.cache.whole()
        for ident in requests:
            assert np.abs(got[ident] - want[ident]).max() < 2e-4 * max(1.0, spread), ident   # float32 stand-ins against float64


def test_a_request_holds_a_state_slot_per_pass_and_a_windows_pages(tmp_path):
    folder = make_kavedra_folder(tmp_path, "A")
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), page_size=4, num_pages=64, max_live=2)
    groups = session.runner.groups
    # the latent's page row is [40 | 8] in one plane that is key and value at once; the attention's three runs share a group
    assert sorted((g.head_dim, g.window, g.num_kv_heads, g.cache_ids, g.planes) for g in groups) == [
        (32, None, 2, (2, 4, 6), 2), (48, 21, 1, (0,), 1)]
    state = session.runner.storage.state
    assert sorted(state) == [1, 3, 5] and all(tuple(s.shape) == (2, 3, 16 * 24) for s in state.values())
    tokens = random_tokens(211, 70, 5)
    session.step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": []}], "end": []})
    for group, table in zip(groups, session.live["a"][0].tables):
        behind = 0 if group.window is None else (70 - group.window + 1) // 4   # the next query, at 70, sees keys from 50 on
        assert int((table.view() < 0).sum()) == behind
    slot = session.live["a"][0].slot
    for cache in (1, 3, 5):
        assert float(state[cache][slot].abs().sum()) > 0 and float(state[cache][1 - slot].abs().sum()) == 0
    assert not torch.equal(state[1][slot], state[3][slot])   # each pass keeps a state of its own
    session.step({"step": 1, "entries": [], "end": ["a"]})
    assert session.runner.cache.whole()
    # the slot's next owner starts from zero state although the kernels left the old one's behind
    session.step({"step": 2, "entries": [{"id": "b", "tokens": tokens[:3], "want": []}], "end": []})
    session.step({"step": 3, "entries": [{"id": "c", "tokens": tokens[:3], "want": []}], "end": []})
    b, c = session.live["b"][0].slot, session.live["c"][0].slot
    assert b != c and all(torch.equal(state[cache][b], state[cache][c]) for cache in (1, 3, 5))


def _one_layer(layer, width=32, vocab=61, **more):
    return dict({"architecture": "Kavedra", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "layers": [layer]}, **more)


def test_the_sink_takes_its_share_of_the_weight(tmp_path):
    """With one sink far above every score, that head's output goes to nothing; the plain implementation agrees, and
    leaving the sink out would change the logits by far more than the tolerance."""
    raw = _one_layer({"type": "attention", "mlp": None,
                      "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25, "rot": {"dims": 16, "base": 100.0}}})

    def plant(tensors):
        tensors["l0.mix.sink"][:] = torch.tensor([9.0, -30.0])   # head 0 loses nearly all its weight, head 1 nearly none

    folder = make_kavedra_folder(tmp_path, "sink", raw=raw, seed=5, change=plant)
    weights = read_weights(folder)
    tokens = random_tokens(61, 23, 8)
    want = pk.forward(raw, weights, tokens).numpy()
    without = pk.forward(raw, dict(weights, **{"l0.mix.sink": torch.full((2,), -80.0)}), tokens).numpy()
    assert np.abs(want - without).max() > 0.05
    for steps in (whole_trace({"a": tokens}), portions_trace({"a": tokens}, [2, 7, 1, 1, 5])):
        got, _ = run(folder, steps, page_size=4, num_pages=8, max_live=1)
        assert np.abs(got["a"] - want).max() < 1e-4


@pytest.mark.parametrize("window", [1, 3, 8, 13])
def test_a_key_at_the_windows_edge_decides(tmp_path, window):
    """Latent attention with one query and one key made large along a shared direction: the logits at the last
    position move when the planted token sits just inside the window and not at all when just outside, whether the
    prompt came whole, in portions that end at the edge, or token by token."""
    raw = _one_layer({"type": "latent_attention", "mlp": None,
                      "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 8, "kv_rank": 12, "scale": 0.5,
                                "rot": {"dims": 4, "base": 20.0}, "mask": {"size": window}}})
    folder = make_kavedra_folder(tmp_path, f"edge{window}", raw=raw, seed=window)
    weights = read_weights(folder)
    count = 30
    base = random_tokens(61, count, 2)
    for back in (window - 1, window):            # the planted token's distance from the last one: seen, not seen
        tokens = list(base)
        other = list(base)
        place = count - 1 - back
        other[place] = (base[place] + 7) % 61
        want, want_other = pk.forward(raw, weights, tokens).numpy()[-1], pk.forward(raw, weights, other).numpy()[-1]
        moved = np.abs(want - want_other).max()
        assert (moved > 1e-3) == (back < window), f"the oracle itself: back {back}, moved {moved}"
        ways = (whole_trace({"a": other}), portions_trace({"a": other}, [place + 1, 2, count]), portions_trace({"a": other}, [1]),
                portions_trace({"a": other}, [max(place, 1), count]))
        for steps in ways:
            got, _ = run(folder, steps, page_size=4, num_pages=10, max_live=1)
            assert np.abs(got["a"][-1] - want_other).max() < 1e-4, f"window {window}, back {back}"


def test_a_lost_or_foreign_state_shows(tmp_path):
    """A decay of exactly 1 keeps the first token for ever: the last logits depend on it, and the engine cut into
    portions carries it."""
    raw = _one_layer({"type": "lightning", "mlp": None, "mixer": {"heads": 2, "dim": 8, "vdim": 16, "decay": [1.0, 0.98]}})
    folder = make_kavedra_folder(tmp_path, "state", raw=raw, seed=11)
    weights = read_weights(folder)
    tokens = random_tokens(61, 90, 4)
    other = [(tokens[0] + 3) % 61] + tokens[1:]
    want, want_other = pk.forward(raw, weights, tokens).numpy(), pk.forward(raw, weights, other).numpy()
    assert np.abs(want[-1] - want_other[-1]).max() > 1e-3
    both = {"a": tokens, "b": other}
    for steps in (whole_trace(both), portions_trace(both, [2, 33, 1, 40, 3]), mixed_trace(both, seed=1, max_live=2)):
        got, session = run(folder, steps, page_size=4, num_pages=2, max_live=2)
        assert np.abs(got["a"] - want).max() < 2e-4 and np.abs(got["b"] - want_other).max() < 2e-4
        assert session.runner.cache.whole()
