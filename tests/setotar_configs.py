"""Tiny Setotar configurations for tests, and model folders with weights that make faults show.

The configurations differ from one another in every size and option: width, vocabulary, the number of
residual streams (one, two, three, four, or the key absent), the order of the two layer types, head counts and
groups (kv heads fewer than heads, one, as many), key size against value size (larger, smaller, equal, no
multiple of sixteen), rotated dimensions fewer than the head's or all of it, frequencies as they are, divided or
stretched (borders inside and outside the range of pairs), convolutions of one to five taps or none, windows
smaller than a page, no multiple of one, or absent, kept first keys fewer than a page, more than one, more than
the window, or none, soft caps that bite and that do not, recurrent heads wider and narrower than their values,
one to all experts chosen, layers without a feed-forward, and layers that read the keys and values of the layer
just before them or of one far back.
"""

from __future__ import annotations

from pathlib import Path

import torch


def _left(heads, kv_heads, dim, vdim, scale, rot=None, conv=None, size=None, keep=0, softcap=None):
    spec = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        spec["rot"] = rot
    if conv is not None:
        spec["conv"] = conv
    if size is not None:
        spec["mask"] = {"size": size, "keep_first": keep}
    if softcap is not None:
        spec["softcap"] = softcap
    return spec


def _parallel(left, right, scales=(1.0, 1.0)):
    return {"type": "parallel", "mixer": {"left": left, "right": dict(zip(("heads", "dim", "vdim"), right)),
                                          "left_scale": scales[0], "right_scale": scales[1]}}


def _attention(heads, kv_heads, dim, vdim, scale, rot=None, kv_from=None):
    spec = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        spec["rot"] = rot
    if kv_from is not None:
        spec["kv_from"] = kv_from
    return {"type": "attention", "mixer": spec}


def _with(layer, experts=None, top=1, ff=8):
    return dict(layer, mlp=None if experts is None else {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}})


def _yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


ATT_B = dict(heads=6, kv_heads=3, dim=16, vdim=32, scale=0.3, rot={"dims": 16, "base": 50.0, "scaling": _yarn(4.0, 64, 8.0, 1.0)})
ATT_C = dict(heads=2, kv_heads=1, dim=24, vdim=8, scale=0.25, rot={"dims": 6, "base": 1000.0, "scaling": {"factor": 2.0}})

SETOTAR = {
    # two streams, both layer types, a window of 21 with 3 kept keys, kv shared two layers back
    "A": {"architecture": "Setotar", "width": 48, "vocab": 211, "norm": {"eps": 1e-5}, "streams": 2, "layers": [
        _with(_parallel(_left(4, 2, 16, 8, 0.3, {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0}}, conv=4, size=21, keep=3, softcap=5.0),
                        (3, 8, 16), (1.2, 0.9)), experts=4, top=1, ff=8),
        _with(_attention(4, 2, 16, 16, 0.25, {"dims": 8, "base": 200.0, "scaling": _yarn(8.0, 32, 4.0, 0.5)}), experts=4, top=2, ff=12),
        _with(_parallel(_left(2, 1, 32, 32, 0.2, {"dims": 32, "base": 30.0}, conv=2, size=130, keep=20, softcap=30.0),
                        (2, 16, 8), (0.7, 1.4))),
        _with(_attention(4, 2, 16, 16, 0.25, {"dims": 8, "base": 200.0, "scaling": _yarn(8.0, 32, 4.0, 0.5)}, kv_from=1), experts=3, top=3, ff=4),
    ]},
    # three streams; attention layers first; keep_first larger than the window; one kv head for every head; no cap
    "B": {"architecture": "Setotar", "width": 96, "vocab": 173, "norm": {"eps": 1e-6}, "streams": 3, "layers": [
        _with(_attention(**ATT_B), experts=5, top=2, ff=16),
        _with(_attention(**ATT_B, kv_from=0)),
        _with(_parallel(_left(3, 3, 8, 24, 0.5, None, conv=5, size=5, keep=9), (1, 40, 8), (1.0, 1.0)), experts=2, top=1, ff=20),
        _with(_attention(**ATT_B, kv_from=0), experts=6, top=1, ff=8),
        _with(_parallel(_left(2, 2, 40, 40, 0.15, {"dims": 10, "base": 10.0}, conv=1, size=64, keep=16, softcap=2.0), (4, 4, 4), (0.5, 2.0))),
    ]},
    # no `streams` key: one residual with the layer scale; no convolution, no window; a stretch whose borders fall outside
    "C": {"architecture": "Setotar", "width": 40, "vocab": 331, "norm": {"eps": 1e-5}, "layers": [
        _with(_parallel(_left(2, 1, 16, 16, 0.3, {"dims": 4, "base": 20.0}, softcap=8.0), (2, 8, 8), (1.0, 1.0)), experts=3, top=1, ff=8),
        _with(_attention(**ATT_C), experts=2, top=2, ff=10),
        _with(_attention(**ATT_C, kv_from=1)),
    ]},
    # four streams, one of them parallel layers only in a row; a window of one key with one kept; wide recurrent heads
    "D": {"architecture": "Setotar", "width": 64, "vocab": 97, "norm": {"eps": 1e-6}, "streams": 4, "layers": [
        _with(_parallel(_left(4, 1, 16, 16, 0.4, {"dims": 16, "base": 500.0, "scaling": {"factor": 1.5}}, conv=3, size=1, keep=1, softcap=4.0),
                        (1, 72, 24), (1.0, 0.5)), experts=4, top=3, ff=6),
        _with(_parallel(_left(8, 4, 8, 16, 0.35, {"dims": 2, "base": 4.0}, conv=2, size=33, keep=17), (2, 8, 72), (2.0, 1.0)), experts=8, top=1, ff=4),
        _with(_attention(8, 8, 8, 8, 0.5, {"dims": 8, "base": 77.0})),
    ]},
    # one stream, learned connections all the same
    "E": {"architecture": "Setotar", "width": 32, "vocab": 61, "norm": {"eps": 1e-5}, "streams": 1, "layers": [
        _with(_parallel(_left(2, 2, 16, 16, 0.3, {"dims": 8, "base": 100.0}, conv=4, size=40, keep=2, softcap=10.0), (2, 8, 8), (1.0, 1.0)), experts=2, top=1, ff=8),
        _with(_attention(2, 1, 16, 16, 0.25, {"dims": 16, "base": 100.0}), experts=2, top=1, ff=8),
    ]},
}
SETOTAR_SEEDS = {"A": 41, "B": 42, "C": 43, "D": 44, "E": 45, "M": 46, "N": 47}

_STRETCH_M = {"dims": 32, "base": 10000.0, "scaling": _yarn(4.0, 256, 16.0, 1.0)}
_STRETCH_N = {"dims": 32, "base": 30000.0, "scaling": _yarn(6.0, 1024, 16.0, 2.0)}
# heads of 64 and 128, the sizes the tcgen05 kernels serve, at widths of a few hundred: prompts of several hundred
# tokens run through those kernels, the kept keys' split, the runs of the recurrence and the clusters of the norm
MEDIUM = {
    "M": {"architecture": "Setotar", "width": 320, "vocab": 1000, "norm": {"eps": 1e-6}, "streams": 3, "layers": [
        _with(_attention(5, 5, 64, 64, 0.125, _STRETCH_M), experts=4, top=2, ff=96),
        _with(_parallel(_left(6, 2, 64, 64, 0.125, {"dims": 64, "base": 5000.0, "scaling": {"factor": 2.0}}, conv=3, size=200, keep=7, softcap=15.0),
                        (2, 64, 32), (1.1, 0.8)), experts=6, top=1, ff=48),
        _with(_attention(5, 5, 64, 64, 0.125, _STRETCH_M, kv_from=0)),
        _with(_parallel(_left(2, 2, 128, 128, 0.09, {"dims": 32, "base": 100.0}, conv=5, size=64, keep=33), (3, 32, 96), (0.5, 1.5)), experts=3, top=3, ff=64),
        _with(_attention(3, 1, 128, 64, 0.1, {"dims": 128, "base": 300.0}), experts=2, top=1, ff=200),
    ]},
    "N": {"architecture": "Setotar", "width": 192, "vocab": 777, "norm": {"eps": 1e-5}, "streams": 2, "layers": [
        _with(_parallel(_left(8, 2, 128, 48, 0.09, {"dims": 64, "base": 30000.0, "scaling": {"factor": 6.0}}, conv=6, size=150, keep=6, softcap=25.0),
                        (4, 48, 64), (1.3, 0.7)), experts=8, top=1, ff=64),
        _with(_parallel(_left(4, 4, 64, 128, 0.12, None, conv=2, size=300, keep=0, softcap=50.0), (1, 200, 40), (1.0, 1.0)), experts=8, top=3, ff=40),
        _with(_attention(4, 2, 64, 64, 0.19, _STRETCH_N), experts=5, top=1, ff=64),
        _with(_attention(4, 2, 64, 64, 0.19, _STRETCH_N, kv_from=2), experts=5, top=1, ff=64),
    ]},
}
SETOTAR.update(MEDIUM)


def sharpened(tensors: dict) -> dict:
    """Random weights as `random_init` makes them, scaled so that faults show: projections large enough for
    softmax rows with a few large entries, gates that open and close, states that matter, routers that decide,
    connections that mix the streams."""
    out = {}
    for name, t in tensors.items():
        t = t.clone()
        last = name.rsplit(".", 1)[-1]
        if ".mix." in name and last in ("q", "k", "v", "f") and t.dim() == 2:
            t *= 12.0
        elif ".mix." in name and last == "o":
            t *= 6.0
        elif ".mlp." in name and last in ("gate", "up", "down"):
            t *= 10.0
        elif last == "router":
            t *= 30.0
        elif name.endswith((".q.b", ".k.b", ".v.b", ".f.b")):
            t *= 20.0
        elif name == "embed":
            t *= 25.0
        elif name.endswith((".hc1.mix", ".hc2.mix")):
            t = t + 0.3 * torch.ones_like(t)
        out[name] = t
    return out


def make_setotar_folder(tmp_path, key: str, dtype: str = "float32", raw: dict | None = None, seed: int | None = None,
                        change=None) -> Path:
    """A model folder (config.json, model.safetensors) of a tiny configuration with sharpened weights.  `change`
    (name -> tensor dictionary, edited in place) lets a test plant a weight of its own."""
    import json

    from shrike_b200 import models  # noqa: F401
    from shrike_b200.config.registry import parse_config
    from shrike_b200.weights.random_init import random_tensors
    from shrike_b200.weights.safetensors_io import write_safetensors

    raw = dict(raw if raw is not None else SETOTAR[key])
    seed = SETOTAR_SEEDS.get(key, 0) if seed is None else seed
    out = Path(tmp_path) / f"setotar_{key}_{dtype}"
    out.mkdir(parents=True, exist_ok=True)
    config = parse_config(raw)
    tensors = sharpened(random_tensors(config, seed, "cpu", torch.float32))
    if change is not None:
        change(tensors)
    tensors = {name: t.to(getattr(torch, dtype)) for name, t in tensors.items()}
    (out / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    write_safetensors(out / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return out


MARK, ASKER = 3, 4   # token ids of `planted_pair`


def planted_pair(raw: dict, strength: float = 2.0, gain: float = 12.0):
    """A `change` for `make_setotar_folder` on a model whose layer 0 is an attention layer or a parallel layer: the
    score between a query of token ASKER and a key of token MARK stands far above every other score, in every head,
    so that whether MARK is seen from ASKER's position decides ASKER's logits however many keys lie between.  In a
    parallel layer the pair is planted in the `left` mixer (its convolutions are made to pass the newest value alone,
    so that a token reaches its neighbours through the window only) and the `right` mixer is silenced.

    Residual axis 0 is nonzero in MARK's embedding only and axis 1 in ASKER's only; one unrotated key dimension reads
    axis 0 alone and the same query dimension reads axis 1 alone."""
    layer = raw["layers"][0]
    parallel = layer["type"] == "parallel"
    spec = layer["mixer"]["left"] if parallel else layer["mixer"]
    prefix = "l0.mix.left." if parallel else "l0.mix."

    def change(tensors):
        embed = tensors["embed"]
        embed[:, 0:2] = 0.0
        embed[MARK, 0] = strength
        embed[ASKER, 1] = strength
        tensors["l0.norm1"][0:2] = 1.0
        tensors[prefix + "o"] *= 4.0
        heads, dim = spec["heads"], spec["dim"]
        at = dim - 1                             # the head's last dimension
        if spec.get("rot") and spec["rot"]["dims"] > at:
            raise ValueError("the planted dimension must lie outside the rotated ones")
        for g in range(spec["kv_heads"]):
            tensors[prefix + "k"][g * dim + at] = 0.0
            tensors[prefix + "k"][g * dim + at, 0] = gain
        for a in range(heads):
            tensors[prefix + "q"][a * dim + at] = 0.0
            tensors[prefix + "q"][a * dim + at, 1] = gain
        if parallel:
            for name in ("q", "k"):
                tensors[f"{prefix}{name}.b"].view(-1, dim)[:, at] = 0.0
            if spec.get("conv"):
                for name in ("q", "k", "v"):   # a token's neighbours reach it through the window alone
                    tensors[f"{prefix}{name}.conv"][:, :-1] = 0.0
                    tensors[f"{prefix}{name}.conv"][:, -1] = 1.0
            tensors["l0.mix.right.o"] *= 0.0
        else:
            for name in ("q", "k"):   # the norm over the whole projection leaves the planted dimension its size
                tensors[f"{prefix}{name}.norm"].view(-1, dim)[:, at] = 3.0

    return change
