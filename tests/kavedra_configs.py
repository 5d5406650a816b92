"""Tiny Kavedra configurations for tests, and model folders with weights that make faults show.

The configurations differ from one another in every size and option: width, vocabulary, the order of
the three mixers, head counts and groups (kv heads fewer than heads, one, as many), key size against
value size (larger, smaller, equal), rotated dimensions fewer than the head's or all of it, with and
without stretched frequencies (borders inside and outside the range of pairs), windows that are no
multiple of a page, smaller than a page, or absent, decays of 1 and far below, layers without a
feed-forward, a logit scale of 1 and another, and the repeated layers at the start, in the middle, at
the end, once, or not at all.
"""

from __future__ import annotations

from pathlib import Path

import torch


def _attention(heads, kv_heads, dim, vdim, scale, rot):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "rot": {"dims": rot[0], "base": rot[1]}}}


def _lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base, window=None, scaling=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer}


def _with(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


# latent first, then lightning, then attention; the repeated layers at the end, three passes; values wider than keys in
# the attention, narrower in the latent; a window that no page size divides; a rotation of part of the head; a layer
# without a feed-forward; a decay of exactly 1
KAVEDRA_A = {
    "architecture": "Kavedra", "width": 96, "vocab": 211, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _with(_latent(3, 24, 8, 16, 40, 0.21, 10000.0, window=21, scaling=(4.0, 64, 8.0, 2.0)), 80),
        _with(_lightning(3, 16, 24, (0.5, 1.0, 0.93)), None),
        _with(_attention(6, 2, 16, 32, 0.3, (8, 1000.0)), 64),
    ],
}

# heads of 64 (the sizes the tensor-core kernels take): attention with one kv head and the whole head rotated, a latent of
# rank 48 + 16 rotated = 64 without a window and without stretched frequencies; no repeated layers; logit scale 1 (absent)
KAVEDRA_B = {
    "architecture": "Kavedra", "width": 128, "vocab": 300, "norm": {"eps": 1e-6},
    "layers": [
        _with(_attention(2, 1, 64, 64, 0.12, (64, 400000.0)), 192),
        _with(_latent(2, 32, 16, 64, 48, 0.15, 100.0), 96),
        _with(_lightning(1, 64, 64, (0.97,)), 160),
        _with(_attention(4, 4, 64, 32, 0.1, (32, 100.0)), None),
    ],
}

# a window of one key and one smaller than a page; one pass "repeated" once at the very start; as many kv heads as heads;
# two rotated dimensions; lightning heads of 40 by 8 and 8 by 40; a quick decay; stretched frequencies whose borders lie
# outside the pairs on both sides
KAVEDRA_C = {
    "architecture": "Kavedra", "width": 72, "vocab": 97, "norm": {"eps": 1e-5}, "logit_scale": 3.0,
    "loop": {"start": 0, "stop": 1, "times": 1},
    "layers": [
        _with(_lightning(2, 40, 8, (0.3, 0.8)), 40),
        _with(_latent(2, 8, 2, 24, 12, 0.4, 10.0, window=1, scaling=(2.0, 4, 1000.0, 0.0001)), None),
        _with(_attention(3, 3, 16, 16, 0.25, (2, 10.0)), 48),
        _with(_latent(1, 16, 4, 8, 20, 0.3, 50.0, window=5, scaling=(16.0, 32, 4.0, 1.0)), 24),
        _with(_lightning(3, 8, 40, (0.9, 0.99, 0.6)), None),
    ],
}

# heads of 128 and a latent whose page row is 128 wide; the repeated layers in the middle, three passes, holding all
# three mixers; a long window
KAVEDRA_D = {
    "architecture": "Kavedra", "width": 64, "vocab": 151, "norm": {"eps": 1e-6}, "logit_scale": 1.5,
    "loop": {"start": 1, "stop": 4, "times": 3},
    "layers": [
        _with(_lightning(2, 16, 16, (0.9995, 0.7)), 96),
        _with(_attention(2, 1, 128, 128, 0.09, (64, 10000.0)), 32),
        _with(_latent(2, 64, 16, 32, 112, 0.1, 30000.0, window=130, scaling=(8.0, 128, 16.0, 1.0)), 48),
        _with(_lightning(1, 48, 32, (0.95,)), None),
        _with(_attention(4, 2, 32, 16, 0.2, (32, 300.0)), 40),
    ],
}

KAVEDRA = {"A": KAVEDRA_A, "B": KAVEDRA_B, "C": KAVEDRA_C, "D": KAVEDRA_D}
KAVEDRA_SEEDS = {"A": 31, "B": 32, "C": 33, "D": 34}


def sharpened(tensors: dict) -> dict:
    """Random weights leave every attention nearly uniform and every gate at a half, which hides a key that is wrongly
    seen, a sink that is left out or a state that was lost.  This scales what sets the size of the scores (query
    and key projections and their biases), of the gates and of the pass vectors, spreads the sinks and the norms'
    weights, and makes the linear attention's keys and values large enough for its state to matter."""
    out = {}
    for name, tensor in tensors.items():
        t = tensor.clone()
        if name.endswith((".mix.q", ".mix.k", ".mix.dkv", ".mix.uk")):
            t *= 6.0
        elif name.endswith((".mix.q.b", ".mix.k.b", ".mix.v.b")):
            t *= 15.0
        elif name.endswith(".mix.g"):
            t *= 30.0
        elif name.endswith(".mix.sink"):
            t *= 2.0
        elif name.endswith((".mix.v", ".mix.uv")):
            t *= 3.0
        elif name == "loop.step":
            t *= 10.0
        elif name.endswith((".norm1", ".norm2")) or name == "final.norm":
            t *= 3.0
        out[name] = t
    return out


def make_kavedra_folder(tmp_path, key: str, dtype: str = "float32", raw: dict | None = None, seed: int | None = None,
                        change=None) -> Path:
    """A model folder (config.json, model.safetensors) of a tiny configuration with sharpened weights.  `change`
    (name -> tensor dictionary, edited in place) lets a test plant a weight of its own."""
    import json

    from shrike_b200 import models  # noqa: F401
    from shrike_b200.config.registry import parse_config
    from shrike_b200.weights.random_init import random_tensors
    from shrike_b200.weights.safetensors_io import write_safetensors

    raw = dict(raw if raw is not None else KAVEDRA[key])
    seed = KAVEDRA_SEEDS.get(key, 0) if seed is None else seed
    out = Path(tmp_path) / f"kavedra_{key}_{dtype}"
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
    """A `change` for `make_kavedra_folder` on a model whose layer 0 is an attention or a latent attention: the
    score between a query of token ASKER and a key of token MARK stands far above every other score, in every
    head, so that whether MARK is seen from ASKER's position decides ASKER's logits however many keys lie between.
    On a linear attention the same pair makes MARK's value stand out in what ASKER reads from the state.

    Residual axis 0 is nonzero in MARK's embedding only and axis 1 in ASKER's only; one unrotated key dimension
    reads axis 0 alone and the same query dimension reads axis 1 alone.  The output projection is made larger so that
    what the heads attend to is a good part of the residual."""
    layer = raw["layers"][0]
    spec = layer["mixer"]

    def change(tensors):
        embed = tensors["embed"]
        embed[:, 0:2] = 0.0
        embed[MARK, 0] = strength
        embed[ASKER, 1] = strength
        tensors["l0.norm1"][0:2] = 0.0
        tensors["l0.mix.o"] *= 4.0
        heads, dim = spec["heads"], spec["dim"]
        if layer["type"] == "latent_attention":
            per_head = dim + spec["rot_dim"]
            tensors["l0.mix.dkv"][0] = 0.0
            tensors["l0.mix.dkv"][0, 0] = gain       # latent component 0 is MARK's alone
            tensors["l0.mix.dkv.norm"][0] = 1.0
            for a in range(heads):
                tensors["l0.mix.uk"][a * dim] = 0.0
                tensors["l0.mix.uk"][a * dim, 0] = 4.0
                tensors["l0.mix.q"][a * per_head] = 0.0
                tensors["l0.mix.q"][a * per_head, 1] = gain
        elif layer["type"] == "attention":
            at = dim - 1                             # the head's last dimension
            if spec["rot"]["dims"] > at:
                raise ValueError("the planted dimension must lie outside the rotated ones")
            for g in range(spec["kv_heads"]):
                tensors["l0.mix.k"][g * dim + at] = 0.0
                tensors["l0.mix.k"][g * dim + at, 0] = gain
                tensors["l0.mix.k.b"][g * dim + at] = 0.0
            for a in range(heads):
                tensors["l0.mix.q"][a * dim + at] = 0.0
                tensors["l0.mix.q"][a * dim + at, 1] = gain
                tensors["l0.mix.q.b"][a * dim + at] = 0.0
        elif layer["type"] == "lightning":
            # key dimension 0 of every head is large for MARK alone, query dimension 0 for ASKER alone: what ASKER reads
            # from the state's row 0 is MARK's value, times the head's decay to the power of the distance
            for a in range(heads):
                tensors["l0.mix.k"][a * dim] = 0.0
                tensors["l0.mix.k"][a * dim, 0] = gain
                tensors["l0.mix.q"][a * dim] = 0.0
                tensors["l0.mix.q"][a * dim, 1] = gain
        else:
            raise ValueError(layer["type"])

    return change
