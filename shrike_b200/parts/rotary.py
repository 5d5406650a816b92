"""Rotary position encoding, rotate-half pairing (j with j + D/2).

inv_freq[j] = 1 / theta^(2j/D) evaluated in float32 exactly as
shrike/models/qwen.py:80 does; the angle is float32(position) * inv_freq[j]
(qwen.py:86) and q' = q cos + rotate_half(q) sin in float32 with one rounding
(qwen.py:91-101).  The table of inverse frequencies is all the fused
rotate-and-store kernel needs, so that is what this part hands to a mixer.
"""

from __future__ import annotations

import torch

from .base import register_part


class Rotary:
    @staticmethod
    def parameters(spec) -> dict:
        return {}

    def __init__(self, spec, tensors, ops, runtime):
        if spec.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {spec.head_dim}")
        self.spec = spec
        exponent = torch.arange(0, spec.head_dim, 2).float() / spec.head_dim
        self.inv_freq = (1.0 / (spec.theta ** exponent)).to(runtime.device)

    def rotary_table(self) -> torch.Tensor:
        return self.inv_freq


register_part("position", "rotary", Rotary)


class PairRotation:
    """What a mixer needs of a `PairRotationSpec` to run it on kernels that pair dimension i with
    i + dims/2 and know nothing of stretches: the table of angles per position, and two changes to
    the ROWS of the projection whose output is rotated, made once when the weights are loaded.

    `order`: old index of each new row inside the rotated dimensions.  With neighbours paired, the
    rows are put as [0, 2, 4, ..., 1, 3, 5, ...], after which pair i sits at (i, i + dims/2); a dot
    product of two vectors reordered alike is unchanged, so queries and keys are both reordered and
    nothing else is.  `gain`: the factor on cos and sin; a rotation is linear, so the rows are
    multiplied by it instead.  Frequencies are formed in float64 and rounded once.
    """

    def __init__(self, spec, device):
        import math

        self.spec = spec
        dims, base = spec.dims, float(spec.base)
        freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        self.gain = 1.0
        if spec.stretch is not None:
            factor, original, fast, slow = (float(v) for v in spec.stretch)

            def border(turns):
                return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

            lo = max(math.floor(border(fast)), 0)
            hi = min(math.ceil(border(slow)), dims - 1)
            for i in range(dims // 2):
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                freq[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp)
            self.gain = 0.1 * math.log(factor) + 1.0
        if getattr(spec, "divide", None) is not None:   # linear scaling: every frequency over one number
            freq = [f / float(spec.divide) for f in freq]
        self.inv_freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(device)
        self.order = list(range(dims))
        if spec.pairing == "neighbours":
            self.order = list(range(0, dims, 2)) + list(range(1, dims, 2))

    def arrange_rows(self, rows: torch.Tensor, heads: int, head_size: int, first: int = 0,
                     fold_gain: bool = True) -> torch.Tensor:
        """`rows` [heads * head_size, ...] (a weight or a bias): inside every head, the `dims` rows from
        `first` on are reordered and scaled as the class comment says; the others stay.  `fold_gain`
        False leaves the scaling to a kernel that takes the gain itself."""
        dims = self.spec.dims
        gain = self.gain if fold_gain else 1.0
        if gain == 1.0 and self.order == list(range(dims)):
            return rows
        shaped = rows.reshape(heads, head_size, *rows.shape[1:]).clone()
        index = torch.tensor(self.order, device=rows.device) + first
        turned = shaped[:, index]
        if gain != 1.0:
            turned = (turned.to(torch.float32) * gain).to(rows.dtype)
        shaped[:, first:first + dims] = turned
        return shaped.reshape(rows.shape)
