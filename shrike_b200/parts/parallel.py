"""Several mixers side by side: each reads the same input, their outputs are added with a scale each.

A branch is any registered mixer; its tensors are named `<branch>.<the mixer's own names>`.  The
branches' outputs are not added here: they go on as a `PendingSum`, and the next norm kernel adds
them to the residual, scales included.  One run of the layer has one cache id; a branch that keeps
keys and values and a branch that keeps state share it (pages under it for the one, a state slot
for the other), so at most one branch of each sort.
"""

from __future__ import annotations

from .base import KVNeed, ParamSpec, PendingSum, StateNeed, part_class, register_part


class ParallelMixer:
    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        params = {}
        for name, branch, _scale in spec.branches:
            for local, param in part_class("mixer", branch.kind).parameters(branch).items():
                params[f"{name}.{local}"] = param
        return params

    @staticmethod
    def cache_needs(spec) -> list:
        needs = []
        for name, branch, _scale in spec.branches:
            needs += part_class("mixer", branch.kind).cache_needs(branch)
        names = [need.name for need in needs if isinstance(need, StateNeed)]
        if sum(isinstance(need, KVNeed) for need in needs) > 1 or len(set(names)) != len(names):
            raise ValueError("a parallel mixer holds at most one branch with pages and one state of each name")
        return needs

    def __init__(self, spec, tensors, ops, runtime):
        self.spec = spec
        self.branches = []
        for name, branch, scale in spec.branches:
            cls = part_class("mixer", branch.kind)
            own = {local: tensors[f"{name}.{local}"] for local in cls.parameters(branch)}
            self.branches.append((cls(branch, own, ops, runtime), float(scale)))
        self.capture_safe = all(getattr(part, "capture_safe", False) for part, _ in self.branches)

    def forward(self, x, ctx, run):
        terms = []
        for part, scale in self.branches:
            terms += PendingSum.of(part.forward(x, ctx, run), scale)
        return PendingSum(terms)


register_part("mixer", "parallel_mixer", ParallelMixer)
