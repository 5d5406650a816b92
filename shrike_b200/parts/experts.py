"""A mixture of gated feed-forward experts with a softmax (or sigmoid) router, and a shared expert beside them.

Router logits are formed in 32-bit; scores are the softmax over ALL experts; the `top` largest are
chosen and their scores divided by their sum (+ a tiny constant); the output is the weighted sum of
the chosen experts' down(act(gate x) * (up x)).  A shared expert, when the spec has one, runs for
every token and is added, times sigmoid(w_sg . x) when it is gated.

How it runs here: every expert's gate and up rows are stacked into one matrix (the shared expert's
last), so one product gives every expert's gate and up columns for every token; the activation
kernel multiplies each column by its expert's weight for that token, which is exactly 0 for an
expert the token did not choose; one product with the stacked down matrices then IS the weighted
sum.  Nothing depends on which experts the tokens chose, so a step's launches are the same for
every batch of a shape and can be replayed.  Options of the spec: `scoring` "sigmoid" (an expert's score
is the sigmoid of its own logit), `renormalise` False (the chosen keep their scores), `weight_on` "input" (an expert
runs on weight * x: gate and up are linear in x, so the activation kernel forms act(w gate) * (w up) from the same
product).  The price is arithmetic: every expert's columns are
computed for every token, experts / top times what the chosen ones alone would take; in decoding,
where the experts' weights are read once whatever the routing, it costs nothing.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, register_part


class RoutedExperts:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        params = {"router.weight": ParamSpec((spec.experts, spec.width), "matrix")}
        sizes = [(f"experts.{e}", spec.intermediate) for e in range(spec.experts)]
        if spec.shared_intermediate is not None:
            sizes.append(("shared", spec.shared_intermediate))
            if spec.shared_gate:
                params["shared_gate.weight"] = ParamSpec((1, spec.width), "matrix")
        for prefix, size in sizes:
            params[f"{prefix}.gate_proj.weight"] = ParamSpec((size, spec.width), "matrix")
            params[f"{prefix}.up_proj.weight"] = ParamSpec((size, spec.width), "matrix")
            params[f"{prefix}.down_proj.weight"] = ParamSpec((spec.width, size), "matrix")
        return params

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        names = [f"experts.{e}" for e in range(spec.experts)]
        if spec.shared_intermediate is not None:
            names.append("shared")
        self.router = tensors.pop("router.weight").to(torch.float32).contiguous()   # the router works in 32-bit
        self.shared_gate = None
        if spec.shared_intermediate is not None and spec.shared_gate:
            self.shared_gate = tensors.pop("shared_gate.weight").to(torch.float32).reshape(-1).contiguous()
        gates = [tensors.pop(f"{name}.gate_proj.weight") for name in names]
        ups = [tensors.pop(f"{name}.up_proj.weight") for name in names]
        self.w_gate_up = torch.cat(gates + ups).contiguous()                      # [2 I, W]: all gate rows, then all up rows
        self.w_down = torch.cat([tensors.pop(f"{name}.down_proj.weight") for name in names], dim=1).contiguous()   # [W, I]
        self.inter = self.w_down.shape[1]
        self.columns = spec.experts + (1 if spec.shared_intermediate is not None else 0)

    def forward(self, x, ctx):
        spec, rt, ops = self.spec, self.runtime, self.ops
        n = x.shape[0]
        share = rt.buffer("expert_share", (n, self.columns), torch.float32)
        ops.route_top(x, self.router, self.shared_gate, share, spec.top, spec.renorm_eps,
                      **({"scoring": spec.scoring} if getattr(spec, "scoring", "softmax") != "softmax" else {}),
                      **({"renormalise": False} if not getattr(spec, "renormalise", True) else {}))
        gate_up = rt.buffer("experts_gate_up", (n, 2 * self.inter), rt.act_dtype)
        ops.linear(x, self.w_gate_up, gate_up)
        act = rt.buffer("experts_act", (n, self.inter), rt.act_dtype)
        ops.act_mul_blocks(gate_up, share, act, spec.experts, spec.intermediate, spec.activation,
                           **({"weight_on": "input"} if getattr(spec, "weight_on", "output") == "input" else {}))
        delta = rt.buffer("ffn_delta", (n, spec.width), torch.float32)
        return ops.linear(act, self.w_down, delta, allow_partials=True)


register_part("feed_forward", "routed_experts", RoutedExperts)
