"""Norms, fused with the residual sum: RMS norm and layer norm.

y = x * rsqrt(mean(x^2) + eps) * w with a plain weight, all in 32-bit, one
rounding at the end (shrike/models/qwen.py:64-74).  The residual stream is kept in
float32; `add_norm` first adds the pending branch output to it, so the sum that
Azimml/shrike does in the model dtype (qwen.py:148-149) is a 32-bit sum here and
costs no pass of its own.

Two ways of sitting in a layer.  Before a branch (`add_norm`): the pending branch output is added to
the residual and the sum is normed.  On a branch's output (`norm_add`): the branch output is normed
and THAT is added to the residual, x += norm(branch(x)); what the next branch reads is then the
residual itself, which `norm_add` returns in the activation type.  `LayerNorm` is
(x - mean) / sqrt(var + eps) * w + b with the variance as the mean squared deviation, in 32-bit.
"""

from __future__ import annotations

import torch

from .base import ParamSpec, PendingSum, register_part


class RMSNorm:
    capture_safe = True   # forward() launches the same kernels for the same batch shape, whatever the positions

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.width,), "around_zero" if getattr(spec, "offset", 0.0) else "norm")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec = spec
        self.ops = ops
        self.runtime = runtime
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        offset = float(getattr(spec, "offset", 0.0))
        if offset:   # the file holds the weight's distance from `offset`: the sum is formed once, in 32-bit
            self.weight = (self.weight + offset).contiguous()

    def add_norm(self, resid, delta, out_name="normed"):
        out = self.runtime.buffer(out_name, (resid.shape[0], self.spec.width), self.runtime.act_dtype)
        self.ops.add_rmsnorm(resid, delta, self.weight, self.spec.eps, out)
        return out

    def gather_norm(self, resid, delta, rows, out_name="normed_rows"):
        out = self.runtime.buffer(out_name, (rows.shape[0], self.spec.width), self.runtime.act_dtype)
        self.ops.gather_add_rmsnorm(resid, delta, rows, self.weight, self.spec.eps, out)
        return out


    def norm_add(self, resid, branch, out_name="hidden"):
        """resid += norm(branch) in 32-bit; returns the new residual in the activation type."""
        return _norm_add(self, resid, branch, None, False, out_name)


def _norm_add(norm, resid, branch, bias, layer_norm, out_name):
    rt = norm.runtime
    # a 32-bit engine reads the residual itself; a 16-bit one gets a rounded copy from the same kernel
    out = None if rt.act_dtype == torch.float32 else rt.buffer(out_name, tuple(resid.shape), rt.act_dtype)
    if branch is not None or out is not None:
        norm.ops.norm_add(resid, branch, norm.weight, bias, norm.spec.eps, out, layer_norm=layer_norm)
    return resid if out is None else out


class LayerNorm:
    capture_safe = True

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        params = {"weight": ParamSpec((spec.width,), "norm")}
        if spec.bias:
            params["bias"] = ParamSpec((spec.width,), "bias")
        return params

    def __init__(self, spec, tensors, ops, runtime):
        self.spec = spec
        self.ops = ops
        self.runtime = runtime
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self.bias = tensors["bias"].to(torch.float32).contiguous() if spec.bias else None

    def norm_add(self, resid, branch, out_name="hidden"):
        """resid += norm(branch) in 32-bit (`branch` None: nothing is added); returns the residual in
        the activation type."""
        return _norm_add(self, resid, branch, self.bias, True, out_name)

    def add_norm(self, resid, delta, out_name="normed"):
        if delta is not None:
            raise NotImplementedError("LayerNorm before a branch with a pending sum: no kernel adds and norms in one pass")
        out = self.runtime.buffer(out_name, tuple(resid.shape), self.runtime.act_dtype)
        rows = self.runtime.buffer("all_rows", (resid.shape[0],), torch.int32)
        torch.arange(resid.shape[0], dtype=torch.int32, device=resid.device, out=rows)
        self.ops.gather_norm(resid, rows, self.weight, self.bias, self.spec.eps, out, layer_norm=True)
        return out

    def gather_norm(self, resid, delta, rows, out_name="normed_rows"):
        if delta is not None:
            raise NotImplementedError("LayerNorm on gathered rows takes a residual with nothing pending")
        out = self.runtime.buffer(out_name, (rows.shape[0], self.spec.width), self.runtime.act_dtype)
        self.ops.gather_norm(resid, rows, self.weight, self.bias, self.spec.eps, out, layer_norm=True)
        return out


class DynamicTanh:
    """tanh(alpha x) * weight + bias with one learned number alpha: a norm that takes no mean and no
    variance, so it is elementwise and several of them can share one pass over a row.  The pending
    branch outputs (a tensor, a K-split stack, or a `PendingSum` of several with a scale each) are
    added to the float32 residual in the same kernel."""

    capture_safe = True
    MAX_TERMS = 4   # pending sums one launch of the kernel adds

    @staticmethod
    def parameters(spec) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.width,), "norm"), "bias": ParamSpec((spec.width,), "bias"),
                "alpha": ParamSpec((), "norm")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self.bias = tensors["bias"].to(torch.float32).contiguous()
        self.alpha = float(tensors["alpha"].to(torch.float32))   # a constant of the model, handed to the kernel by value

    def _flush(self, resid, delta) -> list:
        """The pending terms one launch can take; what is over is added to the residual first."""
        terms = PendingSum.of(delta)
        while len(terms) > self.MAX_TERMS:
            self.ops.tanh_norm(resid, terms[: self.MAX_TERMS])
            terms = terms[self.MAX_TERMS:]
        return terms

    def _triple(self, out):
        return (self.alpha, self.weight, self.bias, out)

    def add_norm(self, resid, delta, out_name="normed"):
        out = self.runtime.buffer(out_name, (resid.shape[0], self.spec.width), self.runtime.act_dtype)
        self.ops.tanh_norm(resid, self._flush(resid, delta), norms=[self._triple(out)])
        return out

    def add_norm_pair(self, resid, delta, other, out_names=("normed", "normed_b")):
        """This norm and `other` (of the same kind) of the same summed row, from one pass over it."""
        if not isinstance(other, DynamicTanh):
            return self.add_norm(resid, delta, out_names[0]), other.add_norm(resid, None, out_names[1])
        shape = (resid.shape[0], self.spec.width)
        first = self.runtime.buffer(out_names[0], shape, self.runtime.act_dtype)
        second = self.runtime.buffer(out_names[1], shape, self.runtime.act_dtype)
        self.ops.tanh_norm(resid, self._flush(resid, delta), norms=[self._triple(first), other._triple(second)])
        return first, second

    def gather_norm(self, resid, delta, rows, out_name="normed_rows"):
        out = self.runtime.buffer(out_name, (rows.shape[0], self.spec.width), self.runtime.act_dtype)
        terms = PendingSum.of(delta)
        if len(terms) > self.MAX_TERMS:
            terms = self._flush(resid, delta)
        self.ops.tanh_norm(resid, terms, rows=rows, norms=[self._triple(out)])
        return out


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
register_part("norm", "layernorm", LayerNorm)
