"""Norms over the model width.  RMSNorm: y = x * w / sqrt(mean(x^2) + eps), all in float32
(crates/bitnet-core/src/llama/model.rs:93-100).  The weight multiplies directly (no 1+w).
``groups`` > 1: the row is cut into that many equal consecutive parts, each divided by its own root mean
square; the weight still spans the whole row.  ``one_plus``: the stored weight lies around zero and multiplies as
1 + w.  ``layer_scale``: a second stored vector ("scale") multiplies the normed row value by value; the two are kept
as one float32 vector.  ``add_to`` is the norm on a sublayer's RESULT: x += norm(y).
LayerNorm: the mean taken off first, and a bias added."""
from __future__ import annotations

import torch

from .base import Norm
from .registry import register_part


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, groups: int = 1, one_plus: bool = False, layer_scale: bool = False):
        self.width, self.eps, self.groups = int(width), float(eps), int(groups)
        self.one_plus, self.layer_scale = bool(one_plus), bool(layer_scale)
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"rmsnorm: a row of {self.width} values is not {self.groups} equal parts")
        self.weight = None

    def weight_shapes(self):
        shapes = {"weight": ((self.width,), "matrix" if self.one_plus else "norm")}
        if self.layer_scale:
            shapes["scale"] = ((self.width,), "norm")
        return shapes

    def bind(self, weights, ops):
        # exact in float32 whatever the stored dtype
        w = weights["weight"].to(torch.float32)
        if self.one_plus:
            w = 1.0 + w
        if self.layer_scale:
            w = w * weights["scale"].to(torch.float32)
        self.weight = w.contiguous()

    def add_to(self, ctx, x, y, want_rounded: bool = False):
        """x (float32 [T, E], the residual stream) += y / rms(y) * weight, y the float32 result of a sublayer; with
        ``want_rounded`` the new rows are also returned in the compute dtype (what the next sublayer reads)."""
        if self.groups != 1:
            raise ValueError("rmsnorm: a norm in groups on a sublayer's result is not built")
        return ctx.ops.norm_add(x, y, self.weight, self.eps, want_rounded=want_rounded)

    def forward(self, ctx, x, out_dtype=None):
        kw = {} if out_dtype is None else {"out_dtype": out_dtype}
        if self.groups > 1:
            return ctx.ops.rmsnorm_grouped(x, self.weight, self.groups, self.eps, **kw)
        return ctx.ops.rmsnorm(x, self.weight, self.eps, **kw)

    def deferred(self, ops):
        """What a product before this norm needs to prepare it, if the operations can fold a norm
        into the products around it (see ``PreNormBlock``); else None."""
        make = getattr(ops, "norm_request", None)
        return make(self.weight, self.eps) if make is not None and self.groups == 1 else None



class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w + b over the width, var the mean of the squared deviations; all in
    float32.  Weights "weight" and "bias" (``bias=False``: none)."""

    def __init__(self, width: int, eps: float, bias: bool = True):
        self.width, self.eps, self.has_bias = int(width), float(eps), bool(bias)
        self.weight = self.bias = None

    def weight_shapes(self):
        shapes = {"weight": ((self.width,), "norm")}
        if self.has_bias:
            shapes["bias"] = ((self.width,), "matrix")
        return shapes

    def bind(self, weights, ops):
        self.weight = weights["weight"].to(torch.float32).contiguous()
        self.bias = weights["bias"].to(torch.float32).contiguous() if self.has_bias else None

    def forward(self, ctx, x):
        return ctx.ops.layernorm(x, self.weight, self.bias, self.eps)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
