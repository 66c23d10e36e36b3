"""What may stand around a sublayer of a block: a filter on what it reads, and a gate on what it adds.

``CausalTapsFilter`` ("input_filter", kind "causal_taps"): the sublayer reads h + conv(h) instead of h, where conv is
a causal convolution over time on every channel, conv(h)_t = sum_j taps[:, j] * h_(t - K + 1 + j) (the last tap is the
current row's; rows before a sequence's start count as zeros; no bias).  The last K - 1 rows h of a sequence are its
state: a ring of K rows by position, float32.

``SigmoidGate`` ("result_gate", kind "sigmoid_linear"): the sublayer's result y enters the residual stream as
x += y * sigmoid(W h + b), value by value, with h the sublayer's input rows before any filter.  The gate's sums, the
sigmoid and the addition are float32.
"""
from __future__ import annotations

import torch

from .base import InputFilter, ResultGate, TokenInput, StateNeed
from .registry import register_part


class CausalTapsFilter(InputFilter):
    def __init__(self, width: int, taps: int):
        self.width, self.taps = int(width), int(taps)
        if self.taps < 1:
            raise ValueError("input filter: at least one tap")
        self.w = None

    def weight_shapes(self):
        return {"taps": ((self.width, self.taps), "matrix")}

    def state_need(self):
        return StateNeed((self.taps, self.width)) if self.taps > 1 else None

    def bind(self, weights, ops):
        self.w = weights["taps"].to(device=ops.device, dtype=torch.float32).contiguous()

    def forward(self, ctx, h, state):
        return ctx.ops.input_filter(h, self.w, state, ctx.meta)


class SigmoidGate(ResultGate):
    def __init__(self, width: int, bias: bool = True):
        self.width, self.has_bias = int(width), bool(bias)
        self.w = self.b = None

    def weight_shapes(self):
        shapes = {"weight": ((self.width, self.width), "matrix")}
        if self.has_bias:
            shapes["bias"] = ((self.width,), "matrix")
        return shapes

    def bind(self, weights, ops):
        self.w = ops.prepare_linear([weights["weight"]])
        self.b = weights["bias"].to(device=ops.device, dtype=torch.float32).contiguous() if self.has_bias else None

    def logits(self, ctx, h):
        return ctx.ops.linear(h, self.w, out_dtype=torch.float32)

    def apply(self, ctx, x, y, logits):
        ctx.ops.gated_add(x, y, logits, self.b)

    def addend(self, y, logits):
        """(y, logits, bias): what ``apply`` would add, for an operation that adds it together with what follows."""
        return y, logits, self.b


register_part("input_filter", "causal_taps", CausalTapsFilter)
register_part("result_gate", "sigmoid_linear", SigmoidGate)


class GatedTokenEmbedding(TokenInput):
    """x += rms(P (gelu_tanh(G x) * e)) * w: e is the row's slice of a second embedding table ("embed": [vocab,
    n_slices * dim], this part's slice is ``index``), G ("gate") is [dim, width], P ("proj") [width, dim], and the RMS
    norm over the width has a plain weight w ("norm").  The table is kept as this part's own [vocab, dim] slice."""

    def __init__(self, width: int, dim: int, vocab: int, index: int, n_slices: int, eps: float):
        self.width, self.dim, self.vocab = int(width), int(dim), int(vocab)
        self.index, self.n_slices, self.eps = int(index), int(n_slices), float(eps)
        if not 0 <= self.index < self.n_slices or self.dim < 1:
            raise ValueError("gated token embedding: the slice must lie inside the table")
        self.table = self.w_gate = self.w_proj = self.norm_w = None

    def weight_shapes(self):
        return {"embed": ((self.vocab, self.n_slices * self.dim), "matrix"), "gate": ((self.dim, self.width), "matrix"),
                "proj": ((self.width, self.dim), "matrix"), "norm": ((self.width,), "norm")}

    def bind(self, weights, ops):
        d = self.dim
        self.table = ops.prepare_embedding(weights["embed"][:, self.index * d:(self.index + 1) * d])
        self.w_gate = ops.prepare_linear([weights["gate"]])
        self.w_proj = ops.prepare_linear([weights["proj"]])
        self.norm_w = weights["norm"].to(device=ops.device, dtype=torch.float32).contiguous()

    def forward(self, ctx, x, h, want_rounded=False):
        ops = ctx.ops
        a = ops.linear(h, self.w_gate, out_dtype=torch.float32)                 # [T, dim]
        g = ops.token_gate(a, self.table, ctx.meta.token_ids)                   # gelu_tanh(a) * e, compute dtype
        y = ops.linear(g, self.w_proj, out_dtype=torch.float32)                 # [T, width]
        return ops.norm_add(x, y, self.norm_w, self.eps, want_rounded=want_rounded)


register_part("token_input", "gated_embedding", GatedTokenEmbedding)
