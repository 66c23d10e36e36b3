"""``GatedLinearAttention``: a mixer that keeps one matrix memory S [head_dim, value_dim] per head and lets every
key channel of it decay at a rate of its own, decided token by token.

From the input rows h, without biases: q = Wq h / sqrt(head_dim) and k = Wk h (``n_heads`` heads of ``head_dim``),
v = Wv h (``n_heads`` heads of ``value_dim``).  The decays come through a low rank:

    z = A2 (A1 h) + b                 A1: [decay_rank, width], A2: [n_heads * head_dim, decay_rank]
    alpha = sigmoid(z)^(1/tau)        one number per head and key channel, in (0, 1)
    S <- diag(alpha) S + k v^T;   o = S^T q                      (the read-out sees the write)
    result = Wo (o / rms(o over value_dim, norm_eps) * w * silu(Wg h))      (w: value_dim values, every head's)

State per sequence: S (float32, kept by value column: [heads, value_dim, head_dim]), zero at the start.  The decays
(their low-rank product's second half, the sigmoid, its logarithm and the power), the memory and its sums, and the
norm per head are float32 in every mode; the projections are one stacked product whose float32 rows feed the
recurrence's kernels.
"""
from __future__ import annotations

import torch

from .base import Mixer, StateNeed
from .registry import register_part


class GatedLinearAttention(Mixer):
    def __init__(self, width: int, n_heads: int, head_dim: int, value_dim: int, decay_rank: int, tau: float,
                 norm_eps: float):
        self.width, self.n_heads, self.head_dim = int(width), int(n_heads), int(head_dim)
        self.value_dim, self.decay_rank = int(value_dim), int(decay_rank)
        self.tau, self.norm_eps = float(tau), float(norm_eps)
        if not self.tau > 0:
            raise ValueError("gated linear attention: tau must be positive")
        if min(self.n_heads, self.head_dim, self.value_dim, self.decay_rank) < 1:
            raise ValueError("gated linear attention: heads, sizes and the decays' rank are at least 1")
        self.w_all = self.w_o = self.a2 = self.a2_bias = self.norm_w = None

    def weight_shapes(self):
        H, D, Dv, E, R = self.n_heads, self.head_dim, self.value_dim, self.width, self.decay_rank
        return {"q": ((H * D, E), "matrix"), "k": ((H * D, E), "matrix"), "v": ((H * Dv, E), "matrix"),
                "g": ((H * Dv, E), "matrix"), "o": ((E, H * Dv), "matrix"), "norm": ((Dv,), "norm"),
                "a1": ((R, E), "matrix"), "a2": ((H * D, R), "matrix"), "a2.b": ((H * D,), "matrix")}

    def state_need(self):
        return {"S": StateNeed((self.n_heads, self.value_dim, self.head_dim))}

    def offsets(self):
        """Columns of the stacked product's rows."""
        H, D, Dv = self.n_heads, self.head_dim, self.value_dim
        return {"q": 0, "k": H * D, "v": 2 * H * D, "g": 2 * H * D + H * Dv, "a": 2 * H * D + 2 * H * Dv}

    def bind(self, weights, ops):
        self.w_all = ops.prepare_linear([weights[k] for k in ("q", "k", "v", "g", "a1")])
        self.w_o = ops.prepare_linear([weights["o"]])
        f32 = dict(device=ops.device, dtype=torch.float32)
        self.a2 = weights["a2"].to(**f32).contiguous()
        self.a2_bias = weights["a2.b"].to(**f32).contiguous()
        self.norm_w = weights["norm"].to(**f32).contiguous()

    def forward(self, ctx, h, entry, accumulate_into=None):
        ops = ctx.ops
        state = ctx.state_view(entry)
        proj = ops.linear(h, self.w_all, out_dtype=torch.float32)        # [T, q | k | v | g | A1 h]
        out = ops.gated_linear_attention(proj, self, state, ctx.meta)    # [T, H Dv], compute dtype
        if accumulate_into is None:
            return ops.linear(out, self.w_o, out_dtype=torch.float32)
        return ops.linear(out, self.w_o, accumulate_into=accumulate_into)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
