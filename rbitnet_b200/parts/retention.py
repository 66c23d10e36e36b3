"""``Retention``: linear attention with one fixed decay per head and neither softmax nor denominator.

From the input rows h, without biases:

    q = rot(W_q h), k = rot(W_k h) / sqrt(head_dim)     [n_heads, head_dim], turned by position (a prefix of every head)
    v = W_v h                                           [n_heads, value_dim]
    S_t = g_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t    a matrix memory per head; g_h is a constant of the head
    result = W_o (o / rms(o) per head  *  silu(W_g h))  the root mean square over the head's value_dim values, no weight

The memory starts at zero, is float32 and belongs to the sequence (``state_need``).  It is gated linear attention whose
decays do not depend on the token: the operations run that recurrence's kernels, token by token for a decode step and
in chunks for a prompt, on a row of decays that every token shares.  The stacked product leaves float32 rows; the
rotation, the recurrence, the norm and the gate are float32.
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, StateNeed
from .registry import register_part, build_part
from .spec import PartSpec


class Retention(Mixer):
    def __init__(self, width: int, n_heads: int, head_dim: int, value_dim: int, decay, norm_eps: float,
                 position: dict = None):
        self.width, self.n_heads, self.head_dim, self.value_dim = int(width), int(n_heads), int(head_dim), int(value_dim)
        self.decay = [float(g) for g in decay]
        self.norm_eps = float(norm_eps)
        if min(self.n_heads, self.head_dim, self.value_dim) < 1:
            raise ValueError("retention: heads and sizes are at least 1")
        if len(self.decay) != self.n_heads or not all(0.0 < g <= 1.0 for g in self.decay):
            raise ValueError(f"retention: one decay in (0, 1] per head, found {self.decay} for {self.n_heads} heads")
        position = position or {"kind": "none", "params": {}}
        self.position = build_part("position", PartSpec(position["kind"], dict(position.get("params", {}))))
        self.w_all = self.w_o = self.decays = self.log_decays = self.norm_w = None

    def weight_shapes(self):
        H, D, Dv, E = self.n_heads, self.head_dim, self.value_dim, self.width
        return {"q": ((H * D, E), "matrix"), "k": ((H * D, E), "matrix"), "v": ((H * Dv, E), "matrix"),
                "g": ((H * Dv, E), "matrix"), "o": ((E, H * Dv), "matrix")}

    def state_need(self):
        return {"S": StateNeed((self.n_heads, self.value_dim, self.head_dim))}

    def offsets(self):
        """Columns of the stacked product's rows."""
        H, D, Dv = self.n_heads, self.head_dim, self.value_dim
        return {"q": 0, "k": H * D, "v": 2 * H * D, "g": 2 * H * D + H * Dv}

    def bind(self, weights, ops):
        self.position.bind({}, ops)
        self.w_all = ops.prepare_linear([weights[k] for k in ("q", "k", "v", "g")])
        self.w_o = ops.prepare_linear([weights["o"]])
        f32 = dict(device=ops.device, dtype=torch.float32)
        per_channel = torch.tensor(self.decay, dtype=torch.float64).repeat_interleave(self.head_dim)
        self.decays = per_channel.to(**f32).contiguous()                 # one row [H * D] that every token shares
        self.log_decays = torch.log(per_channel).to(**f32).contiguous()
        self.norm_w = torch.ones(self.value_dim, **f32)

    def forward(self, ctx, h, entry, accumulate_into=None, scale_result: float = 1.0):
        ops = ctx.ops
        state = ctx.state_view(entry)
        proj = ops.linear(h, self.w_all, out_dtype=torch.float32)        # [T, q | k | v | g]
        out = ops.retention(proj, self, state, ctx.meta)                 # [T, H Dv], compute dtype
        if accumulate_into is None:
            return ops.linear(out, self.w_o, out_dtype=torch.float32, scale=scale_result)
        return ops.linear(out, self.w_o, accumulate_into=accumulate_into, scale=scale_result)


register_part("mixer", "retention", Retention)
