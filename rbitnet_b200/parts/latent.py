"""``LatentAttention``: causal softmax attention whose keys and values are made from one small vector per position,
the only thing the cache keeps.

From the input rows h, without biases and without a position encoding:

    c_q = rmsnorm(W_dq h) * w_dq          [q_rank]      the queries' latent
    q   = W_uq c_q                        [n_heads, head_dim]
    c   = rmsnorm(W_dkv h) * w_dkv        [kv_rank]     the latent that is cached
    k_j = W_uk c_j,  v_j = W_uv c_j       per head: [head_dim], [value_dim]
    score_ij = (q_i . k_j) * scale, j <= i;  softmax over j;  o_i = sum_j p_ij v_j;  result = W_o o

Because k_j and v_j are linear in c_j, the sums over positions can be taken over the latents themselves:
q_i . k_j = (W_uk^T q_i) . c_j and sum_j p_ij v_j = W_uv (sum_j p_ij c_j), head by head.  So a step turns every
query head into the latent's space (a small product per head), runs the library's attention with ONE key/value head
whose keys and values are both the cached latents, and turns every head's result back (another small product per
head).  Nothing but c is stored per position, whole prompts and single tokens take the same path, and every attention
kernel of the library serves it as it serves grouped attention with one key head.  Norms, scores and softmax are
float32 as everywhere.

Options, each off by default:
  q_rank = 0    the queries come straight from the input rows: q = W_q h ("q"), no latent and no norm of their own
  rot_dim > 0   every query head has ``rot_dim`` more values after its ``head_dim`` ones, and W_dkv ``rot_dim`` more
                rows after the latent's (not normed): one key part per position that all heads share.  Both are turned
                by position (``position``: a rotary encoding over ``rot_dim`` values) and the score is
                (q_c . W_uk c + rot(q_r) . rot(k_r)) * scale.  The cache row is [c | rot(k_r)]; a query head enters
                the attention as [W_uk^T q_c | rot(q_r)] (the small product per head carries an identity block for
                the turned part), and the result's columns beyond the latent are dropped by W_uv's zero columns
  sinks         the softmax's denominator also holds exp(s_h), a stored number per head ("sink")
"""
from __future__ import annotations

import dataclasses

import torch

from .base import Mixer, CacheNeed
from .registry import register_part, build_part
from .spec import PartSpec


class LatentAttention(Mixer):
    def __init__(self, width: int, n_heads: int, head_dim: int, value_dim: int, q_rank: int, kv_rank: int,
                 scale: float, norm_eps: float, rot_dim: int = 0, position: dict = None, sinks: bool = False):
        self.width, self.n_heads, self.head_dim, self.value_dim = int(width), int(n_heads), int(head_dim), int(value_dim)
        self.q_rank, self.kv_rank = int(q_rank or 0), int(kv_rank)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.rot_dim, self.sinks = int(rot_dim or 0), bool(sinks)
        if min(self.n_heads, self.head_dim, self.value_dim, self.kv_rank) < 1 or self.q_rank < 0 or self.rot_dim < 0:
            raise ValueError("latent attention: heads, sizes and ranks are at least 1")
        self.position = None
        if self.rot_dim:
            if not position or position.get("kind") != "rotary":
                raise ValueError("latent attention: a turned key part needs a rotary position encoding")
            self.position = build_part("position", PartSpec(position["kind"], dict(position.get("params", {}))))
            if self.position.head_dim != self.rot_dim or self.position.rot_dim != self.rot_dim:
                raise ValueError("latent attention: the position encoding turns the whole turned part")
        self.direct = self.q_rank == 0 or self.rot_dim > 0 or self.sinks
        self.sink_w = None
        self.cache_width = self.kv_rank + self.rot_dim
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = self.q_norm_w = self.kv_norm_w = None

    def weight_shapes(self):
        H, D, Dv, E, Rq, R = self.n_heads, self.head_dim, self.value_dim, self.width, self.q_rank, self.kv_rank
        shapes = {"dkv": ((R + self.rot_dim, E), "matrix"), "dkv.norm": ((R,), "norm"), "uk": ((H * D, R), "matrix"),
                  "uv": ((H * Dv, R), "matrix"), "o": ((E, H * Dv), "matrix")}
        if Rq:
            shapes.update({"dq": ((Rq, E), "matrix"), "dq.norm": ((Rq,), "norm"),
                           "uq": ((H * (D + self.rot_dim), Rq), "matrix")})
        else:
            shapes["q"] = ((H * (D + self.rot_dim), E), "matrix")
        if self.sinks:
            shapes["sink"] = ((H,), "matrix")
        return shapes

    def cache_need(self):
        return CacheNeed(1, self.cache_width, None, streams=((1, self.cache_width),))

    def bind(self, weights, ops):
        H, D, Dv, R, Rr = self.n_heads, self.head_dim, self.value_dim, self.kv_rank, self.rot_dim
        self.cache_width = Rc = ops.cache_head_width(R + Rr, R + Rr)
        if self.q_rank:
            if self.direct:
                raise ValueError("latent attention: a turned key part or sinks go with queries made straight from the "
                                 "input rows (q_rank = 0)")
            self.w_down = ops.prepare_linear([weights["dq"], weights["dkv"]])
            self.w_uq = ops.prepare_linear([weights["uq"]])
        else:
            self.w_down = ops.prepare_linear([weights["q"], weights["dkv"]])
            if self.position is not None:
                self.position.bind({}, ops)
        if self.sinks:
            self.sink_w = weights["sink"].to(device=ops.device, dtype=torch.float32).contiguous()
        self.w_o = ops.prepare_linear([weights["o"]])
        # per head: [Rc, D + Rr] (W_uk of the head, transposed, and an identity block that passes the turned part on)
        # and [Dv, Rc]; the columns beyond kv_rank are zeros
        uk = torch.zeros((H, Rc, D + Rr), dtype=weights["uk"].dtype, device=weights["uk"].device)
        uk[:, :R, :D] = weights["uk"].view(H, D, R).transpose(1, 2)
        if Rr:
            uk[:, R:R + Rr, D:] = torch.eye(Rr, dtype=uk.dtype, device=uk.device)
        uv = torch.zeros((H, Dv, Rc), dtype=weights["uv"].dtype, device=weights["uv"].device)
        uv[:, :, :R] = weights["uv"].view(H, Dv, R)
        self.w_uk_t = ops.prepare_per_head(uk)
        self.w_uv = ops.prepare_per_head(uv)
        f32 = dict(device=ops.device, dtype=torch.float32)
        self.q_norm_w = weights["dq.norm"].to(**f32).contiguous() if self.q_rank else None
        self.kv_norm_w = weights["dkv.norm"].to(**f32).contiguous()

    def forward(self, ctx, h, entry, accumulate_into=None):
        ops = ctx.ops
        view = ctx.cache_view(entry)
        if not view.writes:
            raise ValueError("latent attention reads only its own cache")
        H = self.n_heads
        down = ops.linear(h, self.w_down, out_dtype=torch.float32)                  # [T, W_dq h (or W_q h) | W_dkv h]
        if self.direct:
            table = self.position.table() if self.position is not None else None
            q = ops.latent_rotate_append(down, H, self.head_dim, self.rot_dim, self.kv_rank, table, self.kv_norm_w,
                                         self.norm_eps, ctx.meta, view)            # [T, H * (D + Rr)]; [c | k_r] is cached
        else:
            cq = ops.latent_norm_append(down, self.q_rank, self.kv_rank, self.q_norm_w, self.kv_norm_w, self.norm_eps,
                                        ctx.meta, view)                             # [T, q_rank]; c is in the cache
            q = ops.linear(cq, self.w_uq)                                           # [T, H * D]
        ql = ops.per_head_linear(q, self.w_uk_t)                                    # [T, H * Rc]: W_uk^T q per head
        both = dataclasses.replace(view, v=view.k)                                  # keys and values: the latents
        if self.sinks:
            a = ops.attention(ql.view(ql.shape[0], H, view.head_dim), ctx.meta, both, H, self.scale, None,
                              sinks=self.sink_w)
        else:
            a = ops.attention(ql.view(ql.shape[0], H, view.head_dim), ctx.meta, both, H, self.scale, None)
        o = ops.per_head_linear(a, self.w_uv)                                       # [T, H * Dv]
        if accumulate_into is None:
            return ops.linear(o, self.w_o, out_dtype=torch.float32)
        return ops.linear(o, self.w_o, accumulate_into=accumulate_into)


register_part("mixer", "latent_attention", LatentAttention)
