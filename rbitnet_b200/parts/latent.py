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
"""
from __future__ import annotations

import dataclasses

import torch

from .base import Mixer, CacheNeed
from .registry import register_part


class LatentAttention(Mixer):
    def __init__(self, width: int, n_heads: int, head_dim: int, value_dim: int, q_rank: int, kv_rank: int,
                 scale: float, norm_eps: float):
        self.width, self.n_heads, self.head_dim, self.value_dim = int(width), int(n_heads), int(head_dim), int(value_dim)
        self.q_rank, self.kv_rank = int(q_rank), int(kv_rank)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        if min(self.n_heads, self.head_dim, self.value_dim, self.q_rank, self.kv_rank) < 1:
            raise ValueError("latent attention: heads, sizes and ranks are at least 1")
        self.cache_width = self.kv_rank
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = self.q_norm_w = self.kv_norm_w = None

    def weight_shapes(self):
        H, D, Dv, E, Rq, R = self.n_heads, self.head_dim, self.value_dim, self.width, self.q_rank, self.kv_rank
        return {"dq": ((Rq, E), "matrix"), "dq.norm": ((Rq,), "norm"), "uq": ((H * D, Rq), "matrix"),
                "dkv": ((R, E), "matrix"), "dkv.norm": ((R,), "norm"), "uk": ((H * D, R), "matrix"),
                "uv": ((H * Dv, R), "matrix"), "o": ((E, H * Dv), "matrix")}

    def cache_need(self):
        return CacheNeed(1, self.cache_width, None, streams=((1, self.cache_width),))

    def bind(self, weights, ops):
        H, D, Dv, R = self.n_heads, self.head_dim, self.value_dim, self.kv_rank
        self.cache_width = Rc = ops.cache_head_width(R, R)
        self.w_down = ops.prepare_linear([weights["dq"], weights["dkv"]])
        self.w_uq = ops.prepare_linear([weights["uq"]])
        self.w_o = ops.prepare_linear([weights["o"]])
        # per head: [Rc, D] (W_uk of the head, transposed) and [Dv, Rc]; the columns beyond kv_rank are zeros
        uk = torch.zeros((H, Rc, D), dtype=weights["uk"].dtype, device=weights["uk"].device)
        uk[:, :R] = weights["uk"].view(H, D, R).transpose(1, 2)
        uv = torch.zeros((H, Dv, Rc), dtype=weights["uv"].dtype, device=weights["uv"].device)
        uv[:, :, :R] = weights["uv"].view(H, Dv, R)
        self.w_uk_t = ops.prepare_per_head(uk)
        self.w_uv = ops.prepare_per_head(uv)
        f32 = dict(device=ops.device, dtype=torch.float32)
        self.q_norm_w = weights["dq.norm"].to(**f32).contiguous()
        self.kv_norm_w = weights["dkv.norm"].to(**f32).contiguous()

    def forward(self, ctx, h, entry, accumulate_into=None):
        ops = ctx.ops
        view = ctx.cache_view(entry)
        if not view.writes:
            raise ValueError("latent attention reads only its own cache")
        H = self.n_heads
        down = ops.linear(h, self.w_down, out_dtype=torch.float32)                  # [T, W_dq h | W_dkv h]
        cq = ops.latent_norm_append(down, self.q_rank, self.kv_rank, self.q_norm_w, self.kv_norm_w, self.norm_eps,
                                    ctx.meta, view)                                 # [T, q_rank]; c is in the cache
        q = ops.linear(cq, self.w_uq)                                               # [T, H * D]
        ql = ops.per_head_linear(q, self.w_uk_t)                                    # [T, H * Rc]: W_uk^T q per head
        both = dataclasses.replace(view, v=view.k)                                  # keys and values: the latents
        a = ops.attention(ql.view(ql.shape[0], H, view.head_dim), ctx.meta, both, H, self.scale, None)
        o = ops.per_head_linear(a, self.w_uv)                                       # [T, H * Dv]
        if accumulate_into is None:
            return ops.linear(o, self.w_o, out_dtype=torch.float32)
        return ops.linear(o, self.w_o, accumulate_into=accumulate_into)


register_part("mixer", "latent_attention", LatentAttention)
