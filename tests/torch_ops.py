"""A stand-in for the kernel layer, written with torch on the CPU, for tests only.

It has the same methods as ``rbitnet_b200.kernels.ops.CudaOps`` so that the
package's host logic (parts, cache, paging, step function, generation loop,
trace replay) can be exercised where there is no GPU.  It is not part of the
product: the package never imports it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class _W:
    w: torch.Tensor
    n_out: int
    n_in: int


@dataclass
class _GU:
    w: torch.Tensor
    inner: int
    n_in: int


class TorchOps:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype
        self.device = torch.device("cpu")
        self.calls = 0

    def to_compute(self, t):
        return t.to(self.dtype).contiguous()

    def prepare_embedding(self, table):
        return self.to_compute(table)

    def prepare_linear(self, weights):
        w = torch.cat([self.to_compute(x) for x in weights], dim=0)
        return _W(w, w.shape[0], w.shape[1])

    def rows_of(self, weight, first, count):
        return _W(weight.w[first:first + count], count, weight.n_in)

    def prepare_gate_up(self, gate, up):
        return _GU(torch.cat([self.to_compute(gate), self.to_compute(up)], dim=0), gate.shape[0], gate.shape[1])

    def embed(self, ids, table, scale=1.0):
        return table[ids.long()].to(torch.float32) * scale

    def rmsnorm(self, x, w, eps, out_dtype=None):
        s = (x * x).sum(-1, keepdim=True) / x.shape[-1]
        return (x * w * (1.0 / torch.sqrt(s + eps))).to(out_dtype or self.dtype)

    def layernorm(self, x, w, b, eps, out_dtype=None):
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        y = (x - mu) / torch.sqrt(var + eps) * w
        return (y + b if b is not None else y).to(out_dtype or self.dtype)

    def add_rows(self, x, y):
        x += y
        return x

    def linear(self, x, weight, out_dtype=None, accumulate_into=None, scale=1.0, act=None):
        y = x.to(torch.float32) @ weight.w.to(torch.float32).T * scale
        if act == "relu2":
            y = torch.clamp(y, min=0.0) ** 2
        if accumulate_into is not None:
            accumulate_into += y
            return accumulate_into
        return y.to(out_dtype or self.dtype)

    def gated_linear(self, x, weight, act=None):
        gu = x.to(torch.float32) @ weight.w.to(torch.float32).T
        g, u = gu[:, :weight.inner], gu[:, weight.inner:]
        if act is not None:
            alpha, limit, shift = act
            g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
            return (g / (1.0 + torch.exp(-alpha * g)) * (u + shift)).to(self.dtype)
        return (g / (1.0 + torch.exp(-g)) * u).to(self.dtype)

    def normed(self, rows):
        return rows

    # ---- several residual streams
    fuse_streams = True

    def streams_expand(self, x, s):
        return x.repeat(1, s).contiguous()

    def streams_sum(self, x, s):
        R, E = x.shape[0], x.shape[1] // s
        return x.view(R, s, E).sum(1)

    def normed_mean(self, results, weights, eps):
        out = 0.0
        for y, w in zip(results, weights):
            out = out + y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w
        return out / len(results)

    def stream_step(self, x, s, results=None, result_norms=None, norm_eps=0.0, write=None, read=None, want_result=False):
        T, E = x.shape[0], x.shape[1] // s
        X = x.view(T, s, E)
        y = None
        if results:
            y = self.normed_mean(results, result_norms, norm_eps) if result_norms else results[0]
            mix, w_out = write
            X.copy_(torch.einsum("kj,tke->tje", mix, X) + w_out[None, :, None] * y[:, None, :])
        h = None
        if read is not None:
            w_in, norm_w, eps = read
            u = torch.einsum("k,tke->te", w_in, X)
            h = (u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * norm_w).to(self.dtype)
        return (h, y) if want_result else h

    # ---- attention with a projection norm, a partly turned head, a gate per head
    def cache_head_width(self, head_dim, value_dim):
        return max(head_dim, value_dim)

    def norm_rotate_append(self, proj, table, meta, view, n_heads, head_dim, value_dim, q_norm_w, k_norm_w, eps,
                           head_norm=False):
        T, H, D, Dv, Kh, Dc = proj.shape[0], n_heads, head_dim, value_dim, view.n_kv_heads, view.head_dim
        x = proj.to(torch.float32)
        q, k, v = x[:, :H * D], x[:, H * D:(H + Kh) * D], x[:, (H + Kh) * D:(H + Kh) * D + Kh * Dv]
        if q_norm_w is not None:
            q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * q_norm_w
            k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * k_norm_w
        q, k, v = q.reshape(T, H, D).clone(), k.reshape(T, Kh, D).clone(), v.reshape(T, Kh, Dv)
        if table is not None:
            freq, magnitude, interleaved, rot = table
            ang = meta.tok_pos.to(torch.float64)[:, None] * freq[None, :]
            c, s_ = (torch.cos(ang) * magnitude).float()[:, None, :], (torch.sin(ang) * magnitude).float()[:, None, :]
            for t_ in (q, k):
                if interleaved:
                    a, b = t_[..., 0:rot:2].clone(), t_[..., 1:rot:2].clone()
                    t_[..., 0:rot:2], t_[..., 1:rot:2] = a * c - b * s_, b * c + a * s_
                else:
                    a, b = t_[..., :rot // 2].clone(), t_[..., rot // 2:rot].clone()
                    t_[..., :rot // 2], t_[..., rot // 2:rot] = a * c - b * s_, b * c + a * s_
        if head_norm:
            q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps)
            k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps)
        qo = torch.zeros(T, H, Dc)
        qo[..., :D] = q
        for t in range(T):
            p, slot = int(meta.tok_pos[t]), int(meta.tok_slot[t])
            page = int(view.page_table[slot, p // view.page_size])
            view.k[page, :, p % view.page_size, :] = 0
            view.v[page, :, p % view.page_size, :] = 0
            view.k[page, :, p % view.page_size, :D] = k[t].to(view.k.dtype)
            view.v[page, :, p % view.page_size, :Dv] = v[t].to(view.v.dtype)
        return qo.to(self.dtype)

    def head_gate(self, a, proj, gate_column, n_heads, value_dim, cache_width, per_value=False):
        T = a.shape[0]
        out = a.to(torch.float32).view(T, n_heads, cache_width)[:, :, :value_dim]
        if gate_column is not None and per_value:
            g = proj[:, gate_column:gate_column + n_heads * value_dim].to(torch.float32)
            out = out * torch.sigmoid(g).view(T, n_heads, value_dim)
        elif gate_column is not None:
            out = out * torch.sigmoid(proj[:, gate_column:gate_column + n_heads].to(torch.float32))[:, :, None]
        return out.reshape(T, n_heads * value_dim).to(self.dtype)

    # ---- recurrent mixers
    @staticmethod
    def _runs(meta):
        return [(c.offset, c.n_new, c.slot) for c in meta.seqs]

    def gated_recurrence(self, proj, p, state, meta):
        W, B, K = p.inner, p.blocks, p.taps
        Wb = W // B
        f = p.f32
        out = torch.zeros(proj.shape[0], W)
        sp = p.decay_scale * torch.nn.functional.softplus(f["lam"])
        for first, n, slot in self._runs(meta):
            xx = proj[first:first + n, :W].float() + f["x.b"]
            y = proj[first:first + n, W:].float() + f["y.b"]
            y = 0.5 * y * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (y + 0.044715 * y ** 3)))
            old = state["tail"][slot][1:] if K > 1 else torch.zeros(0, W)     # this stand-in keeps the last K-1 inputs in rows 1..
            hist = torch.cat([old, xx], dim=0)                    # K-1 earlier inputs, then this run's
            S = state["S"][slot].clone()
            for t in range(n):
                u = f["conv.b"] + (hist[t:t + K] * f["conv"].T).sum(0)
                ub = u.view(B, Wb)
                g = torch.einsum("boi,bi->bo", p.w_gates, ub)     # [B, 2 Wb]
                r = torch.sigmoid(g[:, :Wb].reshape(W) + f["ra.b"].reshape(W))
                i = torch.sigmoid(g[:, Wb:].reshape(W) + f["ri.b"].reshape(W))
                a = torch.exp(-sp * r)
                S = a * S + torch.sqrt(1.0 - a * a) * i * u
                out[first + t] = S * y[t]
            state["S"][slot] = S
            if K > 1:
                state["tail"][slot][1:] = hist[n:n + K - 1]
        return out.to(self.dtype)

    def matrix_memory(self, proj, p, state, meta):
        H, D, Dv, cap = p.n_heads, p.head_dim, p.value_dim, p.gate_cap
        at = p.offsets()
        x = proj.float()
        T = x.shape[0]
        o = torch.zeros(T, H, Dv)
        for first, n, slot in self._runs(meta):
            C, nn, m = state["C"][slot].clone(), state["n"][slot].clone(), state["m"][slot].clone()
            for t in range(first, first + n):
                q = x[t, at["q"]:at["q"] + H * D].view(H, D) * D ** -0.5
                k = x[t, at["k"]:at["k"] + H * D].view(H, D)
                v = x[t, at["v"]:at["v"] + H * Dv].view(H, Dv)
                ig = cap * torch.tanh((x[t, at["i"]:at["i"] + H] + p.i_bias) / cap)
                fg = torch.nn.functional.logsigmoid(cap * torch.tanh((x[t, at["f"]:at["f"] + H] + p.f_bias) / cap))
                m_new = torch.maximum(fg + m, ig)
                keep, take = torch.exp(fg + m - m_new), torch.exp(ig - m_new)
                C = keep[:, None, None] * C + take[:, None, None] * k[:, :, None] * v[:, None, :]
                nn = keep[:, None] * nn + take[:, None] * k
                m = m_new
                den = torch.maximum((nn * q).sum(-1).abs(), torch.exp(-m)) + p.floor
                o[t] = torch.einsum("hdv,hd->hv", C, q) / den[:, None]
            state["C"][slot], state["n"][slot], state["m"][slot] = C, nn, m
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + p.norm_eps)
        g = torch.sigmoid(x[:, at["g"]:at["g"] + H * Dv])
        return (o.reshape(T, H * Dv) * p.norm_w * g).to(self.dtype)

    def gated_delta(self, proj, p, state, meta):
        H, G, D, Dv, K = p.n_heads, p.n_kv_heads, p.head_dim, p.value_dim, p.taps
        C = 2 * G * D + H * Dv
        at = p.offsets()
        x = proj.float()
        T = x.shape[0]
        o = torch.zeros(T, H, Dv)
        share = torch.arange(H) // (H // G)
        for first, n, slot in self._runs(meta):
            xin = x[first:first + n, :C]
            old = state["tail"][slot][1:] if K > 1 else torch.zeros(0, C)      # this stand-in keeps the last K-1 inputs in rows 1..
            hist = torch.cat([old, xin], dim=0)
            S = state["S"][slot].clone()                                        # [H, Dv, D]
            for t in range(n):
                u = (hist[t:t + K] * p.conv_w.T).sum(0)
                u = u / (1.0 + torch.exp(-u))
                q, k, v = u[:G * D].view(G, D), u[G * D:2 * G * D].view(G, D), u[2 * G * D:].view(H, Dv)
                q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + p.unit_eps) * D ** -0.5
                k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + p.unit_eps)
                q, k = q[share], k[share]
                row = x[first + t]
                beta = torch.sigmoid(row[at["b"]:at["b"] + H])
                g = torch.exp(-torch.exp(p.a_log) * torch.nn.functional.softplus(row[at["a"]:at["a"] + H] + p.dt_bias))
                S = S * g[:, None, None]
                w = beta[:, None] * (v - torch.einsum("hvd,hd->hv", S, k))
                S = S + w[:, :, None] * k[:, None, :]
                o[first + t] = torch.einsum("hvd,hd->hv", S, q)
            state["S"][slot] = S
            if K > 1:
                state["tail"][slot][1:] = hist[n:n + K - 1]
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + p.norm_eps) * p.norm_w
        gate = x[:, at["g"]:at["g"] + H * Dv]
        return (o.reshape(T, H * Dv) * (gate / (1.0 + torch.exp(-gate)))).to(self.dtype)

    # ---- around a sublayer
    def rmsnorm_grouped(self, x, w, groups, eps, out_dtype=None):
        T, E = x.shape
        parts = x.view(T, groups, E // groups)
        y = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
        return (y.reshape(T, E) * w).to(out_dtype or self.dtype)

    def input_filter(self, h, taps, ring, meta):
        K = taps.shape[1]
        x = h.to(torch.float32)
        out = torch.zeros_like(x)
        for first, n, slot in self._runs(meta):
            old = ring[slot][1:] if K > 1 else torch.zeros(0, x.shape[1])     # this stand-in keeps the last K-1 inputs in rows 1..
            hist = torch.cat([old, x[first:first + n]], dim=0)
            for t in range(n):
                out[first + t] = x[first + t] + (hist[t:t + K] * taps.T).sum(0)
            if K > 1:
                ring[slot][1:] = hist[n:n + K - 1]
        return out.to(self.dtype)

    def gated_add(self, x, y, logits, bias):
        z = logits.to(torch.float32) + (bias if bias is not None else 0.0)
        x += y * torch.sigmoid(z)
        return x

    def add_scaled_rows(self, y, z, gate):
        y += torch.sigmoid(gate[:, :1]) * z
        return y

    def softcap(self, v, cap):
        v.copy_(cap * torch.tanh(v / cap))
        return v

    # ---- gated linear attention
    def gated_linear_attention(self, proj, p, state, meta):
        H, D, Dv, R = p.n_heads, p.head_dim, p.value_dim, p.decay_rank
        at = p.offsets()
        x = proj.float()
        T = x.shape[0]
        z = x[:, at["a"]:at["a"] + R] @ p.a2.T + p.a2_bias
        alpha = torch.exp(torch.nn.functional.logsigmoid(z) / p.tau).view(T, H, D)
        q = x[:, at["q"]:at["q"] + H * D].view(T, H, D) * D ** -0.5
        k = x[:, at["k"]:at["k"] + H * D].view(T, H, D)
        v = x[:, at["v"]:at["v"] + H * Dv].view(T, H, Dv)
        o = torch.zeros(T, H, Dv)
        for first, n, slot in self._runs(meta):
            S = state["S"][slot].clone()                                        # [H, Dv, D]
            for t in range(first, first + n):
                S = S * alpha[t][:, None, :] + v[t][:, :, None] * k[t][:, None, :]
                o[t] = torch.einsum("hvd,hd->hv", S, q[t])
            state["S"][slot] = S
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + p.norm_eps) * p.norm_w
        gate = x[:, at["g"]:at["g"] + H * Dv]
        return (o.reshape(T, H * Dv) * (gate / (1.0 + torch.exp(-gate)))).to(self.dtype)

    # ---- attention through latents
    def latent_norm_append(self, down, q_rank, kv_rank, wq, wkv, eps, meta, view):
        x = down.float()
        cq, c = x[:, :q_rank], x[:, q_rank:q_rank + kv_rank]
        cq = cq / torch.sqrt((cq * cq).mean(-1, keepdim=True) + eps) * wq
        c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * wkv
        for t in range(x.shape[0]):
            p, slot = int(meta.tok_pos[t]), int(meta.tok_slot[t])
            page = int(view.page_table[slot, p // view.page_size])
            view.k[page, 0, p % view.page_size, :] = 0
            view.k[page, 0, p % view.page_size, :kv_rank] = c[t].to(view.k.dtype)
        return cq.to(self.dtype)

    def prepare_per_head(self, w):
        return self.to_compute(w)

    def per_head_linear(self, x, w):
        H, N, K = w.shape
        y = torch.einsum("thk,hnk->thn", x.to(torch.float32).view(x.shape[0], H, K), w.to(torch.float32))
        return y.reshape(x.shape[0], H * N).to(self.dtype)

    # ---- routed experts
    def prepare_expert_gate_up(self, gates, ups):
        w = torch.cat([torch.cat([self.to_compute(g), self.to_compute(u)], dim=0) for g, u in zip(gates, ups)], dim=0)
        return _W(w, w.shape[0], w.shape[1])

    def route_scored(self, h, router, correction, top, groups, keep, scoring="softmax", extra_rows=0, router_tc=None):
        z = h.to(torch.float32) @ router.T
        n = router.shape[0] - extra_rows
        extra = z[:, n:].clone() if extra_rows else None
        z = z[:, :n]
        s = torch.sigmoid(z) if scoring == "sigmoid" else torch.softmax(z, dim=-1)
        choice = s + correction if correction is not None else s.clone()
        if groups > 1 and keep < groups:
            per = n // groups
            best = choice.view(-1, groups, per).max(-1).values
            kept = torch.zeros_like(best, dtype=torch.bool).scatter_(1, best.topk(keep, dim=-1).indices, True)
            choice = choice.masked_fill(~kept.repeat_interleave(per, dim=1), -math.inf)
        ids = choice.topk(top, dim=-1).indices
        return ids.to(torch.int32), s.gather(1, ids), extra

    def route(self, h, router, correction, top, groups, keep):
        s = torch.softmax(h.to(torch.float32) @ router.T, dim=-1)
        choice = s + correction if correction is not None else s.clone()
        if groups > 1 and keep < groups:
            per = s.shape[1] // groups
            best = choice.view(-1, groups, per).max(-1).values
            kept = torch.zeros_like(best, dtype=torch.bool).scatter_(1, best.topk(keep, dim=-1).indices, True)
            choice = choice.masked_fill(~kept.repeat_interleave(per, dim=1), -math.inf)
        ids = choice.topk(top, dim=-1).indices
        return ids.to(torch.int32), s.gather(1, ids)

    def routed_experts(self, h, ids, weights, w_up, w_down, n_experts, inner, accumulate_into=None, act=None,
                       weight_on_input=False):
        T, E = h.shape
        x = h.to(torch.float32)
        out = torch.zeros(T, E)
        for t in range(T):
            for e, w in zip(ids[t].tolist(), weights[t]):
                if e >= n_experts:
                    out[t] += w * x[t]
                    continue
                down = w_down.w[e * E:(e + 1) * E].to(torch.float32)
                xin = (w * x[t]).to(self.dtype).to(torch.float32) if weight_on_input else x[t]
                if act is not None:
                    gu = w_up.w[e * 2 * inner:(e + 1) * 2 * inner].to(torch.float32) @ xin
                    alpha, limit, shift = act
                    g, u = torch.clamp(gu[:inner], max=limit), torch.clamp(gu[inner:], -limit, limit)
                    mid = (g / (1.0 + torch.exp(-alpha * g)) * (u + shift)).to(self.dtype).to(torch.float32)
                else:
                    up = w_up.w[e * inner:(e + 1) * inner].to(torch.float32)
                    mid = (torch.clamp(up @ xin, min=0.0) ** 2).to(self.dtype).to(torch.float32)
                out[t] += (down @ mid) if weight_on_input else w * (down @ mid)
        if accumulate_into is not None:
            accumulate_into += out
            return accumulate_into
        return out

    def project_rotate_append(self, h, weight, rotary, meta, view, n_heads):
        return self.rotate_append(self.linear(h, weight), rotary, meta, view, n_heads)

    def rotate_append(self, qkv, rotary, meta, view, n_heads):
        T = qkv.shape[0]
        D, Kh = view.head_dim, view.n_kv_heads
        x = qkv.to(torch.float32)
        q = x[:, :n_heads * D].reshape(T, n_heads, D)
        pos = meta.tok_pos.long()

        def rot(t):
            if rotary is None:
                return t
            inv, interleaved, _ = rotary
            ang = pos.to(torch.float32)[:, None] * inv[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            out = torch.empty_like(t)
            if interleaved:
                a, b = t[..., 0::2], t[..., 1::2]
                out[..., 0::2], out[..., 1::2] = a * c - b * s, a * s + b * c
            else:
                h = D // 2
                a, b = t[..., :h], t[..., h:]
                out[..., :h], out[..., h:] = a * c - b * s, a * s + b * c
            return out

        q = rot(q)
        if view.writes:
            k = rot(x[:, n_heads * D:(n_heads + Kh) * D].reshape(T, Kh, D))
            v = x[:, (n_heads + Kh) * D:].reshape(T, Kh, D)
            for t in range(T):
                p, slot = int(meta.tok_pos[t]), int(meta.tok_slot[t])
                page = int(view.page_table[slot, p // view.page_size])
                view.k[page, :, p % view.page_size, :] = k[t].to(view.k.dtype)
                view.v[page, :, p % view.page_size, :] = v[t].to(view.v.dtype)
        return q.to(self.dtype)

    def attention(self, q, meta, view, n_heads, scale, window, sinks=None, softcap=0.0):
        T, H, D = q.shape
        G = H // view.n_kv_heads
        out = torch.zeros(T, H * D, dtype=torch.float32)
        for t in range(T):
            p, slot = int(meta.tok_pos[t]), int(meta.tok_slot[t])
            lo = max(0, p - window + 1) if window else 0
            idx = torch.arange(lo, p + 1)
            pages = view.page_table[slot, idx // view.page_size].long()
            ks = view.k[pages, :, idx % view.page_size, :].to(torch.float32)   # [n, Kh, D]
            vs = view.v[pages, :, idx % view.page_size, :].to(torch.float32)
            for h in range(H):
                s = (ks[:, h // G, :] @ q[t, h].to(torch.float32)) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                if sinks is not None:
                    pr = torch.softmax(torch.cat([s, sinks[h:h + 1].float()]), dim=0)[:-1]
                else:
                    pr = torch.softmax(s, dim=0)
                out[t, h * D:(h + 1) * D] = pr @ vs[:, h // G, :]
        return out.to(self.dtype)

    # ---- rows that sublayers read as they are, and results that are normed
    def round_rows(self, x):
        return x.to(self.dtype)

    def norm_add(self, x, y, w, eps, want_rounded=False):
        y = y.float()
        x += y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w
        return x.to(self.dtype) if want_rounded else None

    def token_gate(self, a, table, ids):
        a = a.float()
        g = 0.5 * a * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (a + 0.044715 * a ** 3)))
        return (g * table[ids.long()].float()).to(self.dtype)

    def embed_pairs(self, meta, table, scale, pair_table, pair_hash, previous):
        buckets, mul_prev, mul_cur = pair_hash
        ids = meta.token_ids.long()
        x = table[ids].to(torch.float32) * scale
        for first, n, slot in self._runs(meta):
            for t in range(first, first + n):
                if int(meta.tok_pos[t]) == 0:
                    row = buckets
                else:
                    prev = int(ids[t - 1]) if t > first else int(previous[slot, 0])
                    row = (prev * mul_prev + int(ids[t]) * mul_cur) % buckets
                x[t] += pair_table[row].float()
            previous[slot, 0] = int(ids[first + n - 1])
        return x

    def _turn(self, t_, table, pos):
        """t_ [T, heads, D], changed in place: the first rot values of every head turned by position."""
        freq, magnitude, interleaved, rot = table
        ang = pos.to(torch.float64)[:, None] * freq[None, :]
        c, s_ = (torch.cos(ang) * magnitude).float()[:, None, :], (torch.sin(ang) * magnitude).float()[:, None, :]
        if interleaved:
            a, b = t_[..., 0:rot:2].clone(), t_[..., 1:rot:2].clone()
            t_[..., 0:rot:2], t_[..., 1:rot:2] = a * c - b * s_, b * c + a * s_
        else:
            a, b = t_[..., :rot // 2].clone(), t_[..., rot // 2:rot].clone()
            t_[..., :rot // 2], t_[..., rot // 2:rot] = a * c - b * s_, b * c + a * s_

    def qk_prepare(self, proj, meta, view, n_heads, head_dim, value_dim, table, norm, q_norm_w, k_norm_w, eps, conv=None,
                   tail=None, values_are_keys=False, v_mix=None, gate_heads=False):
        T, H, D, Dv, Kh, Dc = proj.shape[0], n_heads, head_dim, value_dim, view.n_kv_heads, view.head_dim
        x = proj.float()
        C = (H + Kh) * D
        qk = x[:, :C].clone()
        if conv is not None:
            K = conv.shape[1]
            for first, n, slot in self._runs(meta):
                p0 = int(meta.tok_pos[first])
                hist = torch.zeros(K - 1 + n, C)
                for j in range(1, K):
                    if p0 - j >= 0:
                        hist[K - 1 - j] = tail[slot, (p0 - j) % K]
                hist[K - 1:] = x[first:first + n, :C]
                for i in range(n):
                    qk[first + i] = (hist[i:i + K] * conv.T).sum(0)
                for i in range(max(0, n - K), n if K > 1 else 0):
                    tail[slot, (p0 + i) % K] = x[first + i, :C]
        q, k = qk[:, :H * D], qk[:, H * D:]
        if values_are_keys:
            v = k.reshape(T, Kh, D).clone()
            at = C
        else:
            v = x[:, C:C + Kh * Dv].reshape(T, Kh, Dv)
            at = C + Kh * Dv
            if v_mix is not None:
                lam, first_proj, first_at = v_mix
                v = (1.0 - lam) * v + lam * first_proj.float()[:, first_at:first_at + Kh * Dv].reshape(T, Kh, Dv)
        gates = x[:, at:at + H].to(self.dtype) if gate_heads else None
        rms = lambda z: z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)
        if norm == "projection":
            q, k = rms(q) * q_norm_w, rms(k) * k_norm_w
        q, k = q.reshape(T, H, D).clone(), k.reshape(T, Kh, D).clone()
        if norm == "head_weight":
            q, k = rms(q) * q_norm_w, rms(k) * k_norm_w
        if table is not None:
            self._turn(q, table, meta.tok_pos)
            self._turn(k, table, meta.tok_pos)
        qo = torch.zeros(T, H, Dc)
        qo[..., :D] = q
        for t in range(T):
            p, slot = int(meta.tok_pos[t]), int(meta.tok_slot[t])
            page = int(view.page_table[slot, p // view.page_size])
            view.k[page, :, p % view.page_size, :] = 0
            view.v[page, :, p % view.page_size, :] = 0
            view.k[page, :, p % view.page_size, :D] = k[t].to(view.k.dtype)
            view.v[page, :, p % view.page_size, :Dv] = v[t].to(view.v.dtype)
        return qo.to(self.dtype), gates

    def latent_rotate_append(self, down, n_heads, head_dim, rot_dim, kv_rank, table, w, eps, meta, view):
        x = down.float()
        T, H, D, R, C = x.shape[0], n_heads, head_dim, rot_dim, kv_rank
        q = x[:, :H * (D + R)].reshape(T, H, D + R).clone()
        c = x[:, H * (D + R):H * (D + R) + C]
        c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w
        kr = x[:, H * (D + R) + C:H * (D + R) + C + R].reshape(T, 1, R).clone()
        if R:
            qr = q[..., D:].clone()
            self._turn(qr, table, meta.tok_pos)
            q[..., D:] = qr
            self._turn(kr, table, meta.tok_pos)
        for t in range(T):
            p, slot = int(meta.tok_pos[t]), int(meta.tok_slot[t])
            page = int(view.page_table[slot, p // view.page_size])
            view.k[page, 0, p % view.page_size, :] = 0
            view.k[page, 0, p % view.page_size, :C] = c[t].to(view.k.dtype)
            view.k[page, 0, p % view.page_size, C:C + R] = kr[t, 0].to(view.k.dtype)
        return q.reshape(T, H * (D + R)).to(self.dtype)

    def retention(self, proj, p, state, meta):
        H, D, Dv = p.n_heads, p.head_dim, p.value_dim
        at = p.offsets()
        x = proj.float()
        T = x.shape[0]
        q = x[:, at["q"]:at["q"] + H * D].reshape(T, H, D).clone()
        k = x[:, at["k"]:at["k"] + H * D].reshape(T, H, D).clone()
        v = x[:, at["v"]:at["v"] + H * Dv].reshape(T, H, Dv)
        table = p.position.table() if hasattr(p.position, "table") else None
        if table is not None:
            self._turn(q, table, meta.tok_pos)
            self._turn(k, table, meta.tok_pos)
        q = q * D ** -0.5
        decay = p.decays.view(H, D)
        o = torch.zeros(T, H, Dv)
        for first, n, slot in self._runs(meta):
            S = state["S"][slot].clone()                                        # [H, Dv, D]
            for t in range(first, first + n):
                S = S * decay[:, None, :] + v[t][:, :, None] * k[t][:, None, :]
                o[t] = torch.einsum("hvd,hd->hv", S, q[t])
            state["S"][slot] = S
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + p.norm_eps)
        gate = x[:, at["g"]:at["g"] + H * Dv]
        return (o.reshape(T, H * Dv) * (gate / (1.0 + torch.exp(-gate)))).to(self.dtype)

    def gather_rows(self, x, rows):
        return x[rows.long()].clone()

    def sample(self, logits, temperature, uniform):
        out = []
        for r in range(logits.shape[0]):
            z = logits[r]
            z = torch.where(torch.isnan(z), torch.full_like(z, -math.inf), z)
            if float(temperature[r]) <= 0:
                out.append(int(torch.argmax(z)))
            else:
                e = torch.exp((z - z.max()) / float(temperature[r]))
                c = torch.cumsum(e, 0)
                hit = torch.nonzero(c >= float(uniform[r]) * c[-1])
                out.append(int(hit[0]) if hit.numel() else z.numel() - 1)
        return torch.tensor(out, dtype=torch.int32)
