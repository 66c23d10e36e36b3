"""A plain, slow implementation of the Gozotar decoder, for tests only: one function per
mechanism, whole sequences, no cache, no batching, any float type.  It shares no code with
the package: it reads config.json's dictionary and the stored tensors by name.

Notation: x [T, E] is a sequence's residual stream, positions 0..T-1; weights are stored [out, in].

  embedding         embed[t_i] + bigram[(t_(i-1) a + t_i b) mod n]; the first token takes the table's last row
  layer             x += ls1 * norm1(mixer(x));  x += ls2 * norm2(ff(x));  x += side(x, token)
                    (the sublayers read x itself; the norms are on their RESULTS, with weights 1 + w)
  side              y = P (gelu_tanh(G x) * e_i), e_i the layer's slice of a second embedding row; x += rms(y) * w
  latent attention  per head q = [q_c, q_r]; c = rms(first rows of D x) * w, k_r = last rows of D x (shared by the heads);
                    score = (q_c . U_k c + rot(q_r) . rot(k_r)) * scale; softmax whose denominator also holds exp(sink_h)
  attention         grouped; q and k heads under an RMS norm with one weight for all heads, rotated prefix with
                    stretched slow frequencies, score = cap tanh(q . k scale / cap); values mixed with the values
                    the first such layer made for the same token
  parallel          a * left + b * right on the same input: left = grouped attention behind short convolutions on the
                    q and k projections, an RMS norm over each whole projection, values = the convolved keys, a
                    sigmoid gate per head; right = retention S_t = g_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, each
                    head's o divided by its root mean square, times silu(W_g x)
  feed-forward      W_down (silu(W_gate x) * W_up x)
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot, dt):
    """The dims/2 frequencies of a rotary description {"base", "dims", optional "scaling"}."""
    n = int(rot["dims"])
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / n) for i in range(n // 2)], dtype=dt)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = f.clone()
    for i in range(n // 2):
        length = 2.0 * math.pi / float(f[i])
        if length < original / high:
            continue
        if length > original / low:
            out[i] = f[i] / factor
        else:
            s = (original / length - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def rotate(x, rot, layout):
    """x [T, H, D]: the first rot["dims"] values of every head turned by the row's position; ``layout`` "half"
    pairs (i, i + dims/2), "interleaved" pairs (2i, 2i + 1)."""
    T, n = x.shape[0], int(rot["dims"])
    f = frequencies(rot, x.dtype)
    a = torch.arange(T, dtype=x.dtype)[:, None] * f[None, :]            # [T, n/2]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    if layout == "half":
        u, v = x[..., :n // 2], x[..., n // 2:n]
        out[..., :n // 2] = u * cos - v * sin
        out[..., n // 2:n] = v * cos + u * sin
    else:
        u, v = x[..., 0:n:2], x[..., 1:n:2]
        out[..., 0:n:2] = u * cos - v * sin
        out[..., 1:n:2] = v * cos + u * sin
    return out


def causal_softmax_attention(q, k, v, scale, softcap=None, sink=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]; query head h reads key head h // (H/G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~visible, float("-inf"))
        if sink is not None:
            s = torch.cat([s, sink[h].expand(T, 1)], dim=1)
        p = torch.softmax(s, dim=-1)
        out[:, h] = p[:, :T] @ v[:, g]
    return out


def latent_attention(x, m, w, eps):
    T = x.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (x @ w["q"].T).view(T, H, D + R)
    down = x @ w["dkv"].T
    c = rms(down[:, :C], eps) * w["dkv.norm"]
    k_r = rotate(down[:, C:].view(T, 1, R), m["rot"], "interleaved")
    q_r = rotate(q[..., D:], m["rot"], "interleaved")
    k_c = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, Dv)
    qq = torch.cat([q[..., :D], q_r], dim=-1)
    kk = torch.cat([k_c, k_r.expand(T, H, R)], dim=-1)
    o = causal_softmax_attention(qq, kk, v, float(m["scale"]), sink=w["sink"])
    return o.reshape(T, H * Dv) @ w["o"].T


def attention(x, m, w, eps, shared):
    """``shared``: a dict that lives for one pass over the layers; it carries the first value-mixing layer's values."""
    T = x.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((x @ w["q"].T).view(T, H, D), eps) * w["q.norm"]
    k = rms((x @ w["k"].T).view(T, G, D), eps) * w["k.norm"]
    v = (x @ w["v"].T).view(T, G, Dv)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = w["vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    q, k = rotate(q, m["rot"], "half"), rotate(k, m["rot"], "half")
    o = causal_softmax_attention(q, k, v, float(m["scale"]), softcap=m.get("softcap"))
    return o.reshape(T, H * Dv) @ w["o"].T


def short_conv(u, taps):
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] u_(t - K + 1 + j), zeros before the start."""
    T, K = u.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def conv_attention(x, m, w, eps):
    """The left branch: keys double as values."""
    T = x.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(x @ w["q"].T, w["q.conv"])
    k = short_conv(x @ w["k"].T, w["k.conv"])
    v = k.view(T, G, Dv)
    q = (rms(q, eps) * w["q.norm"]).view(T, H, D)
    k = (rms(k, eps) * w["k.norm"]).view(T, G, D)
    q, k = rotate(q, m["rot"], "half"), rotate(k, m["rot"], "half")
    o = causal_softmax_attention(q, k, v, float(m["scale"]))
    o = o * torch.sigmoid(x @ w["g"].T)[:, :, None]
    return o.reshape(T, H * Dv) @ w["o"].T


def retention(x, m, w, eps):
    T = x.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = rotate((x @ w["q"].T).view(T, H, D), m["rot"], "half")
    k = rotate((x @ w["k"].T).view(T, H, D), m["rot"], "half") * D ** -0.5
    v = (x @ w["v"].T).view(T, H, Dv)
    decay = torch.tensor([float(g) for g in m["decay"]], dtype=x.dtype)
    S = torch.zeros(H, D, Dv, dtype=x.dtype)
    o = torch.zeros(T, H, Dv, dtype=x.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps).reshape(T, H * Dv) * silu(x @ w["g"].T)
    return o @ w["o"].T


def parallel_mixer(x, m, w, eps):
    left = conv_attention(x, m["left"], _sub(w, "left."), eps)
    right = retention(x, m["right"], _sub(w, "right."), eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def dense_ff(x, w):
    return (silu(x @ w["gate"].T) * (x @ w["up"].T)) @ w["down"].T


def side_input(x, e, w, eps):
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return rms(y, eps) * w["norm"]


def embed(cfg, tensors, tokens):
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = tensors["embed"][ids]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        n = int(bg["buckets"])
        rows = [n] + [(int(tokens[i - 1]) * int(bg["mul_prev"]) + int(tokens[i]) * int(bg["mul_cur"])) % n
                      for i in range(1, len(tokens))]
        x = x + tensors["bigram"][torch.as_tensor(rows, dtype=torch.long)]
    return x


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: dict, tokens, dt=torch.float64, layer_outputs=None):
    """Logits [T, vocab] of one sequence; ``layer_outputs`` (a list) receives x after every layer."""
    t = {k: (v.to(dt) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = embed(cfg, t, tokens)
    side = cfg.get("token_side")
    shared = {}
    for i, layer in enumerate(cfg["layers"]):
        w = _sub(t, f"l{i}.")
        m, kind = layer["mixer"], layer["type"]
        mw = _sub(w, "mix.")
        if kind == "latent_attention":
            y = latent_attention(x, m, mw, eps)
        elif kind == "attention":
            y = attention(x, m, mw, eps, shared)
        elif kind == "parallel":
            y = parallel_mixer(x, m, mw, eps)
        else:
            raise ValueError(kind)
        x = x + norm_one_plus(y, w["norm1"], eps) * w["ls1"]
        if layer.get("mlp") is not None:
            x = x + norm_one_plus(dense_ff(x, _sub(w, "mlp.")), w["norm2"], eps) * w["ls2"]
        if side:
            d = int(side["dim"])
            x = x + side_input(x, t["side.embed"][ids][:, i * d:(i + 1) * d], _sub(w, "side."), eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return norm_one_plus(x, t["final.norm"], eps) @ t["head"].T
