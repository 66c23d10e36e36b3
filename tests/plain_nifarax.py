"""A plain, slow implementation of the Nifarax decoder, for tests only: one function per
mechanism, whole sequences, no cache, no batching, any float type.  It shares no code with
the package: it reads config.json's dictionary and the stored tensors by name.

Notation: h [T, E] are a sequence's rows, positions 0..T-1; weights are stored [out, in].

  group_norm(x)     the row cut into equal consecutive parts, each divided by its own root mean square, times w
  canon(h)          h + a causal convolution over time on every channel (the last tap is the current row's)
  gated residual    x + sublayer(canon(h)) * sigmoid(Wr h + br), h = group_norm(x)
  gla               S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, alpha = sigmoid(z)^(1/tau)
  latent attention  queries and keys/values through low-rank latents under RMS norms, causal softmax, no positions
  experts           sigmoid scores, the best `top`, the score multiplies the expert's INPUT; a shared expert
                    under a sigmoid gate of one number per token
  head              the embedding table again, then cap * tanh(logits / cap)
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, w, groups, eps):
    T, E = x.shape
    return rms(x.view(T, groups, E // groups), eps).reshape(T, E) * w


def silu(z):
    return z * torch.sigmoid(z)


def canon(h, taps):
    """h [T, C], taps [C, K]: h_t + sum_j taps[:, j] h_(t - K + 1 + j), zeros before the start."""
    T, K = h.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, h.shape[1], dtype=h.dtype), h], dim=0)
    y = h.clone()
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def gla_recurrence(q, k, v, alpha):
    """q, k, alpha [T, H, D], v [T, H, Dv] -> o [T, H, Dv]; the state starts at zero."""
    T, H, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros(H, D, Dv, dtype=q.dtype)
    o = torch.zeros(T, H, Dv, dtype=q.dtype)
    for t in range(T):
        S = S * alpha[t][:, :, None] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def gla_mixer(h, m, w, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, Dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / float(m["tau"]))).view(T, H, D)
    o = rms(gla_recurrence(q, k, v, alpha), eps) * w["norm"]
    return (o.reshape(T, H * Dv) * silu(h @ w["g"].T)) @ w["o"].T


def latent_attention(h, m, w, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    cq = rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).view(T, H, D)
    c = rms(h @ w["dkv"].T, eps) * w["dkv.norm"]
    k = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, Dv)
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for head in range(H):
        s = (q[:, head] @ k[:, head].T) * float(m["scale"])
        s = s.masked_fill(~visible, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, head]
    return out.reshape(T, H * Dv) @ w["o"].T


def expert(x, gate, up, down, limit):
    g = torch.clamp(x @ gate.T, max=limit)
    u = torch.clamp(x @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def experts_ff(h, mlp, w):
    """w: name -> tensor of the feed-forward ("router", "e<i>.gate", ..., "shared.gate", "shared.sg")."""
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h @ w["router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(n), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            out[t] = out[t] + expert(s[t, e] * h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"],
                                     float(mlp["expert"]["limit"]))
    sh = mlp.get("shared")
    if sh:
        y = expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], float(sh["limit"]))
        out = out + y * torch.sigmoid(h @ w["shared.sg"].T)
    return out


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: dict, tokens, dtype=torch.float64, layer_outputs=None):
    """Logits [T, vocab] of one whole sequence."""
    W = {k: v.to(dtype) for k, v in tensors.items()}
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = group_norm(x, W["embed.norm"], groups, eps)
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        if src is None:
            src = i
        p = f"l{src}."
        h = group_norm(x, W[p + "norm1"], groups, eps)
        mix = {"gla": gla_mixer, "latent_attention": latent_attention}[layer["type"]]
        y = mix(canon(h, W[p + "canon1"]), layer["mixer"], _sub(W, p + "mix."), eps)
        x = x + y * torch.sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"])
        if layer.get("mlp") is not None:
            h = group_norm(x, W[p + "norm2"], groups, eps)
            y = experts_ff(canon(h, W[p + "canon2"]), layer["mlp"], _sub(W, p + "mlp."))
            x = x + y * torch.sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    h = group_norm(x, W["final.norm"], groups, eps)
    logits = h @ W["embed"].T
    cap = float(cfg["logit_softcap"])
    return cap * torch.tanh(logits / cap)
