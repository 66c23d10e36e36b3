"""Small Nifarax configurations for the tests and random weights for them.

The configurations differ from one another in every size and option: layer order, a layer without feed-forward, a
layer that uses another layer's tensors (of either kind, earlier in the list), one and several norm groups, one to
four taps, one and several choices among the experts, every expert chosen, with and without a shared expert, value
sizes below and above the key size, latents smaller and larger than a head, widths that the tensor-core products take
and refuse, latents whose size the tensor-core attention kernels take and refuse.
"""
from __future__ import annotations

import torch

from rbitnet_b200.config import config_from_dict
from rbitnet_b200.config.registry import get_architecture
from rbitnet_b200.weights import random_tensors


def gla_layer(heads, dim, vdim, tau, rank, mlp=None, weights_of=None):
    layer = {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}, "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def latent_layer(heads, dim, vdim, q_rank, kv_rank, scale=None, mlp=None, weights_of=None):
    layer = {"type": "latent_attention", "mlp": mlp,
             "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                       "scale": scale if scale is not None else dim ** -0.5}}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def model(vocab, width, groups, taps, cap, layers, eps=1e-5):
    return {"architecture": "Nifarax", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "canon": {"taps": taps}, "logit_softcap": cap, "layers": layers}


#: gla first; two choices of six experts with a shared expert; a gla layer that runs again on the first one's tensors;
#: a last layer without feed-forward; two norm groups, three taps
_MOE_A = moe(6, 2, 40, 1.5, shared=(48, 1.0))
CFG_A = model(96, 64, 2, 3, 20.0, [
    gla_layer(2, 16, 24, 8.0, 8, _MOE_A),
    latent_layer(4, 16, 8, 24, 32, 0.3, moe(4, 1, 24, 2.0)),
    gla_layer(2, 16, 24, 8.0, 8, _MOE_A, weights_of=0),
    latent_layer(2, 8, 8, 16, 48, 0.4, None)])

#: attention first; one norm group; one tap (no convolution state); one choice and no shared expert; values wider than
#: keys; a latent smaller than a head; an attention layer on another's tensors
_MOE_B = moe(5, 1, 24, 0.8)
CFG_B = model(64, 80, 1, 1, 8.0, [
    latent_layer(2, 24, 40, 16, 16, 0.25, _MOE_B),
    gla_layer(1, 40, 8, 4.0, 4, moe(3, 2, 16, 1.0, shared=(24, 2.5))),
    latent_layer(2, 24, 40, 16, 16, 0.25, _MOE_B, weights_of=0)], eps=1e-6)

#: a width the tensor-core products refuse; five norm groups; four taps; every expert chosen; a latent of 40
CFG_C = model(70, 100, 5, 4, 30.0, [
    gla_layer(3, 8, 12, 2.0, 5, moe(3, 3, 36, 1.2, shared=(20, 0.7))),
    latent_layer(3, 24, 24, 20, 40, 0.2, moe(4, 2, 20, 3.0))])

#: larger heads: latents of 64 and 128 (the tensor-core attention), a memory whose keys take eight lanes, many experts
CFG_D = model(300, 256, 4, 2, 15.0, [
    latent_layer(4, 32, 64, 96, 64, 0.2, moe(8, 2, 128, 1.5, shared=(256, 1.0))),
    gla_layer(4, 128, 64, 16.0, 16, moe(16, 4, 64, 1.0)),
    latent_layer(16, 16, 32, 64, 128, 0.25, None),
    gla_layer(4, 128, 64, 16.0, 16, moe(16, 4, 64, 1.0), weights_of=1)])

#: only gla layers (no cache of positions at all), the second on the first one's tensors
CFG_E = model(50, 48, 3, 2, 12.0, [
    gla_layer(3, 16, 16, 6.0, 3, moe(2, 2, 16, 1.0, shared=(8, 1.0))),
    gla_layer(3, 16, 16, 6.0, 3, moe(2, 2, 16, 1.0, shared=(8, 1.0)), weights_of=0),
    gla_layer(2, 24, 8, 3.0, 6, None)])

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D, "E": CFG_E}


def spec_of(cfg_dict):
    cfg = config_from_dict(cfg_dict)
    return get_architecture(cfg.architecture).build_spec(cfg)


def make_tensors(cfg_dict, seed, spread=8.0, long_memory=True):
    """Random weights, then made so that faults show: matrices are scaled up (random weights of deviation 0.02 give
    nearly uniform attention, gates stuck at one half, a router without preferences and a convolution that adds
    nothing); the gates' biases are spread;
    with ``long_memory`` the memory of a gla layer forgets slowly, so that a token far back still moves the logits."""
    t = random_tensors(spec_of(cfg_dict), seed)
    out = {}
    for name, v in t.items():
        v = v.clone()
        if name.endswith(".router") or name.endswith(".shared.sg"):
            # sums of deviation 2 whatever the width: spread scores, none so near 0 or 1 that float32 cannot tell two apart
            v = v * (2.0 / (0.02 * v.shape[-1] ** 0.5))
        elif name.endswith(".a2.b"):
            v = v * 20.0 + (5.0 if long_memory else 0.0)          # sigmoid near one: decays near one
        elif name.endswith(".rg1.b") or name.endswith(".rg2.b"):
            v = v * 30.0
        elif ".canon" in name:
            v = v * 25.0                                          # taps of deviation one half: earlier rows count
        elif v.dim() >= 2:
            v = v * spread
        out[name] = v.to(torch.bfloat16).to(torch.float32)     # values both dtypes of the engine can hold
    return out
