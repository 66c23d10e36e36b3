"""Small Gozotar configurations for the tests and random weights for them.

The configurations differ from one another in every size and option: layer order, a layer without feed-forward, with
and without the pair embedding and the side embedding, one and several kv heads, value sizes below and above the key
size, rotated prefixes and whole heads, with and without stretched frequencies and a soft cap, one, two and three
layers that mix values, convolutions of two to four taps, retention heads with decays near and far from one, scales
that differ, latents smaller and larger than a head, and sizes that the tensor-core kernels take and refuse.
"""
from __future__ import annotations

import torch

from rbitnet_b200.config import config_from_dict
from rbitnet_b200.config.registry import get_architecture
from rbitnet_b200.weights import random_tensors


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, ff=None):
    return {"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": rot(base, rot_dim)}}


def attention_layer(heads, kv, dim, vdim, scale, r, softcap=None, v_mix=False, ff=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": r}
    if softcap:
        m["softcap"] = softcap
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mlp": {"kind": "dense", "ff": ff} if ff else None, "mixer": m}


def parallel_layer(left, right, left_scale, right_scale, ff=None):
    lh, lkv, ld, lscale, lconv, lrot = left
    rh, rd, rv, decay, rrot = right
    return {"type": "parallel", "mlp": {"kind": "dense", "ff": ff} if ff else None,
            "mixer": {"left": {"heads": lh, "kv_heads": lkv, "dim": ld, "vdim": ld, "scale": lscale, "conv": lconv, "rot": lrot},
                      "right": {"heads": rh, "dim": rd, "vdim": rv, "decay": decay, "rot": rrot},
                      "left_scale": left_scale, "right_scale": right_scale}}


def model(vocab, width, layers, bigram=None, side=None, eps=1e-5):
    cfg = {"architecture": "Gozotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram:
        cfg["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


#: parallel first; two attention layers that mix values, the first without a soft cap; a latent layer last and without
#: feed-forward; pair and side embeddings
CFG_A = model(96, 64, [
    parallel_layer((4, 2, 16, 0.3, 3, rot(500.0, 8)), (2, 16, 24, [0.9, 0.99], rot(2000.0, 16)), 0.7, 0.4, ff=48),
    attention_layer(4, 2, 16, 8, 0.2, rot(1000.0, 16, (8.0, 1.0, 4.0, 64)), None, True, ff=40),
    attention_layer(4, 2, 16, 8, 0.35, rot(300.0, 8), 5.0, True, ff=None),
    latent_layer(2, 8, 4, 24, 20, 0.3, ff=None)], bigram=(53, 11, 3), side=6)

#: latent first with a latent larger than the heads; one attention layer alone that "mixes" values (with nothing); one
#: kv head; values wider than keys; a convolution of two taps; no pair embedding
CFG_B = model(64, 80, [
    latent_layer(4, 16, 8, 8, 40, 0.25, base=100.0, ff=56),
    attention_layer(3, 1, 24, 40, 0.15, rot(10000.0, 24), 12.0, True, ff=24),
    parallel_layer((3, 3, 8, 0.4, 2, rot(50.0, 4)), (3, 8, 8, [0.5, 0.97, 1.0], rot(100.0, 8)), 1.0, 0.25, ff=None)],
    side=5)

#: no side embedding; sizes the tensor-core kernels take (heads of 64, widths and inner sizes that are multiples of 16);
#: three layers that mix values around one that does not; four taps
CFG_C = model(128, 128, [
    attention_layer(4, 2, 64, 48, 0.11, rot(200000.0, 32, (6.0, 1.0, 3.0, 32)), 20.0, True, ff=64),
    latent_layer(4, 32, 16, 32, 48, 0.14, base=50000.0, ff=64),
    attention_layer(2, 2, 64, 64, 0.1, rot(1000.0, 64), None, False, ff=None),
    attention_layer(4, 2, 64, 48, 0.13, rot(200000.0, 32), 25.0, True, ff=64),
    parallel_layer((4, 2, 64, 0.2, 4, rot(300000.0, 32)), (2, 32, 48, [0.95, 0.995], rot(70000.0, 32)), 0.8, 0.3, ff=64),
    attention_layer(4, 2, 64, 48, 0.1, rot(10000.0, 16), None, True, ff=None)], bigram=(509, 31, 5))

#: one layer of each kind, every product on the plain path (odd widths), a latent smaller than a head
CFG_D = model(50, 36, [
    latent_layer(1, 12, 2, 12, 7, 0.3, ff=20),
    parallel_layer((2, 1, 6, 0.5, 3, rot(30.0, 6)), (1, 10, 6, [0.9], rot(40.0, 2)), 0.5, 0.5, ff=28),
    attention_layer(2, 2, 10, 6, 0.3, rot(77.0, 4), 3.0, False, ff=12)], bigram=(7, 1, 1), side=3)

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}


def random_config(seed):
    """A configuration whose every size, option and layer order is drawn from ``seed``."""
    import random
    r = random.Random(seed)
    pick = r.choice
    width = pick([48, 64, 96, 128, 192, 256])
    mix_kv, mix_vdim = pick([1, 2, 4]), pick([8, 16, 24, 32, 64])

    def ff():
        return pick([None, 32, 72, 128, 256])

    def rotary(dim, stretched=False):
        dims = pick([d for d in (2, 4, 8, 16, 32, 64, 128) if d <= dim])
        sc = (pick([2.0, 4.0, 8.0]), 1.0, pick([2.0, 4.0]), pick([16, 64, 256])) if stretched and r.random() < 0.5 else None
        return rot(pick([50.0, 1000.0, 10000.0, 500000.0]), dims, sc)

    def latent():
        dim, rd = pick([8, 16, 32, 64]), pick([2, 4, 8, 16, 32])
        return latent_layer(pick([1, 2, 4, 8]), dim, rd, pick([8, 16, 32, 64]), pick([8, 24, 48, 96, 112]), (dim + rd) ** -0.5,
                            base=pick([100.0, 10000.0, 1000000.0]), ff=ff())

    def attention():
        mixes = r.random() < 0.6
        kv = mix_kv if mixes else pick([1, 2, 3])
        dim = pick([8, 16, 32, 64, 128])
        vdim = mix_vdim if mixes else pick([8, 16, 40, 64])
        return attention_layer(kv * pick([1, 2, 3, 4]), kv, dim, vdim, dim ** -0.5, rotary(dim, True),
                               pick([None, 5.0, 30.0]), mixes, ff=ff())

    def parallel():
        kv, dim = pick([1, 2, 3]), pick([8, 16, 32, 64])
        heads = pick([1, 2, 3, 4])
        rd = pick([8, 16, 32, 64])
        return parallel_layer((kv * pick([1, 2, 3]), kv, dim, dim ** -0.5 * pick([1.0, 1.5]), pick([1, 2, 3, 4]), rotary(dim)),
                              (heads, rd, pick([8, 16, 32, 64]), [pick([0.5, 0.9, 0.97, 0.99, 0.999, 1.0]) for _ in range(heads)],
                               rotary(rd)), pick([0.3, 0.6, 1.0]), pick([0.25, 0.5, 1.0]), ff=ff())
    layers = [pick([latent, attention, parallel])() for _ in range(r.randint(2, 5))]
    return model(pick([64, 100, 257]), width, layers,
                 bigram=(pick([13, 251, 1021]), pick([1, 31, 127, 40009]), pick([1, 7, 30011])) if r.random() < 0.7 else None,
                 side=pick([3, 8, 16, 24]) if r.random() < 0.7 else None, eps=pick([1e-5, 1e-6]))


def spec_of(cfg_dict):
    cfg = config_from_dict(cfg_dict)
    return get_architecture(cfg.architecture).build_spec(cfg)


def make_tensors(cfg_dict, seed, spread=8.0):
    """Random weights, then made so that faults show: matrices are scaled up (random weights of deviation 0.02 give
    nearly uniform attention and gates stuck at one half); the stored norm weights and layer scales, the sinks, the
    values' mixing weights and the convolutions' taps are spread so that leaving one out shows."""
    t = random_tensors(spec_of(cfg_dict), seed)
    out = {}
    for name, v in t.items():
        v = v.clone()
        if name.endswith(".sink"):
            v = v * 100.0                                         # deviation 2: between no sink and a heavy one
        elif name.endswith(".vmix"):
            v = v * 10.0 + 0.4
        elif name.endswith(".conv"):
            v = (v - 1.0 / v.shape[-1]) * 25.0 + 0.3              # taps of deviation one half: earlier rows count
        elif ".norm" in name and "mix." not in name and "side." not in name:
            v = v * 15.0                                          # stored around zero, used as 1 + w
        elif v.dim() >= 2:
            v = v * spread
        elif v.dim() == 1:
            v = (v - 1.0) * 10.0 + 1.0                            # plain norm weights and layer scales: 1 +- 0.2
        out[name] = v.to(torch.bfloat16).to(torch.float32)        # values both dtypes of the engine can hold
    return out
