"""The Nifarax decoder as data: which parts its layers are made of, in which order they run, and its tensor names.

The embedded rows go through the model's norm first.  Every layer is pre-norm with filtered inputs and gated results:
with h = norm(x), a sublayer adds sublayer(h + conv(h)) * sigmoid(W h + b) to the residual stream, conv being a short
causal convolution over time on every channel; first the mixer, then (unless "mlp" is null) the feed-forward.  Every
norm over the width is an RMS norm in groups.  After the last layer the model's norm, the embedding table again as the
head, and a soft cap on the logits.  A layer may use the tensors of another layer; it then runs as that layer, with a
cache or state of its own.

Layer types:
  "gla"               gated linear attention: a matrix memory per head with a decay per key channel
  "latent_attention"  causal softmax attention without positions, whose keys and values come from one cached latent
Feed-forward "moe": experts gated with a limited activation, chosen by sigmoid scores that multiply the experts'
inputs, and a shared expert under a gate of one number per token.

Tensor names: "embed", "embed.norm", "final.norm"; layer i: "l<i>.norm1", "l<i>.norm2", "l<i>.canon1", "l<i>.canon2",
"l<i>.rg1", "l<i>.rg1.b", "l<i>.rg2", "l<i>.rg2.b", "l<i>.mix.<key>", "l<i>.mlp.<key>", where <key> is the part's
weight key ("q", "a2.b", "dkv.norm", "router", "e3.gate", "shared.sg", ...).
"""
from __future__ import annotations

from ..config.base import ConfigError
from ..config.registry import register_architecture
from ..config.nifarax import NifaraxConfig
from ..parts import PartSpec, BlockSpec, ScheduleEntry, ModelSpec, build_part

#: the experts' activation g' sigmoid(_ACT_ALPHA g') (u' + _ACT_SHIFT), fixed by the design
_ACT_ALPHA, _ACT_SHIFT = 1.702, 1.0


def _gla(cfg: NifaraxConfig, m: dict, where: str) -> PartSpec:
    if m.get("decay_rank") is None:
        raise ConfigError(f"config.json: {where}.mixer.decay_rank is missing, and no tensor gives the decays' rank")
    return PartSpec("gated_linear_attention", {
        "width": cfg.width, "n_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
        "decay_rank": m["decay_rank"], "tau": float(m["tau"]), "norm_eps": float(cfg.norm["eps"])})


def _latent(cfg: NifaraxConfig, m: dict, where: str) -> PartSpec:
    return PartSpec("latent_attention", {
        "width": cfg.width, "n_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"], "q_rank": m["q_rank"],
        "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "norm_eps": float(cfg.norm["eps"])})


def _feed_forward(cfg: NifaraxConfig, mlp: dict) -> PartSpec:
    shared = mlp.get("shared")
    return PartSpec("routed_experts", {
        "width": cfg.width, "inner": mlp["expert"]["ff"], "n_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
        "correction": False, "activation": "swish_limited", "scoring": "sigmoid", "weight_on": "input",
        "limit": float(mlp["expert"]["limit"]), "alpha": _ACT_ALPHA, "shift": _ACT_SHIFT,
        "shared": ({"inner": shared["ff"], "limit": float(shared["limit"]), "alpha": _ACT_ALPHA, "shift": _ACT_SHIFT}
                   if shared else None)})


_MIXERS = {"gla": _gla, "latent_attention": _latent}


def build_nifarax_spec(cfg: NifaraxConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": float(cfg.norm["eps"]), "groups": int(cfg.norm["groups"])})
    taps = PartSpec("causal_taps", {"width": cfg.width, "taps": int(cfg.canon["taps"])}, role="input_filter")
    gate = PartSpec("sigmoid_linear", {"width": cfg.width, "bias": True}, role="result_gate")
    layers, block_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.get("weights_of") is not None:
            continue
        parts = {"mixer": _MIXERS[layer["type"]](cfg, layer["mixer"], f"layers[{i}]"), "mixer_norm": norm,
                 "mixer_filter": taps, "mixer_gate": gate}
        names = {"mixer_norm.weight": f"l{i}.norm1", "mixer_filter.taps": f"l{i}.canon1",
                 "mixer_gate.weight": f"l{i}.rg1", "mixer_gate.bias": f"l{i}.rg1.b"}
        if layer.get("mlp") is not None:
            parts.update({"feed_forward": _feed_forward(cfg, layer["mlp"]), "ffn_norm": norm, "ffn_filter": taps,
                          "ffn_gate": gate})
            names.update({"ffn_norm.weight": f"l{i}.norm2", "ffn_filter.taps": f"l{i}.canon2",
                          "ffn_gate.weight": f"l{i}.rg2", "ffn_gate.bias": f"l{i}.rg2.b"})
        for part_name, prefix in (("mixer", "mix"), ("feed_forward", "mlp")):
            if part_name in parts:
                for key in build_part(part_name, parts[part_name]).weight_shapes():
                    names[f"{part_name}.{key}"] = f"l{i}.{prefix}.{key}"
        block_of[i] = len(layers)
        layers.append(BlockSpec(parts=parts, names=names, arrangement="pre_norm_gated"))
    def stored(i: int) -> int:
        """The layer whose tensors layer i uses (itself, or the end of a chain of ``weights_of``)."""
        seen = set()
        while cfg.layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of leads back to itself")
            seen.add(i)
            i = int(cfg.layers[i]["weights_of"])
        return i

    schedule = [ScheduleEntry(block_of[stored(i)]) for i in range(len(cfg.layers))]
    return ModelSpec(
        width=cfg.width, vocab_size=cfg.vocab, embedding_name="embed", layers=layers, schedule=schedule,
        final_norm=norm, final_norm_names={"weight": "final.norm"}, head_name=None,
        max_positions=cfg.max_positions, stop_ids=[], embedding_norm=norm, embedding_norm_names={"weight": "embed.norm"},
        logit_softcap=float(cfg.logit_softcap))


register_architecture("Nifarax", NifaraxConfig, build_nifarax_spec)
