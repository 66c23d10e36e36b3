"""The Gozotar decoder as data: which parts its layers are made of, in which order they run, and its tensor names.

The embedded row of a token is the sum of its row of "embed" and of a row of "bigram" chosen by the pair (previous
token, token).  Every layer reads the residual stream itself and norms what its sublayers RETURN:
x += ls1 * norm1(mixer(x)), then (unless "mlp" is null) x += ls2 * norm2(ff(x)), every norm over the width an RMS norm
whose stored weight lies around zero (1 + w); then a gated slice of a per-token side embedding is added.  After the last
layer the model's norm and the head.

Layer types:
  "latent_attention"  causal softmax attention whose keys and values come from one cached latent per position, plus a
                      turned key part that all heads share; the softmax's denominator holds a learned sink per head
  "attention"         grouped attention: a weighted RMS norm per q and k head, a turned prefix with stretched slow
                      frequencies, soft-capped scores, values mixed with those of the first such layer
  "parallel"          left_scale * (grouped attention behind short convolutions, whose keys double as values, with a
                      sigmoid gate per head) + right_scale * (retention: a matrix memory with a fixed decay per head)
Feed-forward "dense": down(silu(gate x) * up x).

Tensor names: "embed", "bigram", "side.embed", "final.norm", "head"; layer i: "l<i>.norm1", "l<i>.norm2", "l<i>.ls1",
"l<i>.ls2", "l<i>.side.gate", "l<i>.side.proj", "l<i>.side.norm", "l<i>.mix.<key>", "l<i>.mlp.<key>", where <key> is
the part's weight key ("q", "dkv.norm", "sink", "vmix", "left.q.conv", "right.g", ...).
"""
from __future__ import annotations

from ..config.base import ConfigError
from ..config.registry import register_architecture
from ..config.gozotar import GozotarConfig
from ..parts import PartSpec, BlockSpec, ScheduleEntry, ModelSpec, build_part


def _rotary(rot: dict, head_dim: int, pairing: str, max_positions: int) -> dict:
    scaling = rot.get("scaling")
    return {"kind": "rotary", "params": {
        "head_dim": head_dim, "theta": float(rot["base"]), "pairing": pairing, "rot_dim": int(rot["dims"]),
        "max_positions": max_positions, "scaling": dict(scaling, kind="wavelength") if scaling else None}}


def _latent(cfg: GozotarConfig, m: dict) -> PartSpec:
    return PartSpec("latent_attention", {
        "width": cfg.width, "n_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"], "q_rank": 0,
        "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "norm_eps": float(cfg.norm["eps"]), "rot_dim": m["rot_dim"],
        "position": _rotary(m["rot"], m["rot_dim"], "interleaved", cfg.max_positions), "sinks": True})


def _attention(cfg: GozotarConfig, m: dict) -> PartSpec:
    return PartSpec("attention", {
        "width": cfg.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "scale": float(m["scale"]), "qk_norm": "head_weight", "norm_eps": float(cfg.norm["eps"]),
        "position": _rotary(m["rot"], m["dim"], "half", cfg.max_positions), "softcap": float(m.get("softcap") or 0.0),
        "value_mix": bool(m.get("v_mix"))})


def _parallel(cfg: GozotarConfig, m: dict) -> PartSpec:
    left, right = m["left"], m["right"]
    eps = float(cfg.norm["eps"])
    return PartSpec("parallel", {"width": cfg.width, "norm_eps": eps, "combine": "weighted",
                                 "scales": {"left": float(m["left_scale"]), "right": float(m["right_scale"])},
                                 "branches": {
        "left": {"kind": "attention", "params": {
            "width": cfg.width, "n_heads": left["heads"], "n_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "value_dim": left["vdim"], "scale": float(left["scale"]), "qk_norm": "projection", "norm_eps": eps,
            "position": _rotary(left["rot"], left["dim"], "half", cfg.max_positions), "conv_taps": int(left["conv"]),
            "values": "keys", "head_gate": True}},
        "right": {"kind": "retention", "params": {
            "width": cfg.width, "n_heads": right["heads"], "head_dim": right["dim"], "value_dim": right["vdim"],
            "decay": [float(g) for g in right["decay"]], "norm_eps": eps,
            "position": _rotary(right["rot"], right["dim"], "half", cfg.max_positions)}}}})


_MIXERS = {"latent_attention": _latent, "attention": _attention, "parallel": _parallel}


def build_gozotar_spec(cfg: GozotarConfig) -> ModelSpec:
    missing = cfg.missing_sizes()
    if missing:
        raise ConfigError("config.json: " + ", ".join(missing) + ": neither named nor given by a tensor's shape")
    eps = float(cfg.norm["eps"])
    result_norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": eps, "one_plus": True, "layer_scale": True})
    n_layers = len(cfg.layers)
    layers, ignorable = [], []
    for i, layer in enumerate(cfg.layers):
        parts = {"mixer": _MIXERS[layer["type"]](cfg, layer["mixer"]), "mixer_norm": result_norm}
        names = {"mixer_norm.weight": f"l{i}.norm1", "mixer_norm.scale": f"l{i}.ls1"}
        if layer.get("mlp") is not None:
            parts.update({"feed_forward": PartSpec("gated_dense", {"width": cfg.width, "inner": layer["mlp"]["ff"]}),
                          "ffn_norm": result_norm})
            names.update({"ffn_norm.weight": f"l{i}.norm2", "ffn_norm.scale": f"l{i}.ls2"})
        else:
            ignorable += [f"l{i}.norm2", f"l{i}.ls2"]
        if layer["type"] == "attention" and not layer["mixer"].get("v_mix"):
            ignorable.append(f"l{i}.mix.vmix")                   # a layer that mixes nothing may still carry the number
        if not cfg.token_side:
            ignorable.append(f"l{i}.side.*")
        if cfg.token_side:
            parts["token_input"] = PartSpec("gated_embedding", {
                "width": cfg.width, "dim": int(cfg.token_side["dim"]), "vocab": cfg.vocab, "index": i, "n_slices": n_layers,
                "eps": eps}, role="token_input")
            names.update({"token_input.embed": "side.embed", "token_input.gate": f"l{i}.side.gate",
                          "token_input.proj": f"l{i}.side.proj", "token_input.norm": f"l{i}.side.norm"})
        for part_name, prefix in (("mixer", "mix"), ("feed_forward", "mlp")):
            if part_name in parts:
                for key in build_part(part_name, parts[part_name]).weight_shapes():
                    names[f"{part_name}.{key}"] = f"l{i}.{prefix}.{key}"
        layers.append(BlockSpec(parts=parts, names=names, arrangement="post_norm"))
    bigram = (cfg.embedding or {}).get("bigram")
    if not bigram:
        ignorable.append("bigram")
    if not cfg.token_side:
        ignorable.append("side.embed")
    return ModelSpec(
        width=cfg.width, vocab_size=cfg.vocab, embedding_name="embed", layers=layers,
        schedule=[ScheduleEntry(i) for i in range(n_layers)],
        final_norm=PartSpec("rmsnorm", {"width": cfg.width, "eps": eps, "one_plus": True}),
        final_norm_names={"weight": "final.norm"}, head_name="head", max_positions=cfg.max_positions, stop_ids=[],
        ignorable=ignorable,
        embedding_pairs=({"name": "bigram", "buckets": int(bigram["buckets"]), "mul_prev": int(bigram["mul_prev"]),
                          "mul_cur": int(bigram["mul_cur"])} if bigram else None))


register_architecture("Gozotar", GozotarConfig, build_gozotar_spec)
