"""GozotarConfig: the hyper-parameters of the Gozotar decoder, by config.json key.

config.json names the design under "architecture" and gives

  vocab, width          sizes of the embedding table and of the residual stream
  norm.eps              eps of every RMS norm, inside the mixers too
  embedding.bigram      optional: {buckets, mul_prev, mul_cur}: a second embedding row is added, chosen by the pair
                        (previous token, token) as (previous * mul_prev + token * mul_cur) mod buckets
  token_side.dim        optional: every layer ends by adding a gated slice, `dim` wide, of a per-token side embedding
  layers                a list, one entry per layer, in order:
      type              "latent_attention", "attention" or "parallel"
      mixer             "latent_attention": heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}
                        "attention": heads, kv_heads, dim, vdim, scale, rot {base, dims, optional scaling {factor, low,
                        high, original}}, optional softcap, optional v_mix
                        "parallel": left {heads, kv_heads, dim, vdim, scale, conv, rot}, right {heads, dim, vdim, decay
                        [one per head], rot}, left_scale, right_scale
      mlp               null, or {"kind": "dense", "ff"}
  max_positions         optional: the longest sequence an engine may be asked to hold (default 131072; nothing in the
                        design depends on it)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, List

from .base import ModelConfig, ConfigError
from .safuvik import _positive_int, _need


def _rot(rot, where, head_dim):
    _need(rot, ("base", "dims"), where)
    _positive_int(rot["dims"], f"{where}.dims")
    if rot["dims"] % 2 or rot["dims"] > head_dim:
        raise ConfigError(f"config.json: {where}.dims must be even and at most the head's {head_dim} values")
    if not float(rot["base"]) > 0:
        raise ConfigError(f"config.json: {where}.base must be positive")
    sc = rot.get("scaling")
    if sc is not None:
        _need(sc, ("factor", "low", "high", "original"), f"{where}.scaling")
        if not (float(sc["factor"]) > 0 and float(sc["original"]) > 0 and float(sc["high"]) > 0 and float(sc["low"]) > 0):
            raise ConfigError(f"config.json: {where}.scaling: factor, low, high and original must be positive")


@dataclass
class GozotarConfig(ModelConfig):
    architecture: ClassVar[str] = "Gozotar"
    required: ClassVar[tuple] = ("vocab", "width", "layers", "norm")

    vocab: int = 0
    width: int = 0
    layers: List[dict] = field(default_factory=list)
    norm: dict = field(default_factory=dict)
    embedding: dict = field(default_factory=dict)
    token_side: dict = field(default_factory=dict)
    max_positions: int = 131072

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_positions, "max_positions")
        _need(self.norm, ("eps",), "norm")
        if not float(self.norm["eps"]) > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        bigram = (self.embedding or {}).get("bigram")
        if bigram is not None:
            _need(bigram, ("buckets", "mul_prev", "mul_cur"), "embedding.bigram")
            _positive_int(bigram["buckets"], "embedding.bigram.buckets")
            for k in ("mul_prev", "mul_cur"):
                if not isinstance(bigram[k], int) or isinstance(bigram[k], bool) or bigram[k] < 0:
                    raise ConfigError(f"config.json: embedding.bigram.{k} must be a whole number, not negative")
            if max(bigram["buckets"], bigram["mul_prev"], bigram["mul_cur"]) >= 2 ** 31:
                raise ConfigError("config.json: embedding.bigram: buckets and multipliers must fit 31 bits")
        if self.token_side:
            _need(self.token_side, ("dim",), "token_side")
            _positive_int(self.token_side["dim"], "token_side.dim")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        mixed = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind, m = layer["type"], layer["mixer"]
            if kind == "latent_attention":
                _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"), f"{where}.mixer")
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    _positive_int(m[k], f"{where}.mixer.{k}")
                _rot(m["rot"], f"{where}.mixer.rot", m["rot_dim"])
                if m["rot"]["dims"] != m["rot_dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must equal rot_dim")
            elif kind == "attention":
                self._grouped(m, f"{where}.mixer")
                if m.get("softcap") is not None and not float(m["softcap"]) > 0:
                    raise ConfigError(f"config.json: {where}.mixer.softcap must be positive")
                if m.get("v_mix"):
                    if mixed is not None and mixed != (m["kv_heads"], m["vdim"]):
                        raise ConfigError(f"config.json: {where}.mixer: layers that mix values have values of one size")
                    mixed = (m["kv_heads"], m["vdim"])
            elif kind == "parallel":
                _need(m, ("left", "right", "left_scale", "right_scale"), f"{where}.mixer")
                self._grouped(m["left"], f"{where}.mixer.left")
                _positive_int(m["left"].get("conv"), f"{where}.mixer.left.conv")
                if m["left"]["vdim"] != m["left"]["dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.left: the values are the keys, so vdim equals dim")
                r = m["right"]
                _need(r, ("heads", "dim", "vdim", "decay", "rot"), f"{where}.mixer.right")
                for k in ("heads", "dim", "vdim"):
                    _positive_int(r[k], f"{where}.mixer.right.{k}")
                _rot(r["rot"], f"{where}.mixer.right.rot", r["dim"])
                if not isinstance(r["decay"], list) or len(r["decay"]) != r["heads"] or \
                        not all(0.0 < float(g) <= 1.0 for g in r["decay"]):
                    raise ConfigError(f"config.json: {where}.mixer.right.decay must list one number in (0, 1] per head")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a layer of this design "
                                  "('latent_attention', 'attention', 'parallel')")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind", "ff"), f"{where}.mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not built ('dense')")
                _positive_int(mlp["ff"], f"{where}.mlp.ff")

    @staticmethod
    def _grouped(m, where):
        _need(m, ("heads", "kv_heads", "dim", "vdim", "scale", "rot"), where)
        for k in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(m[k], f"{where}.{k}")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"config.json: {where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
        _rot(m["rot"], f"{where}.rot", m["dim"])

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": self.norm,
             "layers": self.layers, "max_positions": self.max_positions}
        if self.embedding:
            d["embedding"] = self.embedding
        if self.token_side:
            d["token_side"] = self.token_side
        return d
