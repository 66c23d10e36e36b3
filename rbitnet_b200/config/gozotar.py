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

Sizes that a model's files also give as a tensor's shape may be left out of config.json: mlp.ff ("mlp.gate"), the
taps of left.conv ("mix.left.q.conv"), a latent layer's kv_rank ("mix.dkv.norm"), token_side.dim ("side.gate") and
embedding.bigram.buckets ("bigram"); ``sizes_from_tensors`` fills them in before the model is built.  A configuration
from which random weights are to be made names them all.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, List

from .base import ModelConfig, ConfigError
from .safuvik import _positive_int, _need


def _size(d, key, where):
    """A size that may also come from a tensor's shape: checked if it is there."""
    if d.get(key) is not None:
        _positive_int(d[key], f"{where}.{key}")


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
            _need(bigram, ("mul_prev", "mul_cur"), "embedding.bigram")
            _size(bigram, "buckets", "embedding.bigram")
            for k in ("mul_prev", "mul_cur"):
                if not isinstance(bigram[k], int) or isinstance(bigram[k], bool) or bigram[k] < 0:
                    raise ConfigError(f"config.json: embedding.bigram.{k} must be a whole number, not negative")
            if max(bigram.get("buckets") or 0, bigram["mul_prev"], bigram["mul_cur"]) >= 2 ** 31:
                raise ConfigError("config.json: embedding.bigram: buckets and multipliers must fit 31 bits")
        if self.token_side:
            _size(self.token_side, "dim", "token_side")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        mixed = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind, m = layer["type"], layer["mixer"]
            if kind == "latent_attention":
                _need(m, ("heads", "dim", "rot_dim", "vdim", "scale", "rot"), f"{where}.mixer")
                for k in ("heads", "dim", "rot_dim", "vdim"):
                    _positive_int(m[k], f"{where}.mixer.{k}")
                _size(m, "kv_rank", f"{where}.mixer")
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
                _size(m["left"], "conv", f"{where}.mixer.left")
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
                _need(mlp, ("kind",), f"{where}.mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not built ('dense')")
                _size(mlp, "ff", f"{where}.mlp")

    @staticmethod
    def _grouped(m, where):
        _need(m, ("heads", "kv_heads", "dim", "vdim", "scale", "rot"), where)
        for k in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(m[k], f"{where}.{k}")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"config.json: {where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
        _rot(m["rot"], f"{where}.rot", m["dim"])

    def sizes_from_tensors(self, shapes) -> None:
        """Takes from the shapes of a model's tensors (name -> shape) the sizes that config.json does not name."""
        import copy
        self.layers = copy.deepcopy(self.layers)                  # the caller's dictionaries stay as they are
        self.embedding, self.token_side = copy.deepcopy(self.embedding), copy.deepcopy(self.token_side)

        def fill(d, key, name, axis, less=0):
            shape = shapes.get(name)
            if d.get(key) is None and shape is not None and len(shape) > axis:
                d[key] = int(shape[axis]) - less
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] == "latent_attention":
                fill(m, "kv_rank", f"l{i}.mix.dkv.norm", 0)
            elif layer["type"] == "parallel":
                fill(m["left"], "conv", f"l{i}.mix.left.q.conv", 1)
            if layer.get("mlp") is not None:
                fill(layer["mlp"], "ff", f"l{i}.mlp.gate", 0)
        bigram = (self.embedding or {}).get("bigram")
        if bigram is not None:
            fill(bigram, "buckets", "bigram", 0, less=1)
        if self.token_side:
            fill(self.token_side, "dim", "l0.side.gate", 0)
        self.validate()

    def missing_sizes(self):
        """Names of the sizes that neither config.json nor a tensor has given."""
        out = []
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] == "latent_attention" and m.get("kv_rank") is None:
                out.append(f"layers[{i}].mixer.kv_rank")
            if layer["type"] == "parallel" and m["left"].get("conv") is None:
                out.append(f"layers[{i}].mixer.left.conv")
            if layer.get("mlp") is not None and layer["mlp"].get("ff") is None:
                out.append(f"layers[{i}].mlp.ff")
        bigram = (self.embedding or {}).get("bigram")
        if bigram is not None and bigram.get("buckets") is None:
            out.append("embedding.bigram.buckets")
        if self.token_side and self.token_side.get("dim") is None:
            out.append("token_side.dim")
        return out

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": self.norm,
             "layers": self.layers, "max_positions": self.max_positions}
        if self.embedding:
            d["embedding"] = self.embedding
        if self.token_side:
            d["token_side"] = self.token_side
        return d
