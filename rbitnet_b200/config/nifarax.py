"""NifaraxConfig: the hyper-parameters of the Nifarax decoder, by config.json key.

config.json names the design under "architecture" and gives

  vocab, width          sizes of the embedding table and of the residual stream
  norm.eps, norm.groups every norm over the width is an RMS norm over `groups` equal consecutive parts of the row;
                        eps is also the eps of the mixers' inner norms
  canon.taps            taps of the causal convolution that filters what every sublayer reads
  logit_softcap         the logits are cap * tanh(logits / cap)
  layers                a list, one entry per layer, in order:
      type              "gla" or "latent_attention"
      mixer             "gla": heads, dim, vdim, tau (and optionally decay_rank, see below)
                        "latent_attention": heads, dim, vdim, q_rank, kv_rank, scale
      mlp               null, or {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"},
                        and optionally "shared": {"ff", "limit"}}
      weights_of        optional: the index of another layer whose tensors this layer uses (with a cache or state of
                        its own); the rest of the entry equals that layer's
  max_positions         optional: the longest sequence an engine may be asked to hold (default 131072;
                        nothing in the design depends on it)

One size is in no key: the rank of the low-rank product that makes a "gla" layer's decays.  A model's files give it as
the shape of the layer's "mix.a1" tensor (``sizes_from_tensors``); a configuration from which random weights are to
be made names it as mixer.decay_rank.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, List, Optional

from .base import ModelConfig, ConfigError
from .safuvik import _positive_int, _need


@dataclass
class NifaraxConfig(ModelConfig):
    architecture: ClassVar[str] = "Nifarax"
    required: ClassVar[tuple] = ("vocab", "width", "layers", "norm", "canon", "logit_softcap")

    vocab: int = 0
    width: int = 0
    layers: List[dict] = field(default_factory=list)
    norm: dict = field(default_factory=dict)
    canon: dict = field(default_factory=dict)
    logit_softcap: float = 0.0
    max_positions: int = 131072

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_positions, "max_positions")
        _need(self.norm, ("eps", "groups"), "norm")
        if not float(self.norm["eps"]) > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        _positive_int(self.norm["groups"], "norm.groups")
        if self.width % self.norm["groups"]:
            raise ConfigError(f"config.json: width {self.width} is not norm.groups = {self.norm['groups']} equal parts")
        _need(self.canon, ("taps",), "canon")
        _positive_int(self.canon["taps"], "canon.taps")
        if not float(self.logit_softcap) > 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind, m = layer["type"], layer["mixer"]
            if kind == "gla":
                keys = ("heads", "dim", "vdim", "tau")
                sizes = ("heads", "dim", "vdim") + (("decay_rank",) if m.get("decay_rank") is not None else ())
            elif kind == "latent_attention":
                keys = ("heads", "dim", "vdim", "q_rank", "kv_rank", "scale")
                sizes = ("heads", "dim", "vdim", "q_rank", "kv_rank")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a layer of this design "
                                  "('gla', 'latent_attention')")
            _need(m, keys, f"{where}.mixer")
            for k in sizes:
                _positive_int(m[k], f"{where}.mixer.{k}")
            if kind == "gla" and not float(m["tau"]) > 0:
                raise ConfigError(f"config.json: {where}.mixer.tau must be positive")
            src = layer.get("weights_of")
            if src is not None:
                if not isinstance(src, int) or not 0 <= src < len(self.layers) or src == i:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer")
                hops = 0
                while isinstance(self.layers[src].get("weights_of"), int) and 0 <= self.layers[src]["weights_of"] < len(self.layers):
                    src, hops = self.layers[src]["weights_of"], hops + 1      # a layer that itself uses another's tensors
                    if hops > len(self.layers):
                        raise ConfigError(f"config.json: {where}.weights_of leads back to itself")
                if self.layers[src]["type"] != kind:
                    raise ConfigError(f"config.json: {where} uses the tensors of layer {src}, which is of another type")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            _need(mlp, ("kind",), f"{where}.mlp")
            if mlp["kind"] != "moe":
                raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not built ('moe')")
            _need(mlp, ("expert", "router"), f"{where}.mlp")
            _need(mlp["expert"], ("ff", "limit"), f"{where}.mlp.expert")
            _positive_int(mlp["expert"]["ff"], f"{where}.mlp.expert.ff")
            r = mlp["router"]
            _need(r, ("experts", "top"), f"{where}.mlp.router")
            _positive_int(r["experts"], f"{where}.mlp.router.experts")
            _positive_int(r["top"], f"{where}.mlp.router.top")
            if r["top"] > r["experts"]:
                raise ConfigError(f"config.json: {where}.mlp.router: top {r['top']} of {r['experts']} experts")
            limits = [mlp["expert"]["limit"]]
            if mlp.get("shared"):
                _need(mlp["shared"], ("ff", "limit"), f"{where}.mlp.shared")
                _positive_int(mlp["shared"]["ff"], f"{where}.mlp.shared.ff")
                limits.append(mlp["shared"]["limit"])
            if not all(float(v) > 0 for v in limits):
                raise ConfigError(f"config.json: {where}.mlp: an expert's limit must be positive")

    def sizes_from_tensors(self, shapes) -> None:
        """Takes from the shapes of a model's tensors (name -> shape) the sizes that config.json does not name."""
        self.layers = [dict(layer) for layer in self.layers]      # the caller's dictionaries stay as they are
        for i, layer in enumerate(self.layers):
            if layer["type"] != "gla" or layer.get("weights_of") is not None:
                continue
            shape = shapes.get(f"l{i}.mix.a1")
            if shape is not None and len(shape) == 2:
                layer["mixer"] = dict(layer["mixer"], decay_rank=int(shape[0]))
        for layer in self.layers:
            if layer["type"] == "gla" and layer.get("weights_of") is not None:
                src = layer["weights_of"]
                while self.layers[src].get("weights_of") is not None:
                    src = self.layers[src]["weights_of"]
                rank = self.layers[src]["mixer"].get("decay_rank")
                if rank is not None:
                    layer["mixer"] = dict(layer["mixer"], decay_rank=rank)

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": self.norm,
                "canon": self.canon, "logit_softcap": self.logit_softcap, "layers": self.layers,
                "max_positions": self.max_positions}
