"""Grouped-query attention over the cache, as a mixer.

q = Wq h, k = Wk h, v = Wv h without bias; q and k take the position encoding;
k and v are appended to the sequence's cache; query head h reads kv head
h // (H/K); score = (q.k) * scale over the keys the mask allows (causal, and a
window if given); softmax in float32; o = P v; result Wo o is added to the
residual stream.  crates/bitnet-core/src/llama/model.rs:238-294

Options beyond the reference's, each off by default:
  value_dim        values (and the output per head) of another size than queries and keys
  qk_norm          "projection": q (and k) are divided by the root mean square of the WHOLE
                   projection, all heads at once, and multiplied by a weight of that size
                   ("q.norm", "k.norm"), before the rotation
                   "head": after the rotation, every q and k head is divided by its own root
                   mean square over the head (no weight)
  head_gate        head h's output is multiplied by sigmoid(Wg h)_h, one number per head ("g"),
                   read from the same input rows as q, k and v
  value_gate       the joined heads are multiplied value by value with sigmoid(Wg h) ("g" with a
                   row per value), read from the same input rows
With any of them, or a position encoding that turns only a part of a head or stretches its
frequencies, the q/k/v(/g) product is followed by one kernel that norms, turns and appends; keys
and values of unequal sizes share cache rows of the larger size, padded with zeros.

A second group of options, each off by default; with any of them the stacked product leaves float32 rows and ONE
kernel (``ops.qk_prepare``) does everything between it and the attention:
  qk_norm          "head_weight": BEFORE the rotation every q and k head is divided by its own root mean square and
                   multiplied by a weight of the head's size that all heads share ("q.norm", "k.norm")
  conv_taps        a short causal convolution over time on every channel of the q and k projections ("q.conv",
                   "k.conv": [channels, taps], the last tap is the current row's), directly after the product; the
                   last taps - 1 projected rows of a sequence are its state (one tap only scales the channels)
  values           "keys": there is no value matrix; a position's values are its keys as they leave the convolution,
                   before norm and rotation
  softcap          score <- softcap * tanh(score / softcap) before the softmax
  value_mix        the values of the first layer of a step that has this option are kept for the step; every later
                   such layer caches (1 - l) v + l v_first instead of its own v, l its stored number "vmix"
  sinks            the softmax's denominator also holds exp(s_h), a stored number per head ("sink")
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import Mixer, CacheNeed, StateNeed
from .registry import register_part, build_part
from .spec import PartSpec


class Attention(Mixer):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: Optional[dict] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, value_dim: Optional[int] = None,
                 qk_norm: Optional[str] = None, norm_eps: float = 1e-6, head_gate: bool = False,
                 value_gate: bool = False, conv_taps: int = 0, values: str = "own", softcap: float = 0.0,
                 value_mix: bool = False, sinks: bool = False):
        if n_heads % n_kv_heads:
            raise ValueError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = width, n_heads, n_kv_heads, head_dim
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        position = position or {"kind": "none", "params": {}}
        self.position = build_part("position", PartSpec(position["kind"], dict(position.get("params", {}))))
        self.value_dim = int(value_dim) if value_dim else head_dim
        if qk_norm not in (None, "projection", "head", "head_weight"):
            raise ValueError(f"attention: qk_norm {qk_norm!r} is not built ('projection', 'head', 'head_weight')")
        if values not in ("own", "keys"):
            raise ValueError(f"attention: values {values!r} is not built ('own', 'keys')")
        self.conv_taps, self.values_are_keys = int(conv_taps or 0), values == "keys"
        self.softcap, self.value_mix, self.sinks = float(softcap or 0.0), bool(value_mix), bool(sinks)
        if self.values_are_keys and self.value_dim != head_dim:
            raise ValueError("attention: values that are the keys have the keys' size")
        if self.values_are_keys and value_mix:
            raise ValueError("attention: values that are the keys are not mixed with another layer's")
        #: the options of the module's third paragraph: float32 projections and one kernel before the attention
        self.prepared = bool(self.conv_taps >= 1 or self.values_are_keys or self.softcap or self.value_mix or self.sinks
                             or qk_norm == "head_weight")
        if self.prepared and (qk_norm == "head" or value_gate):
            raise ValueError("attention: a weightless norm per head after the rotation and a gate per value do not go "
                             "with the convolution, the shared values, the soft cap, the mixed values or the sinks")
        if head_gate and value_gate:
            raise ValueError("attention: a gate per head or a gate per value, not both")
        self.qk_norm, self.norm_eps, self.head_gate = qk_norm, float(norm_eps), bool(head_gate)
        self.value_gate = bool(value_gate)
        self.w_qkv = self.w_q = self.w_o = None
        self.q_norm_w = self.k_norm_w = None
        self.cache_width = head_dim

    @property
    def extended(self) -> bool:
        """Whether the options of this module's second paragraph are in use."""
        plain_position = getattr(self.position, "plain", True)
        return bool(self.value_dim != self.head_dim or self.qk_norm or self.head_gate or self.value_gate
                    or not plain_position or self.prepared)

    def weight_shapes(self):
        H, K, D, E, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.width, self.value_dim
        shapes = {"q": ((H * D, E), "matrix"), "k": ((K * D, E), "matrix"),
                  "v": ((K * Dv, E), "matrix"), "o": ((E, H * Dv), "matrix")}
        if self.qk_norm == "projection":
            shapes["q.norm"] = ((H * D,), "norm")
            shapes["k.norm"] = ((K * D,), "norm")
        if self.qk_norm == "head_weight":
            shapes["q.norm"] = ((D,), "norm")
            shapes["k.norm"] = ((D,), "norm")
        if self.values_are_keys:
            del shapes["v"]
        if self.conv_taps >= 1:
            shapes["q.conv"] = ((H * D, self.conv_taps), "taps")
            shapes["k.conv"] = ((K * D, self.conv_taps), "taps")
        if self.value_mix:
            shapes["vmix"] = ((), "matrix")
        if self.sinks:
            shapes["sink"] = ((H,), "matrix")
        if self.head_gate:
            shapes["g"] = ((H, E), "matrix")
        if self.value_gate:
            shapes["g"] = ((H * Dv, E), "matrix")
        return shapes

    def cache_need(self):
        return CacheNeed(self.n_kv_heads, self.cache_width, self.window)

    def state_need(self):
        if self.conv_taps > 1:
            # the last projected q and k rows of a sequence, a row per position modulo the taps
            return {"tail": StateNeed((self.conv_taps, (self.n_heads + self.n_kv_heads) * self.head_dim))}
        return None

    def bind(self, weights, ops):
        self.position.bind({}, ops)
        if self.prepared:
            f32 = dict(device=ops.device, dtype=torch.float32)
            stack = [weights["q"], weights["k"]] + ([] if self.values_are_keys else [weights["v"]]) + \
                ([weights["g"]] if self.head_gate else [])
            self.w_qkv = ops.prepare_linear(stack)
            self.w_o = ops.prepare_linear([weights["o"]])
            if self.qk_norm:
                self.q_norm_w = weights["q.norm"].to(**f32).contiguous()
                self.k_norm_w = weights["k.norm"].to(**f32).contiguous()
            if self.conv_taps >= 1:
                self.conv_w = torch.cat([weights["q.conv"], weights["k.conv"]], dim=0).to(**f32).contiguous()
            if self.value_mix:
                self.mix_weight = float(weights["vmix"].to(torch.float32).reshape(-1)[0])
            if self.sinks:
                self.sink_w = weights["sink"].to(**f32).contiguous()
            self.cache_width = ops.cache_head_width(self.head_dim, self.value_dim)
            return
        if self.extended:
            # one product for q, k, v and the gates: rows [q heads | k heads | v heads | gates]
            stack = [weights["q"], weights["k"], weights["v"]] + ([weights["g"]] if self.head_gate or self.value_gate else [])
            self.w_qkv = ops.prepare_linear(stack)
            self.w_o = ops.prepare_linear([weights["o"]])
            if self.qk_norm == "projection":
                self.q_norm_w = weights["q.norm"].to(torch.float32).contiguous()
                self.k_norm_w = weights["k.norm"].to(torch.float32).contiguous()
            self.cache_width = ops.cache_head_width(self.head_dim, self.value_dim)
            return
        # one product for q, k and v: rows [q heads | k heads | v heads]
        self.w_qkv = ops.prepare_linear([weights["q"], weights["k"], weights["v"]])
        self.w_q = None  # for a run that reads another layer's cache: the q rows of w_qkv, as a view
        self.w_o = ops.prepare_linear([weights["o"]])

    #: ``h`` may be rows with their norm pending, and ``then_norm`` is handed to the last product
    folds_norms = True

    conv_w = sink_w = None
    mix_weight = 0.0

    def _forward_prepared(self, ctx, h, entry, accumulate_into, scale_result):
        ops = ctx.ops
        view = ctx.cache_view(entry)
        if not view.writes:
            raise ValueError("attention behind a convolution, with shared or mixed values, reads only its own cache")
        H, Kh, D, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim
        table = self.position.table() if hasattr(self.position, "table") else None
        proj = ops.linear(ops.normed(h) if hasattr(h, "scaled") else h, self.w_qkv, out_dtype=torch.float32)
        mix = None
        if self.value_mix:
            v_at = (H + Kh) * D
            shared = ctx.pass_state                      # lives for one pass over the layers (see engine/model.py)
            first = shared.get("value_mix_first")
            if first is None:
                shared["value_mix_first"] = (proj, v_at, Kh * Dv)             # this pass's first such layer
            else:
                if first[2] != Kh * Dv:
                    raise ValueError("attention: layers that mix values have values of one size")
                mix = (self.mix_weight, first[0], first[1])
        tail = (ctx.state_view(entry) or {}).get("tail") if self.conv_taps > 1 else None
        q, gates = ops.qk_prepare(proj, ctx.meta, view, H, D, Dv, table, self.qk_norm, self.q_norm_w, self.k_norm_w,
                                  self.norm_eps, conv=self.conv_w, tail=tail, values_are_keys=self.values_are_keys,
                                  v_mix=mix, gate_heads=self.head_gate)
        a = ops.attention(q, ctx.meta, view, H, self.scale, self.window, sinks=self.sink_w, softcap=self.softcap)
        a = ops.head_gate(a, gates, 0 if self.head_gate else None, H, Dv, view.head_dim)
        if accumulate_into is None:
            return ops.linear(a, self.w_o, out_dtype=torch.float32, scale=scale_result)
        return ops.linear(a, self.w_o, accumulate_into=accumulate_into, scale=scale_result)

    def _forward_extended(self, ctx, h, entry, accumulate_into):
        ops = ctx.ops
        view = ctx.cache_view(entry)
        if not view.writes:
            raise ValueError("attention with a projection norm, a head gate or unequal key and value sizes "
                             "reads only its own cache")
        H, Kh, D, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim
        table = self.position.table() if hasattr(self.position, "table") else None
        proj = ops.linear(ops.normed(h) if hasattr(h, "scaled") else h, self.w_qkv)
        if self.qk_norm == "head":
            q = ops.norm_rotate_append(proj, table, ctx.meta, view, H, D, Dv, None, None, self.norm_eps, head_norm=True)
        else:
            q = ops.norm_rotate_append(proj, table, ctx.meta, view, H, D, Dv, self.q_norm_w, self.k_norm_w, self.norm_eps)
        a = ops.attention(q, ctx.meta, view, H, self.scale, self.window)
        gate_column = (H + Kh) * D + Kh * Dv if self.head_gate or self.value_gate else None
        if self.value_gate:
            a = ops.head_gate(a, proj, gate_column, H, Dv, view.head_dim, per_value=True)
        else:
            a = ops.head_gate(a, proj, gate_column, H, Dv, view.head_dim)
        if accumulate_into is None:
            return ops.linear(a, self.w_o, out_dtype=torch.float32)
        return ops.linear(a, self.w_o, accumulate_into=accumulate_into)

    def forward(self, ctx, h, entry, accumulate_into=None, then_norm=None, scale_result: float = 1.0):
        """``scale_result`` multiplies the mixer's result (in the output product's float32 sums); the options of the
        module's third paragraph take it."""
        if self.prepared:
            return self._forward_prepared(ctx, h, entry, accumulate_into, scale_result)
        if scale_result != 1.0:
            raise ValueError("attention: a scaled result goes with the prepared path only")
        if self.extended:
            return self._forward_extended(ctx, h, entry, accumulate_into)
        ops = ctx.ops
        view = ctx.cache_view(entry)
        if view.writes:
            w = self.w_qkv
        else:
            if self.w_q is None:
                self.w_q = ops.rows_of(self.w_qkv, 0, self.n_heads * self.head_dim)
            w = self.w_q
        q = ops.project_rotate_append(h, w, self.position.rotary(), ctx.meta, view, self.n_heads)
        a = ops.attention(q, ctx.meta, view, self.n_heads, self.scale, self.window)
        if accumulate_into is None:
            return ops.linear(a, self.w_o, out_dtype=torch.float32)
        if then_norm is None:
            ops.linear(a, self.w_o, accumulate_into=accumulate_into)
        else:
            ops.linear(a, self.w_o, accumulate_into=accumulate_into, then_norm=then_norm)


register_part("mixer", "attention", Attention)
