"""Mixers side by side: every branch reads the same input rows; each result goes through an RMS
norm over the model width with a weight of its own ("<branch>.out"), and the mixer's result is
their mean.  A branch is any registered mixer; its weights are named "<branch>.<key>", its
state "<branch>.<name>".  At most one branch may keep a cache of keys and values, because a cache
entry belongs to one run of one mixer.

``combine`` "weighted": no norms and no mean; the result is sum_b scales[b] * branch_b, each branch multiplying its own
result in its output product and adding it to the sum of the branches before it.
"""
from __future__ import annotations

import torch

from .base import Mixer
from .registry import register_part, build_part
from .spec import PartSpec


class _BranchContext:
    """The step's context as one branch sees it: its own part of the mixer's state."""

    def __init__(self, ctx, branch: str):
        self._ctx, self._prefix = ctx, branch + "."
        self.ops, self.meta, self.cache = ctx.ops, ctx.meta, getattr(ctx, "cache", None)

    def cache_view(self, entry):
        return self._ctx.cache_view(entry)

    @property
    def pass_state(self):
        return self._ctx.pass_state

    def state_view(self, entry):
        whole = self._ctx.state_view(entry) or {}
        mine = {k[len(self._prefix):]: v for k, v in whole.items() if k.startswith(self._prefix)}
        if list(mine) == [""]:
            return mine[""]
        return mine or None


class ParallelMixers(Mixer):
    def __init__(self, width: int, norm_eps: float, branches: dict, combine: str = "mean_of_norms", scales: dict = None):
        """branches: name -> {"kind": mixer kind, "params": {...}}, in the order they run."""
        self.width, self.norm_eps = int(width), float(norm_eps)
        if combine not in ("mean_of_norms", "weighted"):
            raise ValueError(f"parallel mixers: combine {combine!r} is not built ('mean_of_norms', 'weighted')")
        self.weighted = combine == "weighted"
        self.scales = {k: float(v) for k, v in (scales or {}).items()}
        if self.weighted and set(self.scales) != set(branches):
            raise ValueError("parallel mixers: a weighted sum needs one scale per branch")
        if not branches:
            raise ValueError("parallel mixers: no branch")
        self.branches = {name: build_part("mixer", PartSpec(b["kind"], dict(b.get("params", {}))))
                         for name, b in branches.items()}
        self.out_w = {}

    def weight_shapes(self):
        shapes = {}
        for name, part in self.branches.items():
            for key, v in part.weight_shapes().items():
                shapes[f"{name}.{key}"] = v
            if not self.weighted:
                shapes[f"{name}.out"] = ((self.width,), "norm")
        return shapes

    def bind(self, weights, ops):
        for name, part in self.branches.items():
            pre = name + "."
            part.bind({k[len(pre):]: v for k, v in weights.items() if k.startswith(pre) and k != pre + "out"}, ops)
            if not self.weighted:
                self.out_w[name] = weights[pre + "out"].to(torch.float32).contiguous()

    def cache_need(self):
        needs = [n for n in (p.cache_need() for p in self.branches.values()) if n is not None]
        if len(needs) > 1:
            raise ValueError("parallel mixers: more than one branch keeps a cache; give each a layer of its own")
        return needs[0] if needs else None

    def state_need(self):
        out = {}
        for name, part in self.branches.items():
            need = part.state_need()
            if need is None:
                continue
            if isinstance(need, dict):
                out.update({f"{name}.{k}": v for k, v in need.items()})
            else:
                out[f"{name}."] = need
        return out or None

    def results(self, ctx, h, entry):
        """Every branch's float32 result [T, E], with the weights of their norms."""
        ys = [part.forward(_BranchContext(ctx, name), h, entry, accumulate_into=None)
              for name, part in self.branches.items()]
        return ys, [self.out_w[name] for name in self.branches]

    def _weighted(self, ctx, h, entry):
        y = None
        for name, part in self.branches.items():
            y = part.forward(_BranchContext(ctx, name), h, entry, accumulate_into=y, scale_result=self.scales[name])
        return y

    def forward(self, ctx, h, entry, accumulate_into=None):
        if self.weighted:
            y = self._weighted(ctx, h, entry)
            if accumulate_into is None:
                return y
            accumulate_into += y
            return accumulate_into
        ys, ws = self.results(ctx, h, entry)
        y = ctx.ops.normed_mean(ys, ws, self.norm_eps)
        if accumulate_into is None:
            return y
        accumulate_into += y
        return accumulate_into


register_part("mixer", "parallel", ParallelMixers)
