"""Feed-forwards.  ``GatedDense``, the dense gated one: down( act(gate h) * (up h) ), act = SiLU, no bias
(crates/bitnet-core/src/llama/model.rs:116-120, 296-306).  The activation and
the product are float32 before any rounding to the compute dtype.

``activation`` "swish_limited": with g' = min(gate h, limit) and u' = clamp(up h, -limit, limit),
the inner rows are g' * sigmoid(alpha g') * (u' + shift); alpha = 1.702 and shift = 1 unless given.

``Dense``: down(relu2(up h)), no gate.  ``RoutedExperts``: a router chooses a few of many small feed-forwards
(and identity experts) per token; a shared expert may run beside them."""
from __future__ import annotations

import torch

from .base import FeedForward
from .registry import register_part


class GatedDense(FeedForward):
    def __init__(self, width: int, inner: int, activation: str = "silu", limit: float = 0.0,
                 alpha: float = 1.702, shift: float = 1.0):
        if activation not in ("silu", "swish_limited"):
            raise ValueError(f"gated feed-forward: activation {activation!r} is not built "
                             "(only 'silu' and 'swish_limited')")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        #: (alpha, limit, shift) of the limited activation; None: SiLU(gate) * up
        self.act = None if activation == "silu" else (float(alpha), float(limit), float(shift))
        if self.act is not None and not self.act[1] > 0:
            raise ValueError("gated feed-forward: 'swish_limited' needs a positive limit")
        self.w_gate_up = self.w_down = None

    def weight_shapes(self):
        return {"gate": ((self.inner, self.width), "matrix"), "up": ((self.inner, self.width), "matrix"),
                "down": ((self.width, self.inner), "matrix")}

    def bind(self, weights, ops):
        self.w_gate_up = ops.prepare_gate_up(weights["gate"], weights["up"])
        self.w_down = ops.prepare_linear([weights["down"]])

    #: ``h`` may be rows with their norm pending, and ``then_norm`` is handed to the last product
    folds_norms = True

    def forward(self, ctx, h, accumulate_into=None, then_norm=None):
        if self.act is None:
            t = ctx.ops.gated_linear(h, self.w_gate_up)        # silu(gate h) * (up h)
        else:
            t = ctx.ops.gated_linear(h, self.w_gate_up, act=self.act)
        if accumulate_into is None:
            return ctx.ops.linear(t, self.w_down, out_dtype=torch.float32)
        if then_norm is None:
            ctx.ops.linear(t, self.w_down, accumulate_into=accumulate_into)
        else:
            ctx.ops.linear(t, self.w_down, accumulate_into=accumulate_into, then_norm=then_norm)


class Dense(FeedForward):
    """down(act(up h)) without a gate and without biases; ``activation`` "relu2": max(z, 0)^2, taken of the
    product's float32 sums before they are rounded to the compute dtype."""

    def __init__(self, width: int, inner: int, activation: str = "relu2"):
        if activation != "relu2":
            raise ValueError(f"dense feed-forward: activation {activation!r} is not built (only 'relu2')")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.w_up = self.w_down = None

    def weight_shapes(self):
        return {"up": ((self.inner, self.width), "matrix"), "down": ((self.width, self.inner), "matrix")}

    def bind(self, weights, ops):
        self.w_up = ops.prepare_linear([weights["up"]])
        self.w_down = ops.prepare_linear([weights["down"]])

    def forward(self, ctx, h, accumulate_into=None):
        t = ctx.ops.linear(h, self.w_up, act=self.activation)
        if accumulate_into is None:
            return ctx.ops.linear(t, self.w_down, out_dtype=torch.float32)
        ctx.ops.linear(t, self.w_down, accumulate_into=accumulate_into)


class RoutedExperts(FeedForward):
    """A mixture of ``n_experts`` small feed-forwards without biases of which every token uses ``top``, plus
    ``n_identity`` identity experts whose result is the input row itself.

    Router: z = Wr h in float32 over all n_experts + n_identity outputs; ``scoring`` "softmax": s = softmax(z),
    "sigmoid": s = sigmoid(z), output by output.  The choice is made by s + correction ("correction", one number per
    output), among the outputs of the ``keep`` best of ``groups`` equal groups of neighbouring outputs (a group's score
    is its largest choice score; groups 0 or 1: no groups); the chosen outputs' weights are their s, not
    renormalised.  ``weight_on`` "output": the result is the weighted sum of the chosen experts' results;
    "input": every chosen expert runs on its weight times the input row, and the results are added up as they are.

    ``activation`` "relu2": an expert is down(relu2(up h)) ("e<i>.up" [inner, width], "e<i>.down" [width, inner]).
    "swish_limited": an expert is gated, down(g' sigmoid(alpha g') (u' + shift)) with g' = min(gate h, limit) and
    u' = clamp(up h, -limit, limit) ("e<i>.gate" beside the other two).

    ``shared`` (a dict with "inner", "limit" and optionally "alpha", "shift"): one more gated expert of that form that
    every token uses ("shared.gate", "shared.up", "shared.down"), its result multiplied by sigmoid(w_sg . h), one
    number per token ("shared.sg" [1, width]), and added.  The gate's sum is made beside the router's, in float32.

    Weights: "router" [n_experts + n_identity, width], "correction" (``correction=False``: none), the experts'."""

    def __init__(self, width: int, inner: int, n_experts: int, top: int, n_identity: int = 0, groups: int = 0,
                 keep: int = 0, correction: bool = True, activation: str = "relu2", scoring: str = "softmax",
                 weight_on: str = "output", limit: float = 0.0, alpha: float = 1.702, shift: float = 1.0,
                 shared: dict = None):
        if activation not in ("relu2", "swish_limited"):
            raise ValueError(f"routed experts: activation {activation!r} is not built (only 'relu2' and 'swish_limited')")
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"routed experts: scoring {scoring!r} is not built (only 'softmax' and 'sigmoid')")
        if weight_on not in ("output", "input"):
            raise ValueError(f"routed experts: the weight acts on the 'output' or on the 'input', not on {weight_on!r}")
        self.width, self.inner, self.n_experts, self.top = int(width), int(inner), int(n_experts), int(top)
        self.n_identity, self.groups, self.keep = int(n_identity), int(groups or 0), int(keep or 0)
        self.has_correction = bool(correction)
        self.activation, self.scoring, self.weight_on = activation, scoring, weight_on
        #: (alpha, limit, shift) of a gated expert's activation; None: relu2 without a gate
        self.act = (float(alpha), float(limit), float(shift)) if activation == "swish_limited" else None
        if self.act is not None and not self.act[1] > 0:
            raise ValueError("routed experts: 'swish_limited' needs a positive limit")
        self.shared = None
        if shared:
            self.shared = {"inner": int(shared["inner"]),
                           "act": (float(shared.get("alpha", 1.702)), float(shared["limit"]), float(shared.get("shift", 1.0)))}
            if self.shared["inner"] < 1 or not self.shared["act"][1] > 0:
                raise ValueError("routed experts: the shared expert needs an inner size and a positive limit")
        n = self.n_experts + self.n_identity
        if self.weight_on == "input" and self.n_identity:
            raise ValueError("routed experts: identity experts go with weights on the results")
        if not 1 <= self.top <= n:
            raise ValueError(f"routed experts: {self.top} choices among {n} outputs")
        if self.groups > 1:
            if n % self.groups:
                raise ValueError(f"routed experts: {n} router outputs are not {self.groups} equal groups")
            if not 1 <= self.keep <= self.groups:
                raise ValueError(f"routed experts: {self.keep} of {self.groups} groups kept")
        self.router = self.router_tc = self.correction = self.w_up = self.w_down = None
        self.shared_gate_up = self.shared_down = None

    @property
    def plain(self) -> bool:
        """Softmax scores that weigh the results of ungated experts, and no shared expert."""
        return self.act is None and self.scoring == "softmax" and self.weight_on == "output" and self.shared is None

    def weight_shapes(self):
        n = self.n_experts + self.n_identity
        shapes = {"router": ((n, self.width), "matrix")}
        if self.has_correction:
            shapes["correction"] = ((n,), "matrix")
        for e in range(self.n_experts):
            if self.act is not None:
                shapes[f"e{e}.gate"] = ((self.inner, self.width), "matrix")
            shapes[f"e{e}.up"] = ((self.inner, self.width), "matrix")
            shapes[f"e{e}.down"] = ((self.width, self.inner), "matrix")
        if self.shared is not None:
            f = self.shared["inner"]
            shapes.update({"shared.gate": ((f, self.width), "matrix"), "shared.up": ((f, self.width), "matrix"),
                           "shared.down": ((self.width, f), "matrix"), "shared.sg": ((1, self.width), "matrix")})
        return shapes

    def bind(self, weights, ops):
        # the router's product is float32 whatever the compute dtype; a shared expert's gate is one more row of it
        rows = [weights["router"]] + ([weights["shared.sg"]] if self.shared is not None else [])
        self.router = torch.cat([r.to(device=ops.device, dtype=torch.float32) for r in rows], dim=0).contiguous()
        self.correction = (weights["correction"].to(device=ops.device, dtype=torch.float32).contiguous()
                           if self.has_correction else None)
        # where the operations can make the same float32 sums on the tensor cores, they say so here
        prepare = getattr(ops, "prepare_router", None)
        self.router_tc = prepare(self.router) if prepare is not None else None
        if self.n_experts:
            # the experts' matrices one below the other: [n_experts * rows, width] and [n_experts * width, inner]
            if self.act is None:
                self.w_up = ops.prepare_linear([weights[f"e{e}.up"] for e in range(self.n_experts)])
            else:
                self.w_up = ops.prepare_expert_gate_up([weights[f"e{e}.gate"] for e in range(self.n_experts)],
                                                       [weights[f"e{e}.up"] for e in range(self.n_experts)])
            self.w_down = ops.prepare_linear([weights[f"e{e}.down"] for e in range(self.n_experts)])
        if self.shared is not None:
            self.shared_gate_up = ops.prepare_gate_up(weights["shared.gate"], weights["shared.up"])
            self.shared_down = ops.prepare_linear([weights["shared.down"]])

    def forward(self, ctx, h, accumulate_into=None):
        ops = ctx.ops
        if self.plain:
            if self.router_tc is not None:
                ids, weights = ops.route(h, self.router, self.correction, self.top, self.groups, self.keep, router_tc=self.router_tc)
            else:
                ids, weights = ops.route(h, self.router, self.correction, self.top, self.groups, self.keep)
            return ops.routed_experts(h, ids, weights, self.w_up, self.w_down, self.n_experts, self.inner,
                                      accumulate_into=accumulate_into)
        extra = 1 if self.shared is not None else 0
        ids, weights, gate = ops.route_scored(h, self.router, self.correction, self.top, self.groups, self.keep,
                                              scoring=self.scoring, extra_rows=extra, router_tc=self.router_tc)
        y = ops.routed_experts(h, ids, weights, self.w_up, self.w_down, self.n_experts, self.inner,
                               accumulate_into=accumulate_into, act=self.act, weight_on_input=self.weight_on == "input")
        if self.shared is not None:
            t = ops.gated_linear(h, self.shared_gate_up, act=self.shared["act"])
            z = ops.linear(t, self.shared_down, out_dtype=torch.float32)
            ops.add_scaled_rows(y, z, gate)                      # y += sigmoid(gate) * z, one number per row
        return y


register_part("feed_forward", "gated_dense", GatedDense)
register_part("feed_forward", "dense", Dense)
register_part("feed_forward", "routed_experts", RoutedExperts)
