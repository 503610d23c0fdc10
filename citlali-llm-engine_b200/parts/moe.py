"""Routed experts: a feed-forward made of ``experts`` small gated feed-forwards of which every token uses ``top``.

Router logits z = W_router h in 32-bit; scores s = softmax(z) over all experts (``score`` "sigmoid": s = sigmoid(z), every
expert's score by itself).  The experts form ``groups`` equal groups of
neighbours; a group's score is the largest score in it, and only experts of the ``keep_groups`` best groups can be chosen
(``groups`` None: no groups).  The ``top`` experts with the largest scores among those are chosen; their weights are their
scores times ``weight_scale``, not renormalised.  An expert is  W_down act(W_gate h, W_up h), without biases; the output is
the weighted sum of the chosen experts' outputs, or with ``weight_on`` "input" the sum of the experts applied to the weight
times h (the weight then meets gate and up ahead of the activation: act(w W_gate h, w W_up h)).  ``activation``:

* ``silu`` (the default): act(g, u) = silu(g) u;
* ``clamped_swish``: g' = min(g, limit), u' = clamp(u, -limit, limit); act = g' sigmoid(alpha g') (u' + 1), with ``limit``
  and ``alpha`` (default 1.702) from the parameters.

``shared``: {"intermediate_size", "limit"} of one more expert of the same form that runs for every row and is added with
weight 1; its matrices ride in the same two products, behind the routed experts'.

How it runs: the router is a product with a float32 result; one kernel turns a row's logits into a row of weights (zero
for an expert that was not chosen); the experts' gate and up matrices are ONE product for all experts (the gate in its
epilogue where the shape and the activation allow; otherwise a kernel takes the product's float32 result through the
activation), every expert's activations are multiplied by the row's weight for it, and the experts' output matrices side
by side are ONE product that sums over experts.  Nothing depends on counts known to the host
only, so a decoding step replays as a graph; the price is that every expert's matrices are applied to every row.

Parameters: hidden_size, experts, top, intermediate_size, groups, keep_groups, weight_scale, score, weight_on, activation,
limit, alpha, shared; ``names``: {"router": name, "gate": [names], "up": [names], "down": [names], "shared": {"gate", "up", "down"}}
(default ``<prefix>.router``, ``<prefix>.e<i>.{gate,up,down}`` and ``<prefix>.shared.{gate,up,down}``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import require
from .base import register_part
from .linear import DenseLinear, ExpertDown, ExpertGateUp


class RoutedExperts:
    graph_safe = True
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.E, self.top, self.ff = int(params["experts"]), int(params["top"]), int(params["intermediate_size"])
        self.groups = None if params.get("groups") is None else int(params["groups"])
        self.keep = int(params.get("keep_groups") or (self.groups or 1))
        require(1 <= self.top <= self.E, f"{prefix}: {self.top} of {self.E} experts cannot be chosen")
        require(self.E <= 512, f"{prefix}: {self.E} experts exceed the router kernel's 512")
        if self.groups is not None:
            require(self.groups >= 1 and self.E % self.groups == 0, f"{prefix}: {self.E} experts do not form {self.groups} equal groups")
            require(1 <= self.keep <= self.groups and self.keep * (self.E // self.groups) >= self.top,
                    f"{prefix}: {self.keep} groups of {self.E // self.groups} experts cannot give {self.top} experts")
        self.weight_scale = 1.0 if params.get("weight_scale") is None else float(params["weight_scale"])
        self.score = str(params.get("score") or "softmax")
        require(self.score in ops.ROUTER_SCORES, f"{prefix}: unknown router score '{self.score}'; known: {', '.join(ops.ROUTER_SCORES)}")
        self.weight_input = {"output": False, "input": True}.get(str(params.get("weight_on") or "output"))
        require(self.weight_input is not None, f"{prefix}: weight_on must be 'output' or 'input'")
        self.activation = str(params.get("activation") or "silu")
        require(self.activation in ops.EXPERT_ACTIVATIONS,
                f"{prefix}: unknown expert activation '{self.activation}'; known: {', '.join(ops.EXPERT_ACTIVATIONS)}")
        self.limit = float(params.get("limit") or 0.0)
        self.alpha = 1.702 if params.get("alpha") is None else float(params["alpha"])
        require(self.activation != "clamped_swish" or self.limit > 0.0, f"{prefix}: the clamped activation needs a positive limit")
        n = dict(params.get("names") or {})
        each = lambda role: list(n.get(role) or [f"{prefix}.e{i}.{role}" for i in range(self.E)])
        shared = params.get("shared")
        self.shared_ff, self.shared_limit = 0, 0.0
        gate_up_tail = down_tail = None
        if shared is not None:
            self.shared_ff = int(shared["intermediate_size"])
            self.shared_limit = float(shared.get("limit") or 0.0)
            require(self.shared_ff > 0 and (self.activation != "clamped_swish" or self.shared_limit > 0.0),
                    f"{prefix}: the expert for every row needs a width and, with the clamped activation, a positive limit")
            sn = dict(n.get("shared") or {})
            name = lambda role: str(sn.get(role) or f"{prefix}.shared.{role}")
            gate_up_tail = (name("gate"), name("up"), self.shared_ff)
            down_tail = (name("down"), self.shared_ff)
        self.router = DenseLinear([str(n.get("router") or f"{prefix}.router")], [self.E], self.hidden)
        self.gate_up = ExpertGateUp(each("gate"), each("up"), self.ff, self.hidden, tail=gate_up_tail)
        self.down = ExpertDown(each("down"), self.ff, self.hidden, tail=down_tail)
        self.prefix = prefix
        # the product's own gate epilogue and the scaling kernel serve the plain form; anything else runs the gate kernel
        self.plain = self.activation == "silu" and shared is None and not self.weight_input

    def tensor_specs(self):
        return self.router.tensor_specs() + self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, weights, ctx):
        self.router.bind(weights, ctx)
        self.gate_up.bind(weights, ctx)
        self.down.bind(weights, ctx)
        self.dtype = ctx.dtype

    def route(self, h):
        """The row's weights for every expert, float32 [rows, experts]: its score where chosen, zero elsewhere."""
        logits = self.router.forward(h, out_dtype=torch.float32)
        weights = torch.empty_like(logits)
        ops.moe_route(logits, weights, self.groups, self.keep, self.top, weight_scale=self.weight_scale, score=self.score)
        return weights

    def forward(self, h, batch, residual, overwrite=False):
        weights = self.route(h)
        if self.plain:
            act = self.gate_up.forward_gated(h, self.gate_up.run)
            if act is None:
                act = torch.empty((h.shape[0], self.E * self.ff), dtype=self.dtype, device=h.device)
                ops.swiglu(self.gate_up.forward(h), act, self.gate_up.run)
            ops.moe_scale(act, weights, self.ff)
        else:
            gu = self.gate_up.forward(h, out_dtype=torch.float32)
            act = torch.empty((h.shape[0], self.E * self.ff + self.shared_ff), dtype=self.dtype, device=h.device)
            ops.expert_gate(gu, weights, act, self.E, self.ff, self.gate_up.run, self.activation, self.limit, self.alpha,
                            self.shared_ff, self.gate_up.tail_run, self.shared_limit, weight_input=self.weight_input)
        if overwrite:
            self.down.forward(act, out=residual)
        else:
            self.down.forward(act, accumulate_into=residual)
        return residual


register_part("feed_forward", "routed_experts", RoutedExperts)
