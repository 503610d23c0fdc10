"""The gated feed-forward: act = silu(W_gate h) * (W_up h), y = W_down act, added to the
residual stream (src/model/qwen_model.cpp:360-374; the gate is swiglu_kernel,
src/compute/cuda/kernels.cu:474-482).  The reference runs gate and up as two products; here
their matrices are stacked with rows alternating in runs, so that one product yields both
and matching gate and up values lie next to each other for the gate kernel.

Parameters: hidden_size, intermediate_size; optional ``activation`` ("silu", the default, or "gelu_tanh": z / 2 (1 +
tanh(sqrt(2 / pi) (z + 0.044715 z^3)))), ``biases`` (true: gate, up and down have a bias each) and ``names``: the full
tensor names by role (gate, up, down, gate_bias, up_bias, down_bias; a bias defaults to its matrix's name with ``.b``).
With another activation than SiLU, or with biases, the gate and up product keeps its float32 result, and bias,
activation and gate are one kernel with one rounding at its store.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..errors import require
from ..weights.loader import TensorSpec
from .base import NormedRows, bind_vector, register_part
from .linear import DenseLinear

_RUN = 16


class GatedSiluFeedForward:
    graph_safe = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.run = _RUN if self.inter % _RUN == 0 else self.inter
        self.activation = str(params.get("activation") or "silu")
        require(self.activation in ("silu", "gelu_tanh"), f"{prefix}: unknown activation '{self.activation}'; known: silu, gelu_tanh")
        self.has_biases = bool(params.get("biases", False))
        n = dict(params.get("names") or {})
        nm = {"gate": str(n.get("gate") or f"{prefix}.gate_proj.weight"), "up": str(n.get("up") or f"{prefix}.up_proj.weight"),
              "down": str(n.get("down") or f"{prefix}.down_proj.weight")}
        for r in ("gate", "up", "down"):
            nm[r + "_bias"] = str(n.get(r + "_bias") or nm[r] + ".b")
        self.names = nm
        self.gate_up = DenseLinear([nm["gate"], nm["up"]], [self.inter, self.inter], self.hidden, interleave_run=self.run)
        self.down = DenseLinear([nm["down"]], [self.hidden], self.inter)
        self.plain = self.activation == "silu" and not self.has_biases       # the product's own gate epilogue serves
        self.can_overwrite = not self.plain
        self.bias = self.deferred_bias = None

    def tensor_specs(self):
        specs = self.gate_up.tensor_specs() + self.down.tensor_specs()
        if self.has_biases:
            nm = self.names
            specs += [TensorSpec(nm["gate_bias"], (self.inter,), "state"), TensorSpec(nm["up_bias"], (self.inter,), "state"),
                      TensorSpec(nm["down_bias"], (self.hidden,), "state")]
        return specs

    def bind(self, weights, ctx):
        self.gate_up.bind(weights, ctx)
        self.down.bind(weights, ctx)
        if self.has_biases:
            nm, r = self.names, self.run
            both = torch.stack([bind_vector(weights, nm["gate_bias"], self.inter, ctx).view(-1, r),
                                bind_vector(weights, nm["up_bias"], self.inter, ctx).view(-1, r)], 1)
            self.bias = both.reshape(-1).contiguous()                 # in the order of the interleaved product's columns
            self.deferred_bias = bind_vector(weights, nm["down_bias"], self.hidden, ctx)
        self.dtype = ctx.dtype

    def can_absorb_norm(self) -> bool:
        if not self.plain:
            return False
        return self.run == _RUN and self.gate_up.can_take_normed_rows() and self.down.can_emit_normed_rows()

    def fold_norm_gain(self, gain: torch.Tensor) -> None:
        self.gate_up.fold_input_gain(gain)

    def forward(self, h, batch, residual, emit=None, overwrite=False, defer_bias=False):
        """``h``: the normed rows, or :class:`~.base.NormedRows` (few rows; after :meth:`fold_norm_gain`).  ``emit``: a pair
        of buffers that the down projection fills with what the next norm needs of the updated residual rows.
        ``overwrite``: ``residual`` holds nothing yet and receives the output.  ``defer_bias``: the caller adds
        ``deferred_bias`` (the output's bias) itself."""
        if not self.plain:
            gu = self.gate_up.forward(h, out_dtype=torch.float32)
            act = torch.empty((h.shape[0], self.inter), dtype=self.dtype, device=h.device)
            ops.expert_gate(gu, None, act, 0, 0, 1, self.activation, tail_ff=self.inter, tail_run=self.run, bias=self.bias)
            if overwrite:
                self.down.forward(act, out=residual)
            else:
                self.down.forward(act, accumulate_into=residual)
            if self.deferred_bias is not None and not defer_bias:
                ops.add_row_bias(residual, self.deferred_bias)
            return residual
        if isinstance(h, NormedRows):
            act = self.gate_up.forward_gated(h.rows, self.run, row_scale=h.scale)
        else:
            act = self.gate_up.forward_gated(h, self.run)          # gate in the product's epilogue
            if act is None:
                act = torch.empty((h.shape[0], self.inter), dtype=self.dtype, device=h.device)
                ops.swiglu(self.gate_up.forward(h), act, self.run)
        if overwrite:
            self.down.forward(act, out=residual)
        else:
            self.down.forward(act, accumulate_into=residual, emit=emit)
        return residual


class SquaredReluFeedForward:
    """y = W_down max(W_up h, 0)^2, no gate.  Parameters: hidden_size, intermediate_size; optional ``up`` and ``down``
    (the matrices' full names; default ``<prefix>.up_proj.weight`` and ``<prefix>.down_proj.weight``)."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.up = DenseLinear([str(params.get("up") or f"{prefix}.up_proj.weight")], [self.inter], self.hidden)
        self.down = DenseLinear([str(params.get("down") or f"{prefix}.down_proj.weight")], [self.hidden], self.inter)

    def tensor_specs(self):
        return self.up.tensor_specs() + self.down.tensor_specs()

    def bind(self, weights, ctx):
        self.up.bind(weights, ctx)
        self.down.bind(weights, ctx)
        self.dtype = ctx.dtype

    def forward(self, h, batch, residual, overwrite=False):
        """``overwrite``: ``residual`` holds nothing yet and receives the output instead of being added to."""
        z = self.up.forward(h)
        ops.relu_squared(z, z)
        if overwrite:
            self.down.forward(z, out=residual)
        else:
            self.down.forward(z, accumulate_into=residual)
        return residual


class XieluFeedForward:
    """y = W_down xielu(W_up h + b_up) (+ b_down), no gate.  xielu has two numbers p, q stored as one tensor of two:
    for z > 0: softplus(p) z^2 + z / 2; for z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.  The up product's result
    stays float32 until the activation has been applied (bias, activation and the one rounding are one kernel).

    Parameters: hidden_size, intermediate_size; ``names``: {"up", "down", "act", "up_bias", "down_bias"} (a bias name of
    None: no such bias; defaults ``<prefix>.up``, ``<prefix>.down``, ``<prefix>.act``, ``<prefix>.up.b``,
    ``<prefix>.down.b``).  A block that adds vectors in a kernel of its own may take the output's bias from
    ``deferred_bias`` and pass ``defer_bias=True``."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        n = dict(params.get("names") or {})
        name = lambda role, default: None if (role in n and n[role] is None) else str(n.get(role) or default)
        self.act_name = name("act", f"{prefix}.act")
        self.up_bias_name = name("up_bias", f"{prefix}.up.b")
        self.down_bias_name = name("down_bias", f"{prefix}.down.b")
        self.up = DenseLinear([name("up", f"{prefix}.up")], [self.inter], self.hidden)
        self.down = DenseLinear([name("down", f"{prefix}.down")], [self.hidden], self.inter)
        self.up_bias = self.deferred_bias = None

    def tensor_specs(self):
        specs = self.up.tensor_specs() + self.down.tensor_specs() + [TensorSpec(self.act_name, (2,), "state")]
        if self.up_bias_name is not None:
            specs.append(TensorSpec(self.up_bias_name, (self.inter,), "state"))
        if self.down_bias_name is not None:
            specs.append(TensorSpec(self.down_bias_name, (self.hidden,), "state"))
        return specs

    def bind(self, weights, ctx):
        self.up.bind(weights, ctx)
        self.down.bind(weights, ctx)
        if self.up_bias_name is not None:
            self.up_bias = bind_vector(weights, self.up_bias_name, self.inter, ctx)
        if self.down_bias_name is not None:
            self.deferred_bias = bind_vector(weights, self.down_bias_name, self.hidden, ctx)
        h = weights[self.act_name]
        require(tuple(h.shape) == (2,), f"unexpected tensor shape for {self.act_name}: got {list(h.shape)}, expected [2]")
        p, q = (float(v) for v in h.tensor.to(torch.float64))
        softplus = lambda v: v if v > 30.0 else math.log1p(math.exp(v))
        self.alpha_pos, self.alpha_neg = softplus(p), 0.5 + softplus(q)
        self.dtype = ctx.dtype

    def forward(self, h, batch, residual, overwrite=False, defer_bias=False):
        """``overwrite``: ``residual`` holds nothing yet and receives the output.  ``defer_bias``: the caller adds
        ``deferred_bias`` itself."""
        z = self.up.forward(h, out_dtype=torch.float32)
        act = torch.empty((h.shape[0], self.inter), dtype=self.dtype, device=h.device)
        ops.bias_xielu(z, self.up_bias, self.alpha_pos, self.alpha_neg, act)
        if overwrite:
            self.down.forward(act, out=residual)
        else:
            self.down.forward(act, accumulate_into=residual)
        if self.deferred_bias is not None and not defer_bias:
            ops.add_row_bias(residual, self.deferred_bias)
        return residual


register_part("feed_forward", "gated_silu", GatedSiluFeedForward)
register_part("feed_forward", "gated", GatedSiluFeedForward)          # the same part under the name that fits every activation
register_part("feed_forward", "xielu", XieluFeedForward)
register_part("feed_forward", "relu_squared", SquaredReluFeedForward)
