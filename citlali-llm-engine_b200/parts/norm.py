"""RMSNorm over the hidden size: y = x * rsqrt(mean(x^2) + eps) * gain, eps inside the root,
the gain multiplies (no 1 + gain) -- rms_norm_kernel, src/compute/cuda/kernels.cu:73-92.
Input is the float32 residual stream; the sum of squares, the root and the product are
32-bit, rounded once at the store to the compute dtype.

Parameters: size, eps; optional ``tensor`` (the gain's full name; default ``<prefix>.weight``) and ``offset``
(the factor is ``offset + w``: a gain stored around zero has offset 1; the sum is made once, in 32-bit, and the gain
then stays 32-bit in both paths, since 1 + w rounded to bfloat16 would lose most of w)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import bind_gain, bind_vector, register_part


class RMSNorm:
    graph_safe = True

    def __init__(self, params, prefix: str):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = str(params.get("tensor") or f"{prefix}.weight")
        self.offset = float(params.get("offset", 0.0))
        self.gain = None
        self.gain_downstream = False

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), "gain")]

    def bind(self, weights, ctx):
        self.gain = bind_gain(weights, self.name, self.size, ctx)
        if self.offset != 0.0:
            self.gain = (self.gain.to(torch.float32) + self.offset).contiguous()
        self.dtype = ctx.dtype

    def gain_moves_downstream(self) -> torch.Tensor:
        """The part behind this norm has multiplied its weights by the gain: from now on the norm only divides by the
        root mean square (its kernel gets a gain of ones).  Returns the gain."""
        gain = self.gain
        self.gain = torch.ones_like(gain)
        self.gain_downstream = True
        return gain

    def forward(self, x: torch.Tensor, row_index=None, out_dtype=None) -> torch.Tensor:
        """``out_dtype``: float32 for rows that stay part of the 32-bit residual (a norm on the embedding's rows);
        default: the compute dtype, for rows a product reads."""
        rows = x.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.size), dtype=out_dtype or self.dtype, device=x.device)
        ops.rms_norm(x, self.gain, self.eps, out, row_index)
        return out


class LayerNorm:
    """y = (x - mean) / sqrt(var + eps) * gain (+ bias) with var the mean of the squared deviations, over the hidden size,
    in 32-bit.  ``forward`` norms rows of the residual stream (the norm in front of a sub-layer, a model's last norm);
    ``add_into`` serves a block whose norm sits on a sub-layer's output: ``x += norm(y)``, optionally leaving the updated
    rows in the compute dtype; ``chain_terms`` gives a block what it needs to run this norm inside a kernel of its own.

    Parameters: size, eps; optional ``tensor`` (the gain's full name; default ``<prefix>.weight``) and ``bias`` (the bias's
    full name; None: no bias).  A norm with a bias keeps gain and bias in float32 in both paths."""
    graph_safe = True

    def __init__(self, params, prefix: str):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = str(params.get("tensor") or f"{prefix}.weight")
        self.bias_name = None if params.get("bias") is None else str(params["bias"])
        self.gain = self.bias = None

    def tensor_specs(self):
        specs = [TensorSpec(self.name, (self.size,), "gain")]
        if self.bias_name is not None:
            specs.append(TensorSpec(self.bias_name, (self.size,), "state"))
        return specs

    def bind(self, weights, ctx):
        if self.bias_name is None:
            self.gain = bind_gain(weights, self.name, self.size, ctx)
        else:
            self.gain = bind_vector(weights, self.name, self.size, ctx)
            self.bias = bind_vector(weights, self.bias_name, self.size, ctx)
        self.dtype = ctx.dtype

    def forward(self, x: torch.Tensor, row_index=None) -> torch.Tensor:
        rows = x.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.size), dtype=self.dtype, device=x.device)
        ops.layer_norm_rows(x, self.gain, self.eps, out, row_index, bias=self.bias)
        return out

    def chain_terms(self):
        """(gain, bias or None, eps) with float32 vectors: what ``ops.layer_norm_chain`` takes."""
        return self.gain.float() if self.gain.dtype != torch.float32 else self.gain, self.bias, self.eps

    def add_into(self, y: torch.Tensor, x: torch.Tensor, emit=None) -> torch.Tensor:
        if self.bias is None:
            ops.layer_norm_add(y, self.gain, self.eps, x, emit)
        else:
            ops.layer_norm_chain(y, x, self.gain, self.bias, self.eps, emit=emit)
        return x


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm", LayerNorm)
