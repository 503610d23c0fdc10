"""Grouped-query attention over a sliding window that also keeps a sequence's first tokens, with a short causal
convolution in front and heads whose keys and values may differ in size.

For a token with input h:  q (``heads`` of ``dim``), k (``kv_heads`` of ``dim``) and v (``kv_heads`` of ``vdim``) are
projections of h, without biases unless ``biases`` says otherwise (a bias a channel, added to what the convolution gives;
with no convolution: to the projection); each channel then passes a causal convolution over time (``conv`` taps, no bias, zeros before
the sequence's start; None: none).  q and k heads pass an RMS norm over ``dim`` with a weight shared by the heads
(``qk_norm_eps`` None: none), then the rotation of the first ``rot_dims`` elements of a head in neighbouring pairs
(2i, 2i+1) by position * ``rot_base``^(-2i/rot_dims); the rest of a head, and v, pass unchanged.  Query head j reads key
head j // (heads / kv_heads).  Position p sees key j if j <= p and (p - j < ``window`` or j < ``keep_first``); ``window``
None: every earlier key.  Kept tokens keep their own positions.  Scores times ``scale``, then with ``softcap`` c the
score s becomes c tanh(s / c); an ordinary softmax over the visible keys, the weighted sum of values; with ``gate``
"elements" the heads side by side are multiplied element by element by sigmoid(W_g h), a projection of the same input
without a bias that rides in the q | k | v product; then the output matrix.

The convolution, head norm, rotation and the cache write are one kernel; scores and softmax are float32.  The cache holds
keys and values in pages (``KVRequirement`` with the window and the kept tokens: pages that hold neither are given back);
beside it a sequence keeps the last ``conv - 1`` projected rows in a float32 region, so the mixer asks for two caches.

Parameters: hidden_size, heads, kv_heads, dim, vdim, conv, qk_norm_eps, rot_dims, rot_base, scale, window, keep_first,
softcap, biases, gate; ``names``: full tensor names by role (q, k, v, q_conv, k_conv, v_conv, q_norm, k_norm, o, gate,
q_bias, k_bias, v_bias; the biases default to the matrix's name with ``.b``, the gate to ``<prefix>.g``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KVRequirement, StateRequirement
from ..errors import require
from ..weights.loader import TensorSpec
from .base import bind_vector, register_part
from .delta import bind_float32
from .linear import DenseLinear

_ROLES = ("q", "k", "v", "q_conv", "k_conv", "v_conv", "q_norm", "k_norm", "o")


class WindowAttention:
    graph_safe = True            # slots and positions are read on the device; the launch depends on the row count alone
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.nq, self.nkv = int(params["heads"]), int(params.get("kv_heads") or params["heads"])
        self.d = int(params["dim"])
        self.vd = int(params.get("vdim") or self.d)
        self.has_conv = params.get("conv") is not None
        self.taps = int(params.get("conv") or 1)
        self.eps = params.get("qk_norm_eps")
        self.rot_dims = int(params.get("rot_dims") or 0)
        self.rot_base = float(params.get("rot_base") or 1.0)
        self.scale = float(params["scale"])
        self.window = None if params.get("window") is None else int(params["window"])
        self.keep_first = int(params.get("keep_first") or 0) if self.window is not None else 0
        self.softcap = float(params.get("softcap") or 0.0)
        self.has_biases = bool(params.get("biases", False))
        self.has_gate = params.get("gate") is not None
        require(params.get("gate") in (None, "elements"), f"{prefix}: gate must be 'elements' or None")
        require(self.softcap >= 0.0, f"{prefix}: softcap must be positive or None")
        require(self.nq % self.nkv == 0, f"{prefix}: {self.nq} query heads are not a multiple of {self.nkv} key/value heads")
        require(self.rot_dims % 2 == 0 and self.rot_dims <= self.d,
                f"{prefix}: {self.rot_dims} rotated elements must be even and at most the head size {self.d}")
        require(self.window is None or self.window > 0, f"{prefix}: window must be positive or None")
        require(self.d <= 256 and self.vd <= 256, f"{prefix}: heads of {self.d} / {self.vd} exceed the kernels' 256")
        n = dict(params.get("names") or {})
        self.names = {r: str(n.get(r) or f"{prefix}.{r}") for r in _ROLES}
        self.names["gate"] = str(n.get("gate") or f"{prefix}.g")
        for r in ("q", "k", "v"):
            self.names[r + "_bias"] = str(n.get(r + "_bias") or self.names[r] + ".b")
        self.prefix = prefix
        self.C = (self.nq + self.nkv) * self.d + self.nkv * self.vd
        nm = self.names
        self.sizes = [self.nq * self.d, self.nkv * self.d, self.nkv * self.vd]
        self.qkv = DenseLinear([nm["q"], nm["k"], nm["v"]] + ([nm["gate"]] if self.has_gate else []),
                               self.sizes + ([self.nq * self.vd] if self.has_gate else []), self.hidden)
        self.o = DenseLinear([nm["o"]], [self.hidden], self.nq * self.vd)

    def tensor_specs(self):
        nm = self.names
        specs = self.qkv.tensor_specs() + self.o.tensor_specs()
        if self.has_conv:
            specs += [TensorSpec(nm["q_conv"], (self.nq * self.d, self.taps), "state"),
                      TensorSpec(nm["k_conv"], (self.nkv * self.d, self.taps), "state"),
                      TensorSpec(nm["v_conv"], (self.nkv * self.vd, self.taps), "state")]
        if self.eps is not None:
            specs += [TensorSpec(nm["q_norm"], (self.d,), "gain"), TensorSpec(nm["k_norm"], (self.d,), "gain")]
        if self.has_biases:
            specs += [TensorSpec(nm[r + "_bias"], (size,), "state") for r, size in zip(("q", "k", "v"), self.sizes)]
        return specs

    def cache_requirement(self):
        kv = KVRequirement(self.nkv, self.d, self.window, value_dim=self.vd, keep_first=self.keep_first)
        if self.taps > 1:
            return (kv, StateRequirement(((self.taps - 1) * self.C,), torch.float32))
        return (kv,)

    def bind(self, weights, ctx):
        nm = self.names
        self.qkv.bind(weights, ctx)
        self.o.bind(weights, ctx)
        if self.has_conv:
            self.conv_w = torch.cat([bind_float32(weights, nm["q_conv"], (self.nq * self.d, self.taps), ctx),
                                     bind_float32(weights, nm["k_conv"], (self.nkv * self.d, self.taps), ctx),
                                     bind_float32(weights, nm["v_conv"], (self.nkv * self.vd, self.taps), ctx)], 0).contiguous()
        else:
            self.conv_w = torch.ones((self.C, 1), dtype=torch.float32, device=ctx.device)
        self.q_gain = self.k_gain = None
        if self.eps is not None:
            self.q_gain = bind_float32(weights, nm["q_norm"], (self.d,), ctx)
            self.k_gain = bind_float32(weights, nm["k_norm"], (self.d,), ctx)
        self.bias = None
        if self.has_biases:
            self.bias = torch.cat([bind_vector(weights, nm[r + "_bias"], size, ctx)
                                   for r, size in zip(("q", "k", "v"), self.sizes)]).contiguous()
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        self.inv_freq = (torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / max(self.rot_dims, 1))
                         .to(torch.float32).to(ctx.device))
        self.dtype = ctx.dtype

    def forward(self, h, batch, cache_view, residual, write_cache=True, overwrite=False):
        require(isinstance(cache_view, tuple) and len(cache_view) == (2 if self.taps > 1 else 1),
                f"{self.prefix}: attention behind a convolution needs a key/value cache and a region for its last inputs")
        require(write_cache, f"{self.prefix}: this attention always keeps its own keys and values")
        kv = cache_view[0]
        state = cache_view[1].storage if self.taps > 1 else None
        rows = batch.rows
        proj = self.qkv.forward(h, out_dtype=torch.float32)
        q = torch.empty((rows, self.nq * self.d), dtype=self.dtype, device=proj.device)
        ops.conv_heads_prepare(proj, self.conv_w, state, 0, self.q_gain, self.k_gain, self.inv_freq, self.rot_dims, batch, kv,
                               q, self.nq, self.nkv, self.d, self.vd, float(self.eps or 0.0), bias=self.bias)
        if self.taps > 1:
            ops.conv_keep(proj, proj.shape[1], self.taps, self.C, state, 0, batch)
        out = torch.empty((rows, self.nq * self.vd), dtype=self.dtype, device=proj.device)
        ops.attention_window(q, kv, batch, out, self.nq, self.nkv, self.d, self.vd, self.window, self.keep_first, self.scale,
                             softcap=self.softcap, gate=proj[:, self.C:] if self.has_gate else None)
        if overwrite:
            self.o.forward(out, out=residual)
        else:
            self.o.forward(out, accumulate_into=residual)
        return residual


register_part("mixer", "window_attention", WindowAttention)
