"""Grouped-query attention whose weights are sigmoids instead of a softmax, on scores that the heads mix among themselves.

For a token at position i with input h:  q (``heads`` H of ``dim``), k (``kv_heads`` G of ``dim``), v (G of ``vdim``) and
a gate (one number a head) are projections of h; q, k, v and the output may have biases.  There is no rotation.  Position
enters three ways:

* ``q_temp`` {coef, every}: q is multiplied by 1 + coef ln(floor((i + 1) / every) + 1) (None: not at all);
* ``slope_exp`` c: head g's score to key j loses 2^(-c (g + 1) / H) (i - j) (0: nothing);
* ``window`` w: key j is visible if 0 <= i - j < w (None: every key up to i).

With s_g(j) = (q_g . k_j) ``scale`` minus the distance term (query head g reads key/value head g // (H / G)), the heads'
scores are mixed, m_h = sum_g T[h, g] s_g (``talk``), a number a head is added (``head_bias``), and the weight of a visible
key is sigmoid(m_h): nothing is normalised over the keys.  Head h's sum of weighted values is multiplied by the sigmoid of
its gate, and the output matrix is applied to the heads side by side.  ``talk``, ``head_bias`` and ``gate`` are optional.

A mixer with ``own_kv`` False has no key and value projections: it is given another step's cache to read (the schedule's
``cache_of``) and asks for none.  ``cache_window`` is the reach the kept keys must have (the widest window of this mixer and
of those that read its cache; None: everything is kept).

How it runs: one product for q | k | v | gate with a float32 result; one kernel adds the biases, applies the temperature,
writes k and v to the paged cache and takes the gate's sigmoid.  Single tokens, and everything in 32-bit: one kernel a row
does scores, mix, sigmoid and the sums in float32 over the cache, in an order of sums that depends on the row's position
and the window alone.  Runs of new tokens in bfloat16 (``mma_min_rows`` rows or more): two tensor-core kernels, one that
writes all heads' weights of 8 rows and a run of pages (scores by MMA, mix and sigmoid in float32, rounded to bfloat16), one
that multiplies them with the values a head and 64 rows at a time; the weights in between take at most ``mma_max_scratch``
bytes, else the first form runs.  Then the output product.

Parameters: hidden_size, heads, kv_heads, dim, vdim, scale, window, cache_window, q_temp, slope_exp, own_kv, talk,
head_bias, gate, biases; ``names``: full tensor names by role (q, k, v, o, talk, head_bias, gate, q_bias, k_bias, v_bias,
o_bias).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KVRequirement
from ..errors import require
from ..weights.loader import TensorSpec
from .base import bind_vector, register_part
from .delta import bind_float32
from .linear import DenseLinear

_DEFAULTS = {"q": "q", "k": "k", "v": "v", "o": "o", "talk": "talk", "head_bias": "pb", "gate": "g", "q_bias": "q.b",
             "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b"}


class SigmoidAttention:
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.H, self.G = int(params["heads"]), int(params.get("kv_heads") or params["heads"])
        self.D = int(params["dim"])
        self.V = int(params.get("vdim") or self.D)
        self.scale = float(params["scale"])
        self.window = None if params.get("window") is None else int(params["window"])
        self.cache_window = self.window if "cache_window" not in params else (
            None if params["cache_window"] is None else int(params["cache_window"]))
        qt = params.get("q_temp")
        self.temp_coef, self.temp_every = (float(qt["coef"]), int(qt["every"])) if qt is not None else (0.0, 0)
        self.slope_exp = float(params.get("slope_exp") or 0.0)
        self.own_kv = bool(params.get("own_kv", True))
        self.has_talk = bool(params.get("talk", True))
        self.has_head_bias = bool(params.get("head_bias", True))
        self.has_gate = bool(params.get("gate", True))
        self.has_biases = bool(params.get("biases", True))
        require(self.H % self.G == 0, f"{prefix}: {self.H} query heads are not a multiple of {self.G} key/value heads")
        require(self.window is None or self.window > 0, f"{prefix}: window must be positive or None")
        require(self.cache_window is None or (self.window is not None and self.cache_window >= self.window),
                f"{prefix}: the kept keys reach {self.cache_window} back, the window {self.window}")
        require(qt is None or self.temp_every > 0, f"{prefix}: q_temp.every must be positive")
        n = dict(params.get("names") or {})
        self.names = {r: str(n.get(r) or f"{prefix}.{d}") for r, d in _DEFAULTS.items()}
        self.prefix = prefix
        nm = self.names
        stacked, sizes = [nm["q"]], [self.H * self.D]
        if self.own_kv:
            stacked += [nm["k"], nm["v"]]
            sizes += [self.G * self.D, self.G * self.V]
        if self.has_gate:
            stacked.append(nm["gate"])
            sizes.append(self.H)
        self.sizes = sizes
        self.proj = DenseLinear(stacked, sizes, self.hidden)
        self.o = DenseLinear([nm["o"]], [self.hidden], self.H * self.V)
        self.bias = self.deferred_bias = self.talk = self.head_bias = None
        self.mma_min_rows = int(params.get("mma_min_rows", 64))            # fewer rows a step: the kernel a row
        self.mma_max_scratch = int(params.get("mma_max_scratch", 2 << 30))   # bytes of weights between the two kernels

    @property
    def graph_safe(self):
        # with a window the launch depends on the row count alone; without one the runs follow the longest row
        return self.window is not None

    def _on_tensor_cores(self, batch, kv, rows) -> bool:
        """Runs of new tokens in bfloat16 go to the two tensor-core kernels when these have the sizes and the weights they
        keep in between stay small; single tokens, 32-bit and everything else go to the kernel that walks a row's keys."""
        if self.dtype != torch.bfloat16 or rows < self.mma_min_rows or rows < 8 * len(batch.slots):
            return False
        if not ops.sigmoid_attention_mma_supports(self.H, self.G, self.D, self.V, kv.page_size):
            return False
        need = ops.sigmoid_attention_mma_scratch_bytes(rows, len(batch.slots), max(batch.max_keys, 1), self.H, self.window)
        return need <= self.mma_max_scratch

    def _bias_names(self):
        nm = self.names
        return [nm["q_bias"]] + ([nm["k_bias"], nm["v_bias"]] if self.own_kv else [])

    def tensor_specs(self):
        nm = self.names
        specs = self.proj.tensor_specs() + self.o.tensor_specs()
        if self.has_biases:
            specs += [TensorSpec(b, (s,), "state") for b, s in zip(self._bias_names(), self.sizes)]
            specs.append(TensorSpec(nm["o_bias"], (self.hidden,), "state"))
        if self.has_talk:
            specs.append(TensorSpec(nm["talk"], (self.H, self.H), "state"))
        if self.has_head_bias:
            specs.append(TensorSpec(nm["head_bias"], (self.H,), "state"))
        return specs

    def cache_requirement(self):
        if not self.own_kv:
            return None
        return KVRequirement(self.G, self.D, self.cache_window, value_dim=self.V)

    def bind(self, weights, ctx):
        nm = self.names
        self.proj.bind(weights, ctx)
        self.o.bind(weights, ctx)
        if self.has_biases:
            pieces = [bind_vector(weights, b, s, ctx) for b, s in zip(self._bias_names(), self.sizes)]
            if self.has_gate:
                pieces.append(torch.zeros(self.H, dtype=torch.float32, device=ctx.device))     # the gate has no bias
            self.bias = torch.cat(pieces).contiguous()
            self.deferred_bias = bind_vector(weights, nm["o_bias"], self.hidden, ctx)
        if self.has_talk:
            self.talk = bind_float32(weights, nm["talk"], (self.H, self.H), ctx)
        if self.has_head_bias:
            self.head_bias = bind_vector(weights, nm["head_bias"], self.H, ctx)
        self.dtype = ctx.dtype
        self.run_keys = ops.sigmoid_attention_run_keys()

    def forward(self, h, batch, cache_view, residual, write_cache=True, overwrite=False, defer_bias=False):
        """``overwrite``: ``residual`` holds nothing yet and receives the output.  ``defer_bias``: the caller adds
        ``deferred_bias`` (the output's bias) itself."""
        require(cache_view is not None and not isinstance(cache_view, tuple),
                f"{self.prefix}: this attention reads one key/value cache")
        require(write_cache == self.own_kv,
                f"{self.prefix}: a mixer with key and value projections keeps them in a cache of its own; one without reads another's")
        kv = cache_view
        rows = batch.rows
        proj = self.proj.forward(h, out_dtype=torch.float32)
        q = torch.empty((rows, self.H * self.D), dtype=self.dtype, device=proj.device)
        gate = torch.empty((rows, self.H), dtype=torch.float32, device=proj.device) if self.has_gate else None
        ops.biased_heads_prepare(proj, self.bias, batch, kv, q, gate, self.H, self.G, self.D, self.V, self.own_kv,
                                 self.temp_coef, self.temp_every)
        out = torch.empty((rows, self.H * self.V), dtype=self.dtype, device=proj.device)
        if self._on_tensor_cores(batch, kv, rows):
            ops.sigmoid_attention_mma(q, kv, batch, self.talk, self.head_bias, gate, out, self.H, self.G, self.D, self.V,
                                      self.window, self.scale, self.slope_exp)
        else:
            # few rows: a row's keys are dealt to several blocks, as many as the window (or, without one, the longest row)
            # has runs; with a window the launch then depends on the row count alone
            reach = self.window if self.window is not None else max(batch.max_keys, 1)
            runs = (reach + self.run_keys - 1) // self.run_keys if rows < 512 else 1
            ops.sigmoid_attention(q, kv, batch, self.talk, self.head_bias, gate, out, self.H, self.G, self.D, self.V,
                                  self.window, self.scale, self.slope_exp, runs=runs)
        if overwrite:
            self.o.forward(out, out=residual)
        else:
            self.o.forward(out, accumulate_into=residual)
        if self.deferred_bias is not None and not defer_bias:
            ops.add_row_bias(residual, self.deferred_bias)
        return residual


register_part("mixer", "sigmoid_attention", SigmoidAttention)
