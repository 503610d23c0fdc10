"""Attention through a shared latent, with a sliding window, a sink in the softmax and an output gate.

Per token the cache keeps one vector: the latent c (``kv_rank`` numbers, RMS-normed with a plain weight) and one key
part r (``rot_dim`` numbers, rotated by the position) that all heads share.  Head a's key is [W_uk,a c | r], its value
W_uv,a c, its query [q_plain | q_rot] = W_uq RMSnorm(W_dq h) with q_rot rotated like r.  Since
q_plain . (W_uk c) = (W_uk^T q_plain) . c, the heads' matrices are applied to the query before and to the weighted sum of
latents after the walk over the cache (``ops.heads_product``), and the walk (``ops.latent_attention``) reads the cached
vector once for every head.  Scores are scaled by ``scale``; position i sees j with 0 <= i - j < window (None: every
j <= i); the softmax's denominator also counts exp(sink_a), a learned number per head without key or value (absent
tensor name: none); the heads side by side are multiplied by sigmoid(W_g h), then pass the output matrix.  ``gate``
"elements" (the default): W_g gives a number for every element of every head's output; "heads": one number a head.

A layer with ``kv_projection`` false has no W_dkv and reads the cache of the layer the model's schedule names; the
layer that owns a cache keeps it for the widest window among its readers (``cache_window``).

Rotation: pairs (2i, 2i+1), i < rot_dims / 2, of the key part and of each head's q_rot turn by position * base^(-2i /
rot_dims); the angle is a float32 product of the position and a tabulated frequency.  ``rot_layout`` "halves" pairs
element i with element i + rot_dims / 2 instead (the first of a pair, u, becomes u cos - v sin, the second v cos + u sin).

The result of W_dq / W_dkv / W_g (one product) and the query are kept in float32; norms, rotation, scores and softmax are
float32 in both paths.

Parameters: hidden_size, heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, norm_eps, window, cache_window,
rot_dims, rot_base, rot_layout, gate, kv_projection; ``names``: full tensor names by role (dq, dq_norm, uq, dkv, dkv_norm, uk, uv, sink,
gate, o); ``sink`` may be None.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KVRequirement
from ..errors import require
from ..weights.loader import TensorSpec
from .base import register_part
from .delta import bind_float32
from .linear import DenseLinear


class LatentAttention:
    graph_safe = True
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.H = int(params["heads"])
        self.D = int(params["dim"])
        self.P = int(params["rot_dim"])
        self.V = int(params["vdim"])
        self.RQ = int(params["q_rank"])
        self.R = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["norm_eps"])
        self.window = params.get("window")
        self.cache_window = params.get("cache_window", self.window)
        self.rot_dims = int(params.get("rot_dims") or 0)
        self.rot_base = float(params.get("rot_base") or 1.0)
        self.kv_projection = bool(params.get("kv_projection", True))
        self.rot_halves = {"pairs": False, "halves": True}.get(str(params.get("rot_layout") or "pairs"))
        require(self.rot_halves is not None, f"{prefix}: rot_layout must be 'pairs' or 'halves'")
        self.gate_per_head = {"elements": False, "heads": True}.get(str(params.get("gate") or "elements"))
        require(self.gate_per_head is not None, f"{prefix}: gate must be 'elements' or 'heads'")
        require(self.window is None or int(self.window) > 0, f"{prefix}: window must be positive or None")
        require(self.rot_dims % 2 == 0 and self.rot_dims <= self.P,
                f"{prefix}: {self.rot_dims} rotated dimensions must be even and at most the key part's {self.P}")
        require(self.R + self.P <= 1024, f"{prefix}: a cached vector of {self.R + self.P} exceeds the walk's 1024")
        n = dict(params.get("names") or {})
        roles = ("dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "gate", "o")
        self.names = {r: str(n.get(r) or f"{prefix}.{r}") for r in roles}
        self.names["sink"] = n.get("sink", f"{prefix}.sink")          # None: a plain softmax
        self.prefix = prefix
        nm, hv = self.names, self.H * self.V
        down = [nm["dq"]] + ([nm["dkv"]] if self.kv_projection else []) + [nm["gate"]]
        outs = [self.RQ] + ([self.R + self.P] if self.kv_projection else []) + [self.H if self.gate_per_head else hv]
        self.down = DenseLinear(down, outs, self.hidden)
        self.gate_at = sum(outs[:-1])
        self.uq = DenseLinear([nm["uq"]], [self.H * (self.D + self.P)], self.RQ)
        self.o = DenseLinear([nm["o"]], [self.hidden], hv)

    def tensor_specs(self):
        nm = self.names
        specs = self.down.tensor_specs() + self.uq.tensor_specs() + self.o.tensor_specs() + [
            TensorSpec(nm["dq_norm"], (self.RQ,), "gain"),
            TensorSpec(nm["uk"], (self.H * self.D, self.R), "matrix"),
            TensorSpec(nm["uv"], (self.H * self.V, self.R), "matrix")]
        if self.kv_projection:
            specs.append(TensorSpec(nm["dkv_norm"], (self.R,), "gain"))
        if nm["sink"] is not None:
            specs.append(TensorSpec(nm["sink"], (self.H,), "state"))
        return specs

    def cache_requirement(self):
        if not self.kv_projection:
            return None
        w = self.cache_window
        return KVRequirement(1, self.R + self.P, None if w is None else int(w), value_dim=0)

    def bind(self, weights, ctx):
        nm = self.names
        for part in (self.down, self.uq, self.o):
            part.bind(weights, ctx)
        self.q_weight = bind_float32(weights, nm["dq_norm"], (self.RQ,), ctx)
        self.c_weight = bind_float32(weights, nm["dkv_norm"], (self.R,), ctx) if self.kv_projection else None
        self.sink = bind_float32(weights, nm["sink"], (self.H,), ctx) if nm["sink"] is not None else None
        uk = torch.empty((self.H * self.D, self.R), dtype=ctx.dtype, device=ctx.device)
        self.uv = torch.empty((self.H * self.V, self.R), dtype=ctx.dtype, device=ctx.device)
        for name, dst in ((nm["uk"], uk), (nm["uv"], self.uv)):
            require(tuple(weights[name].shape) == tuple(dst.shape),
                    f"unexpected tensor shape for {name}: got {list(weights[name].shape)}, expected {list(dst.shape)}")
            weights[name].copy_into(dst)
        # W_uk meets the query along its rows (sum over a head's D rows): kept [head, R, D], so that both per-head products
        # read their matrices along the axis they sum over, in 16-byte pieces
        self.uk = uk.view(self.H, self.D, self.R).transpose(1, 2).contiguous()
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        self.inv_freq = (torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / max(self.rot_dims, 1))
                         .to(torch.float32).to(ctx.device)) if self.rot_dims else None
        self.dtype = ctx.dtype

    def forward(self, h, batch, cache_view, residual, write_cache=True, overwrite=False):
        require(cache_view is not None and cache_view.requirement.head_dim == self.R + self.P
                and cache_view.requirement.num_kv_heads == 1,
                f"{self.prefix}: the cache does not hold vectors of {self.R} + {self.P}")
        require(write_cache == self.kv_projection,
                f"{self.prefix}: a layer with a latent projection writes its own cache; one without reads another's")
        rows, H, R, P, D, V = batch.rows, self.H, self.R, self.P, self.D, self.V
        dev = h.device
        pool, table, page = cache_view.keys, cache_view.page_table, cache_view.page_size
        proj = self.down.forward(h, out_dtype=torch.float32)
        cq = torch.empty((rows, self.RQ), dtype=self.dtype, device=dev)
        ops.latent_prepare(proj, self.RQ, R, P, self.kv_projection, self.q_weight, self.c_weight, self.inv_freq,
                           self.rot_dims, batch.row_slot, batch.row_pos, table, pool, page, cq, self.eps,
                           rot_halves=self.rot_halves)
        q = self.uq.forward(cq, out_dtype=torch.float32)                      # [rows, H (D + P)]
        qa = torch.empty((rows, H * (R + P)), dtype=torch.float32, device=dev)
        ops.heads_product(q, H * (D + P), D + P, self.uk, D * R, 1, D, qa, H * (R + P), R + P, rows, H, D, R,
                          tail=P, inv_freq=self.inv_freq, rot_dims=self.rot_dims, row_pos=batch.row_pos,
                          rot_halves=self.rot_halves)
        mixed = torch.empty((rows, H * R), dtype=torch.float32, device=dev)
        ops.latent_attention(qa, pool, table, batch.row_slot, batch.row_pos, self.sink, mixed, H, R, R + P, page,
                             int(self.window or 0), self.scale)
        heads = torch.empty((rows, H * V), dtype=self.dtype, device=dev)
        ops.heads_product(mixed, H * R, R, self.uv, V * R, 1, R, heads, H * V, V, rows, H, R, V,
                          gate=proj[:, self.gate_at:], gate_stride=proj.shape[1], gate_per_head=self.gate_per_head)
        if overwrite:
            self.o.forward(heads, out=residual)
        else:
            self.o.forward(heads, accumulate_into=residual)
        return residual


register_part("mixer", "latent_attention", LatentAttention)
