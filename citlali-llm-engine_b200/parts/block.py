"""Arrangements of a layer's parts around the residual stream.

``pre_norm_residual`` is the reference's layer (src/model/qwen_model.cpp:306-374):
x += mixer(norm(x)); x += feed_forward(norm(x)).  The residual stream is float32 and the two
sums are 32-bit additions.  Either half may be absent from the layer's parts (a layer with a
mixer only, or a feed-forward only).

For few rows in bfloat16 (decoding) the two norms need no kernels of their own: the product that ends a sub-layer also
writes the updated residual rows as bfloat16 with the sums of their squares, the product that begins the next sub-layer
reads those rows and scales its result by the inverse root mean square, and the norm's gain is multiplied into that
product's weights once, when the layer is bound (x . (g W)^T rsqrt(mean x^2 + eps) = (x rsqrt(...) g) . W^T).  That is
an arrangement between this block, RMSNorm and parts that say they can (``can_absorb_norm``); other parts and other
norms run the plain way.

A block is given the layer's description and builds its parts from the registries by the
names it knows; another arrangement (four norms a layer, one norm for a mixer and a
feed-forward side by side) is another class registered under another kind, with part names of
its own.
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import require
from ..weights.loader import TensorSpec
from .base import NormedRows, build_part, register_part
from .linear import DenseLinear
from .norm import RMSNorm

_FEW_ROWS = 128        # up to here the product always runs the form whose epilogue can do a norm's work


class PreNormResidualBlock:
    def __init__(self, layer_spec):
        has = layer_spec.parts.__contains__
        self.mixer = self.mixer_norm = self.feed_forward = self.feed_forward_norm = None
        if has("mixer"):
            self.mixer_norm = build_part("norm", layer_spec.part("mixer_norm"))
            self.mixer = build_part("mixer", layer_spec.part("mixer"))
        if has("feed_forward"):
            self.feed_forward_norm = build_part("norm", layer_spec.part("feed_forward_norm"))
            self.feed_forward = build_part("feed_forward", layer_spec.part("feed_forward"))

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        return [t for p in self.parts() for t in p.tensor_specs()]

    def cache_requirement(self):
        return self.mixer.cache_requirement() if self.mixer is not None else None

    def bind(self, weights, ctx):
        for p in self.parts():
            p.bind(weights, ctx)
        self.norms_in_products = (
            self.mixer is not None and self.feed_forward is not None and ctx.dtype == torch.bfloat16
            and type(self.mixer_norm) is RMSNorm and type(self.feed_forward_norm) is RMSNorm
            and not self.mixer_norm.gain_downstream and not self.feed_forward_norm.gain_downstream
            and self.mixer_norm.size % 32 == 0 and self.mixer_norm.size == self.feed_forward_norm.size
            and callable(getattr(self.mixer, "can_absorb_norm", None)) and self.mixer.can_absorb_norm()
            and callable(getattr(self.feed_forward, "can_absorb_norm", None)) and self.feed_forward.can_absorb_norm())
        if self.norms_in_products:
            self.mixer.fold_norm_gain(self.mixer_norm.gain_moves_downstream())
            self.feed_forward.fold_norm_gain(self.feed_forward_norm.gain_moves_downstream())

    def forward(self, x, batch, cache_view, write_cache=True):
        if getattr(self, "norms_in_products", False) and 0 < batch.rows <= _FEW_ROWS:
            return self._forward_norms_in_products(x, batch, cache_view, write_cache)
        if self.mixer is not None:
            self.mixer.forward(self.mixer_norm.forward(x), batch, cache_view, x, write_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(self.feed_forward_norm.forward(x), batch, x)
        return x

    def _forward_norms_in_products(self, x, batch, cache_view, write_cache):
        rows, hidden = x.shape
        def buffers():
            return (torch.empty((rows, hidden), dtype=torch.bfloat16, device=x.device),
                    torch.empty((rows, hidden // 32), dtype=torch.float32, device=x.device))
        carried = batch.norm_carry_in
        if carried is None or carried.rows.shape != (rows, hidden):
            rows_bf16, sumsq = buffers()                   # the rows came from somewhere that emitted nothing
            ops.norm_inputs(x, rows_bf16, sumsq)
            carried = NormedRows(rows_bf16, sumsq, hidden)
        after_mixer = buffers()
        self.mixer.forward(carried.with_eps(self.mixer_norm.eps), batch, cache_view, x, write_cache, emit=after_mixer)
        after_ff = buffers()
        self.feed_forward.forward(NormedRows(after_mixer[0], after_mixer[1], hidden, self.feed_forward_norm.eps), batch, x,
                                  emit=after_ff)
        batch.norm_carry = NormedRows(after_ff[0], after_ff[1], hidden)
        return x


class SublayerOutputNormBlock:
    """x += norm(mixer(x)); x += norm(feed_forward(x)): the sub-layers read the residual stream itself and the norm sits on
    what they give.  Parts by name: ``mixer``, ``mixer_norm``, ``feed_forward``, ``feed_forward_norm`` (either pair may be
    absent); a norm here is one with ``add_into(y, x, emit)`` (a layer norm).  The sub-layers' outputs are float32 and the
    sum is a 32-bit addition; the rows a sub-layer reads are the residual rounded once to the compute dtype, left behind by
    the kernel that did the sum before (for a model's first layer by a conversion of its own; none in the 32-bit path, where
    the sub-layers read the residual's own memory).  Any registered mixer or feed-forward serves: one that says
    ``can_overwrite`` stores its output, any other adds it into a zeroed buffer."""

    def __init__(self, layer_spec):
        has = layer_spec.parts.__contains__
        self.subs = []
        for role, norm_name in (("mixer", "mixer_norm"), ("feed_forward", "feed_forward_norm")):
            if has(role):
                norm = build_part("norm", layer_spec.part(norm_name))
                if not callable(getattr(norm, "add_into", None)):
                    raise TypeError(f"the norm behind a {role} must offer add_into(y, x, emit); '{layer_spec.part(norm_name).kind}' does not")
                self.subs.append((role, build_part(role, layer_spec.part(role)), norm))
        self.mixer = next((p for r, p, _ in self.subs if r == "mixer"), None)

    def parts(self):
        return [p for _, part, norm in self.subs for p in (part, norm)]

    def tensor_specs(self):
        return [t for p in self.parts() for t in p.tensor_specs()]

    def cache_requirement(self):
        return self.mixer.cache_requirement() if self.mixer is not None else None

    def bind(self, weights, ctx):
        for p in self.parts():
            p.bind(weights, ctx)
        self.dtype = ctx.dtype

    def forward(self, x, batch, cache_view, write_cache=True):
        rows, hidden = x.shape
        h = batch.rows_carry_in if self.dtype != torch.float32 else x
        if h is None or h.shape != x.shape or h.dtype != self.dtype:
            h = torch.empty((rows, hidden), dtype=self.dtype, device=x.device)
            ops.cast_rows(x, h)
        for role, part, norm in self.subs:
            fresh = bool(getattr(part, "can_overwrite", False))
            y = (torch.empty if fresh else torch.zeros)((rows, hidden), dtype=torch.float32, device=x.device)
            extra = {"overwrite": True} if fresh else {}
            if role == "mixer":
                part.forward(h, batch, cache_view, y, write_cache, **extra)
            else:
                part.forward(h, batch, y, **extra)
            if self.dtype != torch.float32:
                h = torch.empty((rows, hidden), dtype=self.dtype, device=x.device)
                norm.add_into(y, x, emit=h)
            else:
                norm.add_into(y, x)
        if self.dtype != torch.float32:
            batch.rows_carry = h             # the residual as the next layer's sub-layers read it
        return x


class SandwichNormBlock:
    """x += norm_out(mixer(norm_in(x))); x += norm_out'(feed_forward(norm_in'(x))): a norm in front of every sub-layer and
    another on what it gives.  Parts by name: ``mixer_norm``, ``mixer``, ``mixer_out_norm``, ``feed_forward_norm``,
    ``feed_forward``, ``feed_forward_out_norm`` (either triple may be absent).  The sub-layers' outputs are float32 and
    the sum is a 32-bit addition.

    Norms that say ``chain_terms()`` (layer norms; gain, bias, eps) are run in one kernel a sub-layer: the norm on the
    sub-layer's output, the sum into the residual, and the norm in front of the NEXT sub-layer read and write a row once.
    The next sub-layer may be the next layer's: this block then leaves the normed rows for it (``StepBatch.normed_carry``:
    the rows and the norm they went through), and a block that finds rows made by its own first norm skips that norm.  A sub-layer that offers ``deferred_bias`` (its output's bias) has it added in the same kernel.
    Other norms run one by one (``forward`` in front, ``add_into`` behind)."""

    def __init__(self, layer_spec):
        has = layer_spec.parts.__contains__
        self.subs = []
        for role in ("mixer", "feed_forward"):
            if has(role):
                self.subs.append((role, build_part("norm", layer_spec.part(role + "_norm")), build_part(role, layer_spec.part(role)),
                                  build_part("norm", layer_spec.part(role + "_out_norm"))))
        self.mixer = next((p for r, _, p, _ in self.subs if r == "mixer"), None)

    def parts(self):
        return [p for _, before, part, after in self.subs for p in (before, part, after)]

    def tensor_specs(self):
        return [t for p in self.parts() for t in p.tensor_specs()]

    def cache_requirement(self):
        return self.mixer.cache_requirement() if self.mixer is not None else None

    def bind(self, weights, ctx):
        for p in self.parts():
            p.bind(weights, ctx)
        self.dtype = ctx.dtype
        self.chained = all(callable(getattr(n, "chain_terms", None)) for _, before, _, after in self.subs for n in (before, after))

    def first_norm(self):
        return self.subs[0][1] if self.subs else None

    def forward(self, x, batch, cache_view, write_cache=True):
        rows, hidden = x.shape
        h = None
        carried = batch.normed_carry_in
        if (self.subs and carried is not None and carried[1] is self.subs[0][1] and carried[0].shape == x.shape
                and carried[0].dtype == self.dtype):
            h = carried[0]                    # the block ahead already ran this block's first norm
        for k, (role, before, part, after) in enumerate(self.subs):
            if h is None:
                h = before.forward(x)
            fresh = bool(getattr(part, "can_overwrite", False))
            y = (torch.empty if fresh else torch.zeros)((rows, hidden), dtype=torch.float32, device=x.device)
            extra = {"overwrite": True} if fresh else {}
            bias = getattr(part, "deferred_bias", None) if self.chained else None
            if bias is not None:
                extra["defer_bias"] = True
            if role == "mixer":
                part.forward(h, batch, cache_view, y, write_cache, **extra)
            else:
                part.forward(h, batch, y, **extra)
            h = None
            if not self.chained:
                after.add_into(y, x)
                continue
            nxt = self.subs[k + 1][1] if k + 1 < len(self.subs) else batch.next_first_norm
            gain, nbias, eps = after.chain_terms()
            if nxt is not None and callable(getattr(nxt, "chain_terms", None)) and nxt.size == hidden:
                g2, b2, eps2 = nxt.chain_terms()
                h = torch.empty((rows, hidden), dtype=self.dtype, device=x.device)
                ops.layer_norm_chain(y, x, gain, nbias, eps, in_bias=bias, next_gain=g2, next_bias=b2, next_eps=eps2, next_out=h)
                if k + 1 == len(self.subs):
                    batch.normed_carry = (h, nxt)
            else:
                ops.layer_norm_chain(y, x, gain, nbias, eps, in_bias=bias)
        return x


class ParallelResidualBlock:
    """h = norm(x); x += mixer(h) + feed_forward(h): one norm, and both sub-layers read what it gives.  Parts by name:
    ``norm``, ``mixer``, ``feed_forward`` (either sub-layer may be absent).  Both outputs are added into the float32
    residual by the products that end the sub-layers (32-bit additions)."""

    def __init__(self, layer_spec):
        has = layer_spec.parts.__contains__
        self.norm = build_part("norm", layer_spec.part("norm"))
        self.mixer = build_part("mixer", layer_spec.part("mixer")) if has("mixer") else None
        self.feed_forward = build_part("feed_forward", layer_spec.part("feed_forward")) if has("feed_forward") else None

    def parts(self):
        return [p for p in (self.norm, self.mixer, self.feed_forward) if p is not None]

    def tensor_specs(self):
        return [t for p in self.parts() for t in p.tensor_specs()]

    def cache_requirement(self):
        return self.mixer.cache_requirement() if self.mixer is not None else None

    def bind(self, weights, ctx):
        for p in self.parts():
            p.bind(weights, ctx)

    def first_norm(self):
        return self.norm

    def forward(self, x, batch, cache_view, write_cache=True):
        h = self.norm.forward(x)
        if self.mixer is not None:
            self.mixer.forward(h, batch, cache_view, x, write_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(h, batch, x)
        return x


class InputInjectionBlock:
    """x <- W [x ; x0] + b_t: the residual is mixed again with the rows the embedding left (x0), by one matrix
    ``[hidden, 2 hidden]`` whose first half meets x, and a vector is added that depends on how often this block has run
    in the step (row t of a table ``[passes, hidden]``; a schedule names the block once ahead of every pass over a run of
    layers that repeats).  No norm, no cache.  The product reads [x ; x0] rounded once to the compute dtype; its result
    and the sum are float32.  ``block_params``: hidden_size, passes, ``matrix`` and ``steps`` (the tensors' full names)."""
    needs_embedding_output = True
    graph_safe = True

    def __init__(self, layer_spec):
        bp = layer_spec.block_params
        self.hidden, self.passes = int(bp["hidden_size"]), int(bp["passes"])
        self.steps_name = str(bp["steps"])
        self.mix = DenseLinear([str(bp["matrix"])], [self.hidden], 2 * self.hidden)

    def parts(self):
        return []

    def tensor_specs(self):
        return self.mix.tensor_specs() + [TensorSpec(self.steps_name, (self.passes, self.hidden), "state")]

    def cache_requirement(self):
        return None

    def bind(self, weights, ctx):
        self.mix.bind(weights, ctx)
        h = weights[self.steps_name]
        require(tuple(h.shape) == (self.passes, self.hidden),
                f"unexpected tensor shape for {self.steps_name}: got {list(h.shape)}, expected {[self.passes, self.hidden]}")
        self.steps = h.tensor.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.dtype = ctx.dtype

    def forward(self, x, batch, cache_view, write_cache=True):
        x0 = batch.embedding_output
        require(x0 is not None and x0.shape == x.shape and x0.data_ptr() != x.data_ptr(),
                "the injection block needs the embedding's rows beside the residual")
        require(0 <= batch.visit < self.passes, f"the injection block has run {batch.visit} times, its table has {self.passes} rows")
        both = torch.empty((x.shape[0], 2 * self.hidden), dtype=self.dtype, device=x.device)
        ops.concat_rows(x, x0, both)
        self.mix.forward(both, out=x)
        ops.add_row_bias(x, self.steps[batch.visit])
        return x


register_part("block", "parallel_residual", ParallelResidualBlock)
register_part("block", "input_injection", InputInjectionBlock)
register_part("block", "pre_norm_residual", PreNormResidualBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("block", "sublayer_output_norm", SublayerOutputNormBlock)
