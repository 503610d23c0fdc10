"""Throughput of a decoder design beside another of the library's designs at equal size, with every kernel of a step timed.

Used by ``bench.py --design lanizen`` (beside the Qwen3 dense decoder), ``--design gidirax`` (beside Lanizen, the
closest design the library has: both mix delta-rule layers with windowed attention) and ``--design sobunex`` (beside
Gidirax: both have windowed attention with key and value sizes of their own, layer norms on the sub-layers' outputs and
experts whose weights are not renormalised) and ``--design pivavik`` (beside Sobunex: both are made of attention layers
only, with windows, output gates, biases, and dense and routed feed-forwards in turn).  A size is a width and a number of layers; both models get that width, that
many layers, feed-forwards of equal parameter count (8 width^2: two matrices of 4 width, or three of 8/3 width) and
the same vocabulary, with random weights in bfloat16.  Measured per model: one prompt in one step (tokens a second),
one decode step of ``batch`` sequences at ``context`` through the session's ``decode`` (the replayed graph where the
model allows one), and the device time of every kernel of both steps, each between two CUDA events, grouped by
kernel, with the bytes it must move or the FLOPs it must do and the fraction of the measured peak that makes.
Between timed steps a buffer larger than L2 is written.
"""
from __future__ import annotations

import statistics
from typing import Dict, List

import torch

from . import ops
from .config.registry import config_from_dict
from .engine.session import InferenceSession
from .engine.step import StepEntry

SIZES = {"small": dict(width=1024, layers=4, vocab=32768), "medium": dict(width=2048, layers=4, vocab=32768),
         "large": dict(width=4096, layers=4, vocab=32768)}


def lanizen_config(width: int, layers: int, vocab: int, streams: int = 4, window: int = 1024):
    """Three delta-rule layers to one latent-attention layer; heads of 128; a latent of 512 + 64."""
    heads = max(1, width // 128)
    delta = {"type": "delta", "mixer": {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4},
             "mlp": {"kind": "dense", "ff": 4 * width}}
    latent = {"type": "latent_attention",
              "mixer": {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": max(256, width * 3 // 8),
                        "kv_rank": 512, "scale": 192 ** -0.5, "mask": {"size": window},
                        "rot": {"base": 10000.0, "dims": 64}},
              "mlp": {"kind": "dense", "ff": 4 * width}}
    return config_from_dict({"architecture": "Lanizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
                             "embedding": {"scale": 1.0}, "streams": streams,
                             "layers": [latent if i % 4 == 3 else delta for i in range(layers)]})


def gidirax_config(width: int, layers: int, vocab: int, window: int = 1024):
    """Layers in turn: delta rule with a decay per key channel, state-space, attention beside a recurrent unit, delta rule.
    Heads of 128 (state-space: heads of 64 over an inner width of 2 x width, a state of 128); sixteen experts of which a
    token uses four, about 8 width^2 parameters in all experts of a layer."""
    heads = max(1, width // 128)
    ff = max(64, (width // 6 + 32) // 64 * 64)
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2}}}
    delta = {"type": "channel_delta", "mlp": mlp,
             "mixer": {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64,
                       "gate_rank": 64}}
    ssm = {"type": "mamba2", "mlp": mlp,
           "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}}
    par = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "conv": 4, "scale": 128 ** -0.5,
                 "mask": {"size": window, "keep_first": 4}, "rot": {"base": 10000.0, "dims": 64}},
        "right": {"width": width, "blocks": heads, "conv": 4}, "left_scale": 1.0, "right_scale": 1.0}}
    order = [delta, ssm, par, delta]
    return config_from_dict({"architecture": "Gidirax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
                             "layers": [order[i % 4] for i in range(layers)]})


def sobunex_config(width: int, layers: int, vocab: int, window: int = 1024):
    """Attention layers only, in pairs: one with keys and values of its own and a dense feed-forward of 4 x width, one that
    reads the first one's keys and has sixteen experts of which a token uses four, plus an expert for every row (about
    8 width^2 parameters in a layer's experts).  Heads of 128, four query heads a key/value head."""
    heads = max(1, width // 128)
    ff = max(64, (width // 6 + 32) // 64 * 64)
    mixer = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
             "mask": {"size": window}, "q_temp": {"coef": 0.1, "every": 512}}
    own = {"type": "attention", "mixer": dict(mixer), "mlp": {"kind": "dense", "ff": 4 * width}}
    moe = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": 16, "top": 4, "scale": 2.0},
           "shared": {"ff": 2 * ff, "limit": 7.0}}
    out = []
    for i in range(layers):
        out.append(own if i % 2 == 0 else {"type": "attention", "mixer": dict(mixer, kv_from=i - 1), "mlp": moe})
    return config_from_dict({"architecture": "Sobunex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": out})


def pivavik_config(width: int, layers: int, vocab: int, window: int = 1024):
    """Latent-attention and windowed-attention layers in turn, heads of 128 (latent layers: 128 unrotated + 64 rotated
    elements a head, a latent of 512); dense feed-forwards of 8/3 width (three matrices: 8 width^2 parameters) and sixteen
    experts of which a token uses four (about 8 width^2 in all experts of a layer) in turn, so that each kind of mixer meets
    each kind of feed-forward.  The middle layers are a repeated run that runs once: the step ahead of it is measured, and
    the model runs as many layers as the design beside it."""
    heads = max(1, width // 128)
    ff = max(64, (width // 6 + 32) // 64 * 64)
    dense = {"kind": "dense", "ff": (8 * width // 3 + 255) // 256 * 256}
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": 16, "top": 4}}
    latent = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": max(256, width * 3 // 8), "kv_rank": 512,
              "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}
    attention = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 30.0,
                 "mask": {"size": window}}
    order = [("latent_attention", latent, dense), ("attention", attention, moe), ("latent_attention", latent, moe),
             ("attention", attention, dense)]
    out = [{"type": t, "mixer": dict(m), "mlp": dict(f)} for t, m, f in (order[i % 4] for i in range(layers))]
    d = {"architecture": "Pivavik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": out}
    if layers >= 3:
        d["loop"] = {"start": 1, "stop": layers - 1, "times": 1}
    return config_from_dict(d)


def qwen3_config(width: int, layers: int, vocab: int):
    heads = max(1, width // 128)
    return config_from_dict(dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads,
        num_key_value_heads=max(1, heads // 4), head_dim=128, intermediate_size=(8 * width // 3 + 255) // 256 * 256,
        vocab_size=vocab, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960))


class KernelTimer:
    """While active, every kernel function of :mod:`ops` runs between two CUDA events."""

    SKIP = {"lib", "launch_count", "sm_count", "zero_counters", "attention", "gemm_tc_plan", "gemm_tc_accepts",
            "gemm_tc_pair_plan", "gemm_tc_runs_on_pairs", "gemm_tc_is_small_form", "gemm_tc_set_pair_rows",
            "attention_steps_from_device", "wait_selftest", "sigmoid_attention_mma_supports",
            "sigmoid_attention_mma_scratch_bytes", "sigmoid_attention_run_keys"}

    def __init__(self):
        self.records: List[tuple] = []
        self._saved: Dict[str, object] = {}

    def __enter__(self):
        for name, fn in list(vars(ops).items()):
            if name.startswith("_") or name in self.SKIP or not callable(fn) or getattr(fn, "__module__", "") != ops.__name__ \
                    or isinstance(fn, type):
                continue
            self._saved[name] = fn

            def timed(*a, _fn=fn, _name=name, **kw):
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                out = _fn(*a, **kw)
                end.record()
                self.records.append((_name, _shape_note(_name, a), start, end))
                return out
            setattr(ops, name, timed)
        return self

    def __exit__(self, *exc):
        for name, fn in self._saved.items():
            setattr(ops, name, fn)
        torch.cuda.synchronize()

    def summary(self) -> Dict[str, dict]:
        out: Dict[str, dict] = {}
        for name, note, a, b in self.records:
            key = name if not note else f"{name} {note}"
            e = out.setdefault(key, {"calls": 0, "us": 0.0})
            e["calls"] += 1
            e["us"] += a.elapsed_time(b) * 1e3
        for e in out.values():
            e["us_per_call"] = round(e["us"] / e["calls"], 2)
            e["us"] = round(e["us"], 1)
        return out


def _shape_note(name, args) -> str:
    if name in ("gemm_tc", "gemm_simt", "gemm_tc_pair"):
        return f"{args[0].shape[0]}x{args[1].shape[0]}x{args[0].shape[1]}"
    return ""


def _flush(buf):
    buf.add_(1.0)


def measure_model(config, prompt_tokens: int, batch: int, context: int, steps: int, warmup: int, seed: int = 1) -> dict:
    dev = torch.device("cuda:0")
    session = InferenceSession().load_random(config, seed=seed, max_context=context + steps + warmup + 8, dtype="bfloat16",
                                             device="cuda:0", max_batch=batch)
    vocab = session.model.spec.vocab_size
    gen = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, vocab, (prompt_tokens,), generator=gen).tolist()
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device=dev)         # 256 MB: larger than L2
    ev = lambda: torch.cuda.Event(enable_timing=True)
    out = {"weights_bytes_per_step": session.model.weight_bytes_read_per_step(), "cache_bytes": session.cache.bytes()}

    # ---- one prompt in one step -------------------------------------------------------------------------------------
    times = []
    for i in range(warmup + 3):
        slot = session.acquire()
        _flush(flush)
        a, b = ev(), ev()
        a.record()
        session.step([StepEntry(slot, prompt, [prompt_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        session.release(slot)
        if i >= warmup:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    out["prefill"] = {"tokens": prompt_tokens, "ms": round(ms, 3), "tokens_per_s": round(prompt_tokens / ms * 1e3, 1)}
    slot = session.acquire()
    with KernelTimer() as timer:
        session.step([StepEntry(slot, prompt, [prompt_tokens - 1])])
    session.release(slot)
    out["prefill"]["kernels"] = timer.summary()

    # ---- decoding: `batch` sequences at `context` ------------------------------------------------------------------
    slots = [session.acquire() for _ in range(batch)]
    for s in slots:
        session.assume_cached(s, context)          # the cache's memory as it is: the time does not depend on its values
    tokens = torch.randint(0, vocab, (batch,), generator=gen).tolist()
    for _ in range(warmup):
        session.decode(slots, tokens, 0.0, [])
    per_step = []
    for _ in range(steps):
        _flush(flush)
        a, b = ev(), ev()
        a.record()
        session.decode(slots, tokens, 0.0, [])
        b.record()
        torch.cuda.synchronize()
        per_step.append(a.elapsed_time(b))
    ms = statistics.median(per_step)
    out["decode"] = {"batch": batch, "context": context, "ms_per_step": round(ms, 4),
                     "tokens_per_s": round(batch / ms * 1e3, 1), "replayed_graph": session.runner is not None,
                     "launches_per_step": (session.runner.kernels_per_replay.get((batch, True)) if session.runner else None)}
    with KernelTimer() as timer:
        session.step([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)])
    out["decode"]["kernels"] = timer.summary()
    for s in slots:
        session.release(s)
    session.check_device_errors()
    del session
    torch.cuda.empty_cache()
    return out


DESIGNS = {"lanizen": (lanizen_config, "qwen3"), "gidirax": (gidirax_config, "lanizen"), "sobunex": (sobunex_config, "gidirax"),
           "pivavik": (pivavik_config, "sobunex"), "qwen3": (qwen3_config, None)}


def run(design: str, sizes, prompt_tokens: int, batch: int, context: int, steps: int, warmup: int) -> dict:
    """The design and the design it is held beside (``DESIGNS``), each at every size."""
    make, beside = DESIGNS[design]
    result = {}
    for name in sizes:
        size = SIZES[name]
        result[name] = {
            "size": dict(size),
            design: measure_model(make(**size), prompt_tokens, batch, context, steps, warmup),
            beside: measure_model(DESIGNS[beside][0](**size), prompt_tokens, batch, context, steps, warmup),
        }
    return result
