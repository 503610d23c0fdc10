"""Configuration of the Pivavik decoder, read from its own config.json keys.

Pivavik is a decoder whose layers run mixer and feed-forward side by side on one norm: h = N(x), x <- x + (mixer(h) +
ff(h)), with N an RMS norm whose stored weight w acts as the factor 1 + w.  The embedding's rows pass such a norm before
the first layer (``embed.norm``), the last norm is ``final.norm``, the head is the embedding table, and the logits are
capped softly: ``logit_softcap`` c makes them c tanh(logits / c).

config ``layers`` lists the layers in order, each with a ``type`` that names its mixer, the mixer's sizes (``mixer``) and
its feed-forward (``mlp``, or null for none):

* ``latent_attention``: causal softmax attention through one cached latent a token (``kv_rank``) and one rotated key part
  that all heads share (``rot_dim``); queries through a latent of their own (``q_rank``), laid out head by head as
  ``dim`` unrotated then ``rot_dim`` rotated elements; the rotation pairs element i with element i + rot.dims / 2 and
  turns them by position * rot.base^(-2i / rot.dims); a sigmoid gate with one number a head on the heads' outputs.
* ``attention``: grouped-query softmax attention without a rotation, with biases on q, k and v, a soft cap on the scaled
  scores (``softcap``), a sliding window (``mask.size``) and a sigmoid gate an element on the heads side by side.

Feed-forwards: ``dense`` (W_down (gelu_tanh(W_gate h) * (W_up h)), every projection with a bias) or ``moe`` (``expert``
{ff}, ``router`` {experts, top}: bias-free SiLU-gated experts; the router's scores are sigmoids of its logits, the ``top``
largest are chosen and used as they are, and a chosen expert reads its score times h).

``loop`` {start, stop, times}: layers start .. stop - 1 run ``times`` times in a row with the same weights and a cache of
their own every time; ahead of every such pass t the residual becomes W_in [x ; x0] + step[t], with x0 the normed
embedding rows, ``loop.in`` [width, 2 width] and ``loop.step`` [times, width].

Tensor names: ``embed``, ``embed.norm``, ``final.norm``, ``loop.in``, ``loop.step``; layer i's tensors start with
``l<i>.``: ``norm1``, ``mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}`` or ``mix.{q,k,v}`` (+ ``.b``) and ``mix.{g,o}``,
``mlp.{gate,up,down}`` (+ ``.b``) or ``mlp.router`` and ``mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..errors import require
from .lanizen import _int, _number
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

ARCHITECTURE = "Pivavik"
MAX_POSITIONS = 1 << 24          # positions are exact as float32 up to here; the design itself sets no limit

_LAYER_TYPES = ("latent_attention", "attention")
_MLP_KINDS = ("dense", "moe")


def _check_latent(m, mw):
    for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
        _int(m, key, mw)
    rot_dim = _int(m, "rot_dim", mw, minimum=0)
    _number(m, "scale", mw)
    if m.get("rot") is not None:
        dims = _int(m["rot"], "dims", mw + ".rot", minimum=0)
        _number(m["rot"], "base", mw + ".rot")
        require(dims % 2 == 0 and dims <= rot_dim, f"config.json: {mw}.rot.dims {dims} must be even and at most rot_dim {rot_dim}")


def _check_attention(m, mw):
    heads = _int(m, "heads", mw)
    kv = _int(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
    require(heads % kv == 0, f"config.json: {mw}.heads {heads} is not a multiple of kv_heads {kv}")
    _int(m, "dim", mw)
    if m.get("vdim") is not None:
        _int(m, "vdim", mw)
    _number(m, "scale", mw)
    if m.get("softcap") is not None:
        _number(m, "softcap", mw)
    if m.get("mask") is not None:
        _int(m["mask"], "size", mw + ".mask")


def _check_mlp(mlp, lw):
    require(isinstance(mlp, dict) and mlp.get("kind") in _MLP_KINDS, f"config.json: {lw}.kind must be one of: {', '.join(_MLP_KINDS)}")
    if mlp["kind"] == "dense":
        _int(mlp, "ff", lw)
        return
    _int(mlp.get("expert"), "ff", lw + ".expert")
    r = mlp.get("router")
    experts, top = _int(r, "experts", lw + ".router"), _int(r, "top", lw + ".router")
    require(top <= experts, f"config.json: {lw}.router.top {top} exceeds experts {experts}")


@dataclass(frozen=True)
class PivavikConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: Optional[float]
    loop: Optional[Tuple[int, int, int]]        # (start, stop, times)
    layers: Tuple[Dict[str, Any], ...]          # as config.json lists them, validated

    # ---- reading -------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PivavikConfig":
        vocab = _int(d, "vocab", "the top level")
        width = _int(d, "width", "the top level")
        eps = _number(d.get("norm"), "eps", "norm")
        cap = None if d.get("logit_softcap") is None else _number(d, "logit_softcap", "the top level")
        layers = d.get("layers")
        require(isinstance(layers, list) and len(layers) > 0, "config.json: 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            require(isinstance(layer, dict), f"config.json: {where} must be an object")
            kind = layer.get("type")
            require(kind in _LAYER_TYPES, f"config.json: {where}.type '{kind}' is unknown; known: {', '.join(_LAYER_TYPES)}")
            require(isinstance(layer.get("mixer"), dict), f"config.json: {where}.mixer must be an object")
            (_check_latent if kind == "latent_attention" else _check_attention)(layer["mixer"], where + ".mixer")
            if layer.get("mlp") is not None:
                _check_mlp(layer["mlp"], where + ".mlp")
            checked.append(copy.deepcopy(layer))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            start, stop = _int(lp, "start", "loop", minimum=0), _int(lp, "stop", "loop", minimum=0)
            times = _int(lp, "times", "loop")
            require(start < stop <= len(layers), f"config.json: loop runs layers {start} .. {stop} - 1, the model has {len(layers)}")
            loop = (start, stop, times)
        return cls(vocab, width, eps, cap, loop, tuple(checked))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": copy.deepcopy(list(self.layers))}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    def describe(self) -> Dict[str, Any]:
        one = lambda l: l["type"] + (" + " + l["mlp"]["kind"] if l.get("mlp") else " (no feed-forward)")
        loop = "none" if self.loop is None else f"layers {self.loop[0]}..{self.loop[1] - 1} x {self.loop[2]}"
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm_eps": self.norm_eps,
                "logit_softcap": self.logit_softcap, "loop": loop, "layers": ", ".join(one(l) for l in self.layers)}

    # ---- the architecture as data ----------------------------------------------------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps, "tensor": name, "offset": 1.0}, name)

    def _mixer(self, p: str, kind: str, m) -> PartSpec:
        if kind == "latent_attention":
            rot = m.get("rot")
            return PartSpec("latent_attention", {
                "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "norm_eps": self.norm_eps,
                "window": None, "rot_dims": rot["dims"] if rot is not None else 0,
                "rot_base": rot["base"] if rot is not None else 1.0, "rot_layout": "halves", "gate": "heads",
                "kv_projection": True,
                "names": {"dq": f"{p}.dq", "dq_norm": f"{p}.dq.norm", "uq": f"{p}.uq", "dkv": f"{p}.dkv",
                          "dkv_norm": f"{p}.dkv.norm", "uk": f"{p}.uk", "uv": f"{p}.uv", "gate": f"{p}.g", "o": f"{p}.o",
                          "sink": None}}, p)
        return PartSpec("window_attention", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m.get("kv_heads") or m["heads"], "dim": m["dim"],
            "vdim": m.get("vdim") or m["dim"], "conv": None, "qk_norm_eps": None, "rot_dims": 0, "scale": m["scale"],
            "window": None if m.get("mask") is None else m["mask"]["size"], "keep_first": 0, "softcap": m.get("softcap"),
            "biases": True, "gate": "elements"}, p)

    def _feed_forward(self, p: str, mlp) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("gated", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "gelu_tanh",
                                      "biases": True, "names": {"gate": f"{p}.gate", "up": f"{p}.up", "down": f"{p}.down"}}, p)
        r = mlp["router"]
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "experts": r["experts"], "top": r["top"], "intermediate_size": mlp["expert"]["ff"],
            "groups": None, "keep_groups": None, "weight_scale": 1.0, "score": "sigmoid", "weight_on": "input",
            "activation": "silu", "shared": None}, p)

    def to_model_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}"
            parts = {"norm": self._norm(f"{p}.norm1"), "mixer": self._mixer(f"{p}.mix", layer["type"], layer["mixer"])}
            if layer.get("mlp") is not None:
                parts["feed_forward"] = self._feed_forward(f"{p}.mlp", layer["mlp"])
            layers.append(LayerSpec(block="parallel_residual", parts=parts))
        n = len(layers)
        if self.loop is None:
            schedule = [ScheduleStep(i) for i in range(n)]
        else:
            start, stop, times = self.loop
            # the step ahead of every pass is a layer of its own, named once a pass: it counts its runs itself
            layers.append(LayerSpec(block="input_injection", parts={}, block_params={
                "hidden_size": self.width, "passes": times, "matrix": "loop.in", "steps": "loop.step"}))
            schedule = [ScheduleStep(i) for i in range(start)]
            for _ in range(times):
                schedule.append(ScheduleStep(n))
                schedule += [ScheduleStep(i) for i in range(start, stop)]
            schedule += [ScheduleStep(i) for i in range(stop, n)]
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
            embedding_name="embed", layers=tuple(layers), schedule=tuple(schedule), final_norm=self._norm("final.norm"),
            head_name="head", tie_head_to_embedding=True, stop_token_ids=(), embedding_norm=self._norm("embed.norm"),
            logit_softcap=self.logit_softcap)
        spec.validate()
        return spec
