"""Configuration of the Sobunex decoder, read from its own config.json keys.

Sobunex is a decoder whose every sub-layer sits between two layer norms (weight and bias): x <- x + LN(mixer(LN(x))), then
x <- x + LN(ff(LN(x))).  config ``layers`` lists the layers in order, each with a ``type`` that names its mixer, the mixer's
sizes (``mixer``) and its feed-forward (``mlp``, or null for none).  The one mixer is ``attention``: grouped-query attention
without a rotation and without a softmax.  A key's weight is a sigmoid of its score; the score loses a slope times the
distance, slope 2^(-8 (h + 1) / H) for head h of H; the heads' scores are mixed by a matrix; a number a head is added; a
gate per head multiplies the head's output; the query is multiplied by a temperature that grows with the logarithm of the
position (``q_temp`` {coef, every}); ``mask`` {size} is a sliding window.  ``kv_from``: j makes the layer read layer j's keys
and values instead of projecting its own.

Feed-forwards: ``dense`` (W_down xielu(W_up h), with biases and the activation's two numbers in a tensor) or ``moe``
(``expert`` {ff, limit}, ``router`` {experts, top, scale}, optional ``shared`` {ff, limit}): experts with a clamped gate
g sigmoid(1.702 g) (u + 1), weights softmax scores times ``router.scale``, not renormalised.  The last norm is a layer norm
with a bias; the head is a matrix of its own.

Tensor names: ``embed``, ``final.norm`` (+ ``.b``), ``head``; layer i's tensors start with ``l<i>.``: ``norm1``, ``norm1b``,
``norm2``, ``norm2b`` (+ ``.b``), ``mix.{q,k,v,o}`` (+ ``.b``), ``mix.talk``, ``mix.pb``, ``mix.g``, ``mlp.{up,down}`` (+ ``.b``),
``mlp.act``, ``mlp.router``, ``mlp.e<j>.{gate,up,down}``, ``mlp.shared.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..errors import require
from .lanizen import _int, _number
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

ARCHITECTURE = "Sobunex"
MAX_POSITIONS = 1 << 24          # positions are exact as float32 up to here; the design itself sets no limit
SLOPE_EXPONENT = 8.0             # head h of H loses 2^(-8 (h + 1) / H) a token of distance
SWISH_ALPHA = 1.702              # of the experts' gate

_LAYER_TYPES = ("attention",)
_MLP_KINDS = ("dense", "moe")
_SHARED_KEYS = ("heads", "kv_heads", "dim", "vdim")      # what a layer and the layer whose keys it reads must agree on


def _kv_heads(m):
    return m["heads"] if m.get("kv_heads") is None else m["kv_heads"]


def _vdim(m):
    return m["dim"] if m.get("vdim") is None else m["vdim"]


def _window(m):
    return None if m.get("mask") is None else m["mask"]["size"]


def _check_mixer(m, mw, i, layers):
    require(isinstance(m, dict), f"config.json: {mw} must be an object")
    heads = _int(m, "heads", mw)
    kv = _int(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
    require(heads % kv == 0, f"config.json: {mw}.heads {heads} is not a multiple of kv_heads {kv}")
    _int(m, "dim", mw)
    if m.get("vdim") is not None:
        _int(m, "vdim", mw)
    _number(m, "scale", mw)
    if m.get("mask") is not None:
        _int(m["mask"], "size", mw + ".mask")
    if m.get("q_temp") is not None:
        _number(m["q_temp"], "coef", mw + ".q_temp", positive=False)
        _int(m["q_temp"], "every", mw + ".q_temp")
    src = m.get("kv_from")
    if src is not None:
        require(isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i
                and layers[src].get("type") == "attention" and layers[src]["mixer"].get("kv_from") is None,
                f"config.json: {mw}.kv_from must name an earlier attention layer with keys and values of its own, got {src!r}")
        other = layers[src]["mixer"]
        require(heads == other["heads"] and kv == _kv_heads(other) and m["dim"] == other["dim"] and _vdim(m) == _vdim(other),
                f"config.json: {mw}: {', '.join(_SHARED_KEYS)} must equal those of layer {src}, whose keys and values it reads")


def _check_expert(e, where):
    _int(e, "ff", where)
    _number(e, "limit", where)


def _check_mlp(mlp, lw):
    require(isinstance(mlp, dict) and mlp.get("kind") in _MLP_KINDS,
            f"config.json: {lw}.kind must be one of: {', '.join(_MLP_KINDS)}")
    if mlp["kind"] == "dense":
        _int(mlp, "ff", lw)
        return
    _check_expert(mlp.get("expert"), lw + ".expert")
    r = mlp.get("router")
    experts, top = _int(r, "experts", lw + ".router"), _int(r, "top", lw + ".router")
    require(top <= experts, f"config.json: {lw}.router.top {top} exceeds experts {experts}")
    if r.get("scale") is not None:
        _number(r, "scale", lw + ".router", positive=False)
    if mlp.get("shared") is not None:
        _check_expert(mlp["shared"], lw + ".shared")


@dataclass(frozen=True)
class SobunexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]          # as config.json lists them, validated

    # ---- reading -------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SobunexConfig":
        vocab = _int(d, "vocab", "the top level")
        width = _int(d, "width", "the top level")
        eps = _number(d.get("norm"), "eps", "norm")
        layers = d.get("layers")
        require(isinstance(layers, list) and len(layers) > 0, "config.json: 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            require(isinstance(layer, dict), f"config.json: {where} must be an object")
            kind = layer.get("type")
            require(kind in _LAYER_TYPES, f"config.json: {where}.type '{kind}' is unknown; known: {', '.join(_LAYER_TYPES)}")
            _check_mixer(layer.get("mixer"), where + ".mixer", i, layers)
            if layer.get("mlp") is not None:
                _check_mlp(layer["mlp"], where + ".mlp")
            checked.append(copy.deepcopy(layer))
        return cls(vocab, width, eps, tuple(checked))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(list(self.layers))}

    def describe(self) -> Dict[str, Any]:
        def one(l):
            m = l["mixer"]
            text = l["type"] + (f" (keys of layer {m['kv_from']})" if m.get("kv_from") is not None else "")
            return text + (" + " + l["mlp"]["kind"] if l.get("mlp") else " (no feed-forward)")
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm_eps": self.norm_eps,
                "layers": ", ".join(one(l) for l in self.layers)}

    # ---- the architecture as data ----------------------------------------------------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("layer_norm", {"size": self.width, "eps": self.norm_eps, "tensor": name, "bias": name + ".b"}, name)

    def _feed_forward(self, p: str, mlp) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("xielu", {"hidden_size": self.width, "intermediate_size": mlp["ff"]}, f"{p}.mlp")
        r, shared = mlp["router"], mlp.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "experts": r["experts"], "top": r["top"], "intermediate_size": mlp["expert"]["ff"],
            "groups": None, "keep_groups": None, "weight_scale": 1.0 if r.get("scale") is None else r["scale"],
            "activation": "clamped_swish", "limit": mlp["expert"]["limit"], "alpha": SWISH_ALPHA,
            "shared": None if shared is None else {"intermediate_size": shared["ff"], "limit": shared["limit"]}}, f"{p}.mlp")

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        readers: Dict[int, list] = {}                 # layer -> the windows of the layers that read its keys and values
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            readers.setdefault(i if m.get("kv_from") is None else m["kv_from"], []).append(_window(m))
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer["mixer"]
            own = m.get("kv_from") is None
            windows = readers[i] if own else []
            parts = {"mixer_norm": self._norm(f"{p}.norm1"), "mixer_out_norm": self._norm(f"{p}.norm1b")}
            parts["mixer"] = PartSpec("sigmoid_attention", {
                "hidden_size": self.width, "heads": m["heads"], "kv_heads": _kv_heads(m), "dim": m["dim"], "vdim": _vdim(m),
                "scale": m["scale"], "window": _window(m),
                "cache_window": None if (not own or None in windows) else max(windows),
                "q_temp": copy.deepcopy(m.get("q_temp")), "slope_exp": SLOPE_EXPONENT, "own_kv": own,
                "talk": True, "head_bias": True, "gate": True, "biases": True}, f"{p}.mix")
            if layer.get("mlp") is not None:
                parts["feed_forward_norm"] = self._norm(f"{p}.norm2")
                parts["feed_forward"] = self._feed_forward(p, layer["mlp"])
                parts["feed_forward_out_norm"] = self._norm(f"{p}.norm2b")
            layers.append(LayerSpec(block="sandwich_norm", parts=parts))
            schedule.append(ScheduleStep(i, None if own else int(m["kv_from"])))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
            embedding_name="embed", layers=tuple(layers), schedule=tuple(schedule), final_norm=self._norm("final.norm"),
            head_name="head", tie_head_to_embedding=False, stop_token_ids=())
        spec.validate()
        return spec
