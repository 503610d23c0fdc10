"""A plain, slow restatement of the Sobunex decoder for tests: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the package.  Weights come as a ``{name: tensor}`` mapping and the configuration as
the dictionary config.json holds.

Notation: T tokens, W the model's width, H query heads, G key/value heads; ``h`` is a sub-layer's input ``[T, W]``.  A
layer is  x <- x + LN_1b(mixer(LN_1(x)));  x <- x + LN_2b(ff(LN_2(x)))  with layer norms that have a weight and a bias.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def f64(t):
    return t.to(F)


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean of squared deviations."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * f64(w) + f64(b)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def linear(h, w, name, bias=True):
    y = h @ f64(w[name]).T
    return y + f64(w[name + ".b"]) if bias else y


# ---- attention --------------------------------------------------------------------------------------------------------

def query_temperature(positions, coef, every):
    """1 + coef ln(floor((p + 1) / every) + 1) for every position p."""
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in positions], dtype=F)


def head_slopes(H):
    """2^(-8 (h + 1) / H) for h = 0 .. H-1."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F)


def raw_scores(q, k, scale, H, G):
    """q [T, H, D], k [T, G, D] -> [H, T, T]: (q_i . k_j) scale minus slope_h (i - j); head h reads key head h // (H/G)."""
    T = q.shape[0]
    i = torch.arange(T, dtype=F)
    dist = i[:, None] - i[None, :]
    s = torch.empty(H, T, T, dtype=F)
    slopes = head_slopes(H)
    for h in range(H):
        s[h] = q[:, h] @ k[:, h // (H // G)].T * scale - slopes[h] * dist
    return s


def mix_heads(s, talk):
    """s_h <- sum_g talk[h, g] s_g."""
    return torch.einsum("hg,gij->hij", f64(talk), s)


def visible(T, window):
    """[T, T] bool: j <= i and (window is None or i - j < window)."""
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    ok = d >= 0
    if window is not None:
        ok &= d < window
    return ok


def sigmoid_weights(s, pb, mask):
    """sigmoid(s_h + pb_h) where visible, 0 elsewhere; nothing is normalised over keys."""
    return torch.sigmoid(s + f64(pb)[:, None, None]) * mask[None].to(F)


def attention_keys_values(h, w, p, m):
    G, D = m.get("kv_heads") or m["heads"], m["dim"]
    V = m.get("vdim") or D
    T = h.shape[0]
    return linear(h, w, p + ".k").view(T, G, D), linear(h, w, p + ".v").view(T, G, V)


def attention_mixer(h, w, p, m, kv=None, store=None):
    """``kv``: the (keys, values) of the layer this one borrows from (None: its own).  ``store``: how keys and values are
    rounded when they are kept (None: not at all)."""
    T = h.shape[0]
    H, G, D = m["heads"], m.get("kv_heads") or m["heads"], m["dim"]
    V = m.get("vdim") or D
    q = linear(h, w, p + ".q").view(T, H, D)
    if kv is None:
        k, v = attention_keys_values(h, w, p, m)
        if store is not None:
            k, v = store(k), store(v)
    else:
        k, v = kv
    qt = m.get("q_temp")
    if qt is not None:
        q = q * query_temperature(range(T), qt["coef"], qt["every"])[:, None, None]
    s = mix_heads(raw_scores(q, k, m["scale"], H, G), w[p + ".talk"])
    mask = m.get("mask")
    a = sigmoid_weights(s, w[p + ".pb"], visible(T, mask["size"] if mask is not None else None))
    o = torch.empty(T, H, V, dtype=F)
    for hd in range(H):
        o[:, hd] = a[hd] @ v[:, hd // (H // G)]
    gate = torch.sigmoid(h @ f64(w[p + ".g"]).T)                      # [T, H], no bias
    o = o * gate[:, :, None]
    return linear(o.reshape(T, H * V), w, p + ".o"), (k, v)


# ---- feed-forwards ----------------------------------------------------------------------------------------------------

def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    ap = softplus(torch.as_tensor(p, dtype=F))
    an = 0.5 + softplus(torch.as_tensor(q, dtype=F))
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(neg) - neg) + 0.5 * z)


def dense_ff(h, w, p):
    act = f64(w[p + ".act"])
    return linear(xielu(linear(h, w, p + ".up"), act[0], act[1]), w, p + ".down")


def clamped_expert(h, w, p, limit):
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1)); no biases."""
    g = torch.clamp(linear(h, w, p + ".gate", bias=False), max=limit)
    u = torch.clamp(linear(h, w, p + ".up", bias=False), -limit, limit)
    return linear(g * torch.sigmoid(1.702 * g) * (u + 1.0), w, p + ".down", bias=False)


def route(h, w, p, r):
    """[T, E] weights: softmax over all experts, the ``top`` largest kept (lowest index wins a tie), times ``scale``, not
    renormalised; zero elsewhere.  Also the chosen indices and the margin between the last chosen and the first left out."""
    s = torch.softmax(h @ f64(w[p + ".router"]).T, -1)
    E, top = r["experts"], r["top"]
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices
    chosen = order[:, :top]
    out = torch.zeros_like(s)
    out.scatter_(1, chosen, s.gather(1, chosen) * float(r.get("scale", 1.0)))
    if top < E:
        margin = s.gather(1, order[:, top - 1:top]) - s.gather(1, order[:, top:top + 1])
    else:
        margin = torch.full((s.shape[0], 1), float("inf"), dtype=F)
    return out, chosen, margin[:, 0]


def moe_ff(h, w, p, mlp):
    weights, _, _ = route(h, w, p, mlp["router"])
    y = torch.zeros(h.shape[0], w[p + ".e0.down"].shape[0], dtype=F)
    for e in range(mlp["router"]["experts"]):
        rows = torch.nonzero(weights[:, e] != 0)[:, 0]
        if rows.numel():
            y[rows] += weights[rows, e:e + 1] * clamped_expert(h[rows], w, f"{p}.e{e}", mlp["expert"]["limit"])
    if mlp.get("shared") is not None:
        y = y + clamped_expert(h, w, p + ".shared", mlp["shared"]["limit"])
    return y


def feed_forward(h, w, p, mlp):
    return dense_ff(h, w, p) if mlp["kind"] == "dense" else moe_ff(h, w, p, mlp)


# ---- the model ----------------------------------------------------------------------------------------------------------

def forward(config, w, tokens, round_inputs=None, store=None, return_layers=False):
    """Logits [T, vocab] (float64) for one sequence.  ``round_inputs``: applied to what a product reads (None: nothing);
    ``store``: how kept keys and values are rounded."""
    eps = config["norm"]["eps"]
    rin = round_inputs or (lambda t: t)
    x = f64(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    kept, per_layer = {}, []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        ln = lambda t, n: layer_norm(t, w[f"{p}.{n}"], w[f"{p}.{n}.b"], eps)
        src = m.get("kv_from")
        y, kept[i] = attention_mixer(rin(ln(x, "norm1")), w, p + ".mix", m, kv=None if src is None else kept[src], store=store)
        x = x + ln(y, "norm1b")
        if layer.get("mlp") is not None:
            x = x + ln(feed_forward(rin(ln(x, "norm2")), w, p + ".mlp", layer["mlp"]), "norm2b")
        per_layer.append(x.clone())
    logits = rin(layer_norm(x, w["final.norm"], w["final.norm.b"], eps)) @ f64(w["head"]).T
    return (logits, torch.stack(per_layer)) if return_layers else logits
