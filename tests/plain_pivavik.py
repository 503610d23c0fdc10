"""A plain, slow restatement of the Pivavik decoder for tests: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the package.  Weights come as a ``{name: tensor}`` mapping and the configuration as
the dictionary config.json holds.

Notation: T tokens, W the model's width, H query heads, G key/value heads; ``h`` is a layer's normed input ``[T, W]``.
A layer is  h = N(x);  x <- x + (mixer(h) + ff(h))  with N an RMS norm whose stored weight w acts as the factor 1 + w.
The embedding's rows pass such a norm too.  Layers ``loop.start .. loop.stop - 1`` run ``loop.times`` times over with
the same weights; ahead of every such pass t the residual becomes  W_in [x ; x0] + step[t]  (x0: the normed embedding).
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def f64(t):
    return t.to(F)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """rms(x) (1 + w): the layers' norm, the embedding's and the last one."""
    return rms(x, eps) * (1.0 + f64(w))


def plain_norm(x, w, eps):
    """rms(x) w: the norms of the latents."""
    return rms(x, eps) * f64(w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def soft_cap(s, cap):
    """cap tanh(s / cap)."""
    return cap * torch.tanh(s / cap)


def rotate_halves(x, positions, dims, base):
    """x [T, ..., n]: of the first ``dims`` elements, element i < dims/2 and element i + dims/2 turn by the angle
    p base^(-2i/dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    freq = torch.tensor(float(base), dtype=F) ** (-2.0 * i / dims)
    ang = torch.as_tensor(list(positions), dtype=F)[:, None] * freq[None, :]            # [T, half]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * torch.cos(ang) - v * torch.sin(ang), v * torch.cos(ang) + u * torch.sin(ang), x[..., dims:]], -1)


def causal(T, window=None):
    """[T, T] bool: j <= i and (window is None or i - j < window)."""
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    ok = d >= 0
    if window is not None:
        ok &= d < window
    return ok


def softmax_visible(s, mask):
    """Softmax over the visible keys of [.., T, T] scores."""
    return torch.softmax(s.masked_fill(~mask, float("-inf")), -1)


# ---- mixers -------------------------------------------------------------------------------------------------------------

def latent_cache_entries(h, w, p, m, eps, positions):
    """What a token leaves behind: the normed latent c [T, kv_rank] and the rotated shared key part r [T, rot_dim]."""
    R, P = m["kv_rank"], m["rot_dim"]
    down = h @ f64(w[p + ".dkv"]).T
    c = plain_norm(down[:, :R], w[p + ".dkv.norm"], eps)
    r = rotate_halves(down[:, R:R + P], positions, m["rot"]["dims"], m["rot"]["base"])
    return c, r


def latent_queries(h, w, p, m, eps, positions):
    """[T, H, dim] unrotated and [T, H, rot_dim] rotated query parts."""
    T, H, D, P = h.shape[0], m["heads"], m["dim"], m["rot_dim"]
    cq = plain_norm(h @ f64(w[p + ".dq"]).T, w[p + ".dq.norm"], eps)
    q = (cq @ f64(w[p + ".uq"]).T).view(T, H, D + P)
    return q[..., :D], rotate_halves(q[..., D:], positions, m["rot"]["dims"], m["rot"]["base"])


def latent_attention(h, w, p, m, eps, store=None):
    T, H, D, V = h.shape[0], m["heads"], m["dim"], m["vdim"]
    pos = range(T)
    c, r = latent_cache_entries(h, w, p, m, eps, pos)
    if store is not None:
        c, r = store(c), store(r)
    qn, qr = latent_queries(h, w, p, m, eps, pos)
    k = (c @ f64(w[p + ".uk"]).T).view(T, H, D)
    v = (c @ f64(w[p + ".uv"]).T).view(T, H, V)
    s = (torch.einsum("ihd,jhd->hij", qn, k) + torch.einsum("ihd,jd->hij", qr, r)) * m["scale"]
    a = softmax_visible(s, causal(T))
    o = torch.einsum("hij,jhv->ihv", a, v)
    gate = torch.sigmoid(h @ f64(w[p + ".g"]).T)                       # [T, H]: a number a head
    return (o * gate[:, :, None]).reshape(T, H * V) @ f64(w[p + ".o"]).T


def window_attention(h, w, p, m, store=None):
    T, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    lin = lambda n: h @ f64(w[f"{p}.{n}"]).T + f64(w[f"{p}.{n}.b"])
    q, k, v = lin("q").view(T, H, D), lin("k").view(T, G, D), lin("v").view(T, G, V)
    if store is not None:
        k, v = store(k), store(v)
    mask = causal(T, m["mask"]["size"] if m.get("mask") is not None else None)
    o = torch.empty(T, H, V, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        s = soft_cap(q[:, hd] @ k[:, g].T * m["scale"], m["softcap"])
        o[:, hd] = softmax_visible(s, mask) @ v[:, g]
    gate = torch.sigmoid(h @ f64(w[p + ".g"]).T)                       # [T, H V]: a number an element, no bias
    return (o.reshape(T, H * V) * gate) @ f64(w[p + ".o"]).T


# ---- feed-forwards ------------------------------------------------------------------------------------------------------

def dense_ff(h, w, p):
    lin = lambda x, n: x @ f64(w[f"{p}.{n}"]).T + f64(w[f"{p}.{n}.b"])
    return lin(gelu_tanh(lin(h, "gate")) * lin(h, "up"), "down")


def expert(h, w, p):
    lin = lambda x, n: x @ f64(w[f"{p}.{n}"]).T
    return lin(silu(lin(h, "gate")) * lin(h, "up"), "down")


def route(h, w, p, r):
    """[T, E] weights: sigmoid scores, the ``top`` largest kept as they are (lowest index wins a tie), zero elsewhere;
    also the margin between the last chosen score and the first left out."""
    s = torch.sigmoid(h @ f64(w[p + ".router"]).T)
    E, top = r["experts"], r["top"]
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices
    chosen = order[:, :top]
    out = torch.zeros_like(s)
    out.scatter_(1, chosen, s.gather(1, chosen))
    if top < E:
        margin = s.gather(1, order[:, top - 1:top]) - s.gather(1, order[:, top:top + 1])
    else:
        margin = torch.full((s.shape[0], 1), float("inf"), dtype=F)
    return out, chosen, margin[:, 0]


def moe_ff(h, w, p, mlp):
    """sum over the chosen experts of expert(weight h): the weight scales what the expert reads."""
    weights, chosen, _ = route(h, w, p, mlp["router"])
    y = torch.zeros(h.shape[0], w[p + ".e0.down"].shape[0], dtype=F)
    for e in range(mlp["router"]["experts"]):
        rows = torch.nonzero((chosen == e).any(-1))[:, 0]
        if rows.numel():
            y[rows] += expert(weights[rows, e:e + 1] * h[rows], w, f"{p}.e{e}")
    return y


def feed_forward(h, w, p, mlp):
    return dense_ff(h, w, p) if mlp["kind"] == "dense" else moe_ff(h, w, p, mlp)


# ---- the model ------------------------------------------------------------------------------------------------------------

def run_order(config):
    """[(layer, pass or None, first of its pass)] in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    return order + [(i, None, False) for i in range(b, n)]


def layer(x, w, i, spec, eps, round_inputs, store):
    p = f"l{i}"
    h = round_inputs(offset_norm(x, w[p + ".norm1"], eps))
    if spec["type"] == "latent_attention":
        y = latent_attention(h, w, p + ".mix", spec["mixer"], eps, store)
    else:
        y = window_attention(h, w, p + ".mix", spec["mixer"], store)
    if spec.get("mlp") is not None:
        y = y + feed_forward(h, w, p + ".mlp", spec["mlp"])
    return x + y


def forward(config, w, tokens, round_inputs=None, store=None, return_layers=False):
    """Logits [T, vocab] (float64) for one sequence.  ``round_inputs``: applied to what a product reads (None: nothing);
    ``store``: how kept keys, values and latents are rounded."""
    eps = config["norm"]["eps"]
    rin = round_inputs or (lambda t: t)
    emb = f64(w["embed"])
    x0 = offset_norm(emb[torch.as_tensor(list(tokens), dtype=torch.long)], w["embed.norm"], eps)
    x = x0
    per_layer = []
    for i, t, first in run_order(config):
        if first:
            x = rin(torch.cat([x, x0], -1)) @ f64(w["loop.in"]).T + f64(w["loop.step"])[t]
        x = layer(x, w, i, config["layers"][i], eps, rin, store)
        per_layer.append(x.clone())
    logits = rin(offset_norm(x, w["final.norm"], eps)) @ emb.T
    logits = soft_cap(logits, config["logit_softcap"])
    return (logits, torch.stack(per_layer)) if return_layers else logits
