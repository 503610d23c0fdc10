"""Small Sobunex configurations and weights for tests.

The configurations differ from one another in every size and option: layer orders, head counts and group sizes (one
key/value head for all, one for every query head, groups of two and four), head sizes that are no multiple of 32, key and
value sizes that differ or are left to default, windows (one token, shorter than a page, a page and one, several pages,
none), a query temperature that changes every token, every few tokens, or is absent, layers that read an earlier layer's
keys through a window of their own, dense and routed feed-forwards with and without the expert every row uses, top = 1 and
top = experts, a router scale that is absent, layers without a feed-forward, widths and vocabularies that are no multiples
of 8.  Weights are drawn so that every mechanism matters to the logits and stored in bfloat16 so that both compute paths
and the plain implementation read the same numbers.
"""
import json
import os

import torch

import citlali_b200 as cb


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def att(heads, kv_heads, dim, vdim, scale, window, q_temp, mlp, kv_from=None):
    m = {"heads": heads, "dim": dim, "scale": scale}
    if kv_heads is not None:
        m["kv_heads"] = kv_heads
    if vdim is not None:
        m["vdim"] = vdim
    if window is not None:
        m["mask"] = {"size": window}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


CONFIGS = {
    # a window shorter than a page; a reader with a wider window than the layer whose keys it reads; a temperature that
    # steps every 7 tokens; values wider than keys; the first layer is routed
    "P": {"architecture": "Sobunex", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        att(4, 2, 16, 24, 0.25, 9, (0.5, 7), moe(6, 2, 32, 1.5, 2.0, (48, 0.8))),
        att(4, 2, 16, 24, 0.2, 20, (0.3, 3), dense(96), kv_from=0),
        att(2, 1, 40, 8, 0.15, 65, None, None),
        att(4, 2, 16, 24, 0.3, 4, (0.5, 7), moe(4, 1, 16, 3.0), kv_from=0)]},
    # odd width and vocabulary, no window at all, no temperature, a head size over 64, one key head a query head, value
    # size left to default, top = experts
    "Q": {"architecture": "Sobunex", "vocab": 333, "width": 60, "norm": {"eps": 1e-6}, "layers": [
        att(3, None, 20, 44, 0.2, None, None, dense(100)),
        att(3, 3, 80, None, 0.08, None, (1.0, 1), moe(3, 3, 24, 1.0, 0.7)),
        att(3, 3, 80, None, 0.1, 70, None, None, kv_from=1)]},
    # windows over several pages and of one token, one key/value head for eight query heads, sixteen experts with the
    # expert for every row, a reader without a window of an owner with one
    "R": {"architecture": "Sobunex", "vocab": 512, "width": 96, "norm": {"eps": 1e-6}, "layers": [
        att(8, 1, 32, 32, 0.125, 130, (0.25, 64), moe(16, 4, 16, 2.0, 2.5, (32, 1.0))),
        att(2, 2, 24, 40, 0.2, 1, None, dense(64)),
        att(8, 1, 32, 32, 0.1, None, (0.25, 64), dense(200), kv_from=0),
        att(6, 3, 16, 16, 0.3, 64, (2.0, 100), moe(8, 2, 40, 0.5, None, (8, 4.0)))]},
}


def config(name):
    return cb.config_from_dict(json.loads(json.dumps(CONFIGS[name])))


def make_weights(cfg, seed):
    """{name: bfloat16 tensor} for every tensor the model reads."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in cb.expected_tensors(cfg.to_model_spec()):
        if spec.optional:
            continue
        n, shape = spec.name, tuple(spec.shape)
        r = torch.randn(shape, generator=g)
        if n == "embed":
            t = r
        elif n.endswith(".b"):
            t = 0.3 * r                                    # biases of norms and projections
        elif n.endswith((".norm1", ".norm2", ".norm1b", ".norm2b")) or n == "final.norm":
            t = 1.0 + 0.3 * r
        elif n.endswith(".talk"):
            t = torch.eye(shape[0]) + 0.4 * r              # every head hears every other
        elif n.endswith(".pb"):
            t = -1.0 + r                                   # weights of ordinary keys well inside (0, 1)
        elif n.endswith(".act"):
            t = r
        elif n.endswith(".router"):
            t = 3.0 * r / shape[1] ** 0.5
        elif n.endswith((".mix.q", ".mix.k")):
            t = 2.0 * r / shape[1] ** 0.5                  # scores of a few units, so that the sigmoids spread
        elif n.endswith((".gate", ".up")) and ".mlp." in n:
            t = 2.0 * r / shape[1] ** 0.5                  # some of the experts' inputs reach their limits
        else:
            t = r / shape[-1] ** 0.5                       # matrices [out, in]
        out[n] = t.to(torch.bfloat16)
    return out


def write_model(path, name, seed):
    cfg = config(name)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    w = make_weights(cfg, seed)
    cb.write_safetensors(os.path.join(path, "model.safetensors"), lambda: iter(w.items()), metadata={"format": "pt"})
    return cfg, w
