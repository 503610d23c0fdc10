"""Small Pivavik configurations and weights for tests.

The configurations differ from one another in every size and option: layer orders (attention first, latent first, one kind
only), repeated runs of layers that start at the first layer, in the middle, reach the last layer, cover the whole model,
run once, or are absent; head counts and groupings (one key/value head for all, one a query head, groups of two and
four); head sizes that are no multiple of 32; key and value sizes that differ; latent ranks that are and are not sizes the
tensor-core walk takes; a rotated part smaller and larger than the unrotated one, and a rotation of only some of its
elements; windows of one token, shorter than a page, a page and one, several pages, none; soft caps that bite and that
hardly matter; dense and routed feed-forwards, top = 1, top > 1 and top = experts, layers without a feed-forward; widths and
vocabularies that are no multiples of 8.  Weights are drawn so that every mechanism matters to the logits and stored in
bfloat16 so that both compute paths and the plain implementation read the same numbers.
"""
import json
import os

import torch

import citlali_b200 as cb


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def att(heads, kv_heads, dim, vdim, scale, softcap, window, mlp):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, mlp, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def model(vocab, width, eps, cap, loop, layers):
    d = {"architecture": "Pivavik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_softcap": cap, "layers": layers}
    if loop is not None:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


CONFIGS = {
    # the repeated run sits in the middle and holds one layer of each kind; a window shorter than a page; values wider than
    # keys; a rotated part smaller than the unrotated one; top = 2 of 6; a soft cap that bites
    "P": model(200, 64, 1e-5, 12.0, (1, 3, 2), [
        att(4, 2, 16, 24, 0.25, 3.0, 9, moe(6, 2, 32)),
        lat(3, 16, 8, 24, 40, 48, 0.2, 10000.0, dense(96)),
        att(2, 1, 40, 8, 0.15, 50.0, 65, None),
        lat(2, 8, 24, 12, 24, 32, 0.18, 500.0, moe(4, 1, 16))]),
    # odd width and vocabulary, no repeated run at all, latent layers only at first, one key head a query head, a window
    # wider than any sequence of the tests' short requests, top = experts, only some of the rotated part's elements turn
    "Q": model(333, 60, 1e-6, 40.0, None, [
        lat(5, 12, 20, 12, 36, 44, 0.25, 100.0, moe(3, 3, 24), rot_dims=12),
        lat(2, 20, 4, 36, 16, 20, 0.2, 1000000.0, None),
        att(3, 3, 20, 44, 0.2, 8.0, 300, dense(100))]),
    # the repeated run is the whole model and runs twice; sizes the tensor-core kernels take (a latent of 64 + 16, heads
    # of 64 and of 32 with equal key and value sizes); windows of several pages and of one token; sixteen experts
    "R": model(512, 96, 1e-6, 25.0, (0, 4, 2), [
        att(8, 2, 64, 64, 0.125, 10.0, 130, moe(16, 4, 16)),
        lat(5, 32, 16, 32, 48, 64, 0.15, 200000.0, dense(200)),
        att(2, 2, 32, 32, 0.2, 4.0, 1, dense(64)),
        lat(16, 16, 16, 16, 64, 64, 0.2, 10000.0, dense(80))]),
    # the repeated run reaches the last layer and runs three times; attention layers only inside it; no window on one of them
    "S": model(130, 40, 1e-5, 30.0, (1, 3, 3), [
        lat(2, 16, 16, 16, 24, 24, 0.2, 10000.0, dense(48)),
        att(4, 1, 8, 16, 0.3, 6.0, None, moe(5, 5, 8)),
        att(6, 3, 12, 12, 0.3, 2.0, 64, dense(24))]),
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
        elif n == "loop.step":
            t = 0.5 * r
        elif n.endswith(".b"):
            t = 0.3 * r                                    # biases of projections
        elif n.endswith((".dq.norm", ".dkv.norm")):
            t = 1.0 + 0.3 * r                              # plain weights
        elif n.endswith(".norm1") or n in ("final.norm", "embed.norm"):
            t = 0.3 * r                                    # stored around zero: the factor is 1 + w
        elif n.endswith(".router"):
            t = 3.0 * r / shape[1] ** 0.5
        elif n.endswith((".mix.q", ".mix.k", ".mix.uq", ".mix.uk", ".mix.dkv")):
            t = 2.0 * r / shape[1] ** 0.5                  # scores of several units: the softmax is no average, the cap bites
        elif n.endswith(".mix.g"):
            t = 2.0 * r / shape[1] ** 0.5                  # gates that spread over (0, 1)
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
