"""Pivavik configurations drawn at random (fixed seed): layer counts and orders, a repeated run of layers anywhere (or none)
that runs one to three times, head counts and groupings, head sizes that are odd multiples of 4 and sizes the tensor cores
like, key and value sizes equal or not, latent ranks and rotated parts of many sizes, windows from 1 to 300 or none, caps
from 2 to 50, dense and routed feed-forwards, top from 1 to all experts, layers without a feed-forward; both dtypes.  Each is
run whole, with its tail decoded and in a batch of two with unequal lengths, against the plain implementation."""
import json
import os
import random

import pytest

import citlali_b200 as cb
import plain_pivavik as plain
import replay
from helpers import random_tokens
from pivavik_models import att, dense, lat, make_weights, model, moe

pytestmark = pytest.mark.gpu


def draw(i):
    rng = random.Random(8100 + i)
    width = rng.choice([40, 64, 72, 128])

    def mlp():
        kind = rng.random()
        if kind < 0.15:
            return None
        if kind < 0.5:
            return dense(rng.choice([24, 100, 128, 200]))
        experts = rng.choice([2, 3, 4, 8, 12, 16])
        return moe(experts, rng.randint(1, min(experts, 4)) if rng.random() < 0.8 else experts, rng.choice([16, 24, 40, 64]))

    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.5:
            kv = rng.randint(1, 3)
            dim = rng.choice([8, 12, 16, 32, 48, 64, 80, 128])
            vdim = dim if rng.random() < 0.5 else rng.choice([8, 20, 24, 64])
            layers.append(att(kv * rng.choice([1, 1, 2, 3, 4]), kv, dim, vdim, rng.choice([0.1, 0.2, dim ** -0.5]),
                              rng.choice([2.0, 5.0, 20.0, 50.0]), rng.choice([None, 1, 7, 64, 65, 100, 300]), mlp()))
        else:
            rot_dim = rng.choice([4, 8, 16, 32, 64])
            kv_rank = rng.choice([16, 24, 48, 64, 128])
            layers.append(lat(rng.choice([1, 2, 3, 6, 16, 17]), rng.choice([8, 12, 16, 32, 64]), rot_dim, rng.choice([8, 12, 32, 64]),
                              rng.choice([16, 24, 64]), kv_rank, rng.choice([0.1, 0.2]), rng.choice([100.0, 10000.0, 200000.0]), mlp(),
                              rot_dims=rot_dim if rng.random() < 0.8 else rot_dim // 2))
    loop = None
    if rng.random() < 0.8:
        start = rng.randrange(len(layers))
        loop = (start, rng.randint(start + 1, len(layers)), rng.randint(1, 3))
    return model(rng.choice([130, 256, 500]), width, rng.choice([1e-5, 1e-6]), rng.choice([10.0, 30.0, 50.0]), loop, layers)


@pytest.mark.parametrize("i", range(12))
def test_random_configuration(i, tmp_path):
    d = draw(i)
    cfg = cb.config_from_dict(json.loads(json.dumps(d)))
    w = make_weights(cfg, 900 + i)
    path = str(tmp_path / "m")
    os.makedirs(path)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    cb.write_safetensors(os.path.join(path, "model.safetensors"), lambda: iter(w.items()), metadata={"format": "pt"})
    reqs = [("a", random_tokens(d["vocab"], 150, 3 * i + 1)), ("b", random_tokens(d["vocab"], 47, 3 * i + 2))]
    want = {rid: plain.forward(cfg.to_dict(), w, toks) for rid, toks in reqs}
    # 32-bit: every position within rounding of the exact evaluation.  bfloat16: a router's close call may fall the other
    # way, and every position behind it in the sequence then differs: most positions must agree and the median error must be
    # small; each bfloat16 kernel is held strictly where it is tested alone
    for dtype, tol, most in (("float32", 2e-5, 1.0), ("bfloat16", 5e-2, 0.6)):
        s = cb.InferenceSession().load_model(path, max_context=256, dtype=dtype, max_batch=2)
        for what, steps in (("whole", replay.whole(reqs)), ("tail", replay.tail(reqs, last=40)),
                            ("batched", replay.batched(reqs, [100, 20], 2))):
            got = replay.run_in_process(s, steps)
            good, errs = 0, []
            for (rid, pos), row in got.items():
                ref = want[rid][pos]
                diff = row.double() - ref
                # root mean square over the vocabulary, means taken off, relative to the logits' own spread
                err = float((diff - diff.mean()).pow(2).mean().sqrt() / (ref - ref.mean()).pow(2).mean().sqrt())
                errs.append(err)
                if err <= tol:
                    good += 1
                else:
                    assert dtype != "float32", f"configuration {i} {what}: {rid} position {pos}: {err:.3e}"
            assert good >= most * len(got), f"configuration {i} {dtype} {what}: only {good} of {len(got)} positions agree"
            assert sorted(errs)[len(errs) // 2] <= 0.6 * tol, f"configuration {i} {dtype} {what}: median error {sorted(errs)[len(errs) // 2]:.3e}"
