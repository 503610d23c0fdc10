"""The Pivavik configuration on the CPU: read, written back, described as data; the repeated run of layers as schedule
steps with a cache of their own every time; constants reaching the parts; rejections that name the key; and the plain
implementation against elementary identities."""
import copy
import json
import math

import pytest
import torch

import citlali_b200 as cb
import plain_pivavik as plain
from citlali_b200.engine.model import cache_requirements_of
from pivavik_models import CONFIGS, config, make_weights


def test_round_trip_and_spec_as_data():
    for name, d in CONFIGS.items():
        cfg = config(name)
        assert cb.config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
        spec = cfg.to_model_spec()
        assert spec.architecture == "Pivavik" and spec.tie_head_to_embedding is True
        assert spec.embedding_norm.params["tensor"] == "embed.norm" and spec.logit_softcap == d["logit_softcap"]
        n = len(d["layers"])
        assert len(spec.layers) == n + (1 if "loop" in d else 0)
        for layer, described in zip(spec.layers, d["layers"]):
            assert layer.block == "parallel_residual" and set(layer.parts) == {"norm", "mixer"} | ({"feed_forward"} if described["mlp"] else set())
            assert layer.parts["mixer"].kind == ("latent_attention" if described["type"] == "latent_attention" else "window_attention")
            assert layer.parts["norm"].params["offset"] == 1.0
        names = [t.name for t in cb.expected_tensors(spec)]
        assert len(names) == len(set(names)) and {"embed", "embed.norm", "final.norm"} <= set(names)
        assert ("loop.in" in names) == ("loop.step" in names) == ("loop" in d)


def test_the_repeated_run_as_schedule_steps():
    order = lambda name: [s.layer for s in config(name).to_model_spec().schedule]
    assert order("P") == [0, 4, 1, 2, 4, 1, 2, 3]                 # layer 4 is the step ahead of every pass
    assert order("Q") == [0, 1, 2]
    assert order("R") == [4, 0, 1, 2, 3] * 2
    assert order("S") == [0, 3, 1, 2, 3, 1, 2, 3, 1, 2]
    spec = config("P").to_model_spec()
    assert all(s.cache_of is None for s in spec.schedule)
    caches = cache_requirements_of(spec)
    assert [c is None for c in caches] == [False, True, False, False, True, False, False, False]   # a cache every time a layer runs
    inj = spec.layers[4]
    assert inj.block == "input_injection" and inj.block_params == {"hidden_size": 64, "passes": 2, "matrix": "loop.in", "steps": "loop.step"}
    shapes = {t.name: tuple(t.shape) for t in cb.expected_tensors(spec)}
    assert shapes["loop.in"] == (64, 128) and shapes["loop.step"] == (2, 64)
    assert plain.run_order(CONFIGS["P"]) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (3, None, False)]


def test_constants_reach_the_parts():
    spec = config("P").to_model_spec()
    a = spec.layers[0].parts["mixer"].params
    assert (a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["scale"], a["softcap"], a["window"]) == (4, 2, 16, 24, 0.25, 3.0, 9)
    assert a["biases"] is True and a["gate"] == "elements" and a["rot_dims"] == 0 and a["conv"] is None and a["qk_norm_eps"] is None
    b = spec.layers[1].parts["mixer"].params
    assert (b["heads"], b["dim"], b["rot_dim"], b["vdim"], b["q_rank"], b["kv_rank"], b["scale"]) == (3, 16, 8, 24, 40, 48, 0.2)
    assert (b["rot_dims"], b["rot_base"], b["rot_layout"], b["gate"], b["window"], b["norm_eps"]) == (8, 10000.0, "halves", "heads", None, 1e-5)
    assert b["names"]["sink"] is None and b["names"]["dq_norm"] == "l1.mix.dq.norm" and b["names"]["gate"] == "l1.mix.g"
    ff = spec.layers[0].parts["feed_forward"]
    assert ff.kind == "routed_experts" and (ff.params["experts"], ff.params["top"], ff.params["intermediate_size"]) == (6, 2, 32)
    assert (ff.params["score"], ff.params["weight_on"], ff.params["activation"]) == ("sigmoid", "input", "silu")
    d = spec.layers[1].parts["feed_forward"]
    assert d.kind == "gated" and d.params["activation"] == "gelu_tanh" and d.params["biases"] is True
    assert d.params["names"] == {"gate": "l1.mlp.gate", "up": "l1.mlp.up", "down": "l1.mlp.down"}
    names = {t.name for t in cb.expected_tensors(spec) if not t.optional}
    assert {"l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b", "l0.mix.g", "l0.mix.o", "l0.mlp.router", "l0.mlp.e5.down", "l1.mlp.gate.b",
            "l1.mlp.down.b", "l1.mix.uk", "l1.mix.dkv.norm", "l3.mlp.e3.up"} <= names
    assert not ({"l0.mix.o.b", "l0.mix.g.b", "l2.mlp.gate", "l1.mix.sink", "l3.mlp.e4.up", "head"} & names)
    q = config("Q").to_model_spec().layers
    assert q[0].parts["mixer"].params["rot_dims"] == 12 and q[0].parts["mixer"].params["rot_dim"] == 20
    assert config("S").to_model_spec().layers[1].parts["mixer"].params["window"] is None


@pytest.mark.parametrize("edit,match", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d.pop("norm"), "eps"),
    (lambda d: d["layers"][0].update(type="conv"), "type 'conv'"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][0]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda d: d["layers"][1]["mlp"].pop("ff"), "ff"),
    (lambda d: d["loop"].update(stop=5), "loop"),
    (lambda d: d["loop"].update(start=3), "loop"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d.update(logit_softcap=0.0), "logit_softcap"),
])
def test_rejections_name_the_key(edit, match):
    d = copy.deepcopy(CONFIGS["P"])
    edit(d)
    with pytest.raises(cb.CitlaliError, match=match):
        cb.config_from_dict(d)


# ---- the plain implementation against elementary identities ---------------------------------------------------------------

def test_plain_norms_and_activations():
    x = torch.randn(5, 12, dtype=torch.float64)
    y = plain.offset_norm(x, torch.zeros(12), 0.0)
    assert torch.allclose((y * y).mean(-1), torch.ones(5, dtype=torch.float64))
    assert torch.allclose(plain.plain_norm(x, torch.full((12,), 2.0), 0.0), 2.0 * y)
    z = torch.linspace(-4, 4, 9, dtype=torch.float64)
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
    assert torch.allclose(plain.silu(z), torch.nn.functional.silu(z))
    assert abs(float(plain.soft_cap(torch.tensor(1e6, dtype=torch.float64), 7.0)) - 7.0) < 1e-9
    assert abs(float(plain.soft_cap(torch.tensor(1e-3, dtype=torch.float64), 7.0)) - 1e-3) < 1e-9


def test_plain_rotation_pairs_halves_keeps_norms_and_depends_on_distance_only():
    x = torch.randn(6, 3, 10, dtype=torch.float64)
    r = plain.rotate_halves(x, range(6), 8, 100.0)
    assert torch.allclose(r[..., 8:], x[..., 8:])
    assert torch.allclose(r[0], x[0])                                   # position 0 turns nothing
    assert torch.allclose((r[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))
    # element 1 pairs with element 5: at position 1 the angle is 100^(-2/8)
    a = 100.0 ** (-0.25)
    assert abs(float(r[1, 0, 1]) - (float(x[1, 0, 1]) * math.cos(a) - float(x[1, 0, 5]) * math.sin(a))) < 1e-12
    assert abs(float(r[1, 0, 5]) - (float(x[1, 0, 5]) * math.cos(a) + float(x[1, 0, 1]) * math.sin(a))) < 1e-12
    q, k = torch.randn(1, 8, dtype=torch.float64), torch.randn(1, 8, dtype=torch.float64)
    dot = lambda i, j: float(plain.rotate_halves(q, [i], 8, 50.0) @ plain.rotate_halves(k, [j], 8, 50.0).T)
    assert abs(dot(9, 4) - dot(105, 100)) < 1e-9


def test_plain_router_and_weighted_input():
    cfg, w = CONFIGS["P"], make_weights(config("P"), 3)
    h = torch.randn(7, 64, dtype=torch.float64)
    weights, chosen, margin = plain.route(h, w, "l0.mlp", cfg["layers"][0]["mlp"]["router"])
    assert chosen.shape == (7, 2) and bool(((weights != 0).sum(-1) == 2).all()) and bool((margin >= 0).all())
    s = torch.sigmoid(h @ w["l0.mlp.router"].double().T)
    assert torch.allclose(weights.max(-1).values, s.max(-1).values)       # the scores themselves, not renormalised
    # a weight on the input is no weight on the output: the gate's activation is not linear
    one = plain.expert(0.5 * h, w, "l0.mlp.e0")
    assert not torch.allclose(one, 0.5 * plain.expert(h, w, "l0.mlp.e0"), rtol=1e-3, atol=1e-6)


def test_plain_causality_and_windows():
    cfg, w = CONFIGS["P"], make_weights(config("P"), 4)
    toks = [5, 9, 100, 3, 77, 8, 1, 150, 60, 2, 31, 44, 12, 199, 0, 6]
    full = plain.forward(cfg, w, toks)
    assert torch.allclose(plain.forward(cfg, w, toks[:9]), full[:9], atol=1e-9)
    assert bool((full.abs() < cfg["logit_softcap"]).all())
    see = plain.causal(12, 4)
    assert bool(see[7, 4]) and not bool(see[7, 3]) and not bool(see[3, 4]) and bool(plain.causal(12)[11, 0])
