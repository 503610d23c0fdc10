"""The Sobunex configuration on the CPU: read, written back, described as data; constants reaching the parts; layers that
read another layer's keys as schedule steps, and the reach the owner's cache must keep; rejections that name the key; and
the plain implementation against elementary identities."""
import json
import math

import pytest
import torch

import citlali_b200 as cb
import plain_sobunex as plain
from sobunex_models import CONFIGS, config, make_weights


def test_round_trip_and_spec_as_data():
    for name, d in CONFIGS.items():
        cfg = config(name)
        assert cb.config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
        spec = cfg.to_model_spec()
        assert spec.architecture == "Sobunex" and spec.tie_head_to_embedding is False and spec.head_name == "head"
        assert len(spec.layers) == len(d["layers"]) == len(spec.schedule)
        for i, (layer, described, step) in enumerate(zip(spec.layers, d["layers"], spec.schedule)):
            assert layer.block == "sandwich_norm" and layer.parts["mixer"].kind == "sigmoid_attention"
            assert ("feed_forward" in layer.parts) == (described["mlp"] is not None)
            assert ("feed_forward_norm" in layer.parts) == ("feed_forward_out_norm" in layer.parts) == (described["mlp"] is not None)
            src = described["mixer"].get("kv_from")
            assert step.layer == i and step.cache_of == src
            assert layer.parts["mixer"].params["own_kv"] == (src is None)
        names = [t.name for t in cb.expected_tensors(spec)]
        assert len(names) == len(set(names)) and {"embed", "final.norm", "final.norm.b", "head"} <= set(names)


def test_a_reader_has_no_key_and_value_tensors():
    names = {t.name for t in cb.expected_tensors(config("P").to_model_spec())}
    assert {"l0.mix.k", "l0.mix.k.b", "l0.mix.v", "l0.mix.v.b", "l2.mix.k"} <= names
    for reader in (1, 3):
        assert not any(n.startswith(f"l{reader}.mix.k") or n.startswith(f"l{reader}.mix.v") for n in names)
        assert {f"l{reader}.mix.q", f"l{reader}.mix.q.b", f"l{reader}.mix.talk", f"l{reader}.mix.pb", f"l{reader}.mix.g",
                f"l{reader}.mix.o", f"l{reader}.mix.o.b"} <= names
    assert "l2.mlp.up" not in names and "l2.norm2" not in names and "l2.norm1b.b" in names
    assert {"l0.mlp.router", "l0.mlp.e5.gate", "l0.mlp.shared.down", "l1.mlp.act", "l1.mlp.up.b"} <= names
    assert "l3.mlp.shared.gate" not in names and "l3.mlp.e3.down" in names and "l3.mlp.e4.down" not in names


def test_constants_reach_the_parts():
    spec = config("P").to_model_spec()
    a = spec.layers[0].parts["mixer"].params
    assert (a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["scale"], a["window"]) == (4, 2, 16, 24, 0.25, 9)
    assert a["q_temp"] == {"coef": 0.5, "every": 7} and a["slope_exp"] == 8.0
    assert a["cache_window"] == 20                       # the widest window among the layer and its two readers
    b = spec.layers[1].parts["mixer"].params
    assert (b["window"], b["cache_window"], b["own_kv"], b["q_temp"]["every"]) == (20, None, False, 3)
    assert spec.layers[2].parts["mixer"].params["q_temp"] is None
    ff = spec.layers[0].parts["feed_forward"].params
    assert (ff["experts"], ff["top"], ff["intermediate_size"], ff["weight_scale"], ff["limit"], ff["alpha"]) == (6, 2, 32, 2.0, 1.5, 1.702)
    assert ff["shared"] == {"intermediate_size": 48, "limit": 0.8} and ff["activation"] == "clamped_swish"
    last = spec.layers[3].parts["feed_forward"].params
    assert last["shared"] is None and last["weight_scale"] == 1.0
    assert spec.layers[1].parts["feed_forward"].kind == "xielu"
    assert spec.layers[0].parts["mixer_norm"].params == {"size": 64, "eps": 1e-5, "tensor": "l0.norm1", "bias": "l0.norm1.b"}
    # absent sizes default: key/value heads to the query heads, the value size to the key size
    q = config("Q").to_model_spec().layers
    assert (q[0].parts["mixer"].params["kv_heads"], q[1].parts["mixer"].params["vdim"]) == (3, 80)
    # an owner with a window whose reader has none keeps every key
    r = config("R").to_model_spec().layers
    assert r[0].parts["mixer"].params["window"] == 130 and r[0].parts["mixer"].params["cache_window"] is None
    assert r[1].parts["mixer"].params["cache_window"] == 1


@pytest.mark.parametrize("edit,match", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d.pop("norm"), "eps"),
    (lambda d: d["layers"][0].update(type="conv"), "type 'conv'"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"].pop("dim"), "dim"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda d: d["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda d: d["layers"][1]["mixer"].update(vdim=16), "layer 0"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda d: d["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda d: d["layers"][0]["mlp"].update(kind="gated"), "kind"),
    (lambda d: d["layers"][1]["mlp"].pop("ff"), "ff"),
])
def test_rejections_name_the_key(edit, match):
    d = json.loads(json.dumps(CONFIGS["P"]))
    edit(d)
    with pytest.raises(cb.CitlaliError, match=match):
        cb.config_from_dict(d)


def test_plain_identities():
    torch.manual_seed(0)
    x = torch.randn(5, 12, dtype=torch.float64)
    y = plain.layer_norm(x, torch.ones(12), torch.zeros(12), 0.0)
    assert float(y.mean(-1).abs().max()) < 1e-12 and float(((y * y).mean(-1) - 1).abs().max()) < 1e-12
    assert torch.allclose(plain.layer_norm(x, torch.zeros(12), torch.full((12,), 3.0), 1e-5), torch.full((5, 12), 3.0, dtype=torch.float64))
    # the temperature is 1 until position every - 1 and steps there
    t = plain.query_temperature(range(10), 0.5, 4)
    assert t[:3].tolist() == [1.0, 1.0, 1.0] and abs(float(t[3]) - (1 + 0.5 * math.log(2))) < 1e-15
    assert abs(float(t[7]) - (1 + 0.5 * math.log(3))) < 1e-15 and t[6] == t[3]
    # slopes halve geometrically down to 2^-8
    s = plain.head_slopes(4)
    assert torch.allclose(s, torch.tensor([0.25, 0.0625, 0.015625, 0.00390625], dtype=torch.float64))
    # a window that covers everything is no window; a window of one sees the token itself
    assert torch.equal(plain.visible(9, 100), plain.visible(9, None))
    assert torch.equal(plain.visible(5, 1), torch.eye(5, dtype=torch.bool))
    assert plain.visible(9, 3)[8].tolist() == [False] * 6 + [True] * 3
    # mixing by the identity changes nothing; a zero score weighs one half; hidden keys weigh nothing
    sc = torch.randn(3, 6, 6, dtype=torch.float64)
    assert torch.equal(plain.mix_heads(sc, torch.eye(3)), sc)
    a = plain.sigmoid_weights(torch.zeros(2, 4, 4, dtype=torch.float64), torch.zeros(2), plain.visible(4, 2))
    assert a[0].tolist() == [[.5, 0, 0, 0], [.5, .5, 0, 0], [0, .5, .5, 0], [0, 0, .5, .5]]
    # xielu is continuous at zero with slope one half on both sides, and quadratic for large inputs
    z = torch.tensor([-1e-6, 0.0, 1e-6, 3.0], dtype=torch.float64)
    v = plain.xielu(z, 0.3, -0.2)
    assert float(v[1]) == 0.0 and abs(float(v[2] - v[0]) / 2e-6 - 0.5) < 1e-5
    assert abs(float(v[3]) - (math.log1p(math.exp(0.3)) * 9 + 1.5)) < 1e-12
    # the expert's gate stops at the limit from above only, its other input on both sides
    w = {"p.gate": torch.eye(2), "p.up": torch.eye(2), "p.down": torch.eye(2)}
    h = torch.tensor([[5.0, 5.0], [-5.0, -5.0]], dtype=torch.float64)
    e = plain.clamped_expert(h, w, "p", 2.0)
    assert torch.allclose(e[0], torch.full((2,), 2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0, dtype=torch.float64))
    assert torch.allclose(e[1], torch.full((2,), -5.0 / (1 + math.exp(1.702 * 5.0)) * -1.0, dtype=torch.float64))
    # routing: weights are the softmax scores themselves times the scale, not renormalised; a tie goes to the lower index
    wr = {"p.router": torch.tensor([[1.0], [1.0], [0.0], [2.0]])}
    out, chosen, _ = plain.route(torch.ones(1, 1, dtype=torch.float64), wr, "p", {"experts": 4, "top": 2, "scale": 3.0})
    sm = torch.softmax(torch.tensor([1.0, 1.0, 0.0, 2.0], dtype=torch.float64), -1)
    assert chosen.tolist() == [[3, 0]] and torch.allclose(out[0], torch.stack([3 * sm[0], sm[1] * 0, sm[2] * 0, 3 * sm[3]]))


def test_plain_model_runs_on_every_configuration():
    for name in CONFIGS:
        cfg = config(name)
        w = make_weights(cfg, 1)
        toks = list(range(1, 40))
        logits, layers = plain.forward(cfg.to_dict(), w, toks, return_layers=True)
        assert logits.shape == (39, CONFIGS[name]["vocab"]) and bool(torch.isfinite(logits).all())
        assert layers.shape == (len(CONFIGS[name]["layers"]), 39, CONFIGS[name]["width"])
        # causality: a later token changes no earlier logits
        again = plain.forward(cfg.to_dict(), w, toks[:20] + [0] + toks[21:])
        assert float((again[:20] - logits[:20]).abs().max()) < 1e-12 and float((again[20:] - logits[20:]).abs().max()) > 1e-3
