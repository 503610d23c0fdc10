"""Each mechanism of the Sobunex design alone, built through the registries at sizes no model uses, against the plain
implementation: the layer norm with a bias and the kernel that chains two of them around the residual sum; attention with
sigmoid weights (the distance bias, the heads' mix, the number a head, the temperature, the gates, each also switched off),
whole, token by token and in portions through one cache, with one key made to stand out just inside and just outside the
window, over page borders, in prompts and in decoding, and far back among hundreds; a mixer that reads another's cache
through a window of its own; the xIELU feed-forward; the routed experts with clamped inputs, scaled weights and the expert
every row uses; and the block with its four norms."""
import math

import pytest
import torch

import citlali_b200 as cb
import plain_sobunex as plain
from citlali_b200 import ops
from citlali_b200.config.spec import LayerSpec, PartSpec
from citlali_b200.engine.step import StepEntry, pack_step
from citlali_b200.parts.base import BuildContext, build_part, part_class
from citlali_b200.weights.loader import WeightHandle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def ctx_for(dtype):
    return BuildContext(torch.device(DEV), dtype, torch.zeros(4, dtype=torch.int32, device=DEV))


def handles(weights):
    return {n: WeightHandle(n, t.dtype, tuple(t.shape), tensor=t) for n, t in weights.items()}


def draw(specs, seed):
    """Random bfloat16 weights for a part's tensors, sized so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for s in specs:
        r = torch.randn(tuple(s.shape), generator=g)
        n = s.name
        if s.role == "gain":
            t = 1.0 + 0.3 * r
        elif n.endswith("talk"):
            t = torch.eye(s.shape[0]) + 0.4 * r
        elif n.endswith("pb"):
            t = -1.0 + r
        elif n.endswith(("act", "router")):
            t = r
        elif len(s.shape) == 1:
            t = 0.4 * r
        elif n.endswith((".q", ".k")):
            t = 2.0 * r / s.shape[-1] ** 0.5
        else:
            t = r / s.shape[-1] ** 0.5
        out[n] = t.to(torch.bfloat16)
    return out


def inputs(T, hidden, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, hidden, generator=g).to(torch.bfloat16).double()       # what both paths read exactly


def close(got, want, dtype, what):
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert err <= TOL[dtype] * scale, f"{what}: |diff| {err:.3e} of {scale:.3e}"


class Harness:
    """An attention mixer with a cache of its own, and optionally a second mixer that reads that cache: feeds sequences in
    the given portions and returns each mixer's output rows."""

    def __init__(self, params, dtype, weights=None, seed=1, reader=None, slots=3, capacity=1024, max_seq=1024):
        self.parts = [build_part("mixer", PartSpec("sigmoid_attention", params, "m"))]
        if reader is not None:
            self.parts.append(build_part("mixer", PartSpec("sigmoid_attention", reader, "r")))
        self.weights = weights if weights is not None else draw([s for p in self.parts for s in p.tensor_specs()], seed)
        self.ctx = ctx_for(dtype)
        for p in self.parts:
            p.bind(handles(self.weights), self.ctx)
        assert reader is None or self.parts[1].cache_requirement() is None
        self.cache = cb.SequenceCache([self.parts[0].cache_requirement()], slots, capacity, max_seq, dtype, DEV)
        self.hidden = params["hidden_size"]
        self.dtype = dtype

    def run(self, sequences, portions):
        """``sequences``: {name: h [T, hidden] float64}; ``portions``: a list of steps, each {name: n new tokens}.  Returns
        one {name: rows} per mixer."""
        slots, done = {}, {}
        out = [{n: [] for n in sequences} for _ in self.parts]
        for step in portions:
            names = [n for n in step if step[n] > 0]
            for n in names:
                if n not in slots:
                    slots[n] = self.cache.acquire()
                    done[n] = 0
            entries = [StepEntry(slots[n], [0] * step[n], []) for n in names]
            batch = pack_step(entries, [done[n] for n in names], 1, DEV)
            for n in names:
                self.cache.reserve(slots[n], done[n] + step[n])
            h = torch.cat([sequences[n][done[n]:done[n] + step[n]] for n in names]).to(DEV).to(self.dtype).contiguous()
            for k, part in enumerate(self.parts):
                y = torch.empty((h.shape[0], self.hidden), dtype=torch.float32, device=DEV)
                part.forward(h, batch, self.cache.view(0), y, k == 0, overwrite=True)
                at = 0
                for n in names:
                    out[k][n].append(y[at:at + step[n]].double().cpu())
                    at += step[n]
            for n in names:
                done[n] += step[n]
                self.cache.commit(slots[n], done[n])
        for n in list(slots):
            self.cache.release(slots.pop(n))
        assert self.cache.pages_held() == 0
        assert not any(self.ctx.error_flag.tolist())
        return [{n: torch.cat(v) for n, v in o.items()} for o in out]


def cuts(T):
    """Ways of feeding T tokens of sequence 'a': whole, one by one, portions of two (and a last odd one), mixed."""
    two = [{"a": 2}] * (T // 2) + ([{"a": 1}] if T % 2 else [])
    mixed, left = [], T
    for n in (3, 1, 7, 2, 64, 5, 1, 1, 40):
        if left <= 0:
            break
        mixed.append({"a": min(n, left)})
        left -= min(n, left)
    if left:
        mixed.append({"a": left})
    return {"whole": [{"a": T}], "one by one": [{"a": 1}] * T, "twos": two, "mixed": mixed}


def mixer_config(params):
    m = {k: params[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale")}
    if params.get("window") is not None:
        m["mask"] = {"size": params["window"]}
    if params.get("q_temp") is not None:
        m["q_temp"] = params["q_temp"]
    return m


def plain_mixer(params, prefix, kv=None):
    """The plain mixer with the options a part may switch off restated as the weights that do nothing."""
    def fn(h, w):
        H = params["heads"]
        w = dict(w)
        if not params.get("talk", True):
            w[prefix + ".talk"] = torch.eye(H)
        if not params.get("head_bias", True):
            w[prefix + ".pb"] = torch.zeros(H)
        if not params.get("gate", True):
            w[prefix + ".g"] = torch.zeros(H, params["hidden_size"])
        if not params.get("biases", True):
            for n, size in (("q", H * params["dim"]), ("k", params["kv_heads"] * params["dim"]),
                            ("v", params["kv_heads"] * params["vdim"]), ("o", params["hidden_size"])):
                w[f"{prefix}.{n}.b"] = torch.zeros(size)
        y, kept = plain.attention_mixer(h, w, prefix, mixer_config(params), kv=kv(h, w) if kv is not None else None)
        if not params.get("gate", True):
            y = 2.0 * (y - w[prefix + ".o.b"].double()) + w[prefix + ".o.b"].double()      # a gate of sigmoid(0) undone
        if params.get("slope_exp", 8.0) == 0.0:
            raise AssertionError("the plain mixer always has the distance bias")
        return y
    return fn


ATT = [
    # a window shorter than a page, values wider than keys, a temperature that steps every 7 tokens
    dict(hidden_size=40, heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, window=9, q_temp={"coef": 0.5, "every": 7}),
    # a window of a page and one, a head size over 64 and no multiple of 32, one key head a query head, no temperature
    dict(hidden_size=48, heads=3, kv_heads=3, dim=80, vdim=12, scale=0.08, window=65, q_temp=None),
    # no window, one key/value head for all, a temperature that steps at every token
    dict(hidden_size=32, heads=8, kv_heads=1, dim=32, vdim=32, scale=0.15, window=None, q_temp={"coef": 1.0, "every": 1}),
    # a window of one token: a row sees itself alone
    dict(hidden_size=24, heads=2, kv_heads=2, dim=24, vdim=40, scale=0.2, window=1, q_temp={"coef": 0.3, "every": 100}),
    # several pages of window, sizes the tensor cores like, many heads
    dict(hidden_size=64, heads=16, kv_heads=4, dim=64, vdim=64, scale=0.125, window=130, q_temp={"coef": 0.3, "every": 64}),
    # one head; the options off: no mix, no number a head, no gate, no biases
    dict(hidden_size=32, heads=1, kv_heads=1, dim=16, vdim=8, scale=0.3, window=20, q_temp=None, talk=False, head_bias=False,
         gate=False, biases=False),
    dict(hidden_size=32, heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, window=70, q_temp=None, talk=False, gate=False),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("params", ATT)
def test_sigmoid_attention_mixer(params, dtype):
    T, seed = 150, 3
    params = dict(params, slope_exp=8.0)
    h = inputs(T, params["hidden_size"], seed)
    hs = Harness(params, dtype, seed=seed)
    fn = plain_mixer(params, "m")
    want = fn(h, hs.weights)
    results = {}
    for what, portions in cuts(T).items():
        results[what] = hs.run({"a": h}, portions)[0]["a"]
        close(results[what], want, dtype, f"{dtype} {what}")
    if dtype == torch.float32:
        for what in results:
            assert torch.equal(results[what], results["whole"]), f"'{what}' gives other bits than 'whole'"
    # two unequal sequences in one batch, a third that takes a slot which was given back
    other = inputs(37, params["hidden_size"], seed + 1)
    both = hs.run({"a": h, "b": other}, [{"a": 50, "b": 20}, {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": T - 52, "b": 15}])[0]
    close(both["a"], want, dtype, f"{dtype} batched a")
    close(both["b"], fn(other, hs.weights), dtype, f"{dtype} batched b")
    if dtype == torch.float32:
        assert torch.equal(both["a"], results["whole"])
    again = hs.run({"c": other}, [{"c": 37}])[0]["c"]                   # the slot's pages were used before
    close(again, fn(other, hs.weights), dtype, f"{dtype} reused slot")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("own_window,reader_window", [(9, 30), (70, 5), (20, None), (None, 64)])
def test_a_mixer_that_reads_anothers_keys(own_window, reader_window, dtype):
    """The second mixer has queries, mix, gates, window and temperature of its own and no keys or values: it reads what the
    first left in the cache, which must reach as far back as the wider of the two windows."""
    T = 200
    own = dict(hidden_size=40, heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, window=own_window,
               q_temp={"coef": 0.5, "every": 7}, slope_exp=8.0)
    reach = [own_window, reader_window]
    own["cache_window"] = None if None in reach else max(reach)
    reader = dict(own, window=reader_window, q_temp={"coef": 0.2, "every": 3}, scale=0.2, own_kv=False, cache_window=None)
    hs = Harness(own, dtype, reader=reader, seed=5, capacity=256 if None not in reach else 1024)
    names = {t.name for t in hs.parts[1].tensor_specs()}
    assert "r.q" in names and not ({"r.k", "r.v", "r.k.b", "r.v.b"} & names)
    h = inputs(T, 40, 6)
    kept = lambda hh, w: plain.attention_keys_values(hh, w, "m", mixer_config(own))
    want = [plain_mixer(own, "m")(h, hs.weights), plain_mixer(reader, "r", kv=kept)(h, hs.weights)]
    base = None
    for what, portions in cuts(T).items():
        got = hs.run({"a": h}, portions)
        for k in (0, 1):
            close(got[k]["a"], want[k], dtype, f"{dtype} {what} mixer {k}")
        if dtype == torch.float32:
            base = base or got
            assert torch.equal(got[1]["a"], base[1]["a"])


def standing_out(d, window, talk=None):
    params = dict(hidden_size=d, heads=1, kv_heads=1, dim=d, vdim=d, scale=1.0, window=window, q_temp=None, slope_exp=8.0,
                  gate=False, biases=False)
    eye = torch.eye(d).to(torch.bfloat16)
    # ordinary keys weigh sigmoid(1 - 30) or less; the long key sigmoid(20 - 30 + 20 - distance / 256): about one
    weights = {"m.q": eye, "m.k": eye, "m.v": eye, "m.o": eye, "m.talk": torch.ones(1, 1).to(torch.bfloat16),
               "m.pb": torch.tensor([-10.0]).to(torch.bfloat16)}
    return params, weights


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode_from", [None, 40])
@pytest.mark.parametrize("window", [9, 64, 65, 130, 1, None])
def test_window_edges_with_one_key_that_stands_out(window, decode_from, dtype):
    """Queries, keys and values are the inputs themselves.  Ordinary keys weigh next to nothing; one key is made long and
    weighs about one for every later query that sees it, so a row's output is that key's value exactly while the key is
    inside the window: the row at distance window - 1 has it, the next one has lost it; over page borders; in prompts and in
    decoding."""
    d, T = 16, 210
    params, weights = standing_out(d, window)
    for special in (0, 1, 62, 63, 64, 100):
        g = torch.Generator().manual_seed(special)
        h = 0.05 * torch.randn(T, d, generator=g)
        h[:, 0] = 1.0                                       # every query has a part along the first axis ...
        h[special, 0] = 30.0                                # ... and one key is long along it
        h[special, 1] = 7.0                                 # and carries a value no other has
        h = h.to(torch.bfloat16).double()
        hs = Harness(params, dtype, weights=weights)
        portions = [{"a": T}] if decode_from is None else [{"a": decode_from}] + [{"a": 1}] * (T - decode_from)
        got = hs.run({"a": h}, portions)[0]["a"]
        want = plain_mixer(params, "m")(h, weights)
        allowed = (1e-4 if dtype == torch.float32 else 0.03) * want.abs().amax(-1, keepdim=True).clamp(min=1.0)
        assert bool(((got - want).abs() <= allowed).all()), (window, special)
        see = plain.visible(T, window)
        for i in range(special + 1, T):                     # the test's point: the special key decides the row
            assert (float(got[i][1]) > 3.0) == bool(see[i, special]), (window, special, i)
            assert (float(want[i][1]) > 3.0) == bool(see[i, special])


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds(dtype):
    """One long key at position 3 among 900 ordinary ones, over fifteen pages, two query heads on one key head: every later
    row must find it whether it comes in the prompt, in a later portion or token by token.  The distance bias of the second
    head (2^-8 a token) has taken 3.5 off the score by the end, which the key's length allows for."""
    d, T = 32, 900
    params = dict(hidden_size=d, heads=2, kv_heads=1, dim=d // 2, vdim=d // 2, scale=1.0, window=None, q_temp=None,
                  slope_exp=8.0, gate=False, biases=False, talk=False)
    eye = torch.eye(d).to(torch.bfloat16)
    weights = {"m.q": eye, "m.k": eye[:d // 2], "m.v": eye[d // 2:], "m.o": eye, "m.pb": torch.tensor([-12.0, -12.0]).to(torch.bfloat16)}
    g = torch.Generator().manual_seed(11)
    h = 0.05 * torch.randn(T, d, generator=g)
    h[:, 0] = 1.0
    h[:, d // 2] = 1.0                                       # both query heads look along the first key axis
    h[3, 0] = 90.0                                           # head 0 loses 1/16 a token: 56 by the end
    h[3, d // 2:] = 7.0                                      # the far token's value
    h = h.to(torch.bfloat16).double()
    want = plain_mixer(params, "m")(h, weights)
    assert float((want[10:, d // 2:] - 7.0).abs().max()) < 0.2       # head 1 returns the far value everywhere
    hs = Harness(params, dtype, weights=weights, capacity=1024)
    for portions in ([{"a": T}], [{"a": 500}, {"a": 300}] + [{"a": 1}] * 100, [{"a": 2}] * 450):
        got = hs.run({"a": h}, portions)[0]["a"]
        assert float((got - want).abs().max()) < (1e-3 if dtype == torch.float32 else 0.1), len(portions)
        assert float((got[10:, d // 2:] - 7.0).abs().max()) < 0.3


@pytest.mark.parametrize("dtype", DTYPES)
def test_each_position_term_alone(dtype):
    """With everything else neutral, a row's output shows one term at a time: the distance bias (weights fall with the
    distance at the head's own rate), the heads' mix (a head with a zero row in the mix weighs every key one half), and the
    temperature (no effect before position every - 1)."""
    d, H, T = 8, 2, 40
    params = dict(hidden_size=H * d, heads=H, kv_heads=H, dim=d, vdim=d, scale=1.0, window=None, q_temp=None, slope_exp=8.0,
                  gate=False, biases=False)
    z = torch.zeros(H * d, H * d)
    eye = torch.eye(H * d)
    talk = torch.tensor([[1.0, 0.0], [0.0, 0.0]])
    w = {"m.q": z, "m.k": z, "m.v": eye, "m.o": eye, "m.talk": talk, "m.pb": torch.zeros(H)}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    h = torch.ones(T, H * d, dtype=torch.float64)
    got = Harness(params, dtype, weights=w).run({"a": h}, [{"a": 30}] + [{"a": 1}] * 10)[0]["a"]
    slope = 2.0 ** (-8.0 / H)
    for i in (0, 5, 29, 30, 39):
        head0 = sum(1.0 / (1.0 + math.exp(slope * (i - j))) for j in range(i + 1))
        assert abs(float(got[i, 0]) - head0) < (1e-4 if dtype == torch.float32 else 0.02 * head0)
        assert abs(float(got[i, d]) - 0.5 * (i + 1)) < (1e-4 if dtype == torch.float32 else 0.02 * (i + 1))
    # the temperature: queries along the keys, a large coefficient; rows before position every - 1 do not move
    params2 = dict(params, q_temp={"coef": 3.0, "every": 16}, talk=False, head_bias=False)
    w2 = {"m.q": eye, "m.k": eye, "m.v": eye, "m.o": eye}
    w2 = {k: v.to(torch.bfloat16) for k, v in w2.items()}
    h2 = inputs(T, H * d, 4) * 0.5
    hot = Harness(params2, dtype, weights=w2).run({"a": h2}, [{"a": 10}] + [{"a": 1}] * 30)[0]["a"]
    cold = Harness(dict(params2, q_temp=None), dtype, weights=w2).run({"a": h2}, [{"a": T}])[0]["a"]
    close(hot[:15], cold[:15], dtype, "before the first step of the temperature")
    assert float((hot[15:] - cold[15:]).abs().max()) > 0.05
    close(hot, plain_mixer(params2, "m")(h2, {**w2, "m.talk": torch.eye(H), "m.pb": torch.zeros(H)}), dtype, "temperature")


# ---- norms ------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("hidden", [60, 75, 256, 1000, 4100, 4102, 9000])   # 75, 4102: no multiple of four (one element a thread)
def test_layer_norm_with_bias_and_the_chain(hidden):
    g = torch.Generator().manual_seed(hidden)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    y, x = (3.0 * rnd(7, hidden) + 2.0).to(DEV), rnd(7, hidden).to(DEV)
    w1, b1, w2, b2, yb = (1.0 + 0.3 * rnd(hidden)).to(DEV), rnd(hidden).to(DEV), (1.0 + 0.3 * rnd(hidden)).to(DEV), rnd(hidden).to(DEV), rnd(hidden).to(DEV)
    c = lambda t: t.double().cpu()
    idx = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty((3, hidden), dtype=torch.float32, device=DEV)
    ops.layer_norm_rows(y, w1, 1e-5, out, idx, bias=b1)
    assert float((c(out) - plain.layer_norm(c(y)[[5, 0, 5]], w1.cpu(), b1.cpu(), 1e-5)).abs().max()) < 1e-5
    # x += LN(y + a bias) w + b; then the next norm of the updated rows, in one kernel
    want_x = c(x) + plain.layer_norm(c(y) + c(yb), w1.cpu(), b1.cpu(), 1e-5)
    want_next = plain.layer_norm(want_x, w2.cpu(), b2.cpu(), 1e-6)
    for dtype in DTYPES:
        x2 = x.clone()
        nxt = torch.empty((7, hidden), dtype=dtype, device=DEV)
        ops.layer_norm_chain(y, x2, w1, b1, 1e-5, in_bias=yb, next_gain=w2, next_bias=b2, next_eps=1e-6, next_out=nxt)
        assert float((c(x2) - want_x).abs().max()) < 1e-5
        assert float((c(nxt) - want_next).abs().max()) < (2e-5 if dtype == torch.float32 else 0.03)
    x3 = x.clone()
    emit = torch.empty((7, hidden), dtype=torch.bfloat16, device=DEV)
    ops.layer_norm_chain(y, x3, w1, b1, 1e-5, emit=emit)
    assert float((c(x3) - (c(x) + plain.layer_norm(c(y), w1.cpu(), b1.cpu(), 1e-5))).abs().max()) < 1e-5
    assert torch.equal(emit, x3.to(torch.bfloat16))


# ---- feed-forwards ------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,ff,act", [(64, 96, (0.3, -0.4)), (60, 100, (-2.0, 1.5)), (128, 512, (0.0, 0.0)), (64, 90, (0.5, 0.2))])
def test_xielu_feed_forward(hidden, ff, act, dtype):
    part = build_part("feed_forward", PartSpec("xielu", {"hidden_size": hidden, "intermediate_size": ff}, "f"))
    w = draw(part.tensor_specs(), ff)
    w["f.act"] = torch.tensor(act).to(torch.bfloat16)
    w["f.up"] = (2.0 * w["f.up"].float()).to(torch.bfloat16)            # both branches of the activation well used
    part.bind(handles(w), ctx_for(dtype))
    h = inputs(70, hidden, 9)
    want = plain.dense_ff(h, {k.replace("f.", "p.", 1): v for k, v in w.items()}, "p")
    y = torch.empty((70, hidden), dtype=torch.float32, device=DEV)
    part.forward(h.to(DEV).to(dtype), None, y, overwrite=True)
    close(y.double().cpu(), want, dtype, f"xielu {dtype}")
    y2 = torch.ones_like(y)
    part.forward(h.to(DEV).to(dtype), None, y2)                         # the adding form
    close(y2.double().cpu() - 1.0, want, dtype, "xielu, added")
    y3 = torch.empty_like(y)
    part.forward(h.to(DEV).to(dtype), None, y3, overwrite=True, defer_bias=True)
    close(y3.double().cpu() + w["f.down.b"].double(), want, dtype, "xielu, the output's bias left to the caller")


def test_xielu_values():
    z = torch.tensor([[-20.0, -3.0, -1e-3, 0.0, 1e-3, 0.5, 4.0, 30.0]], device=DEV)
    out = torch.empty_like(z)
    ap, an = math.log1p(math.exp(0.7)), 0.5 + math.log1p(math.exp(-0.3))
    ops.bias_xielu(z, None, ap, an, out)
    want = plain.xielu(z.double().cpu(), 0.7, -0.3)
    assert float(((out.double().cpu() - want).abs() / want.abs().clamp(min=1e-3)).max()) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,ff,limit,scale,shared,hidden", [
    (8, 2, 32, 1.5, 2.5, (48, 0.8), 64), (5, 1, 24, 0.5, None, None, 60), (4, 4, 16, 3.0, 0.5, (8, 4.0), 32),
    (16, 4, 48, 1.0, 1.0, (128, 1.0), 128), (3, 2, 40, 2.0, 3.0, None, 40)])
def test_routed_experts_with_clamps_scale_and_an_expert_for_every_row(E, top, ff, limit, scale, shared, hidden, dtype):
    params = {"hidden_size": hidden, "experts": E, "top": top, "intermediate_size": ff, "groups": None, "keep_groups": None,
              "weight_scale": scale, "activation": "clamped_swish", "limit": limit, "alpha": 1.702,
              "shared": None if shared is None else {"intermediate_size": shared[0], "limit": shared[1]}}
    part = build_part("feed_forward", PartSpec("routed_experts", params, "f"))
    w = draw(part.tensor_specs(), E)
    for n in w:
        if n.endswith((".gate", ".up")):
            w[n] = (2.5 * w[n].float()).to(torch.bfloat16)                # many inputs beyond the limits
    w["f.router"] = (0.5 * w["f.router"].float()).to(torch.bfloat16)
    part.bind(handles(w), ctx_for(dtype))
    T = 70
    h = inputs(T, hidden, 9)
    mlp = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": E, "top": top}}
    if scale is not None:
        mlp["router"]["scale"] = scale
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    pw = {k.replace("f.", "p.", 1): v for k, v in w.items()}
    want = plain.moe_ff(h, pw, "p", mlp)
    _, _, margin = plain.route(h, pw, "p", mlp["router"])
    sure = margin > 1e-5                      # rows whose choice rounding cannot change (the router reads exact inputs)
    assert int(sure.sum()) > T // 2
    y = torch.empty((T, hidden), dtype=torch.float32, device=DEV)
    part.forward(h.to(DEV).to(dtype), None, y, overwrite=True)
    close(y.double().cpu()[sure], want[sure], dtype, f"experts {dtype}")
    y2 = torch.ones_like(y)
    part.forward(h.to(DEV).to(dtype), None, y2)                         # the adding form
    close(y2.double().cpu()[sure] - 1.0, want[sure], dtype, "experts, added")
    # a row's result does not depend on the rows beside it
    y1 = torch.empty((1, hidden), dtype=torch.float32, device=DEV)
    part.forward(h[11:12].to(DEV).to(dtype), None, y1, overwrite=True)
    if dtype == torch.float32:
        assert torch.equal(y1[0], y[11])


def test_router_scale_and_no_renormalisation():
    g = torch.Generator().manual_seed(3)
    logits = 2.0 * torch.randn(200, 12, generator=g)
    weights = torch.empty(200, 12, device=DEV)
    chosen = torch.empty(200, 3, dtype=torch.int32, device=DEV)
    ops.moe_route(logits.to(DEV), weights, None, None, 3, chosen, weight_scale=2.5)
    s = torch.softmax(logits.double(), -1)
    top = torch.topk(s, 3).indices
    for r in range(200):
        assert sorted(chosen[r].tolist()) == sorted(top[r].tolist())
        row = weights[r].double().cpu()
        assert int((row != 0).sum()) == 3 and float((row[top[r]] - 2.5 * s[r, top[r]]).abs().max()) < 1e-6


# ---- the block ------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("with_ff", [True, False])
def test_block_with_norms_on_both_sides_of_every_sublayer(with_ff, dtype):
    hidden, T = 48, 90
    norm = lambda n: PartSpec("layer_norm", {"size": hidden, "eps": 1e-5, "tensor": n, "bias": n + ".b"}, n)
    att = dict(hidden_size=hidden, heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, window=20, q_temp={"coef": 0.5, "every": 7},
               slope_exp=8.0)
    parts = {"mixer_norm": norm("b.norm1"), "mixer": PartSpec("sigmoid_attention", att, "b.mix"), "mixer_out_norm": norm("b.norm1b")}
    if with_ff:
        parts.update({"feed_forward_norm": norm("b.norm2"), "feed_forward_out_norm": norm("b.norm2b"),
                      "feed_forward": PartSpec("xielu", {"hidden_size": hidden, "intermediate_size": 80}, "b.mlp")})
    block = part_class("block", "sandwich_norm")(LayerSpec(block="sandwich_norm", parts=parts))
    w = draw(block.tensor_specs(), 21)
    ctx = ctx_for(dtype)
    block.bind(handles(w), ctx)
    cache = cb.SequenceCache([block.cache_requirement()], 2, 256, 256, dtype, DEV)
    g = torch.Generator().manual_seed(2)
    x0 = torch.randn(T, hidden, generator=g)
    # the plain block
    ln = lambda t, n: plain.layer_norm(t, w[n], w[n + ".b"], 1e-5)
    rin = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(torch.bfloat16).double())
    xd = x0.double()
    y, _ = plain.attention_mixer(rin(ln(xd, "b.norm1")), w, "b.mix", mixer_config(att))
    want = xd + ln(y, "b.norm1b")
    if with_ff:
        want = want + ln(plain.dense_ff(rin(ln(want, "b.norm2")), w, "b.mlp"), "b.norm2b")
    for portions in ([T], [40, 1, 1, 48], [1] * T):
        slot, done, rows = cache.acquire(), 0, []
        for n in portions:
            batch = pack_step([StepEntry(slot, [0] * n, [])], [done], 1, DEV)
            cache.reserve(slot, done + n)
            x = x0[done:done + n].to(DEV).contiguous()
            block.forward(x, batch, cache.view(0))
            rows.append(x.double().cpu())
            done += n
            cache.commit(slot, done)
        cache.release(slot)
        close(torch.cat(rows), want, dtype, f"block {dtype} {len(portions)} portions")
    assert not any(ctx.error_flag.tolist())


MMA = [
    # head counts that are no multiple of eight, keys and values of different sizes, a window inside one page
    dict(hidden_size=48, heads=6, kv_heads=3, dim=48, vdim=80, scale=0.15, window=40, q_temp={"coef": 0.4, "every": 5}),
    # a window over several pages that ends inside a page, one key/value head
    dict(hidden_size=64, heads=8, kv_heads=1, dim=32, vdim=16, scale=0.2, window=150, q_temp=None),
    # no window, the largest head size
    dict(hidden_size=32, heads=2, kv_heads=2, dim=256, vdim=32, scale=0.06, window=None, q_temp={"coef": 0.2, "every": 64}),
    # twelve heads, a window of exactly two pages; no mix and no gate
    dict(hidden_size=96, heads=12, kv_heads=4, dim=16, vdim=128, scale=0.3, window=128, q_temp=None, talk=False, gate=False),
]


@pytest.mark.parametrize("params", MMA)
def test_tensor_core_form_of_new_tokens(params):
    """Runs of new tokens in bfloat16 take the two tensor-core kernels; the same rows through the kernel that walks a row's
    keys, and the plain implementation, must agree: whole prompts, portions that start inside a group of rows and inside a
    page, unequal sequences in one step (the second starts at a row that is no multiple of eight), a slot used again."""
    dtype = torch.bfloat16
    T = 333
    params = dict(params, slope_exp=8.0)
    h, other = inputs(T, params["hidden_size"], 21), inputs(77, params["hidden_size"], 22)
    fast = Harness(dict(params, mma_min_rows=8), dtype, seed=9, capacity=2048)
    slow = Harness(dict(params, mma_min_rows=10 ** 9), dtype, weights=fast.weights, capacity=2048)
    taken = []
    real = ops.sigmoid_attention_mma
    ops.sigmoid_attention_mma = lambda *a, **k: (taken.append(a[0].shape[0]), real(*a, **k))[1]
    try:
        fn = plain_mixer(params, "m")
        want, want_other = fn(h, fast.weights), fn(other, fast.weights)
        for portions in ([{"a": T}], [{"a": 13}, {"a": 120}, {"a": 1}, {"a": 9}, {"a": 190}], [{"a": 64}, {"a": 64}, {"a": 205}]):
            got = fast.run({"a": h}, portions)[0]["a"]
            ref = slow.run({"a": h}, portions)[0]["a"]
            close(got, want, dtype, f"tensor cores {portions}")
            close(got, ref, dtype, f"tensor cores against rows {portions}")
        assert taken and 1 not in taken and 13 in taken and 333 in taken
        both = fast.run({"a": h, "b": other}, [{"a": 101, "b": 30}, {"a": 1, "b": 1}, {"a": 231, "b": 46}])[0]
        close(both["a"], want, dtype, "batched a")
        close(both["b"], want_other, dtype, "batched b")
        again = fast.run({"c": other}, [{"c": 77}])[0]["c"]
        close(again, want_other, dtype, "reused slot")
        n = len(taken)
        slow.run({"a": h}, [{"a": T}])
        assert len(taken) == n
    finally:
        ops.sigmoid_attention_mma = real


@pytest.mark.parametrize("window", [9, 64, 65, 130, 1, None])
def test_window_edges_on_the_tensor_cores(window):
    """The key that stands out, with every portion on the tensor-core kernels: the row at distance window - 1 has it, the next
    one has lost it, also when the key came in an earlier portion and when the edge falls between two groups of rows."""
    d, T = 16, 210
    params, weights = standing_out(d, window)
    params = dict(params, mma_min_rows=8)
    for special in (0, 7, 8, 63, 64, 100):
        g = torch.Generator().manual_seed(special)
        h = 0.05 * torch.randn(T, d, generator=g)
        h[:, 0] = 1.0
        h[special, 0] = 30.0
        h[special, 1] = 7.0
        h = h.to(torch.bfloat16).double()
        want = plain_mixer(params, "m")(h, weights)
        see = plain.visible(T, window)
        for portions in ([{"a": T}], [{"a": 101}, {"a": 109}], [{"a": 9}, {"a": 60}, {"a": 141}]):
            got = Harness(params, torch.bfloat16, weights=weights).run({"a": h}, portions)[0]["a"]
            allowed = 0.03 * want.abs().amax(-1, keepdim=True).clamp(min=1.0)
            assert bool(((got - want).abs() <= allowed).all()), (window, special, portions)
            for i in range(special + 1, T):
                assert (float(got[i][1]) > 3.0) == bool(see[i, special]), (window, special, i)
