"""Each mechanism of the Pivavik design alone, built through the registries at sizes no model uses, against the plain
implementation: latent attention with pairs of halves turned and one gate number a head (whole, token by token, in portions
and in batches through one cache; a rotated part of which only some elements turn; a far key among hundreds); attention with
biases, a soft cap, a window and a gate an element (one key made to stand out just inside and just outside the window, over
page borders, in prompts and in decoding; a cap that decides which key wins); the GELU feed-forward with biases; the router
with sigmoid scores and experts that read their weighted input; the block with one norm for both sub-layers; the step ahead
of a repeated run of layers; the soft cap on logits."""
import pytest
import torch

import citlali_b200 as cb
import plain_pivavik as plain
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
        if n.endswith((".dq.norm", ".dkv.norm")):
            t = 1.0 + 0.3 * r
        elif s.role == "gain":
            t = 0.3 * r                                   # stored around zero
        elif n.endswith("router"):
            t = 3.0 * r / s.shape[-1] ** 0.5
        elif len(s.shape) == 1:
            t = 0.4 * r
        elif n.endswith((".q", ".k", ".uq", ".uk", ".dkv", ".g")):
            t = 2.0 * r / s.shape[-1] ** 0.5
        else:
            t = r / s.shape[-1] ** 0.5
        out[n] = t.to(torch.bfloat16)
    return out


def inputs(T, hidden, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, hidden, generator=g).to(torch.bfloat16).double()       # what both paths read exactly


def close(got, want, dtype, what, tol=None):
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert err <= (tol or TOL[dtype]) * scale, f"{what}: |diff| {err:.3e} of {scale:.3e}"


class Harness:
    """A mixer with a cache of its own: feeds sequences in the given portions and returns its output rows."""

    def __init__(self, kind, params, dtype, weights=None, seed=1, slots=3, capacity=1024, max_seq=1024):
        self.part = build_part("mixer", PartSpec(kind, params, "m"))
        self.weights = weights if weights is not None else draw(self.part.tensor_specs(), seed)
        self.ctx = ctx_for(dtype)
        self.part.bind(handles(self.weights), self.ctx)
        self.cache = cb.SequenceCache([self.part.cache_requirement()], slots, capacity, max_seq, dtype, DEV)
        self.hidden = params["hidden_size"]
        self.dtype = dtype

    def run(self, sequences, portions):
        """``sequences``: {name: h [T, hidden] float64}; ``portions``: a list of steps, each {name: n new tokens}."""
        slots, done = {}, {}
        out = {n: [] for n in sequences}
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
            y = torch.empty((h.shape[0], self.hidden), dtype=torch.float32, device=DEV)
            self.part.forward(h, batch, self.cache.view(0), y, True, overwrite=True)
            at = 0
            for n in names:
                out[n].append(y[at:at + step[n]].double().cpu())
                at += step[n]
            for n in names:
                done[n] += step[n]
                self.cache.commit(slots[n], done[n])
        for n in list(slots):
            self.cache.release(slots.pop(n))
        assert self.cache.pages_held() == 0
        assert not any(self.ctx.error_flag.tolist())
        return {n: torch.cat(v) for n, v in out.items()}


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


def every_way(hs, fn, h, other, dtype):
    """The mixer against ``fn`` (the plain one) however the sequence is cut; two unequal sequences in a batch; a slot and
    pages that are used again.  In 32-bit every cut must give the same bits."""
    T = h.shape[0]
    want = fn(h)
    results = {}
    for what, portions in cuts(T).items():
        results[what] = hs.run({"a": h}, portions)["a"]
        close(results[what], want, dtype, f"{dtype} {what}")
    if dtype == torch.float32:
        for what in results:
            assert torch.equal(results[what], results["whole"]), f"'{what}' gives other bits than 'whole'"
    n = other.shape[0]
    both = hs.run({"a": h, "b": other}, [{"a": 50, "b": 20}, {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": T - 52, "b": n - 22}])
    close(both["a"], want, dtype, f"{dtype} batched a")
    close(both["b"], fn(other), dtype, f"{dtype} batched b")
    if dtype == torch.float32:
        assert torch.equal(both["a"], results["whole"])
    close(hs.run({"c": other}, [{"c": n}])["c"], fn(other), dtype, f"{dtype} reused slot")


# ---- latent attention -------------------------------------------------------------------------------------------------------

def latent_params(hidden, heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, rot_dims=None):
    return dict(hidden_size=hidden, heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale,
                norm_eps=1e-5, window=None, rot_dims=rot_dim if rot_dims is None else rot_dims, rot_base=base, rot_layout="halves",
                gate="heads", kv_projection=True,
                names={"dq": "m.dq", "dq_norm": "m.dq.norm", "uq": "m.uq", "dkv": "m.dkv", "dkv_norm": "m.dkv.norm", "uk": "m.uk",
                       "uv": "m.uv", "gate": "m.g", "o": "m.o", "sink": None})


def latent_config(p):
    return {"heads": p["heads"], "dim": p["dim"], "rot_dim": p["rot_dim"], "vdim": p["vdim"], "q_rank": p["q_rank"],
            "kv_rank": p["kv_rank"], "scale": p["scale"], "rot": {"dims": p["rot_dims"], "base": p["rot_base"]}}


LATENT = [
    latent_params(40, 3, 16, 8, 24, 24, 48, 0.2, 10000.0),                 # a rotated part smaller than the rest
    latent_params(48, 5, 12, 20, 12, 36, 44, 0.25, 100.0, rot_dims=12),    # only 12 of 20 elements turn; odd sizes
    latent_params(64, 16, 16, 16, 32, 64, 64, 0.2, 200000.0),              # sizes the tensor-core walk takes, sixteen heads
    latent_params(32, 1, 8, 32, 8, 16, 128, 0.15, 500.0),                  # one head; the rotated part carries the score
    latent_params(64, 20, 32, 64, 16, 32, 128, 0.1, 10000.0),              # more heads than one tile of the walk holds
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("params", LATENT)
def test_latent_attention_mixer(params, dtype):
    hs = Harness("latent_attention", params, dtype, seed=3)
    fn = lambda h: plain.latent_attention(h, hs.weights, "m", latent_config(params), 1e-5)
    every_way(hs, fn, inputs(150, params["hidden_size"], 3), inputs(37, params["hidden_size"], 4), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_rotation_alone_carries_the_scores(dtype):
    """No unrotated key part (W_uk = 0): a row's scores come from the turned pairs alone.  The plain implementation says that
    the turning matters here (another base gives other outputs, and so does pairing neighbours instead of halves); the
    mixer must follow it in prompts, portions and decoding."""
    p = latent_params(32, 2, 8, 16, 8, 16, 16, 1.0, 30.0)
    w = draw(build_part("mixer", PartSpec("latent_attention", p, "m")).tensor_specs(), 9)
    w["m.uk"] = torch.zeros_like(w["m.uk"])
    T = 140
    h = inputs(T, 32, 5)
    want = plain.latent_attention(h, w, "m", latent_config(p), 1e-5)
    other = plain.latent_attention(h, w, "m", latent_config(dict(p, rot_base=300.0)), 1e-5)
    assert float((want - other).abs().max()) > 0.05 * float(want.abs().max())
    hs = Harness("latent_attention", p, dtype, weights=w)
    for portions in ([{"a": T}], [{"a": 66}, {"a": 10}] + [{"a": 1}] * (T - 76)):
        close(hs.run({"a": h}, portions)["a"], want, dtype, f"{dtype} rotation alone")
    neighbours = Harness("latent_attention", dict(p, rot_layout="pairs"), dtype, weights=w).run({"a": h}, [{"a": T}])["a"]
    assert float((neighbours - want).abs().max()) > 0.05 * float(want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_finds_a_far_key_among_hundreds(dtype):
    """Queries and keys look along one axis of the latent; one token at position 3 is long along it, 900 ordinary ones are
    not: every later row's softmax gives it nearly all the weight, over fifteen pages, whether the row comes in the prompt, in
    a later portion or token by token.  Its value (the latent's second axis) is what every later row must return."""
    hidden, T = 32, 900
    p = latent_params(hidden, 2, 1, 4, 1, hidden, hidden, 8.0, 10000.0)
    eye = torch.eye(hidden)
    pick = lambda rows: eye[rows].contiguous()
    w = {"m.dq": eye, "m.dq.norm": torch.ones(hidden), "m.dkv": torch.cat([eye, torch.zeros(4, hidden)]), "m.dkv.norm": torch.ones(hidden),
         # both heads' queries: the first axis, nothing along the rotated part; keys: the first axis; values: the second axis
         "m.uq": torch.cat([pick([0]), torch.zeros(4, hidden), pick([0]), torch.zeros(4, hidden)]),
         "m.uk": pick([0, 0]), "m.uv": pick([1, 1]), "m.g": torch.zeros(2, hidden), "m.o": torch.cat([torch.eye(2), torch.zeros(hidden - 2, 2)])}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    g = torch.Generator().manual_seed(11)
    h = torch.randn(T, hidden, generator=g)
    h[:, 0] = 1.0                                    # after the norm: about one along the first axis
    h[3] = 0.0
    h[3, 0], h[3, 1] = 30.0, -20.0                   # after the norm: 4.7 along the first axis, -3.1 along the second
    h = h.to(torch.bfloat16).double()
    want = plain.latent_attention(h, w, "m", latent_config(p), 1e-5)
    far = float(want[3, 0])
    assert far < -1.0 and float((want[10:, :2] - far).abs().max()) < 0.05 * abs(far)
    hs = Harness("latent_attention", p, dtype, weights=w, capacity=1024)
    for portions in ([{"a": T}], [{"a": 500}, {"a": 300}] + [{"a": 1}] * 100, [{"a": 2}] * 450):
        got = hs.run({"a": h}, portions)["a"]
        assert float((got - want).abs().max()) < (1e-3 if dtype == torch.float32 else 0.08), len(portions)
        assert float((got[10:, :2] - far).abs().max()) < 0.1 * abs(far)


# ---- attention with biases, a soft cap, a window and a gate -------------------------------------------------------------------

def attention_params(hidden, heads, kv_heads, dim, vdim, scale, softcap, window):
    return dict(hidden_size=hidden, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=None, qk_norm_eps=None, rot_dims=0,
                scale=scale, window=window, keep_first=0, softcap=softcap, biases=True, gate="elements")


def attention_config(p):
    m = {k: p[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale", "softcap")}
    m["mask"] = {"size": p["window"] if p["window"] is not None else 1 << 30}
    return m


ATT = [
    attention_params(40, 4, 2, 16, 24, 0.25, 3.0, 9),          # a window shorter than a page, values wider than keys, a cap that bites
    attention_params(48, 3, 3, 80, 12, 0.08, 30.0, 65),        # a page and one; a head over 64 and no multiple of 32; one key head a query head
    attention_params(32, 8, 1, 32, 32, 0.15, 5.0, None),       # no window, one key/value head for all
    attention_params(24, 2, 2, 24, 40, 0.2, 2.0, 1),           # a window of one token: a row sees itself alone
    attention_params(64, 16, 4, 64, 64, 0.125, 10.0, 130),     # several pages of window, sizes the tensor cores like
    attention_params(32, 4, 2, 16, 16, 0.3, 1.5, 70),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("params", ATT)
def test_attention_mixer(params, dtype):
    hs = Harness("window_attention", params, dtype, seed=3)
    fn = lambda h: plain.window_attention(h, hs.weights, "m", attention_config(params))
    every_way(hs, fn, inputs(150, params["hidden_size"], 3), inputs(37, params["hidden_size"], 4), dtype)


def test_biases_cap_and_gate_each_matter():
    """Switching one of them off changes the output: none is silently dropped on the way to the kernels."""
    params = ATT[0]
    h = inputs(60, 40, 8)
    base = Harness("window_attention", params, torch.float32, seed=3)
    full = base.run({"a": h}, [{"a": 60}])["a"]
    for change in (dict(softcap=None), dict(biases=False), dict(gate=None)):
        other = Harness("window_attention", dict(params, **change), torch.float32, weights=base.weights)
        assert float((other.run({"a": h}, [{"a": 60}])["a"] - full).abs().max()) > 1e-2, change


def standing_out(d, window, cap):
    params = attention_params(d, 1, 1, d, d, 1.0, cap, window)
    eye = torch.eye(d).to(torch.bfloat16)
    zero = torch.zeros(d).to(torch.bfloat16)
    weights = {"m.q": eye, "m.k": eye, "m.v": eye, "m.o": eye, "m.g": torch.zeros(d, d).to(torch.bfloat16),
               "m.q.b": zero, "m.k.b": zero, "m.v.b": zero}
    return params, weights


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode_from", [None, 40])
@pytest.mark.parametrize("window", [9, 64, 65, 130, 1, None])
def test_window_edges_with_one_key_that_stands_out(window, decode_from, dtype):
    """Queries, keys and values are the inputs themselves.  One key is made long: its capped score is 18 where an ordinary
    key's is about 1, so a row returns that key's value (times the gate's one half) while the key is inside the window: the
    row at distance window - 1 has it, the next one has lost it; over page borders; in prompts and in decoding."""
    d, T = 16, 210
    params, weights = standing_out(d, window, 20.0)
    for special in (0, 1, 62, 63, 64, 100):
        g = torch.Generator().manual_seed(special)
        h = 0.05 * torch.randn(T, d, generator=g)
        h[:, 0] = 1.0                                       # every query has a part along the first axis ...
        h[special, 0] = 30.0                                # ... and one key is long along it
        h[special, 1] = 14.0                                # and carries a value no other has
        h = h.to(torch.bfloat16).double()
        hs = Harness("window_attention", params, dtype, weights=weights)
        portions = [{"a": T}] if decode_from is None else [{"a": decode_from}] + [{"a": 1}] * (T - decode_from)
        got = hs.run({"a": h}, portions)["a"]
        want = plain.window_attention(h, weights, "m", attention_config(params))
        allowed = (1e-4 if dtype == torch.float32 else 0.03) * want.abs().amax(-1, keepdim=True).clamp(min=1.0)
        assert bool(((got - want).abs() <= allowed).all()), (window, special)
        see = plain.causal(T, window)
        for i in range(special + 1, T):                     # the test's point: the special key decides the row
            assert (float(got[i][1]) > 3.0) == bool(see[i, special]), (window, special, i)
            assert (float(want[i][1]) > 3.0) == bool(see[i, special])


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_cap_decides_between_two_long_keys(dtype):
    """Two keys with raw scores 40 and 80: under a cap of 10 both sit at the cap and share the weight; without the cap the
    second would take all of it.  Prompt and decoding."""
    d, T = 16, 100
    params, weights = standing_out(d, None, 10.0)
    h = torch.zeros(T, d)
    h[:, 0] = 1.0
    h[5, 0], h[5, 1] = 40.0, 8.0
    h[70, 0], h[70, 1] = 80.0, -8.0
    h = h.to(torch.bfloat16).double()
    want = plain.window_attention(h, weights, "m", attention_config(params))
    assert abs(float(want[90, 1])) < 0.1 and float(want[60, 1]) > 3.5          # shared after 70, key 5 alone before
    for portions in ([{"a": T}], [{"a": 30}] + [{"a": 1}] * 70):
        got = Harness("window_attention", params, dtype, weights=weights).run({"a": h}, portions)["a"]
        close(got, want, dtype, f"{dtype} two long keys", tol=1e-5 if dtype == torch.float32 else 1e-2)
        assert abs(float(got[90, 1])) < 0.15 and float(got[60, 1]) > 3.5


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_among_hundreds(dtype):
    d, T = 32, 900
    params = attention_params(d, 2, 1, d // 2, d // 2, 1.0, 25.0, 1000)
    eye = torch.eye(d)
    weights = {"m.q": eye, "m.k": eye[:d // 2], "m.v": eye[d // 2:], "m.o": eye, "m.g": torch.zeros(d, d), "m.q.b": torch.zeros(d),
               "m.k.b": torch.zeros(d // 2), "m.v.b": torch.zeros(d // 2)}
    weights = {k: v.to(torch.bfloat16) for k, v in weights.items()}
    g = torch.Generator().manual_seed(11)
    h = 0.05 * torch.randn(T, d, generator=g)
    h[:, 0] = 1.0
    h[:, d // 2] = 1.0                                       # both query heads look along the first key axis
    h[3, 0] = 30.0
    h[3, d // 2:] = 7.0                                      # the far token's value
    h = h.to(torch.bfloat16).double()
    want = plain.window_attention(h, weights, "m", attention_config(params))
    assert float((want[10:] - 3.5).abs().max()) < 0.1        # the far value times the gate's one half, everywhere
    hs = Harness("window_attention", params, dtype, weights=weights, capacity=1024)
    for portions in ([{"a": T}], [{"a": 500}, {"a": 300}] + [{"a": 1}] * 100, [{"a": 2}] * 450):
        got = hs.run({"a": h}, portions)["a"]
        assert float((got - want).abs().max()) < (1e-3 if dtype == torch.float32 else 0.05), len(portions)


# ---- feed-forwards -----------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,ff", [(40, 96), (60, 100), (32, 24), (64, 256)])
def test_gelu_feed_forward_with_biases(hidden, ff, dtype):
    names = {"gate": "f.gate", "up": "f.up", "down": "f.down"}
    part = build_part("feed_forward", PartSpec("gated", {"hidden_size": hidden, "intermediate_size": ff, "activation": "gelu_tanh",
                                                           "biases": True, "names": names}, "f"))
    w = draw(part.tensor_specs(), 5)
    assert {"f.gate.b", "f.up.b", "f.down.b"} <= set(w)
    part.bind(handles(w), ctx_for(dtype))
    h = 1.5 * inputs(70, hidden, 6)
    want = plain.dense_ff(h, w, "f")
    base = torch.randn(70, hidden, dtype=torch.float64)
    for rows in (70, 1):
        y = base[:rows].float().to(DEV).contiguous()
        part.forward(h[:rows].to(DEV).to(dtype).contiguous(), None, y)
        close(y.double().cpu() - base[:rows], want[:rows], dtype, f"{dtype} {rows} rows")
    y = torch.empty(70, hidden, dtype=torch.float32, device=DEV)
    part.forward(h.to(DEV).to(dtype).contiguous(), None, y, overwrite=True)
    close(y.double().cpu(), want, dtype, f"{dtype} overwrite")


@pytest.mark.parametrize("experts,top", [(6, 2), (3, 3), (16, 4), (10, 1), (40, 5)])
def test_sigmoid_router(experts, top):
    g = torch.Generator().manual_seed(experts)
    logits = (3.0 * torch.randn(50, experts, generator=g)).float()
    logits[0, :] = 1.25                                    # ties: the lower indices win
    logits[1, : min(3, experts)] = 100.0                   # scores that saturate at one
    out = torch.empty(50, experts, dtype=torch.float32, device=DEV)
    chosen = torch.empty(50, top, dtype=torch.int32, device=DEV)
    ops.moe_route(logits.to(DEV), out, None, None, top, chosen=chosen, score="sigmoid")
    s = torch.sigmoid(logits.double())
    order = torch.sort(s.float(), dim=-1, descending=True, stable=True).indices[:, :top]
    assert torch.equal(chosen.cpu().long(), order)
    want = torch.zeros_like(s).scatter_(1, order, s.gather(1, order))
    assert float((out.double().cpu() - want).abs().max()) < 1e-6
    assert chosen[0].tolist() == list(range(top))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,experts,top,ff", [(40, 6, 2, 32), (60, 3, 3, 24), (64, 16, 4, 16), (32, 10, 1, 40)])
def test_experts_that_read_their_weighted_input(hidden, experts, top, ff, dtype):
    part = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": hidden, "experts": experts, "top": top, "intermediate_size": ff, "score": "sigmoid", "weight_on": "input",
        "activation": "silu"}, "f"))
    w = draw(part.tensor_specs(), 7)
    part.bind(handles(w), ctx_for(dtype))
    h = 1.5 * inputs(90, hidden, 8)
    mlp = {"router": {"experts": experts, "top": top}}
    want = plain.moe_ff(h, w, "f", mlp)
    _, _, margin = plain.route(h, w, "f", mlp["router"])
    y = torch.zeros(90, hidden, dtype=torch.float32, device=DEV)
    part.forward(h.to(DEV).to(dtype).contiguous(), None, y)
    got = y.double().cpu()
    sure = margin > 1e-3                                   # rows whose choice no rounding can change
    assert int(sure.sum()) > 60
    close(got[sure], want[sure], dtype, f"{dtype} experts")
    # the weight is on the input: weighting the output instead gives other numbers
    other = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": hidden, "experts": experts, "top": top, "intermediate_size": ff, "score": "sigmoid", "weight_on": "output",
        "activation": "silu"}, "f"))
    other.bind(handles(w), ctx_for(dtype))
    y2 = torch.zeros(90, hidden, dtype=torch.float32, device=DEV)
    other.forward(h.to(DEV).to(dtype).contiguous(), None, y2)
    assert float((y2.double().cpu() - want).abs().max()) > 0.05 * float(want.abs().max())


# ---- the block, the step ahead of a repeated run, the caps ----------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
def test_block_with_one_norm_for_both_sublayers(dtype):
    hidden = 40
    norm = PartSpec("rms_norm", {"size": hidden, "eps": 1e-5, "tensor": "l0.norm1", "offset": 1.0}, "l0.norm1")
    mixer = PartSpec("window_attention", attention_params(hidden, 4, 2, 16, 24, 0.25, 3.0, 9), "l0.mix")
    ff = PartSpec("gated", {"hidden_size": hidden, "intermediate_size": 48, "activation": "gelu_tanh", "biases": True,
                            "names": {"gate": "l0.mlp.gate", "up": "l0.mlp.up", "down": "l0.mlp.down"}}, "l0.mlp")
    for parts in ({"norm": norm, "mixer": mixer, "feed_forward": ff}, {"norm": norm, "mixer": mixer}):
        block = part_class("block", "parallel_residual")(LayerSpec("parallel_residual", parts))
        w = draw(block.tensor_specs(), 2)
        block.bind(handles(w), ctx_for(dtype))
        cache = cb.SequenceCache([block.cache_requirement()], 1, 256, 256, dtype, DEV)
        slot = cache.acquire()
        T = 50
        x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(4)).float()
        batch = pack_step([StepEntry(slot, [0] * T, [])], [0], 1, DEV)
        cache.reserve(slot, T)
        xd = x.to(DEV).clone()
        block.forward(xd, batch, cache.view(0), True)
        spec = {"type": "attention", "mixer": attention_config(mixer.params), "mlp": {"kind": "dense", "ff": 48} if "feed_forward" in parts else None}
        rin = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(torch.bfloat16).double())
        want = plain.layer(x.double(), w, 0, spec, 1e-5, rin, None)
        close(xd.double().cpu(), want, dtype, f"{dtype} block")


@pytest.mark.parametrize("dtype", DTYPES)
def test_step_ahead_of_a_repeated_run(dtype):
    hidden, passes, T = 24, 3, 20
    block = part_class("block", "input_injection")(LayerSpec("input_injection", {}, {
        "hidden_size": hidden, "passes": passes, "matrix": "loop.in", "steps": "loop.step"}))
    assert block.parts() == [] and block.cache_requirement() is None and block.needs_embedding_output
    g = torch.Generator().manual_seed(6)
    w = {"loop.in": (torch.randn(hidden, 2 * hidden, generator=g) / 7.0).to(torch.bfloat16),
         "loop.step": torch.randn(passes, hidden, generator=g).to(torch.bfloat16)}
    block.bind(handles(w), ctx_for(dtype))
    x, x0 = inputs(T, hidden, 1), inputs(T, hidden, 2)
    batch = pack_step([StepEntry(0, [0] * T, [])], [0], 1, DEV)
    for t in range(passes):
        batch.visit, batch.embedding_output = t, x0.float().to(DEV)
        xd = x.float().to(DEV).clone()
        block.forward(xd, batch, None)
        want = torch.cat([x, x0], -1) @ w["loop.in"].double().T + w["loop.step"].double()[t]
        close(xd.double().cpu(), want, dtype, f"{dtype} pass {t}", tol=1e-5 if dtype == torch.float32 else 1e-2)
    batch.visit = passes
    with pytest.raises(cb.CitlaliError, match="has run"):
        block.forward(x.float().to(DEV), batch, None)


def test_soft_cap_and_concat_kernels():
    x = torch.linspace(-200.0, 200.0, 4001)
    y = x.to(DEV).clone()
    ops.soft_cap_(y, 30.0)
    assert float((y.double().cpu() - plain.soft_cap(x.double(), 30.0)).abs().max()) < 1e-5
    for width in (10, 12, 64, 200):                       # rows that are and are not multiples of four floats
        a, b = torch.randn(7, width), torch.randn(7, width)
        for dtype in DTYPES:
            out = torch.empty(7, 2 * width, dtype=dtype, device=DEV)
            ops.concat_rows(a.to(DEV), b.to(DEV), out)
            assert torch.equal(out.cpu(), torch.cat([a, b], -1).to(dtype))
        table = torch.randn(3, width)
        y = a.to(DEV).clone()
        ops.add_row_bias(y, table.to(DEV)[2])
        assert torch.equal(y.cpu(), a + table[2])
