"""Tutizen on the native sequence engine against the plain oracle (tests/tutizen_oracle.py): every mechanism alone, then whole models
through prompts, decoding, portions, mixed batches, reused slots and pages, the scheduler and the command line.  Configurations and
weights are made here."""
import json
import math

import numpy as np
import pytest
import torch

import tutizen_oracle as O

pytestmark = pytest.mark.gpu


def attn(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.25, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": None}


def dense(ff=40, limit=1.75):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=8, top=3, count=4, keep=2, ff=20, limit=1.25, scale=1.75, shared=(12, 2.5)):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "scale": scale}}
    if count:
        f["router"]["groups"] = {"count": count, "keep": keep}
    if shared:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def with_ff(layer, ff):
    return dict(layer, mlp=ff)


def config(layers, width=48, vocab=70, eps=2e-5, mult=0.4):
    return {"architecture": "Tutizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


CFG_MIXED = config([with_ff(attn(), dense()), with_ff(attn(kv_from=0), moe()), with_ff(attn(heads=6, kv_heads=3, dim=8, vdim=12, scale=0.5), moe(experts=6, top=2, count=2, keep=1, ff=16)),
                    attn(heads=6, kv_heads=3, dim=8, vdim=12, scale=0.3, kv_from=2)])
# equal head counts, one key/value head, one group, top 1, no shared expert, two layers reading the same earlier cache
CFG_ODD = config([with_ff(attn(heads=3, kv_heads=3, dim=12, vdim=20, scale=0.2), moe(experts=5, top=1, count=1, keep=1, ff=10, shared=None)),
                  with_ff(attn(heads=3, kv_heads=3, dim=12, vdim=20, scale=0.4, kv_from=0), dense(ff=24, limit=0.7)),
                  with_ff(attn(heads=3, kv_heads=3, dim=12, vdim=20, scale=0.1, kv_from=0), moe(experts=4, top=4, count=0, ff=8, scale=0.7)),
                  with_ff(attn(heads=5, kv_heads=1, dim=24, vdim=8, scale=0.15), dense(ff=56, limit=3.0))], width=40, vocab=33, eps=1e-3, mult=1.0)
CFG_WIDE = config([with_ff(attn(heads=8, kv_heads=2, dim=64, vdim=32, scale=0.1), moe(experts=16, top=4, count=4, keep=3, ff=48, shared=(64, 1.5))),
                   with_ff(attn(heads=8, kv_heads=2, dim=64, vdim=32, scale=0.1, kv_from=0), dense(ff=192))], width=128, vocab=150, mult=0.25)
# nothing here is a multiple of 8: rows of every matrix start unaligned, so the vector / TMA forms of the products must step aside
CFG_THIN = config([with_ff(attn(heads=3, kv_heads=1, dim=10, vdim=14, scale=0.3), moe(experts=6, top=2, count=3, keep=1, ff=13, shared=(9, 1.0))),
                   with_ff(attn(heads=2, kv_heads=2, dim=6, vdim=10, scale=0.5), dense(ff=21))], width=36, vocab=31)
CONFIGS = {"mixed": CFG_MIXED, "odd": CFG_ODD, "wide": CFG_WIDE, "thin": CFG_THIN}


def make_weights(cfg, seed):
    """name -> float32 array whose values are exactly representable in bfloat16 (so both engine dtypes hold the same model)."""
    return {k: v.numpy() for k, v in O.random_weights(cfg, seed).items()}


def build(cfg, weights, dtype="float32", max_tokens=256, slots=4, page_size=4, max_step_tokens=64):
    from wf_bitnet import registry
    cls = registry.resolve(cfg)
    model = cls(cfg, dtype=dtype, max_tokens=max_tokens, slots=slots, page_size=page_size, max_step_tokens=max_step_tokens)
    model.load_weights((k, v, "F32") for k, v in weights.items())
    return model


def t64(weights):
    return {k: torch.from_numpy(np.asarray(v)).double() for k, v in weights.items()}


def oracle_logits(cfg, weights, tokens):
    return O.forward(list(tokens), t64(weights), cfg)[0].numpy()


def rel_err(got, want):
    """per row: RMS of the difference (mean taken off) over the RMS of the expected row"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / (np.sqrt((want ** 2).mean(-1)) + 1e-12)


TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def assert_close(got, want, dtype, what):
    """float32: every row within tolerance.  bfloat16: a router whose scores nearly tie may choose another expert after rounding, which
    moves that position by far more than rounding does; such positions are few, so most rows must be within tolerance."""
    err = rel_err(got, want)
    if dtype == "float32":
        assert err.max() < TOL[dtype], (what, int(err.argmax()), err.max())
    else:
        assert (err < 2.5 * TOL[dtype]).mean() >= 0.8 and np.median(err) < TOL[dtype], (what, int(err.argmax()), err.max(), np.median(err))


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def bf16_exact(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def _rows(n, W, seed, scale=1.0):
    return bf16_exact(np.random.default_rng(seed).standard_normal((n, W)) * scale)


def run_alone(m, tokens, cuts):
    """one request through the engine in portions `cuts`; logits of every position"""
    s = m.admit()
    out, a = [], 0
    for c in cuts:
        out.append(m.step([s], [c], tokens[a:a + c], list(range(c))))
        a += c
    m.release(s)
    return np.concatenate(out)


# ---------------------------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_vectors_and_output_norm(dtype):
    """One layer without feed-forward whose attention output is forced to a constant (zero weights, output bias only): the stream after
    it is embedding + position vector + mult * gain * rms(bias) — checked at positions 0, 1 and a few thousand."""
    cfg = config([attn(heads=2, kv_heads=1, dim=8, vdim=8)], width=24, vocab=11, mult=0.7)
    w = make_weights(cfg, 3)
    w["l0.mix.o"] = np.zeros_like(w["l0.mix.o"])
    m = build(cfg, w, dtype, max_tokens=4096, page_size=64, max_step_tokens=512)
    n = 2100
    toks = tokens_for(cfg, n, 4)
    s = m.admit()
    taps = []
    for a in range(0, n, 500):
        taps.append(m.engine.step_with_layer_tap([s], [len(toks[a:a + 500])], toks[a:a + 500])[1][0])
    got = np.concatenate(taps)
    b = torch.from_numpy(w["l0.mix.o.b"]).double()
    want = torch.from_numpy(w["embed"]).double()[toks] + O.position_vectors(torch.arange(n), 24) + 0.7 * O.scalar_rms_norm(b, float(w["l0.norm1"]), 2e-5)
    assert np.abs(got - want.numpy()).max() < 2e-5
    # the position vector itself: even entries sines, odd entries cosines of the same angle
    pv = O.position_vectors(torch.tensor([0, 1, 2000]), 24).numpy()
    assert np.allclose(pv[0, 0::2], 0) and np.allclose(pv[0, 1::2], 1)
    assert abs(pv[1, 0] - math.sin(1.0)) < 1e-12 and abs(pv[1, 1] - math.cos(1.0)) < 1e-12
    assert abs(pv[2, 2] - math.sin(2000 * 10000 ** (-2 / 24))) < 1e-9 and abs(pv[2, 3] - math.cos(2000 * 10000 ** (-2 / 24))) < 1e-9
    m.close()


@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "thin"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_alone_whole_and_in_portions(name, dtype):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 11)
    eps = cfg["norm"]["eps"]
    for li, L in enumerate(cfg["layers"]):
        src = L["mixer"].get("kv_from")
        m = build(cfg, w, dtype)
        n = 23
        x = _rows(n, cfg["width"], 12 + li)
        xs = _rows(n, cfg["width"], 40 + li)                 # what the source layer saw (other rows than this layer's)
        kv = None
        if src is not None:
            kv = O.attention_keys_values(torch.from_numpy(xs).double(), t64(O.sub(w, f"l{src}.mix.")), cfg["layers"][src]["mixer"], eps)
        want = O.attention(torch.from_numpy(x).double(), t64(O.sub(w, f"l{li}.mix.")), L["mixer"], eps, kv)[0].numpy()
        for cuts in ([n], [5, 1, 1, 9, 2, 5], [1] * n):
            s = m.admit()
            got, a = [], 0
            for c in cuts:
                if src is not None:                           # the source layer writes its cache rows first, as in a step
                    m.engine.run_part(src, 2, [s], [c], xs[a:a + c])
                    m.engine.set_length(s, a)
                got.append(m.engine.run_part(li, 2, [s], [c], x[a:a + c]))
                a += c
            m.release(s)
            err = rel_err(np.concatenate(got), want)
            assert err.max() < (TOL[dtype] if dtype == "float32" else 3e-2), (name, li, cuts[:3], int(err.argmax()), err.max())
        m.close()


def test_attention_parts_matter():
    """The oracle itself reacts to each part of the mixer, so agreement with it checks each: gate, distance penalty, value norm,
    key norm, grouping of the heads."""
    cfg = CONFIGS["mixed"]
    w = t64(make_weights(cfg, 11))
    mx, P = cfg["layers"][0]["mixer"], O.sub(w, "l0.mix.")
    x = torch.from_numpy(_rows(23, 48, 5)).double()
    base = O.attention(x, P, mx, 2e-5)[0]
    assert (O.attention(x, dict(P, g=P["g"] * 0), mx, 2e-5)[0] - base).abs().max() > 1e-2
    assert (O.attention(x, P, dict(mx, scale=mx["scale"] * 1.1), 2e-5)[0] - base).abs().max() > 1e-3
    assert (O.attention(x, P, mx, 1e-1)[0] - base).abs().max() > 1e-3
    swapped = dict(P, q=P["q"].reshape(4, 16, 48)[[0, 2, 1, 3]].reshape(64, 48))     # heads 1 and 2 use different key/value heads
    assert (O.attention(x, swapped, mx, 2e-5)[0] - base).abs().max() > 1e-2
    assert abs(float(O.head_slopes(4)[0]) - 0.25) < 1e-12 and abs(float(O.head_slopes(4)[3]) - 2.0 ** -8) < 1e-12


@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "thin"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forwards_alone(name, dtype):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 21)
    m = build(cfg, w, dtype, max_step_tokens=256)
    for li, L in enumerate(cfg["layers"]):
        if L["mlp"] is None:
            continue
        for n in (1, 7, 150):                               # per-pair expert path, and the sorted grouped path
            x = _rows(n, cfg["width"], 22 + li + n, scale=2.0)     # large enough that the clamps act
            want = O.feed_forward(torch.from_numpy(x).double(), t64(O.sub(w, f"l{li}.mlp.")), L["mlp"]).numpy()
            s = m.admit()
            got = m.engine.run_part(li, 3, [s], [n], x)
            m.release(s)
            if dtype == "float32":
                assert rel_err(got, want).max() < TOL[dtype], (name, li, n)
            else:
                assert np.median(rel_err(got, want)) < 3e-2, (name, li, n)
    m.close()


def test_clamped_unit_limits():
    g = torch.tensor([-5.0, 0.5, 3.0, 9.0], dtype=torch.float64)
    u = torch.tensor([-7.0, 0.25, 1.0, 4.0], dtype=torch.float64)
    y = O.clamped_glu(g, u, 2.0)
    gc, uc = torch.tensor([-5.0, 0.5, 2.0, 2.0]), torch.tensor([-2.0, 0.25, 1.0, 2.0])
    assert torch.allclose(y, (gc * torch.sigmoid(1.702 * gc) * (uc + 1)).double())


def test_router_choice_rules():
    """Engine against hand-made router inputs: the correction moves the choice but not the weight; a group is ranked by the SUM of its two
    best choice scores (not by its best); experts of dropped groups are never chosen even when every kept choice score is negative;
    weights are the chosen sigmoid scores over their sum, times the scale."""
    f = moe(experts=8, top=3, count=4, keep=2, ff=4, scale=1.5, shared=None)
    z = torch.tensor([[3.0, -4.0, 2.0, 2.1, -9.0, -9.0, 1.9, 1.8],        # group 0 has the best single score, groups 1 and 3 the best pairs
                      [-3.0, -3.5, -9.0, -9.0, -4.0, -3.2, -9.0, -9.0]], dtype=torch.float64)
    ids, wts = O.route(z, torch.zeros(8, dtype=torch.float64), 3, 4, 2, 1.5)
    assert sorted(ids[0].tolist()) == [2, 3, 6]
    assert sorted(ids[1].tolist()) == [0, 1, 5]
    s = torch.sigmoid(z[0, [2, 3, 6]])
    assert torch.allclose(wts[0].sort().values, (s / s.sum() * 1.5).sort().values)
    corr = torch.tensor([0, 0, 0, 0, 0, 0, 0, 0.5], dtype=torch.float64)
    ids2, wts2 = O.route(z, corr, 3, 4, 2, 1.5)
    assert sorted(ids2[0].tolist()) == [2, 3, 7]
    k = ids2[0].tolist().index(7)
    s2 = torch.sigmoid(z[0, ids2[0]])
    assert abs(float(wts2[0, k]) - float(s2[k] / s2.sum() * 1.5)) < 1e-12        # from sigmoid(z) alone
    # negative choice scores everywhere: with a large negative correction the kept groups' experts are still the only candidates
    ids3, _ = O.route(z, torch.full((8,), -2.0, dtype=torch.float64), 3, 4, 2, 1.5)
    assert sorted(ids3[0].tolist()) == [2, 3, 6]
    # the engine's router on the same logits: a width-8 model whose router matrix is the identity, so that z = h
    cfg = config([with_ff(attn(heads=1, kv_heads=1, dim=8, vdim=8), f)], width=8, vocab=9)
    for correction in (np.zeros(8, np.float32), corr.numpy().astype(np.float32), np.full(8, -2.0, np.float32)):
        w = make_weights(cfg, 31)
        w["l0.mlp.router"] = np.eye(8, dtype=np.float32)
        w["l0.mlp.correction"] = correction
        m = build(cfg, w, "float32")
        x = z.numpy().astype(np.float32)
        want = O.feed_forward(torch.from_numpy(x).double(), t64(O.sub(w, "l0.mlp.")), f).numpy()
        s = m.admit()
        got = m.engine.run_part(0, 3, [s], [2], x)
        assert rel_err(got, want).max() < TOL["float32"]
        m.close()


def test_router_reads_the_unrounded_stream():
    """bfloat16 engine: two router logits that differ by less than bfloat16 resolves (1 and 1 + 2^-9, the larger at the higher index).  The
    router multiplies the float stream in float, so the larger one wins; on the rounded input they would tie and the lower index would."""
    f = moe(experts=8, top=1, count=1, keep=1, ff=8, shared=None)
    cfg = config([with_ff(attn(heads=1, kv_heads=1, dim=8, vdim=8), f)], width=8, vocab=9)
    w = make_weights(cfg, 35)
    w["l0.mlp.router"] = np.eye(8, dtype=np.float32)
    w["l0.mlp.correction"] = np.zeros(8, np.float32)
    x = np.zeros((9, 8), np.float32)
    x[:, 3] = 1.0
    x[:, 6] = 1.0 + 2.0 ** -9
    ids, _ = O.route(torch.from_numpy(x).double(), torch.zeros(8, dtype=torch.float64), 1, 1, 1, f["router"]["scale"])
    assert ids[:, 0].tolist() == [6] * 9
    want = O.feed_forward(torch.from_numpy(x).double(), t64(O.sub(w, "l0.mlp.")), f).numpy()
    tipped = x.copy()
    tipped[:, 3] += 2.0 ** -7                                  # what choosing expert 3 instead would give
    other = O.feed_forward(torch.from_numpy(tipped).double(), t64(O.sub(w, "l0.mlp.")), f).numpy()
    assert rel_err(other, want).min() > 0.3
    m = build(cfg, w, "bfloat16")
    for n in (1, 9):                                           # few-row product, and the plain FMA product
        s = m.admit()
        got = m.engine.run_part(0, 3, [s], [n], x[:n])
        m.release(s)
        assert rel_err(got, want[:n]).max() < 3e-2, n
    m.close()


# ---------------------------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "thin"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_decode_and_portions_agree_with_the_oracle(name, dtype):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 41)
    m = build(cfg, w, dtype)
    n = 37
    toks = tokens_for(cfg, n, 42)
    want = oracle_logits(cfg, w, toks)
    for cuts in ([n], [1] * n, [20] + [1] * 17, [2, 2, 3, 16, 2, 1, 4, 4, 3], [4] * 9 + [1], [7, 30]):
        assert sum(cuts) == n
        assert_close(run_alone(m, toks, cuts), want, dtype, (name, cuts[:4]))
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_streams_and_first_positions(dtype):
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 51)
    m = build(cfg, w, dtype)
    for n in (1, 2, 3, 5):
        toks = tokens_for(cfg, n, 52 + n)
        logits, taps = O.forward(toks, t64(w), cfg)
        s = m.admit()
        got, tap = m.engine.step_with_layer_tap([s], [n], toks, list(range(n)))
        m.release(s)
        assert_close(got, logits.numpy(), dtype, n)
        if dtype == "float32":
            assert np.abs(tap - taps.numpy()).max() < 1e-4
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_equal_each_request_alone(dtype):
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 61)
    m = build(cfg, w, dtype, max_tokens=256, slots=4)
    reqs = [tokens_for(cfg, n, 62 + n) for n in (31, 9, 18, 2)]
    want = [oracle_logits(cfg, w, r) for r in reqs]
    plan = [[(0, 5), (1, 2)], [(0, 1), (1, 1), (2, 7)], [(0, 9), (2, 1), (3, 2)], [(1, 6), (2, 10)], [(0, 16)]]
    slots = [m.admit() for _ in reqs]
    fed = [0] * 4
    got = [[] for _ in reqs]
    for step in plan:
        sl, cn, tk, wn = [], [], [], []
        for r, c in step:
            sl.append(slots[r]); cn.append(c); tk += reqs[r][fed[r]:fed[r] + c]
        out = m.step(sl, cn, tk, list(range(len(tk))))
        a = 0
        for r, c in step:
            got[r].append(out[a:a + c]); a += c; fed[r] += c
    for r in range(4):
        assert fed[r] == len(reqs[r])
        assert_close(np.concatenate(got[r]), want[r], dtype, r)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_are_used_again(dtype):
    """Six requests through a pool of 10 pages and 2 slots; a neighbour fills pages in between, so a request that read a stale row or
    a page of its predecessor would differ from the oracle."""
    cfg = CONFIGS["odd"]
    w = make_weights(cfg, 71)
    m = build(cfg, w, dtype, max_tokens=40, slots=2, page_size=4)
    for k in range(6):
        toks = tokens_for(cfg, 9 + 3 * (k % 3), 72 + k)
        other = m.admit()
        m.step([other], [5], tokens_for(cfg, 5, 90 + k), [])
        s = m.admit()
        assert s >= 0
        a, got = 0, []
        for c in (4, 1, len(toks) - 5):
            got.append(m.step([s, other], [c, 1], toks[a:a + c] + [k % cfg["vocab"]], list(range(c))))
            a += c
        assert_close(np.concatenate(got), oracle_logits(cfg, w, toks), dtype, k)
        m.release(s)
        m.release(other)
        assert m.free_pages() == 10 and m.free_slots() == 2
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 63, 64, 65, 127, 128])
def test_far_key_among_hundreds(dtype, far):
    """One key far back is made the only one the last query looks at: query and key projections read the first 16 input coordinates,
    which are zero in every row but the far one and the last.  Its score is dim * scale, all others are the (negative) distance penalty, so
    the output of the last position is that key's value; a lost page, a wrong slot in the page or a key cut off at a page border (pages
    of 64 tokens, far key at both sides of two borders) shows as an error of order 1.  The last token is decoded alone."""
    cfg = config([attn(heads=2, kv_heads=1, dim=16, vdim=24, scale=1.0)], width=40, vocab=20)
    w = make_weights(cfg, 81)
    sel = np.zeros((16, 40), np.float32)
    sel[np.arange(16), np.arange(16)] = 1.0
    w["l0.mix.q"] = np.concatenate([sel, sel])
    w["l0.mix.k"] = sel.copy()
    for b in ("q", "k"):
        w[f"l0.mix.{b}.b"] = np.zeros_like(w[f"l0.mix.{b}.b"])
    n = 400
    x = _rows(n, 40, 82)
    x[:, :16] = 0
    u = bf16_exact(np.random.default_rng(83).standard_normal(16))
    x[far, :16] = u
    x[n - 1, :16] = u
    P, mx = t64(O.sub(w, "l0.mix.")), cfg["layers"][0]["mixer"]
    want = O.attention(torch.from_numpy(x).double(), P, mx, 2e-5)[0].numpy()
    blind = x.copy()
    blind[far, :16] = 0
    assert rel_err(O.attention(torch.from_numpy(blind).double(), P, mx, 2e-5)[0].numpy()[-1:], want[-1:])[0] > 0.1
    m = build(cfg, w, dtype, max_tokens=512, slots=2, page_size=64, max_step_tokens=256)
    s = m.admit()
    got, a = [], 0
    for c in (130, 2, 200, 67, 1):
        got.append(m.engine.run_part(0, 2, [s], [c], x[a:a + c]))
        a += c
    err = rel_err(np.concatenate(got), want)
    assert err[-1] < (TOL[dtype] if dtype == "float32" else 2e-2), err[-1]
    assert err.max() < (TOL[dtype] if dtype == "float32" else 5e-2)
    m.close()


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(8, 2, 64, 64), (3, 3, 128, 128), (16, 1, 32, 96), (12, 4, 72, 40), (2, 1, 8, 24)])
def test_attention_on_tensor_cores_prompts_decoding_and_key_splits(heads, kv_heads, dim, vdim):
    """Sizes the tensor-core kernel takes (group sizes 1, 3, 4, 16 and 2; per-head sizes that fill or do not fill its 64 / 128 wide tiles):
    three sequences of unequal length read as prompt portions in one ragged batch (the prompt form, tiles that end inside a sequence), then
    decoded together one token each for a few steps in a pool large enough that the key range is cut over several CTAs (the decode form
    with its merge), all against the oracle."""
    cfg = config([attn(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=2.0 / math.sqrt(dim))], width=64, vocab=20)
    w = make_weights(cfg, 121)
    P, mx = t64(O.sub(w, "l0.mix.")), cfg["layers"][0]["mixer"]
    lens = (333, 70, 129)
    xs = [_rows(n + 4, 64, 122 + n) for n in lens]
    want = [O.attention(torch.from_numpy(x).double(), P, mx, 2e-5)[0].numpy() for x in xs]
    m = build(cfg, w, "bfloat16", max_tokens=4096, slots=4, page_size=16, max_step_tokens=512)
    slots = [m.admit() for _ in lens]
    got = [[] for _ in lens]
    fed = [0, 0, 0]
    for counts in ((200, 70, 100), (133, 0, 29)):
        act = [k for k in range(3) if counts[k]]
        out = m.engine.run_part(0, 2, [slots[k] for k in act], [counts[k] for k in act], np.concatenate([xs[k][fed[k]:fed[k] + counts[k]] for k in act]))
        a = 0
        for k in act:
            got[k].append(out[a:a + counts[k]]); a += counts[k]; fed[k] += counts[k]
    for _ in range(4):
        out = m.engine.run_part(0, 2, slots, [1, 1, 1], np.stack([xs[k][fed[k]] for k in range(3)]))
        for k in range(3):
            got[k].append(out[k:k + 1]); fed[k] += 1
    for k in range(3):
        err = rel_err(np.concatenate(got[k]), want[k])
        assert err.max() < 3e-2, (k, int(err.argmax()), err.max())
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_page_borders(dtype):
    cfg = CONFIGS["thin"]
    w = make_weights(cfg, 91)
    m = build(cfg, w, dtype, max_tokens=256, slots=2, page_size=4)
    n = 150
    toks = tokens_for(cfg, n, 92)
    assert_close(run_alone(m, toks, [6] + [1] * (n - 6)), oracle_logits(cfg, w, toks), dtype, "long")
    m.close()


def test_greedy_generation_through_the_scheduler():
    from wf_bitnet.scheduler import Request, Scheduler
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 101)
    m = build(cfg, w, "float32", max_tokens=96, slots=2, page_size=4, max_step_tokens=16)
    sched = Scheduler(m, max_prefill_chunk=5)
    prompts = [tokens_for(cfg, n, 102 + n) for n in (11, 3, 17, 6, 1)]
    for i, p in enumerate(prompts):
        sched.add(Request(f"r{i}", p, max_new_tokens=6))
    done = {r.rid: r for r in sched.run()}
    assert len(done) == 5 and m.free_slots() == 2
    for i, p in enumerate(prompts):
        seq = list(p)
        for t in done[f"r{i}"].output:
            lg = oracle_logits(cfg, w, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if top2[1] - top2[0] > 1e-3 * np.abs(lg).max():
                assert int(np.argmax(lg)) == t
            seq.append(t)
    m.close()


def _write_model_dir(path, cfg, weights):
    import struct
    header, blob = {}, b""
    for name, a in weights.items():
        a = np.asarray(a, dtype=np.float32)
        raw = torch.from_numpy(a.copy()).to(torch.bfloat16).view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header).encode()
    (path / "config.json").write_text(json.dumps(cfg))
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + blob)


def test_command_line_trace_replay_and_generate(tmp_path):
    """`trace` (bin/trace_run) replays a schedule with mixed batches, a pause, and a finished request whose slot and pages go to the next
    one; `generate` runs the scheduler.  The model class comes from config.json.  Both against the oracle."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 111)
    _write_model_dir(tmp_path, cfg, w)
    reqs = {"a": tokens_for(cfg, 21, 112), "b": tokens_for(cfg, 9, 113), "c": tokens_for(cfg, 14, 114)}
    want = {k: oracle_logits(cfg, w, v) for k, v in reqs.items()}
    plan = [[("a", 6)], [("a", 1), ("b", 8)], [("a", 10), ("b", 1)], [("a", 4)], [("c", 2)], [("c", 11)], [("c", 1)]]
    fed, lines, expect = {k: 0 for k in reqs}, [], []
    for n, step in enumerate(plan):
        ents, end, rows = [], [], []
        for rid, c in step:
            ents.append({"id": rid, "tokens": reqs[rid][fed[rid]:fed[rid] + c], "want": list(range(c))})
            rows += [(rid, fed[rid] + k) for k in range(c)]
            fed[rid] += c
            if fed[rid] == len(reqs[rid]):
                end.append(rid)
        lines.append(json.dumps({"step": n, "entries": ents, "end": end}))
        expect.append(rows)
    out = tmp_path / "out"
    out.mkdir()
    for dtype in ("float32", "bfloat16"):
        r = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", dtype, "--out", str(out), "--max-tokens", "64", "--slots", "2"],
                           input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
        for n, rows in enumerate(expect):
            got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"])
            assert_close(got, np.stack([want[rid][pos] for rid, pos in rows]), dtype, n)
    r = subprocess.run([sys.executable, "-m", "wf_bitnet.cli", "generate", "--model", str(tmp_path), "--dtype", "float32", "--max-new-tokens", "5",
                        "--prompt-ids", ",".join(map(str, reqs["a"])), "--prompt-ids", ",".join(map(str, reqs["b"])), "--slots", "1", "--prefill-chunk", "4"],
                       capture_output=True, text=True, timeout=600, env=dict(__import__("os").environ, PYTHONPATH=str(root / "wrinklefree-inference-engine_b200")))
    assert r.returncode == 0, r.stderr[-2000:]
    outs = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert [o["id"] for o in outs] == ["r0", "r1"]
    for o, rid in zip(outs, ("a", "b")):
        seq = list(reqs[rid])
        for t in o["output_ids"]:
            lg = oracle_logits(cfg, w, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if top2[1] - top2[0] > 1e-3 * np.abs(lg).max():
                assert int(np.argmax(lg)) == t
            seq.append(t)
