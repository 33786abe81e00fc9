"""Karusun on the native sequence engine against the plain oracle (tests/karusun_oracle.py): every mechanism alone, then whole models
through prompts, decoding, portions, mixed batches, reused slots and pages, and the scheduler.  Configurations and weights are made here."""
import math

import numpy as np
import pytest
import torch

import karusun_oracle as O

pytestmark = pytest.mark.gpu

LAT = "latent_attention"


def lat(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, window=6, scale=None, base=10000.0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    return {"type": LAT, "mixer": m}


def delta(heads=2, kv_heads=1, dim=16, vdim=24, conv=3):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def moe(experts=6, identity=2, top=3, count=4, keep=2, ff=20):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": count, "keep": keep}}}


def config(layers, width=48, vocab=70, groups=2, taps=3, eps=1e-6):
    return {"architecture": "Karusun", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "canon": {"taps": taps}, "layers": layers}


def with_ff(layer, ff):
    return dict(layer, mlp=ff)


def bf16_exact(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def make_weights(cfg, seed):
    """name -> float32 array whose values are exactly representable in bfloat16 (so both engine dtypes hold the same model)."""
    rng = np.random.default_rng(seed)
    W, w = cfg["width"], {}

    def lin(o, i, gain=1.0):
        return bf16_exact(rng.standard_normal((o, i)) * gain / math.sqrt(i))

    def near_one(n):
        return bf16_exact(1.0 + 0.2 * rng.standard_normal(n))
    w["embed"] = bf16_exact(rng.standard_normal((cfg["vocab"], W)))
    w["final.norm"] = near_one(W)
    w["head"] = lin(cfg["vocab"], W)
    taps = cfg["canon"]["taps"]
    for li, L in enumerate(cfg["layers"]):
        p, m = f"l{li}.", L["mixer"]
        for nm in ("norm1", "norm1b"):
            w[p + nm] = near_one(W)
        w[p + "canon1"] = bf16_exact(0.4 * rng.standard_normal((W, taps)))
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == LAT:
            r, R = m["rot_dim"], m["kv_rank"]
            w[p + "mix.q"] = lin(H * (d + r), W, 2.0)
            w[p + "mix.dkv"] = lin(R + r, W, 2.0)
            w[p + "mix.dkv.norm"] = near_one(R)
            w[p + "mix.uk"] = lin(H * d, R, 2.0)
            w[p + "mix.uv"] = lin(H * dv, R)
            w[p + "mix.g"] = lin(H * dv, W)
        else:
            Hk, c = m["kv_heads"], m["conv"]
            for nm, rows in (("q", Hk * d), ("k", Hk * d), ("v", H * dv)):
                w[p + f"mix.{nm}"] = lin(rows, W, 1.5)
                w[p + f"mix.{nm}.conv"] = bf16_exact(0.5 * rng.standard_normal((rows, c)))
            w[p + "mix.b"] = lin(H, W, 2.0)
            w[p + "mix.a"] = lin(H, W, 2.0)
            w[p + "mix.A_log"] = bf16_exact(rng.uniform(-2.0, 0.5, H))
            w[p + "mix.dt_bias"] = bf16_exact(rng.standard_normal(H))
            w[p + "mix.norm"] = near_one(dv)
            w[p + "mix.g"] = lin(H * dv, W)
        w[p + "mix.o"] = lin(W, H * dv)
        f = L.get("mlp")
        if f is not None:
            for nm in ("norm2", "norm2b"):
                w[p + nm] = near_one(W)
            w[p + "canon2"] = bf16_exact(0.4 * rng.standard_normal((W, taps)))
            r = f["router"]
            N = r["experts"] + r.get("identity", 0)
            w[p + "mlp.router"] = lin(N, W, 3.0)
            w[p + "mlp.correction"] = bf16_exact(0.05 * rng.standard_normal(N))
            for e in range(r["experts"]):
                w[p + f"mlp.e{e}.gate"] = lin(f["expert"]["ff"], W, 1.5)
                w[p + f"mlp.e{e}.up"] = lin(f["expert"]["ff"], W, 1.5)
                w[p + f"mlp.e{e}.down"] = lin(W, f["expert"]["ff"], 1.5)
    return w


def build(cfg, weights, dtype="float32", max_tokens=256, slots=4, page_size=4, max_step_tokens=64):
    from wf_bitnet import registry
    cls = registry.resolve(cfg)
    model = cls(cfg, dtype=dtype, max_tokens=max_tokens, slots=slots, page_size=page_size, max_step_tokens=max_step_tokens)
    model.load_weights((k, v, "F32") for k, v in weights.items())
    return model


def oracle_logits(cfg, weights, tokens):
    w64 = {k: torch.from_numpy(v).double() for k, v in weights.items()}
    return O.forward(cfg, w64, list(tokens)).numpy()


def rel_err(got, want):
    """per row: RMS of the difference (mean taken off) over the RMS of the expected row"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / (np.sqrt((want ** 2).mean(-1)) + 1e-12)


TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def assert_close(got, want, dtype, what, f32_tol=None):
    """float32: every row within tolerance.  bfloat16: a router whose two best scores nearly tie may choose the other expert after
    rounding, which moves that position (and what later positions read from it) by far more than rounding does; such positions are
    few, so most rows must be within tolerance and the typical row well inside it."""
    err = rel_err(got, want)
    if dtype == "float32":
        assert err.max() < (f32_tol or TOL[dtype]), (what, int(err.argmax()), err.max())
    else:                                   # models this narrow (tens of channels) average little rounding noise away
        assert (err < 2.5 * TOL[dtype]).mean() >= 0.8 and np.median(err) < TOL[dtype], (what, int(err.argmax()), err.max(), np.median(err))

CFG_MIXED = config([with_ff(lat(window=6), moe()), with_ff(delta(), moe(experts=4, identity=0, top=1, count=2, keep=1, ff=12)), lat(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, window=9)],
                   width=48, vocab=70, groups=2, taps=3)
CFG_ODD = config([with_ff(delta(heads=4, kv_heads=2, dim=12, vdim=8, conv=2), moe(experts=3, identity=1, top=2, count=1, keep=1, ff=10)),
                  with_ff(lat(heads=1, dim=12, rot_dim=6, vdim=20, kv_rank=40, window=5, base=100.0), moe(experts=8, identity=0, top=2, count=4, keep=4, ff=8))],
                 width=40, vocab=33, groups=1, taps=4)
CFG_WIDE = config([with_ff(lat(heads=2, dim=32, rot_dim=32, vdim=32, kv_rank=64, window=40), moe(experts=8, identity=2, top=3, count=5, keep=3, ff=48)),
                   with_ff(delta(heads=2, kv_heads=2, dim=72, vdim=40, conv=4), moe(experts=8, identity=2, top=3, count=5, keep=3, ff=48))],
                  width=128, vocab=150, groups=4, taps=2)
# nothing here is a multiple of 8: rows of every matrix start unaligned, so the vector / TMA forms of the products must step aside
CFG_THIN = config([with_ff(lat(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=22, window=7), moe(experts=5, identity=1, top=2, count=3, keep=2, ff=13)),
                   with_ff(delta(heads=3, kv_heads=3, dim=10, vdim=14, conv=3), moe(experts=2, identity=2, top=2, count=2, keep=2, ff=9))],
                  width=36, vocab=31, groups=3, taps=3)
CONFIGS = {"mixed": CFG_MIXED, "odd": CFG_ODD, "wide": CFG_WIDE, "thin": CFG_THIN}


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


# ---------------------------------------------------------------------------------------------------------------- mechanisms alone
def _rows(n, W, seed, scale=1.0):
    return bf16_exact(np.random.default_rng(seed).standard_normal((n, W)) * scale)


@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_and_input_convolution(name, dtype):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 1)
    m = build(cfg, w, dtype)
    W, n = cfg["width"], 11
    x = _rows(n, W, 2, 3.0)
    s = m.admit()
    got = m.engine.run_part(0, 0, [s], [n], x)
    want = O.group_rms_norm(torch.from_numpy(x).double(), torch.from_numpy(w["l0.norm1"]).double(), cfg["norm"]["groups"], cfg["norm"]["eps"]).numpy()
    assert np.abs(got - want).max() < 1e-5 * (1 + np.abs(want).max())
    m.release(s)
    # the convolution in three portions (1, 2 and the rest) must equal the whole: its tail is carried in the slot
    s = m.admit()
    want = O.input_conv(torch.from_numpy(x).double(), torch.from_numpy(w["l0.canon1"]).double()).numpy()
    parts = [m.engine.run_part(0, 1, [s], [c], x[a:a + c]) for a, c in ((0, 1), (1, 2), (3, n - 3))]
    assert np.abs(np.concatenate(parts) - want).max() < 1e-5 * (1 + np.abs(want).max())
    m.close()


@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixers_alone(name, dtype):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 3)
    m = build(cfg, w, dtype)
    W, n = cfg["width"], 23
    x = _rows(n, W, 4)
    for li, L in enumerate(cfg["layers"]):
        P = {k: torch.from_numpy(v).double() for k, v in O.sub(w, f"l{li}.mix.").items()}
        fn = O.latent_attention if L["type"] == LAT else O.gated_delta
        want = fn(torch.from_numpy(x).double(), P, L["mixer"], cfg["norm"]["eps"]).numpy()
        for cuts in ([n], [5, 1, 1, 2, n - 9]):            # whole, and in portions through the cache / state
            s = m.admit()
            got, a = [], 0
            for c in cuts:
                got.append(m.engine.run_part(li, 2, [s], [c], x[a:a + c]))
                a += c
            m.release(s)
            err = rel_err(np.concatenate(got), want).max()
            assert err < TOL[dtype], (name, li, L["type"], cuts, err)
    m.close()


@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_alone(name, dtype):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 5)
    m = build(cfg, w, dtype)
    W, n = cfg["width"], 37
    x = _rows(n, W, 6)
    for li, L in enumerate(cfg["layers"]):
        if L.get("mlp") is None:
            continue
        P = {k: torch.from_numpy(v).double() for k, v in O.sub(w, f"l{li}.mlp.").items()}
        want = O.moe(torch.from_numpy(x).double(), P, L["mlp"]).numpy()
        s = m.admit()
        got = m.engine.run_part(li, 3, [s], [n], x)
        m.release(s)
        # a token whose router scores nearly tie may legitimately choose another expert in reduced precision: compare the others
        err = rel_err(got, want)
        ok = err < TOL[dtype]
        assert ok.mean() >= (1.0 if dtype == "float32" else 0.9), (name, li, err.max())
    m.close()


def test_router_choice_rules():
    """correction changes the choice but not the weight; experts of dropped groups are never chosen even when scores are negative."""
    cfg = config([with_ff(lat(), moe(experts=6, identity=2, top=2, count=4, keep=2, ff=12))], width=32, vocab=20)
    w = make_weights(cfg, 7)
    w["l0.mlp.correction"] = bf16_exact(np.array([-3.0, -3.0, 2.0, -3.0, -3.0, -3.0, -3.0, 1.0]))   # groups (0,1) (2,3) (4,5) (6,7)
    m = build(cfg, w, "float32")
    x = _rows(9, 32, 8)
    P = {k: torch.from_numpy(v).double() for k, v in O.sub(w, "l0.mlp.").items()}
    idx, _ = O.route(torch.from_numpy(x).double(), P, cfg["layers"][0]["mlp"]["router"])
    assert set(idx.flatten().tolist()) <= {2, 3, 6, 7} and (idx == 7).any()     # kept groups only; an identity expert is in use
    want = O.moe(torch.from_numpy(x).double(), P, cfg["layers"][0]["mlp"]).numpy()
    s = m.admit()
    got = m.engine.run_part(0, 3, [s], [9], x)
    assert rel_err(got, want).max() < 2e-4
    m.close()


# ---------------------------------------------------------------------------------------------------------------- whole models
def run_alone(m, tokens, cuts):
    """one request through the engine in portions `cuts`; logits of every position"""
    s = m.admit()
    out, a = [], 0
    for c in cuts:
        out.append(m.step([s], [c], tokens[a:a + c], list(range(c))))
        a += c
    m.release(s)
    return np.concatenate(out)


@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "thin"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_decode_and_portions_agree_with_the_oracle(name, dtype):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 11)
    m = build(cfg, w, dtype, page_size=4)
    n = 53
    toks = tokens_for(cfg, n, 12)
    want = oracle_logits(cfg, w, toks)
    schedules = {
        "whole": [n],
        "token by token": [1] * n,
        "prompt then decode": [n - 20] + [1] * 20,
        "portions": [2, 7, 2, 1, 16, 3, 2, 2, 9, 1, 1, n - 46],
        "page-sized": [4] * 13 + [1],
    }
    for label, cuts in schedules.items():
        assert sum(cuts) == n
        assert_close(run_alone(m, toks, cuts), want, dtype, (name, label))
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_single_token_prompt_and_first_positions(dtype):
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 13)
    m = build(cfg, w, dtype)
    for n in (1, 2, 3, 4):
        toks = tokens_for(cfg, n, 14 + n)
        assert_close(run_alone(m, toks, [n]), oracle_logits(cfg, w, toks), dtype, n)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_equal_each_request_alone(dtype):
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 17)
    m = build(cfg, w, dtype, max_tokens=160, page_size=4, max_step_tokens=32)
    lens = [29, 3, 41, 17]
    reqs = [tokens_for(cfg, n, 20 + i) for i, n in enumerate(lens)]
    want = [oracle_logits(cfg, w, t) for t in reqs]
    # a schedule in which requests start at different steps, bring portions of unequal size beside single tokens, and pause
    plan = [
        [(0, 5)], [(0, 2), (1, 1)], [(0, 1), (1, 1), (2, 16)], [(0, 1), (2, 9), (3, 2)], [(1, 1), (2, 1), (3, 7)],
        [(0, 12), (2, 1), (3, 1)], [(0, 1), (2, 1), (3, 1)], [(0, 7), (2, 13), (3, 6)],
    ]
    slots, fed, got = {}, [0] * 4, [[] for _ in reqs]
    for step in plan:
        s_, c_, t_, w_, owner = [], [], [], [], []
        for r, c in step:
            if r not in slots:
                slots[r] = m.admit()
            s_.append(slots[r]); c_.append(c)
            base = len(t_)
            t_.extend(reqs[r][fed[r]:fed[r] + c])
            w_.extend(range(base, base + c)); owner.extend([r] * c)
            fed[r] += c
        out = m.step(s_, c_, t_, w_)
        for row, r in zip(out, owner):
            got[r].append(row)
    for r in range(4):
        assert fed[r] == lens[r]
        assert_close(np.stack(got[r]), want[r], dtype, r)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_are_used_again(dtype):
    """A pool of 8 pages and 2 slots serves six requests one after another and two at a time: stale state or cache rows would show."""
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 23)
    m = build(cfg, w, dtype, max_tokens=32, slots=2, page_size=4, max_step_tokens=32)
    assert m.free_pages() == 8 and m.free_slots() == 2
    for i, n in enumerate((15, 16, 9, 13, 16, 5)):
        toks = tokens_for(cfg, n, 30 + i)
        other = tokens_for(cfg, 11, 40 + i)
        s2 = m.admit()
        m.step([s2], [len(other)], other)                      # a neighbour that dirties pages and a slot
        got = run_alone(m, toks, [n // 2, n - n // 2])
        m.release(s2)
        assert_close(got, oracle_logits(cfg, w, toks), dtype, i)
        assert m.free_pages() == 8 and m.free_slots() == 2
    with pytest.raises(ValueError):                            # more than the pool holds: refused, nothing kept
        s = m.admit()
        m.step([s], [32], tokens_for(cfg, 32, 1))
        m.step([s], [1], [0])
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edges_far_keys_and_long_decoding(dtype):
    """Sharp softmax (large score scale): single keys dominate, at every distance inside the window, so a window that is one token off,
    a wrong page or a wrong slot in a page changes the logits outright.  Page size 4 and windows 6 / 37 put edges inside pages, on
    page borders and many pages back; decoding runs for three windows."""
    cfg = config([with_ff(lat(window=6, scale=1.5), moe()), lat(heads=1, dim=8, rot_dim=8, vdim=8, kv_rank=16, window=37, scale=2.0), delta()], width=48, vocab=50)
    w = make_weights(cfg, 29)
    m = build(cfg, w, dtype, max_tokens=160, page_size=4, max_step_tokens=160)
    n = 131
    toks = tokens_for(cfg, n, 31)
    want = oracle_logits(cfg, w, toks)
    # the oracle itself must be sensitive: shrinking either window by one token moves the logits far beyond the tolerance
    for li in (0, 1):
        c2 = config([dict(L, mixer=dict(L["mixer"], mask={"size": L["mixer"]["mask"]["size"] - 1})) if i == li else L for i, L in enumerate(cfg["layers"])], width=48, vocab=50)
        assert rel_err(oracle_logits(c2, w, toks), want).max() > 0.3
    for cuts in ([n], [20] + [1] * 111, [3, 37, 2, 38, 36, 1, 1, 1, 12]):
        assert_close(run_alone(m, toks, cuts), want, dtype, cuts[:3], f32_tol=1e-3)   # sharp softmax amplifies rounding too
    m.close()


def test_far_key_among_hundreds():
    """Window 300, one key made to dominate from 290 tokens back: the value it carries must arrive."""
    cfg = config([lat(heads=1, dim=8, rot_dim=0, vdim=8, kv_rank=16, window=300, scale=6.0)], width=32, vocab=40, groups=1, taps=1)
    cfg["layers"][0]["mixer"]["rot"] = {"base": 10000.0, "dims": 0}
    w = make_weights(cfg, 37)
    m = build(cfg, w, "float32", max_tokens=512, page_size=16, max_step_tokens=128)
    n = 310
    x = _rows(n, 32, 38, 0.05)
    x[5] = _rows(1, 32, 39, 4.0)[0]                       # the key 290 .. 299 tokens back for the last queries
    x[300:] = x[5] * 0.9 + x[300:]                         # queries aligned with it
    P = {k: torch.from_numpy(v).double() for k, v in O.sub(w, "l0.mix.").items()}
    want = O.latent_attention(torch.from_numpy(x).double(), P, cfg["layers"][0]["mixer"], 1e-6).numpy()
    s = m.admit()
    got = np.concatenate([m.engine.run_part(0, 2, [s], [c], x[a:a + c]) for a, c in ((0, 128), (128, 128), (256, 44), (300, 1), (301, 9))])
    assert rel_err(got, want).max() < 2e-4
    # position 304 still sees key 5 (distance 299), position 305 does not
    assert np.abs(want[304] - want[305]).max() > 1e-2
    m.close()


def test_greedy_generation_through_the_scheduler():
    from wf_bitnet.scheduler import Request, Scheduler
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 41)
    m = build(cfg, w, "float32", max_tokens=96, slots=2, page_size=4, max_step_tokens=16)
    prompts = [tokens_for(cfg, n, 50 + i) for i, n in enumerate((19, 4, 11, 7, 2))]
    sched = Scheduler(m, max_prefill_chunk=6)
    for i, p in enumerate(prompts):
        sched.add(Request(f"r{i}", p, max_new_tokens=9))
    done = {r.rid: r for r in sched.run()}
    assert len(done) == 5 and m.free_slots() == 2 and m.free_pages() == 24
    for i, p in enumerate(prompts):
        seq = list(p)
        for t in done[f"r{i}"].output:
            lg = oracle_logits(cfg, w, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if top2[1] - top2[0] > 1e-3 * np.abs(lg).max():     # not a near tie
                assert int(np.argmax(lg)) == t, (i, len(seq))
            seq.append(t)
    m.close()


def test_sampling_kernel():
    cfg = CONFIGS["odd"]
    w = make_weights(cfg, 43)
    m = build(cfg, w, "float32")
    toks = tokens_for(cfg, 6, 44)
    s = m.admit()
    lg = m.step([s], [6], toks, list(range(6)))
    assert (m.sample(6, 0.0) == lg.argmax(-1)).all()
    # top_k = 1 and a tiny top_p are greedy whatever the draw; a full draw follows the distribution
    u = np.linspace(0.01, 0.99, 6).astype(np.float32)
    assert (m.sample(6, 1.0, 1, 1.0, u) == lg.argmax(-1)).all()
    assert (m.sample(6, 1.0, 0, 1e-6, u) == lg.argmax(-1)).all()
    p = torch.softmax(torch.from_numpy(lg[0]).double() / 0.7, -1).numpy()
    cdf = np.cumsum(p)
    for uu in (0.03, 0.31, 0.62, 0.97):
        got = int(m.sample(1, 0.7, 0, 1.0, np.array([uu], dtype=np.float32))[0])
        lo = cdf[got - 1] if got else 0.0
        assert lo - 1e-4 <= uu <= cdf[got] + 1e-4
    top3 = set(np.argsort(lg[0])[-3:].tolist())
    for uu in np.linspace(0.0, 0.999, 23):
        assert int(m.sample(1, 1.5, 3, 1.0, np.array([uu], dtype=np.float32))[0]) in top3
    m.close()


def test_registry_and_config_reader():
    from wf_bitnet import registry
    cls = registry.resolve({"architecture": "Karusun"})
    assert cls.__name__ == "KarusunForCausalLM"
    assert registry.resolve({"architectures": ["BitNetForCausalLM"]}).__name__ == "BitNetForCausalLM"
    with pytest.raises(KeyError):
        registry.resolve({"architecture": "Nope"})


# ---------------------------------------------------------------------------------------------------------------- matrix products
def _gemm(dtype, A, B, M, N, K, algo, tile_group=None, group_stride=0, n_groups=1, c_f32=True):
    from wf_bitnet._lib import seq_check, seq_lib
    C_ = torch.full((M, N), float("nan"), dtype=torch.float32 if c_f32 else A.dtype, device="cuda")
    tg = tile_group.data_ptr() if tile_group is not None else None
    seq_check(seq_lib().wf_seq_op_gemm(1 if dtype == torch.bfloat16 else 0, A.data_ptr(), 1 if (A.dtype == torch.float32 and dtype == torch.bfloat16) else 0,
                                       A.stride(0), B.data_ptr(), B.stride(-2), C_.data_ptr(), 1 if c_f32 else 0, N, M, N, K, tg, group_stride, n_groups, algo,
                                       torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return C_


@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (5, 300, 200), (8, 1000, 2560), (17, 72, 48), (130, 257, 96), (300, 1000, 2560), (1100, 640, 520)])
def test_matrix_product_forms_agree(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    A = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    B = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    want = A.double() @ B.double().T
    for algo in (1, 2, 3) + ((4,) if M <= 8 else ()):
        got = _gemm(torch.bfloat16, A, B, M, N, K, algo)
        assert torch.isfinite(got).all(), algo
        assert (got.double() - want).abs().max() < 2e-3 * (1 + want.abs().max()), (algo, M, N, K)
    Af, Bf = A.float(), B.float()
    for algo in (1,) + ((4,) if M <= 8 else ()):
        got = _gemm(torch.float32, Af, Bf, M, N, K, algo)
        assert (got.double() - want).abs().max() < 1e-4 * (1 + want.abs().max()), (algo, M, N, K)
    out16 = _gemm(torch.bfloat16, A, B, M, N, K, 3, c_f32=False)
    assert (out16.double() - want).abs().max() < 2e-2 * (1 + want.abs().max())


def test_grouped_matrix_product_on_the_tensor_cores():
    E, N, K, tiles = 5, 200, 192, 9
    g = torch.Generator(device="cuda").manual_seed(3)
    A = torch.randn(tiles * 128, K, device="cuda", generator=g).to(torch.bfloat16)
    B = (torch.randn(E, N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    tg = torch.tensor([0, 0, 3, -1, 4, 1, -1, 2, 2], dtype=torch.int32, device="cuda")
    for algo in (1, 2, 3):
        got = _gemm(torch.bfloat16, A, B, tiles * 128, N, K, algo, tile_group=tg, group_stride=N * K, n_groups=E)
        for t, e in enumerate(tg.tolist()):
            rows = slice(t * 128, (t + 1) * 128)
            if e < 0:
                assert torch.isnan(got[rows]).all()          # skipped tiles are not touched
            else:
                want = A[rows].double() @ B[e].double().T
                assert (got[rows].double() - want).abs().max() < 2e-3 * (1 + want.abs().max()), (algo, t)


@pytest.mark.parametrize("heads,kv_rank,rot_dim", [(20, 128, 16), (5, 512, 32), (33, 256, 8), (7, 80, 24), (32, 48, 0)])
def test_latent_attention_on_tensor_cores_with_key_splits(heads, kv_rank, rot_dim):
    """Sizes that take the tensor-core attention kernel (latent a multiple of 32): padded head tiles, several head tiles, and a window
    long enough that single decoded tokens have their keys split over several CTAs and merged."""
    cfg = config([lat(heads=heads, dim=16, rot_dim=rot_dim, vdim=16, kv_rank=kv_rank, window=600, scale=0.5)], width=64, vocab=40, groups=1, taps=2)
    w = make_weights(cfg, 61)
    m = build(cfg, w, "bfloat16", max_tokens=768, page_size=16, max_step_tokens=256)
    n = 700
    x = _rows(n, 64, 62)
    P = {k: torch.from_numpy(v).double() for k, v in O.sub(w, "l0.mix.").items()}
    want = O.latent_attention(torch.from_numpy(x).double(), P, cfg["layers"][0]["mixer"], 1e-6).numpy()
    s = m.admit()
    cuts = [256, 256, 170, 3, 2] + [1] * 13
    got, a = [], 0
    for c in cuts:
        got.append(m.engine.run_part(0, 2, [s], [c], x[a:a + c]))
        a += c
    err = rel_err(np.concatenate(got), want)
    assert err.max() < TOL["bfloat16"], (int(err.argmax()), err.max())
    m.close()


def _write_model_dir(path, cfg, weights):
    import json
    import struct
    header, blob = {}, b""
    for name, a in weights.items():
        raw = torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header).encode()
    (path / "config.json").write_text(json.dumps(cfg))
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + blob)


def test_command_line_trace_replay_and_generate(tmp_path):
    """The two commands on a model folder written here: `trace` (bin/trace_run) replays a schedule with mixed batches, a pause, a
    finished request whose slot and pages go to the next one; `generate` runs the scheduler.  Both against the oracle."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cfg = CONFIGS["mixed"]
    w = make_weights(cfg, 71)
    _write_model_dir(tmp_path, cfg, w)
    reqs = {"a": tokens_for(cfg, 21, 72), "b": tokens_for(cfg, 9, 73), "c": tokens_for(cfg, 14, 74)}
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
    for dtype, tol in (("float32", 2e-4), ("bfloat16", None)):
        r = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", dtype, "--out", str(out), "--max-tokens", "64", "--slots", "2"],
                           input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
        for n, rows in enumerate(expect):
            got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"])
            ref = np.stack([want[rid][pos] for rid, pos in rows])
            if tol:
                assert rel_err(got, ref).max() < tol, (dtype, n)
            else:
                assert_close(got, ref, dtype, n)
    sys.path.insert(0, str(root / "wrinklefree-inference-engine_b200"))
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_delta_rule_long_memory_across_portions(dtype):
    """Decay made almost 1 (large negative A_log and dt_bias): what a token wrote 300 tokens ago is still read, so a state that is lost,
    zeroed or carried in the wrong slot at any portion border changes every later output — with quick decay it would fade unnoticed."""
    cfg = config([delta(heads=4, kv_heads=2, dim=24, vdim=40, conv=4)], width=64, vocab=40, groups=1, taps=1)
    w = make_weights(cfg, 81)
    w["l0.mix.A_log"] = bf16_exact(np.full(4, -8.0))
    w["l0.mix.dt_bias"] = bf16_exact(np.full(4, -4.0))
    m = build(cfg, w, dtype, max_tokens=512, slots=2, page_size=16, max_step_tokens=160)
    n = 300
    x = _rows(n, 64, 82)
    P = {k: torch.from_numpy(v).double() for k, v in O.sub(w, "l0.mix.").items()}
    want = O.gated_delta(torch.from_numpy(x).double(), P, cfg["layers"][0]["mixer"], 1e-6).numpy()
    # sensitivity of the oracle itself: forgetting the first 150 tokens moves the last outputs far beyond the tolerance
    late = O.gated_delta(torch.from_numpy(x[150:]).double(), P, cfg["layers"][0]["mixer"], 1e-6).numpy()
    assert rel_err(late[-20:], want[-20:]).min() > 0.1
    other = m.admit()                                            # a neighbour in the other slot, stepped in between
    s = m.admit()
    got, a = [], 0
    for c in (128, 3, 2, 1, 1, 100, 65):
        got.append(m.engine.run_part(0, 2, [s], [c], x[a:a + c]))
        m.engine.run_part(0, 2, [other], [2], _rows(2, 64, 83 + a))
        a += c
    err = rel_err(np.concatenate(got), want)
    assert err.max() < (1e-3 if dtype == "float32" else TOL[dtype]), (int(err.argmax()), err.max())
    m.close()
