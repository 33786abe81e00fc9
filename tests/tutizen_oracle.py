"""Slow plain-PyTorch statement of the Tutizen design, one function per mechanism, whole sequence at once, float64 on the CPU.

Test infrastructure only: it shares no code with the product path.  Notation: W = model width, n = tokens of ONE sequence,
positions 0..n-1.  Weights come as a dict name -> tensor with the checkpoint's names ('l<i>.mix.q', 'l<i>.mlp.e<j>.gate', ...).

The design: token embedding plus a sinusoidal position vector; every sublayer reads the residual stream itself and its OUTPUT is
normalised (RMS norm with a single gain) and added with a constant multiplier; the mixer is grouped-query softmax attention without
rotation, with unit-RMS queries, keys and values, a linear distance penalty per head, a per-head sigmoid output gate, and optionally the
cached keys / values of an earlier layer; the feed-forward is a clamped gated unit, dense or routed (sigmoid router, additive choice
correction, groups ranked by their two best choice scores) with a gated shared expert.
"""
import math

import torch


def position_vectors(positions, width, dtype=torch.float64):
    """[n, W]: entry 2i = sin(p * 10000^(-2i / W)), entry 2i + 1 = cos of the same angle."""
    e = torch.arange(width)
    i = (e // 2).to(torch.float64)
    ang = positions.to(torch.float64)[:, None] * (10000.0 ** (-2.0 * i / width))[None, :]
    return torch.where((e % 2 == 0)[None, :], torch.sin(ang), torch.cos(ang)).to(dtype)


def scalar_rms_norm(x, g, eps):
    """x / sqrt(mean(x^2) + eps) * g with ONE gain g for all coordinates."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis (no weight)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def head_slopes(H, dtype=torch.float64):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=dtype)


def attention_keys_values(h, P, m, eps):
    """The cached quantities of a layer that owns its projections: k [n, G, d] and v [n, G, dv], both already unit-RMS per head."""
    n = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ P["k"].T + P["k.b"]).reshape(n, G, d)
    v = (h @ P["v"].T + P["v.b"]).reshape(n, G, dv)
    return unit_rms(k, eps), unit_rms(v, eps)


def attention(h, P, m, eps, kv=None):
    """h [n, W]; P: this mixer's tensors by short name (q, q.b, k, k.b, v, v.b, g, o, o.b); m: the mixer's config.
    kv: (k, v) of the layer whose cache this layer reads (None: its own).  Returns (output [n, W], (k, v))."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ P["q"].T + P["q.b"]).reshape(n, H, d), eps)
    k, v = kv if kv is not None else attention_keys_values(h, P, m, eps)
    rep = H // G
    pos = torch.arange(n)
    dist = (pos[:, None] - pos[None, :]).to(h.dtype)          # i - j
    out = h.new_zeros(n, H, dv)
    slopes = head_slopes(H, h.dtype)
    for hh in range(H):
        g = hh // rep
        s = (q[:, hh] @ k[:, g].T) * m["scale"] - slopes[hh] * dist
        s = s.masked_fill(dist < 0, float("-inf"))
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    gate = torch.sigmoid(h @ P["g"].T)                         # [n, H]
    out = out * gate[:, :, None]
    return out.reshape(n, H * dv) @ P["o"].T + P["o.b"], (k, v)


def clamped_glu(g, u, limit):
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, -limit, limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


def gated_unit(h, gate, up, down, limit):
    """One feed-forward unit (dense layer, expert or shared expert): W_down (act(W_gate h, W_up h))."""
    return clamped_glu(h @ gate.T, h @ up.T, limit) @ down.T


def route(z, correction, top, groups, keep, scale):
    """z [n, E] router logits -> (ids [n, top], weights [n, top]).  Choice by sigmoid(z) + correction inside the `keep` groups whose
    two best choice scores sum highest; weights from sigmoid(z) alone, normalised over the chosen and scaled."""
    n, E = z.shape
    s = torch.sigmoid(z)
    c = s + correction
    per = E // groups
    cg = c.reshape(n, groups, per)
    gs = cg.topk(min(2, per), -1).values.sum(-1)               # [n, groups]
    best = gs.topk(keep, -1).indices
    allowed = torch.zeros(n, groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    c = cg.masked_fill(~allowed[:, :, None], float("-inf")).reshape(n, E)
    ids = c.topk(top, -1).indices
    w = s.gather(1, ids)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * scale
    return ids, w


def routed_ff(h, P, f):
    """h [n, W]; P: the feed-forward's tensors by short name (router, correction, e<j>.gate/up/down, shared.gate/up/down/sg)."""
    r = f["router"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    ids, w = route(h @ P["router"].T, P["correction"], r["top"], g["count"], g["keep"], r.get("scale", 1.0))
    out = torch.zeros_like(h)
    lim = f["expert"]["limit"]
    for t in range(h.shape[0]):
        for k in range(ids.shape[1]):
            e = int(ids[t, k])
            out[t] += w[t, k] * gated_unit(h[t:t + 1], P[f"e{e}.gate"], P[f"e{e}.up"], P[f"e{e}.down"], lim)[0]
    if f.get("shared"):
        sh = gated_unit(h, P["shared.gate"], P["shared.up"], P["shared.down"], f["shared"]["limit"])
        out = out + sh * torch.sigmoid(h @ P["shared.sg"].T)
    return out


def feed_forward(h, P, f):
    if f["kind"] == "dense":
        return gated_unit(h, P["gate"], P["up"], P["down"], f["limit"])
    return routed_ff(h, P, f)


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(tokens, weights, cfg, dtype=torch.float64):
    """tokens: list of ids of one sequence.  Returns (logits [n, vocab], residual stream after every layer [layers, n, W])."""
    Wt = {k: v.to(dtype) for k, v in weights.items()}
    eps, mult, W = cfg["norm"]["eps"], cfg["residual_mult"], cfg["width"]
    t = torch.as_tensor(tokens, dtype=torch.long)
    x = Wt["embed"][t] + position_vectors(torch.arange(len(tokens)), W, dtype)
    caches, taps = {}, []
    for li, L in enumerate(cfg["layers"]):
        if L["type"] != "attention":
            raise ValueError(L["type"])
        m = L["mixer"]
        src = m.get("kv_from")
        y, kv = attention(x, sub(Wt, f"l{li}.mix."), m, eps, caches[src] if src is not None else None)
        caches[li] = kv
        x = x + mult * scalar_rms_norm(y, Wt[f"l{li}.norm1"], eps)
        if L.get("mlp") is not None:
            y = feed_forward(x, sub(Wt, f"l{li}.mlp."), L["mlp"])
            x = x + mult * scalar_rms_norm(y, Wt[f"l{li}.norm2"], eps)
        taps.append(x)
    x = scalar_rms_norm(x, Wt["final.norm"], eps)
    return x @ Wt["head"].T, torch.stack(taps)


def random_weights(cfg, seed=0, scale=1.0):
    """Random weights with the checkpoint's names and shapes, values representable in bfloat16."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def mat(name, o, i, s=None):
        out[name] = (torch.randn(o, i, generator=g) * (s if s is not None else scale / math.sqrt(i))).bfloat16().float()

    def vec(name, n, s=0.1):
        out[name] = (torch.randn(n, generator=g) * s).bfloat16().float()

    out["embed"] = torch.randn(V, W, generator=g).bfloat16().float()
    mat("head", V, W)
    out["final.norm"] = torch.tensor(1.0 + 0.1 * float(torch.randn((), generator=g))).bfloat16().float()
    for li, L in enumerate(cfg["layers"]):
        p, m = f"l{li}.", L["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "norm1"] = torch.tensor(1.0 + 0.1 * float(torch.randn((), generator=g))).bfloat16().float()
        mat(p + "mix.q", H * d, W); vec(p + "mix.q.b", H * d)
        if m.get("kv_from") is None:
            mat(p + "mix.k", G * d, W); vec(p + "mix.k.b", G * d)
            mat(p + "mix.v", G * dv, W); vec(p + "mix.v.b", G * dv)
        mat(p + "mix.g", H, W)
        mat(p + "mix.o", W, H * dv); vec(p + "mix.o.b", W)
        f = L.get("mlp")
        if f is None:
            continue
        out[p + "norm2"] = torch.tensor(1.0 + 0.1 * float(torch.randn((), generator=g))).bfloat16().float()
        if f["kind"] == "dense":
            mat(p + "mlp.gate", f["ff"], W); mat(p + "mlp.up", f["ff"], W); mat(p + "mlp.down", W, f["ff"])
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            for e in range(E):
                mat(p + f"mlp.e{e}.gate", ff, W); mat(p + f"mlp.e{e}.up", ff, W); mat(p + f"mlp.e{e}.down", W, ff)
            mat(p + "mlp.router", E, W, 2.0 / math.sqrt(W))
            vec(p + "mlp.correction", E, 0.2)
            if f.get("shared"):
                sf = f["shared"]["ff"]
                mat(p + "mlp.shared.gate", sf, W); mat(p + "mlp.shared.up", sf, W); mat(p + "mlp.shared.down", W, sf)
                mat(p + "mlp.shared.sg", 1, W)
    return out
