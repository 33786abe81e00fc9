"""Slow plain-PyTorch statement of the Karusun design, one function per mechanism, whole sequence at once, float32 (or float64) on the CPU.

Test infrastructure only: it shares no code with the product path.  Notation: W = model width, n = tokens of ONE sequence,
positions 0..n-1.  Weights come as a dict name -> tensor with the checkpoint's names ('l<i>.mix.q', 'l<i>.mlp.e<j>.gate', ...).
"""
import math

import torch
import torch.nn.functional as F


def group_rms_norm(x, w, groups, eps):
    """x [n, W]: every one of `groups` equal consecutive parts divided by its own sqrt(mean(part^2) + eps); then times w."""
    n, W = x.shape
    p = x.reshape(n, groups, W // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(n, W) * w


def causal_taps(h, w):
    """h [n, C], w [C, taps]; y_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    n, C = h.shape
    taps = w.shape[1]
    pad = torch.cat([h.new_zeros(taps - 1, C), h], 0)
    y = torch.zeros_like(h)
    for j in range(taps):
        y = y + pad[j:j + n] * w[:, j]
    return y


def input_conv(h, w):
    return h + causal_taps(h, w)


def rotate_half_pairs(x, pos, base, dims):
    """x [n, ..., D]: the first `dims` dimensions rotated, pair (i, i + dims/2), angle pos * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    a = pos.to(torch.float64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(a).to(x.dtype).reshape(shape), torch.sin(a).to(x.dtype).reshape(shape)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * c - v * s, v * c + u * s, rest], -1)


def latent_attention(h, P, m, eps):
    """h [n, W]; P: dict of this mixer's tensors by short name (q, dkv, dkv.norm, uk, uv, g, o); m: the mixer's config."""
    n = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(n)
    q = (h @ P["q"].T).reshape(n, H, d + r)
    qn, qr = q[..., :d], q[..., d:]
    ckr = h @ P["dkv"].T
    c = ckr[:, :R]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * P["dkv.norm"]
    kr = ckr[:, R:]
    rot = m["rot"]
    qr = rotate_half_pairs(qr, pos, rot["base"], rot["dims"])
    kr = rotate_half_pairs(kr[:, None, :], pos, rot["base"], rot["dims"])[:, 0]
    kn = (c @ P["uk"].T).reshape(n, H, d)
    v = (c @ P["uv"].T).reshape(n, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    i, j = pos[:, None], pos[None, :]
    vis = (i - j >= 0) & (i - j < m["mask"]["size"])
    s = s.masked_fill(~vis, float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * dv)
    o = o * torch.sigmoid(h @ P["g"].T)
    return o @ P["o"].T


def gated_delta(h, P, m, eps):
    """h [n, W]; P: q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, norm, g, o."""
    n = h.shape[0]
    H, Hk, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(causal_taps(h @ P["q"].T, P["q.conv"])).reshape(n, Hk, d)
    k = F.silu(causal_taps(h @ P["k"].T, P["k.conv"])).reshape(n, Hk, d)
    v = F.silu(causal_taps(h @ P["v"].T, P["v.conv"])).reshape(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ P["b"].T)
    g = torch.exp(-torch.exp(P["A_log"]) * F.softplus(h @ P["a"].T + P["dt_bias"]))
    rep = H // Hk
    o = h.new_zeros(n, H, dv)
    for hd in range(H):
        S = h.new_zeros(d, dv)
        kh = hd // rep
        for t in range(n):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            o[t, hd] = S.T @ q[t, kh]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * P["norm"]
    o = o.reshape(n, H * dv) * F.silu(h @ P["g"].T)
    return o @ P["o"].T


def route(h, P, r):
    """-> chosen [n, top] expert indices (identity experts have index >= experts), weights [n, top]."""
    E, I = r["experts"], r.get("identity", 0)
    z = h @ P["router"].T
    s = torch.softmax(z, -1)
    choice = s + P["correction"]
    G, keep = r["groups"]["count"], r["groups"]["keep"]
    n = h.shape[0]
    gs = choice.reshape(n, G, (E + I) // G).max(-1).values
    kept = torch.zeros(n, G, dtype=torch.bool)
    kept.scatter_(1, gs.topk(keep, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(n, G, (E + I) // G).reshape(n, E + I)
    choice = choice.masked_fill(~allowed, float("-inf"))
    idx = choice.topk(r["top"], dim=-1).indices
    return idx, s.gather(1, idx)


def moe(h, P, f):
    r = f["router"]
    E = r["experts"]
    idx, w = route(h, P, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(idx[t].tolist(), w[t]):
            if e >= E:
                y = h[t]
            else:
                y = (F.silu(h[t] @ P[f"e{e}.gate"].T) * (h[t] @ P[f"e{e}.up"].T)) @ P[f"e{e}.down"].T
            out[t] = out[t] + wt * y
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, taps_out=None):
    """tokens: list of ids of one sequence -> logits [n, vocab].  taps_out: list that receives the residual after every layer."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = weights["embed"][torch.tensor(tokens)]
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        hin = input_conv(group_rms_norm(x, weights[p + "norm1"], groups, eps), weights[p + "canon1"])
        mixer = latent_attention if L["type"] == "latent_attention" else gated_delta
        y = mixer(hin, sub(weights, p + "mix."), L["mixer"], eps)
        x = x + group_rms_norm(y, weights[p + "norm1b"], groups, eps)
        if L.get("mlp") is not None:
            hin = input_conv(group_rms_norm(x, weights[p + "norm2"], groups, eps), weights[p + "canon2"])
            y = moe(hin, sub(weights, p + "mlp."), L["mlp"])
            x = x + group_rms_norm(y, weights[p + "norm2b"], groups, eps)
        if taps_out is not None:
            taps_out.append(x.clone())
    x = group_rms_norm(x, weights["final.norm"], groups, eps)
    return x @ weights["head"].T
