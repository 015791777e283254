"""Plain, slow implementation of the Meropel decoder: the oracle of its tests.

Whole sequences, no cache, one function per mechanism, float64 on the CPU.  It shares no code with the product
package (only the oracles' reader of a model folder, which is test code too).

In this file's notation (n tokens, width d, x the residual stream, rms(x, w) = x / sqrt(mean(x^2) + eps) * w):

    x = E[token] + B[(prev * mul_prev + token * mul_cur) mod buckets]          (B's last row at a sequence's start)
    for every entry of `layers`:
        x += rms(mixer(rms(x, w1)), w1b);   x += rms(ffn(rms(x, w2)), w2b)      (the second line if it has an ffn)
    logits = logit_scale * H rms(x, w_final)

Mixers: `parallel` (softmax attention with a per-head sigmoid gate beside a selective scan with a state per channel,
summed with two factors), `parallel_2` (softmax attention with biases and a norm over the whole q and k projections
beside a scalar-decay state-space recurrence per head, each output normed over the width, half their sum), `gla`
(linear attention whose state decays per key channel by sigmoid(z)^(1/tau)).  Feed-forwards: a gated one, or experts
chosen among groups by corrected softmax scores, some of which hand their input through unchanged.
"""
from __future__ import annotations

import math

import torch

from .qwen3_plain import read_model_folder  # noqa: F401  (re-exported: the folder reader of the oracles)

F64 = torch.float64


def _same(t):
    return t


def rms(x, w, eps):
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def embed(tokens, table, bigram, cfg_bigram, prev_token=None):
    """Rows of the token table plus rows of the bigram table; prev_token: the token before the first one given."""
    buckets, mp, mc = int(cfg_bigram["buckets"]), int(cfg_bigram["mul_prev"]), int(cfg_bigram["mul_cur"])
    rows = []
    prev = prev_token
    for t in tokens:
        r = buckets if prev is None else (int(prev) * mp + int(t) * mc) % buckets
        rows.append(table[int(t)] + bigram[r])
        prev = t
    return torch.stack(rows)


def rotate(t, positions, dims: int, base: float, layout: str):
    """t: [n, heads, e]; the first `dims` elements of every head turn by position * base^(-2i/dims)."""
    out = t.clone()
    half = dims // 2
    for i in range(half):
        f = base ** (-2.0 * i / dims)
        a = torch.tensor([float(p) * f for p in positions], dtype=F64)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        iu, iv = (2 * i, 2 * i + 1) if layout == "pairs" else (i, i + half)
        u, v = t[:, :, iu], t[:, :, iv]
        out[:, :, iu] = u * c - v * s
        out[:, :, iv] = v * c + u * s
    return out


def causal_softmax_attention(q, k, v, scale: float, q_positions=None, k_positions=None):
    """q: [n, H, dim], k: [m, G, dim], v: [m, G, vdim]; query head h reads kv head h // (H / G); a query at position p
    sees the keys at positions <= p.  Returns [n, H, vdim]."""
    n, H, _ = q.shape
    m, G, _ = k.shape
    qp = list(range(n)) if q_positions is None else q_positions
    kp = list(range(m)) if k_positions is None else k_positions
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for i in range(n):
        vis = [j for j in range(m) if kp[j] <= qp[i]]
        for h in range(H):
            g = h // (H // G)
            s = (k[vis, g] @ q[i, h]) * scale
            w = torch.softmax(s, dim=0)
            out[i, h] = w @ v[vis, g]
    return out


def causal_conv(x, w, b, before=None):
    """x: [n, C]; w: [C, taps] whose last column meets the current token; zeros (or `before`, [taps - 1, C]) ahead."""
    n, C = x.shape
    taps = w.shape[1]
    pad = torch.zeros(taps - 1, C, dtype=F64) if before is None else before
    xx = torch.cat([pad, x], dim=0)
    out = torch.zeros(n, C, dtype=F64)
    for t in range(n):
        for j in range(taps):
            out[t] += xx[t + j] * w[:, j]
    return out + b


def attention_left(h, w, p, mx, eps, positions, variant: str, rnd=_same):
    n = h.shape[0]
    H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if variant == "parallel_2":
        q, k, v = q + w[p + "q.b"], k + w[p + "k.b"], v + w[p + "v.b"]
        q, k = rms(q, w[p + "q.norm"], eps), rms(k, w[p + "k.norm"], eps)
    q, k, v = q.view(n, H, dim), k.view(n, G, dim), v.view(n, G, vdim)
    rot = mx.get("rot")
    if rot is not None and rot["dims"] > 0:
        layout = "pairs" if variant == "parallel_2" else "halves"
        q = rotate(q, positions, rot["dims"], float(rot["base"]), layout)
        k = rotate(k, positions, rot["dims"], float(rot["base"]), layout)
    q, k, v = rnd(q), rnd(k), rnd(v)
    o = causal_softmax_attention(q, k, v, float(mx["scale"]))
    if variant == "parallel":
        gate = torch.sigmoid(h @ w[p + "g"].T)           # one number per head
        o = o * gate[:, :, None]
    return rnd(o.reshape(n, H * vdim)) @ w[p + "o"].T


def selective_scan(h, w, p, mx, rnd=_same):
    """Mamba: a state per channel and state index, decays exp(dt A)."""
    n = h.shape[0]
    inner, N, R = mx["inner"], mx["state"], mx["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = rnd(silu(causal_conv(x, w[p + "conv"], w[p + "conv.b"])))
    proj = x @ w[p + "x"].T
    dt, B, C = proj[:, :R], proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    dt = softplus(rnd(dt) @ w[p + "dt"].T + w[p + "dt.b"])         # [n, inner]
    A = -torch.exp(w[p + "A_log"])                                 # [inner, N]
    S = torch.zeros(inner, N, dtype=F64)
    y = torch.zeros(n, inner, dtype=F64)
    for t in range(n):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + "D"] * x[t]
    y = y * silu(z)
    return rnd(y) @ w[p + "o"].T


def state_space_dual(h, w, p, mx, eps, rnd=_same):
    """Mamba-2: a state N x vdim per head with one decay per head and token."""
    n = h.shape[0]
    Hh, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = Hh * P
    proj = h @ w[p + "in"].T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt = proj[:, 2 * inner + 2 * G * N:]
    xbc = rnd(silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"])))
    x = xbc[:, :inner].view(n, Hh, P)
    B = xbc[:, inner:inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = softplus(dt + w[p + "dt_bias"])                          # [n, heads]
    a = torch.exp(w[p + "A_log"])
    S = torch.zeros(Hh, N, P, dtype=F64)
    y = torch.zeros(n, Hh, P, dtype=F64)
    for t in range(n):
        for hh in range(Hh):
            g = hh // (Hh // G)
            S[hh] = math.exp(-float(a[hh]) * float(dt[t, hh])) * S[hh] + float(dt[t, hh]) * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + w[p + "D"][hh] * x[t, hh]
    y = y.reshape(n, inner) * silu(z)
    parts = mx["norm_groups"]
    y = rms(y.view(n, parts, inner // parts), None, eps).reshape(n, inner) * w[p + "norm"]
    return rnd(y) @ w[p + "o"].T


def gated_linear_attention(h, w, p, mx, eps, rnd=_same):
    n = h.shape[0]
    H, dim, vdim, tau = mx["heads"], mx["dim"], mx["vdim"], float(mx["tau"])
    q = (h @ w[p + "q"].T * dim ** -0.5).view(n, H, dim)
    k = (h @ w[p + "k"].T).view(n, H, dim)
    v = (h @ w[p + "v"].T).view(n, H, vdim)
    z = rnd(h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(n, H, dim)
    S = torch.zeros(H, dim, vdim, dtype=F64)
    o = torch.zeros(n, H, vdim, dtype=F64)
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms(o, w[p + "norm"], eps).reshape(n, H * vdim)
    o = o * silu(h @ w[p + "g"].T)
    return rnd(o) @ w[p + "o"].T


def mixer(kind, h, w, p, mx, eps, positions, rnd=_same):
    if kind == "gla":
        return gated_linear_attention(h, w, p, mx, eps, rnd)
    left = attention_left(h, w, p + "left.", mx["left"], eps, positions, kind, rnd)
    if kind == "parallel":
        right = selective_scan(h, w, p + "right.", mx["right"], rnd)
        return float(mx["left_scale"]) * left + float(mx["right_scale"]) * right
    if kind == "parallel_2":
        right = state_space_dual(h, w, p + "right.", mx["right"], eps, rnd)
        return 0.5 * (rms(left, w[p + "left.out"], eps) + rms(right, w[p + "right.out"], eps))
    raise ValueError(kind)


def gated_mlp(h, gate, up, down, rnd=_same):
    return rnd(silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, w_router, correction, router: dict):
    """[(expert, weight), ...] per token; experts from `experts` on hand their input through."""
    real, ident, top = int(router["experts"]), int(router.get("identity", 0)), int(router["top"])
    E = real + ident
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    s = torch.softmax(h @ w_router.T, dim=-1)
    out = []
    for t in range(h.shape[0]):
        choice = (s[t] + correction).tolist()
        size = E // count
        best = sorted(range(count), key=lambda g: (-max(choice[g * size:(g + 1) * size]), g))[:keep]
        allowed = [e for e in range(E) if e // size in best]
        chosen = sorted(allowed, key=lambda e: (-choice[e], e))[:top]
        total = sum(float(s[t, e]) for e in chosen) + 1e-20
        out.append([(e, float(s[t, e]) / total * float(router.get("scale", 1.0))) for e in chosen])
    return out


def expert_mlp(h, w, p, mlp, rnd=_same):
    router = mlp["router"]
    real = int(router["experts"])
    picks = route(h, w[p + "router"], w[p + "correction"], router)
    out = torch.zeros_like(h)
    for t, row in enumerate(picks):
        for e, wt in row:
            if e >= real:
                out[t] += wt * h[t]
            else:
                q = f"{p}e{e}."
                out[t] += wt * gated_mlp(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"], rnd)[0]
    if mlp.get("shared"):
        out = out + gated_mlp(h, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], rnd)
    return out


def feed_forward(h, w, p, mlp, rnd=_same):
    if mlp["kind"] == "dense":
        return gated_mlp(h, w[p + "gate"], w[p + "up"], w[p + "down"], rnd)
    return expert_mlp(h, w, p, mlp, rnd)


def to_bfloat16_and_back(t):
    return t.to(torch.bfloat16).to(F64)


def forward(config: dict, weights: dict, tokens, return_layers: bool = False, rnd=_same):
    """Logits [n, vocab] of a whole sequence (float64); with return_layers also the residual stream after every layer.
    rnd: applied to what a 16-bit engine stores between kernels (identity: exact arithmetic)."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    n = len(tokens)
    positions = list(range(n))
    x = embed(tokens, w["embed"], w["bigram"], config["embedding"]["bigram"])
    layers = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rnd(rms(x, w[p + "norm1"], eps))
        x = x + rms(mixer(layer["type"], h, w, p + "mix.", layer["mixer"], eps, positions, rnd), w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rnd(rms(x, w[p + "norm2"], eps))
            x = x + rms(feed_forward(h, w, p + "mlp.", layer["mlp"], rnd), w[p + "norm2b"], eps)
        layers.append(x.clone())
    logits = rnd(rms(x, w["final.norm"], eps)) @ w["head"].T * float(config.get("logit_scale", 1.0))
    return (logits, layers) if return_layers else logits
