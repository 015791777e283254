"""Plain, slow implementation of the Nikonex decoder: the oracle of its tests.

Whole sequences, no cache, one function per mechanism, float64 on the CPU.  It shares no code
with the product package (only the oracles' reader of a model folder, which is test code too).

The design in this file's notation (n tokens, width d, x the residual stream, m = residual_mult):

    x = E[token]
    for every entry of `layers`:   x += m * (mixer(rms(x, w1)) + ffn(rms(x, w2)))     (two norms of the same x)
    logits = H rms(x, w_final)

rms(x, w) = x / sqrt(mean(x^2) + eps) * w.

Mixers:
  `latent_attention`: queries through a normed latent (W_dq, norm, W_uq), keys and values from ONE normed latent c per
      token (W_dkv -> [c | one rotated key part shared by the heads], W_uk c, W_uv c); every head's query and key are
      [unrotated part | rotated part]; the rotated parts turn in the interleaved layout (2i with 2i+1) with frequencies
      scaled by a ramp over the pair index and cos, sin multiplied by 0.1 ln(factor) + 1; sliding window; softmax.
  `retention`: q, k rotated in the rotate-half layout (i with i + dims/2), k scaled by dim^-1/2 afterwards,
      S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, every head's o divided by its root mean square,
      times silu(W_g h), then W_o.
Feed-forward: experts W_down relu(W_up h)^2 chosen by a sigmoid router inside the best groups of neighbouring
experts, weights = chosen scores / their sum * router.scale, plus a shared expert times sigmoid(w_sg . h).
"""
from __future__ import annotations

import math

import torch

from .qwen3_plain import read_model_folder  # noqa: F401  (re-exported: the folder reader of the oracles)

F64 = torch.float64


def rms(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def ramp_frequencies(dims: int, base: float, scaling: dict | None):
    """(frequencies of the dims/2 pairs, factor on cos and sin)."""
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling is None:
        return freqs, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:   # the (real-valued) pair whose wavelength fits `turns` times into `orig`
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * r + f * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(t: torch.Tensor, positions, freqs, gain: float, layout: str) -> torch.Tensor:
    """t: [n, heads, e]; the first 2 * len(freqs) elements of every head turn, the rest pass.
    layout "pairs": element 2i with 2i + 1; "halves": element i with i + len(freqs)."""
    half = len(freqs)
    out = t.clone()
    for n in range(t.shape[0]):
        for i, f in enumerate(freqs):
            a = float(positions[n]) * f
            c, s = math.cos(a) * gain, math.sin(a) * gain
            iu, iv = (2 * i, 2 * i + 1) if layout == "pairs" else (i, i + half)
            u, v = t[n, :, iu], t[n, :, iv]
            out[n, :, iu] = u * c - v * s
            out[n, :, iv] = v * c + u * s
    return out


def windowed_softmax_attention(q, k, v, scale: float, window: int) -> torch.Tensor:
    """q, k: [n, H, e], v: [n, H, ev]; query i sees key j when 0 <= i - j < window (window 0: every j <= i)."""
    n, H = q.shape[0], q.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for i in range(n):
        j0 = 0 if window <= 0 else max(0, i - window + 1)
        for h in range(H):
            s = (k[j0:i + 1, h] @ q[i, h]) * scale
            p = torch.softmax(s, dim=0)
            out[i, h] = p @ v[j0:i + 1, h]
    return out


def _same(t):
    return t


def to_bfloat16_and_back(t: torch.Tensor) -> torch.Tensor:
    """What a tensor loses when it is stored in bfloat16: the `rnd` of the functions below, to see how far rounding
    of activations alone moves a result (the tolerance of a comparison in bfloat16 is taken from that)."""
    return t.to(torch.bfloat16).to(t.dtype)


def latent_attention(h, w, p, mx, eps, positions=None, rnd=_same):
    n = h.shape[0]
    H, e, r, ev, kv_rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    positions = list(range(n)) if positions is None else positions
    cq = rnd(rms(h @ w[p + "dq"].T, w[p + "dq.norm"], eps))
    q = rnd(cq @ w[p + "uq"].T).view(n, H, e + r)
    down = h @ w[p + "dkv"].T
    c = rnd(rms(down[:, :kv_rank], w[p + "dkv.norm"], eps))
    k_rot = down[:, kv_rank:].view(n, 1, r)
    rot = mx["rot"]
    freqs, gain = ramp_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q_rot = rotate(q[:, :, e:], positions, freqs, gain, "pairs")
    k_rot = rnd(rotate(k_rot, positions, freqs, gain, "pairs"))
    k_flat = (c @ w[p + "uk"].T).view(n, H, e)
    v = (c @ w[p + "uv"].T).view(n, H, ev)
    qq = torch.cat([q[:, :, :e], q_rot], dim=2)
    kk = torch.cat([k_flat, k_rot.expand(n, H, r)], dim=2)
    window = (mx.get("mask") or {}).get("size", 0)
    o = windowed_softmax_attention(qq, kk, v, float(mx["scale"]), window)
    return rnd(o.reshape(n, H * ev)) @ w[p + "o"].T


def retention(h, w, p, mx, eps, positions=None, state=None, rnd=_same):
    """state: None (a sequence from its start) or a list of H [e, ev] matrices that is updated in place."""
    n = h.shape[0]
    H, e, ev = mx["heads"], mx["dim"], mx["vdim"]
    positions = list(range(n)) if positions is None else positions
    q = (h @ w[p + "q"].T).view(n, H, e)
    k = (h @ w[p + "k"].T).view(n, H, e)
    v = (h @ w[p + "v"].T).view(n, H, ev)
    rot = mx.get("rot")
    if rot is not None and rot.get("dims", 0) > 0:
        freqs, gain = ramp_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q = rotate(q, positions, freqs, gain, "halves")
        k = rotate(k, positions, freqs, gain, "halves")
    k = k * float(e) ** -0.5
    o = torch.zeros(n, H, ev, dtype=F64)
    for hd in range(H):
        S = torch.zeros(e, ev, dtype=F64) if state is None else state[hd]
        for t in range(n):
            S = float(mx["decay"][hd]) * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
        if state is not None:
            state[hd] = S
    o = rms(o, None, eps)
    g = h @ w[p + "g"].T
    y = o.reshape(n, H * ev) * (g * torch.sigmoid(g))
    return rnd(y) @ w[p + "o"].T


def relu2_mlp(h, up, down, rnd=_same):
    return rnd(torch.relu(h @ up.T) ** 2) @ down.T


def route(h, w_router, router: dict):
    """(chosen experts [n, top], their weights [n, top])."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    G, keep = groups["count"], groups["keep"]
    s = torch.sigmoid(h @ w_router.T)
    ids, wts = [], []
    per = E // G
    for t in range(h.shape[0]):
        row = s[t]
        gscore = [float(torch.sort(row[g * per:(g + 1) * per], descending=True).values[:2].sum()) for g in range(G)]
        best = sorted(range(G), key=lambda g: (-gscore[g], g))[:keep]
        allowed = [e for e in range(E) if e // per in best]
        chosen = sorted(allowed, key=lambda e: (-float(row[e]), e))[:top]
        wt = torch.stack([row[e] for e in chosen])
        wt = wt / (wt.sum() + 1e-20) * float(router.get("scale", 1.0))
        ids.append(chosen)
        wts.append(wt)
    return ids, torch.stack(wts)


def expert_mlp(h, w, p, mlp, rnd=_same):
    ids, wts = route(h, w[p + "router"], mlp["router"])
    out = torch.zeros(h.shape[0], h.shape[1], dtype=F64)
    for t in range(h.shape[0]):
        for k, e in enumerate(ids[t]):
            out[t] += wts[t, k] * relu2_mlp(h[t:t + 1], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], rnd)[0]
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)      # [n, 1]
        out = out + gate * relu2_mlp(h, w[p + "shared.up"], w[p + "shared.down"], rnd)
    return out


def forward(config: dict, weights: dict, tokens, return_layers: bool = False, rnd=_same):
    """Logits [n, vocab] of a whole sequence (and the residual stream after every layer).  rnd: applied to what a
    16-bit engine would store in 16 bits (what a matrix product reads, cached rows); the identity by default."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, m = float(config["norm"]["eps"]), float(config.get("residual_mult", 1.0))
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h1 = rnd(rms(x, w[p + "norm1"], eps))
        if layer["type"] == "latent_attention":
            upd = latent_attention(h1, w, p + "mix.", layer["mixer"], eps, rnd=rnd)
        elif layer["type"] == "retention":
            upd = retention(h1, w, p + "mix.", layer["mixer"], eps, rnd=rnd)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        if layer.get("mlp") is not None:
            upd = upd + expert_mlp(rnd(rms(x, w[p + "norm2"], eps)), w, p + "mlp.", layer["mlp"], rnd)
        x = x + m * upd
        streams.append(x.clone())
    logits = rnd(rms(x, w["final.norm"], eps)) @ w["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
