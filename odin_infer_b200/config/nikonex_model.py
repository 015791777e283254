"""The Nikonex decoder written out in parts.

x = E[token].  Every layer is a parallel block with two norms and one factor m: x += m * (mixer(norm1(x)) +
feed_forward(norm2(x))), both norms plain RMSNorms of the same x.  Mixers: attention through latents (rotation in
pairs (2i, 2i+1) with frequencies ramped down by pair and a gain on cos and sin, sliding window), or retention
(rotation in halves (i, i + dims/2), a fixed decay per head).  Feed-forward: experts W_down relu(W_up h)^2 chosen by
a sigmoid router inside the best groups, a shared expert behind a per-token sigmoid gate.  Then the norm and the head.
Tensor names: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|o` or `l<i>.mix.q|k|v|g|o`,
`l<i>.mlp.router`, `l<i>.mlp.e<n>.up|down`, `l<i>.mlp.shared.up|down|sg`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..parts.base import PartSpec
from ..parts.spec import ModelSpec, ScheduleEntry
from .nikonex import NikonexConfig
from .registry import register_architecture


def build_nikonex_spec(cfg: NikonexConfig) -> ModelSpec:
    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight=weight))

    blocks, encodings, tolerated = [], {}, []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        pe = None
        if l.rot_dims > 0:
            latent = l.type == "latent_attention"
            pe = f"rope_{l.type}_{l.rot_dims}_{l.rot_base!r}_{l.rot_scaling!r}"
            ramp = dict(zip(("factor", "original", "fast", "slow"), l.rot_scaling)) if l.rot_scaling else None
            encodings[pe] = PartSpec("rope", dict(rotary_dim=l.rot_dims, theta=l.rot_base, ramp=ramp, precise=True,
                                                  layout="pairs" if latent else "halves", exact_angles=True))
        if l.type == "latent_attention":
            mixer = PartSpec("latent_attention", dict(
                width=cfg.width, n_heads=l.heads, head_dim=l.dim, rot_dim=l.rot_dim, v_head_dim=l.vdim, q_rank=l.q_rank,
                kv_rank=l.kv_rank, position_encoding=pe, eps=cfg.norm_eps, scale=l.scale, window=l.window,
                names={"dq": m + "dq", "dq_norm": m + "dq.norm", "uq": m + "uq", "dkv": m + "dkv", "dkv_norm": m + "dkv.norm",
                       "uk": m + "uk", "uv": m + "uv", "o": m + "o"}))
        else:
            mixer = PartSpec("retention", dict(
                width=cfg.width, n_heads=l.heads, head_dim=l.dim, v_head_dim=l.vdim, decay=list(l.decay),
                position_encoding=pe, eps=cfg.norm_eps,
                names={"q": m + "q", "k": m + "k", "v": m + "v", "g": m + "g", "o": m + "o"}))
        ffn, norm2 = None, None
        if l.has_mlp:
            f = p + "mlp."
            names = {"router": f + "router", "up": f + "e{e}.up", "down": f + "e{e}.down", "shared_up": f + "shared.up",
                     "shared_down": f + "shared.down", "shared_token_gate": f + "shared.sg"}
            ffn = PartSpec("routed_experts", dict(
                width=cfg.width, inner=l.ff, n_experts=l.experts, top=l.top, activation="relu2", gated=False,
                shared_inner=l.shared_ff, score="sigmoid_in_groups", groups=l.groups, keep=l.keep,
                route_scale=l.route_scale, shared_gate=l.shared_ff > 0, names=names))
            norm2 = norm(p + "norm2")
        else:
            tolerated.append(p + "norm2")   # a layer without feed-forward reads no second norm
        blocks.append(PartSpec("parallel", dict(mixer=mixer, feed_forward=ffn, norm=norm(p + "norm1"),
                                                norm_feed_forward=norm2, residual_mult=cfg.residual_mult)))
    return ModelSpec(
        width=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=cfg.width, weight="embed")),
        position_encodings=encodings,
        layers=tuple(blocks),
        schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=cfg.width, weight="head")),
        tolerated_tensors=tuple(tolerated),
    )


register_architecture("Nikonex", NikonexConfig, build_nikonex_spec)
