"""The Meropel decoder written out in parts.

x = E[token] + P[hash of (token before, token)].  Every layer is a pre-norm block with a second norm on each sublayer's
output: x += norm1b(mixer(norm1(x))), x += norm2b(feed_forward(norm2(x))).  Mixers: `parallel`, attention (rotation in
halves, a sigmoid gate per head) beside a selective scan, summed with two factors; `parallel_2`, attention (biases, one
norm over the whole q and one over the whole k projection, rotation in pairs) beside a scalar-decay recurrence per head,
each normed over the width, half their sum; `gla`, gated linear attention.  Feed-forwards: SwiGLU, or experts chosen in
groups by corrected softmax scores with pass-through rows and a shared expert.  Then the norm, the head and a factor.
Tensor names: `embed`, `bigram`, `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.left.q|k|v|g|o|q.b|k.b|v.b|q.norm|k.norm|out`,
`l<i>.mix.right.in|conv|conv.b|x|dt|dt.b|dt_bias|A_log|D|norm|o|out`, `l<i>.mix.q|k|v|g|o|norm|a1|a2|a2.b`,
`l<i>.mlp.gate|up|down`, `l<i>.mlp.router|correction`, `l<i>.mlp.e<n>.gate|up|down`, `l<i>.mlp.shared.gate|up|down`,
`final.norm`, `head`.
"""
from __future__ import annotations

from ..parts.base import PartSpec
from ..parts.spec import ModelSpec, ScheduleEntry
from .meropel import MeropelConfig
from .registry import register_architecture


def build_meropel_spec(cfg: MeropelConfig) -> ModelSpec:
    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight=weight))

    blocks, encodings, tolerated = [], {}, []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        if l.type == "gla":
            mixer = PartSpec("gated_linear_attention", dict(
                width=cfg.width, n_heads=l.heads, head_dim=l.dim, v_head_dim=l.vdim, tau=l.tau, eps=cfg.norm_eps,
                names={"q": m + "q", "k": m + "k", "v": m + "v", "g": m + "g", "o": m + "o", "norm": m + "norm",
                       "a1": m + "a1", "a2": m + "a2", "a2_bias": m + "a2.b"}))
        else:
            a, second = l.left, l.type == "parallel_2"
            lm, rm = m + "left.", m + "right."
            pe = None
            if a.rot_dims > 0:
                layout = "pairs" if second else "halves"
                pe = f"rope_{layout}_{a.rot_dims}_{a.rot_base!r}"
                encodings[pe] = PartSpec("rope", dict(rotary_dim=a.rot_dims, theta=a.rot_base, precise=True, layout=layout,
                                                      exact_angles=True))
            names = {"q": lm + "q", "k": lm + "k", "v": lm + "v", "o": lm + "o"}
            more = {}
            if second:
                names.update({"q_norm": lm + "q.norm", "k_norm": lm + "k.norm"})
                more = dict(qk_norm="whole", biases={"q": lm + "q.b", "k": lm + "k.b", "v": lm + "v.b"})
            else:
                more = dict(qk_norm=False, gate=lm + "g", gate_per_head=True)
            left = PartSpec("gqa_attention", dict(
                width=cfg.width, n_q_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim, v_head_dim=a.vdim,
                position_encoding=pe, eps=cfg.norm_eps, scale=a.scale, names=names, **more))
            if second:
                right = PartSpec("state_space_dual", dict(
                    width=cfg.width, n_heads=l.heads, head_dim=l.vdim, state=l.state, groups=l.groups,
                    norm_groups=l.norm_groups, taps=l.conv, eps=cfg.norm_eps,
                    names={"in": rm + "in", "conv": rm + "conv", "conv_bias": rm + "conv.b", "dt_bias": rm + "dt_bias",
                           "A_log": rm + "A_log", "D": rm + "D", "norm": rm + "norm", "o": rm + "o"}))
                mixer = PartSpec("side_by_side", dict(left=left, right=right, width=cfg.width, left_scale=0.5, right_scale=0.5,
                                                      norms={"left": lm + "out", "right": rm + "out"}, eps=cfg.norm_eps))
            else:
                right = PartSpec("selective_scan", dict(
                    width=cfg.width, inner=l.inner, state=l.state, dt_rank=l.dt_rank, taps=l.conv,
                    names={"in": rm + "in", "conv": rm + "conv", "conv_bias": rm + "conv.b", "x": rm + "x", "dt": rm + "dt",
                           "dt_bias": rm + "dt.b", "A_log": rm + "A_log", "D": rm + "D", "o": rm + "o"}))
                mixer = PartSpec("side_by_side", dict(left=left, right=right, width=cfg.width, left_scale=l.left_scale,
                                                      right_scale=l.right_scale))
        ffn, norm2, norm2b = None, None, None
        f = p + "mlp."
        if l.mlp_kind == "dense":
            ffn = PartSpec("swiglu", dict(width=cfg.width, inner=l.ff, names={"gate": f + "gate", "up": f + "up", "down": f + "down"}))
        elif l.mlp_kind == "moe":
            ffn = PartSpec("routed_experts", dict(
                width=cfg.width, inner=l.ff, n_experts=l.experts, top=l.top, activation="silu", shared_inner=l.shared_ff,
                score="softmax_corrected_in_groups", groups=l.expert_groups, keep=l.keep, route_scale=l.route_scale,
                n_pass=l.identity,
                names={"router": f + "router", "router_bias": f + "correction", "gate": f + "e{e}.gate", "up": f + "e{e}.up",
                       "down": f + "e{e}.down", "shared_gate": f + "shared.gate", "shared_up": f + "shared.up",
                       "shared_down": f + "shared.down"}))
        if ffn is not None:
            norm2, norm2b = norm(p + "norm2"), norm(p + "norm2b")
        else:
            tolerated += [p + "norm2", p + "norm2b"]   # a layer without feed-forward reads neither
        blocks.append(PartSpec("prenorm", dict(mixer=mixer, feed_forward=ffn, norm_mixer=norm(p + "norm1"),
                                               norm_feed_forward=norm2, post_norm_mixer=norm(p + "norm1b"),
                                               post_norm_feed_forward=norm2b)))
    pair = None
    if cfg.bigram is not None:
        pair = {"weight": "bigram", "buckets": cfg.bigram[0], "mul_prev": cfg.bigram[1], "mul_cur": cfg.bigram[2]}
    return ModelSpec(
        width=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=cfg.width, weight="embed", pair=pair)),
        position_encodings=encodings,
        layers=tuple(blocks),
        schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=cfg.width, weight="head", scale=cfg.logit_scale)),
        tolerated_tensors=tuple(tolerated),
    )


register_architecture("Meropel", MeropelConfig, build_meropel_spec)
