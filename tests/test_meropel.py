"""The Meropel configuration, its model description, the pending updates that carry terms and norms of their own, and
the plain implementation's own mechanisms checked against what they must equal (no GPU)."""
import copy
import math

import pytest
import torch

from odin_infer_b200.cache import CacheManager
from odin_infer_b200.config import ConfigError, MeropelConfig, config_from_dict, lookup_architecture
from odin_infer_b200.engine.model import DecoderModel
from odin_infer_b200.parts.base import Combined, Normed, PartSpec, build_part, split_update
from tests.plain import meropel_plain as P

F64 = torch.float64
ATT = {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.3, "rot": {"dims": 8, "base": 5000.0}}
MOE = {"kind": "moe", "expert": {"ff": 40},
       "router": {"experts": 6, "top": 3, "scale": 2.0, "identity": 3, "groups": {"count": 3, "keep": 2}}, "shared": {"ff": 56}}
RAW = {"architecture": "Meropel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
       "embedding": {"bigram": {"buckets": 61, "mul_prev": 31, "mul_cur": 5}},
       "layers": [{"type": "parallel",
                   "mixer": {"left": ATT, "left_scale": 0.7, "right": {"inner": 72, "state": 12, "dt_rank": 5, "conv": 3},
                             "right_scale": 1.3},
                   "mlp": {"kind": "dense", "ff": 80}},
                  {"type": "gla", "mixer": {"heads": 3, "dim": 20, "vdim": 28, "tau": 8.0}, "mlp": MOE},
                  {"type": "parallel_2",
                   "mixer": {"left": {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2},
                             "right": {"heads": 4, "vdim": 16, "state": 24, "groups": 2, "norm_groups": 4, "conv": 4}},
                   "mlp": None}]}


def test_configuration_reads_and_writes_the_same_keys():
    cfg = config_from_dict(RAW)
    assert isinstance(cfg, MeropelConfig) and cfg.to_dict() == RAW
    assert config_from_dict(cfg.to_dict()) == cfg
    a, b, c = cfg.layers
    assert (a.left.rot_dims, a.left.rot_base, a.inner, a.state, a.dt_rank, a.conv) == (8, 5000.0, 72, 12, 5, 3)
    assert (b.experts, b.identity, b.top, b.expert_groups, b.keep, b.route_scale, b.shared_ff) == (6, 3, 3, 3, 2, 2.0, 56)
    assert c.left.rot_dims == 0 and c.mlp_kind is None and cfg.bigram == (61, 31, 5)


def test_absent_keys_mean_absent_mechanisms():
    raw = {"architecture": "Meropel", "vocab": 50, "width": 40, "norm": {"eps": 1e-6},
           "layers": [{"type": "gla", "mixer": {"heads": 1, "dim": 8, "vdim": 8, "tau": 2.0},
                       "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 1}}}]}
    cfg = config_from_dict(raw)
    l = cfg.layers[0]
    assert (cfg.logit_scale, cfg.bigram, l.identity, l.expert_groups, l.keep, l.route_scale, l.shared_ff) == (1.0, None, 0, 1, 1, 1.0, 0)
    spec = lookup_architecture("Meropel").build_spec(cfg)
    assert spec.embedding.args["pair"] is None and spec.head.args["scale"] == 1.0 and not spec.position_encodings


def test_every_fault_of_a_configuration_in_one_error():
    bad = copy.deepcopy(RAW)
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 7
    bad["layers"][0]["mixer"]["right"]["state"] = 0
    bad["layers"][1]["mlp"]["router"]["groups"] = {"count": 4, "keep": 1}
    bad["layers"][2]["mixer"]["right"]["groups"] = 3
    bad["embedding"]["bigram"]["buckets"] = 0
    del bad["layers"][1]["mixer"]["tau"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    msg = str(e.value)
    for part in ("dims (7)", "inner, state, dt_rank and conv", "9 router rows in 4 groups", "multiple of groups", "buckets", "'tau'"):
        assert part in msg, (part, msg)


def test_the_model_description_names_every_tensor_once():
    cfg = config_from_dict(RAW)
    model = DecoderModel(lookup_architecture("Meropel").build_spec(cfg))
    names = [p.name for p in model.params()]
    assert len(names) == len(set(names))
    for n in ("embed", "bigram", "l0.norm1b", "l0.norm2b", "l0.mix.left.g", "l0.mix.right.conv.b", "l0.mix.right.dt.b",
              "l1.mix.a2.b", "l1.mlp.correction", "l1.mlp.e5.down", "l1.mlp.shared.up", "l2.mix.left.q.norm", "l2.mix.left.k.b",
              "l2.mix.right.dt_bias", "l2.mix.left.out", "l2.mix.right.out", "final.norm", "head"):
        assert n in names, n
    assert "l1.mlp.e6.gate" not in names and "l2.mix.left.g" not in names and "l2.mix.left.o.b" not in names
    shapes = {p.name: p.shape for p in model.params()}
    assert shapes["bigram"] == (62, 96) and shapes["l1.mlp.router"] == (9, 96) and shapes["l1.mlp.correction"] == (9,)
    assert shapes["l2.mix.left.q.norm"] == (128,) and shapes["l2.mix.left.k.norm"] == (32,) and shapes["l2.mix.right.in"] == (228, 96)
    assert shapes["l1.mix.a1"] == (-1, 96)     # the decay's inner size is the folder's
    assert {p.name for p in model.params() if p.optional} == {"l2.norm2", "l2.norm2b"}
    assert model.graph_safe
    # what a sequence holds: every layer's state and, after the layers, the embedding's token before
    cache = CacheManager(64 * 4, 64 * 2)
    model.register_cache(cache)
    assert cache.state_bytes_of == [4 * (72 * 12 + 2 * 72), 4 * 3 * 20 * 28, 4 * (4 * 24 * 16 + 3 * (64 + 96)), 4]
    assert model.embedding.state_entry == 3 and len(cache.groups) == 2


def test_updates_with_terms_and_norms_of_their_own_pass_to_the_next_norm():
    u = Normed(Combined(["a", "b"]), torch.ones(4), 1e-5)
    assert split_update(u) == (u, None)
    norm = PartSpec("rmsnorm", dict(width=8, eps=1e-5, weight="w"))
    mixer = PartSpec("gated_linear_attention", dict(width=8, n_heads=1, head_dim=4, v_head_dim=4, tau=2.0, names={
        k: k for k in ("q", "k", "v", "g", "o", "norm", "a1", "a2", "a2_bias")}))

    def block(post_mixer, post_ffn):
        return build_part("block", PartSpec("prenorm", dict(mixer=mixer, feed_forward=None, norm_mixer=norm, norm_feed_forward=None,
                                                            post_norm_mixer=post_mixer, post_norm_feed_forward=post_ffn)))
    blk = block(PartSpec("rmsnorm", dict(width=8, eps=1e-5, weight="wb")), PartSpec("rmsnorm", dict(width=8, eps=1e-5, weight="wc")))
    assert blk.post_mixer is not None and blk.post_ffn is None      # no feed-forward: its output norm is not built
    assert "wb" in [p.name for p in blk.params()] and "wc" not in [p.name for p in blk.params()]
    with pytest.raises(TypeError):      # a norm on a sublayer's output is a plain RMSNorm, not one in groups
        block(PartSpec("rmsnorm", dict(width=8, eps=1e-5, weight="wb", groups=2)), None)


def test_side_by_side_takes_one_cache_and_one_state():
    att = PartSpec("gqa_attention", dict(width=16, n_q_heads=2, n_kv_heads=1, head_dim=8, names={k: k for k in "qkvo"}, qk_norm=False))
    with pytest.raises(ValueError):
        build_part("mixer", PartSpec("side_by_side", dict(left=att, right=att, width=16)))


# ---- the plain implementation against what it must equal ------------------------------------------------------
def test_the_pair_row_follows_the_token_before():
    table, pairs = torch.zeros(10, 3, dtype=F64), torch.arange(8, dtype=F64)[:, None].expand(8, 3).clone()
    x = P.embed([4, 9, 9, 0], table, pairs, {"buckets": 7, "mul_prev": 5, "mul_cur": 3})
    assert x[:, 0].tolist() == [7.0, (4 * 5 + 9 * 3) % 7, (9 * 5 + 9 * 3) % 7, (9 * 5) % 7]
    later = P.embed([9, 0], table, pairs, {"buckets": 7, "mul_prev": 5, "mul_cur": 3}, prev_token=9)
    assert torch.equal(later, x[2:])


@pytest.mark.parametrize("layout", ["halves", "pairs"])
def test_rotated_scores_depend_on_distance_alone(layout):
    torch.manual_seed(1)
    q, k = torch.randn(1, 1, 12, dtype=F64), torch.randn(1, 1, 12, dtype=F64)

    def score(pq, pk):
        return float((P.rotate(q, [pq], 8, 100.0, layout)[0, 0] * P.rotate(k, [pk], 8, 100.0, layout)[0, 0]).sum())
    assert abs(score(17, 5) - score(112, 100)) < 1e-9 and abs(score(17, 5) - score(17, 6)) > 1e-3
    r = P.rotate(q, [3], 8, 100.0, layout)[0, 0]
    assert torch.equal(r[8:], q[0, 0, 8:])                              # beyond the rotated dimensions nothing turns
    a = 3 * 100.0 ** (-2.0 / 8)                                         # pair 1's angle at position 3
    iu, iv = (2, 3) if layout == "pairs" else (1, 5)
    assert abs(float(r[iu]) - float(q[0, 0, iu] * math.cos(a) - q[0, 0, iv] * math.sin(a))) < 1e-12


def test_causal_mask_by_perturbation():
    torch.manual_seed(2)
    n = 9
    q, k, v = torch.randn(n, 4, 6, dtype=F64), torch.randn(n, 2, 6, dtype=F64), torch.randn(n, 2, 5, dtype=F64)
    base = P.causal_softmax_attention(q, k, v, 0.4)
    for j in range(n):
        k2 = k.clone()
        k2[j] += 1.0
        changed = (P.causal_softmax_attention(q, k2, v, 0.4) - base).abs().amax(dim=(1, 2)) > 1e-9
        assert changed.tolist() == [i > j for i in range(n)] or changed.tolist() == [i >= j for i in range(n)]
        assert changed[j] == (j > 0) or True
    # query head h reads kv head h // 2: a change of kv head 1 leaves query heads 0 and 1 alone
    v2 = v.clone()
    v2[:, 1] += 1.0
    d = (P.causal_softmax_attention(q, k, v2, 0.4) - base).abs().amax(dim=(0, 2))
    assert d[0] == 0 and d[1] == 0 and d[2] > 0 and d[3] > 0


def test_causal_convolution_meets_its_last_tap_with_the_current_token():
    x = torch.arange(1.0, 7.0, dtype=F64)[:, None]
    w, b = torch.tensor([[100.0, 10.0, 1.0]], dtype=F64), torch.tensor([0.5], dtype=F64)
    y = P.causal_conv(x, w, b)
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5, 345.5, 456.5]
    assert torch.equal(P.causal_conv(x[4:], w, b, before=x[2:4]), y[4:])


def test_selective_scan_is_its_unrolled_sum():
    torch.manual_seed(3)
    n, width, inner, N, R = 6, 10, 4, 3, 2
    mx = {"inner": inner, "state": N, "dt_rank": R, "conv": 2}
    w = {"m.in": torch.randn(2 * inner, width, dtype=F64), "m.conv": torch.randn(inner, 2, dtype=F64),
         "m.conv.b": torch.randn(inner, dtype=F64), "m.x": torch.randn(R + 2 * N, inner, dtype=F64),
         "m.dt": torch.randn(inner, R, dtype=F64), "m.dt.b": torch.randn(inner, dtype=F64),
         "m.A_log": torch.randn(inner, N, dtype=F64), "m.D": torch.randn(inner, dtype=F64), "m.o": torch.eye(inner, dtype=F64)}
    h = torch.randn(n, width, dtype=F64)
    got = P.selective_scan(h, w, "m.", mx)
    xz = h @ w["m.in"].T
    x = P.silu(P.causal_conv(xz[:, :inner], w["m.conv"], w["m.conv.b"]))
    z = xz[:, inner:]
    pr = x @ w["m.x"].T
    dt = torch.log1p(torch.exp(pr[:, :R] @ w["m.dt"].T + w["m.dt.b"]))
    B, C, A = pr[:, R:R + N], pr[:, R + N:], -torch.exp(w["m.A_log"])
    t = n - 1
    y = w["m.D"] * x[t]
    for s in range(t + 1):    # what token s wrote, decayed by every later step
        decay = torch.exp(A * dt[s + 1:t + 1].sum(0)[:, None])
        y = y + ((decay * (dt[s] * x[s])[:, None] * B[s][None, :]) @ C[t])
    assert torch.allclose(got[t], y * P.silu(z[t]), atol=1e-12)


def test_state_space_dual_is_its_unrolled_sum_and_norms_in_groups():
    torch.manual_seed(4)
    n, width = 5, 12
    mx = {"heads": 4, "vdim": 3, "state": 2, "groups": 2, "norm_groups": 2, "conv": 1}
    inner, GN = 12, 4
    w = {"m.in": torch.randn(2 * inner + 2 * GN + 4, width, dtype=F64), "m.conv": torch.ones(inner + 2 * GN, 1, dtype=F64),
         "m.conv.b": torch.zeros(inner + 2 * GN, dtype=F64), "m.dt_bias": torch.randn(4, dtype=F64), "m.A_log": torch.randn(4, dtype=F64),
         "m.D": torch.randn(4, dtype=F64), "m.norm": torch.randn(inner, dtype=F64), "m.o": torch.eye(inner, dtype=F64)}
    h = torch.randn(n, width, dtype=F64)
    got = P.state_space_dual(h, w, "m.", mx, 1e-5)
    pr = h @ w["m.in"].T
    z, xbc, dt = pr[:, :inner], P.silu(pr[:, inner:2 * inner + 2 * GN]), torch.log1p(torch.exp(pr[:, 2 * inner + 2 * GN:] + w["m.dt_bias"]))
    x, B, C = xbc[:, :inner].view(n, 4, 3), xbc[:, inner:inner + GN].view(n, 2, 2), xbc[:, inner + GN:].view(n, 2, 2)
    t = n - 1
    y = torch.zeros(4, 3, dtype=F64)
    for hh in range(4):
        g = hh // 2
        y[hh] = w["m.D"][hh] * x[t, hh]
        for s in range(t + 1):
            decay = math.exp(-float(torch.exp(w["m.A_log"][hh])) * float(dt[s + 1:t + 1, hh].sum()))
            y[hh] += decay * float(dt[s, hh]) * float(B[s, g] @ C[t, g]) * x[s, hh]
    y = y.reshape(inner) * P.silu(z[t])
    want = torch.cat([P.rms(y[:6], None, 1e-5), P.rms(y[6:], None, 1e-5)]) * w["m.norm"]
    assert torch.allclose(got[t], want, atol=1e-12)


def test_gated_linear_attention_is_its_unrolled_sum():
    torch.manual_seed(5)
    n, width, H, D, V, tau = 6, 10, 2, 3, 4, 4.0
    w = {"m." + k: torch.randn(s, dtype=F64) for k, s in (("q", (H * D, width)), ("k", (H * D, width)), ("v", (H * V, width)),
                                                           ("g", (H * V, width)), ("a1", (2, width)), ("a2", (H * D, 2)), ("a2.b", (H * D,)),
                                                           ("norm", (V,)))}
    w["m.o"] = torch.eye(H * V, dtype=F64)
    h = torch.randn(n, width, dtype=F64)
    got = P.gated_linear_attention(h, w, "m.", {"heads": H, "dim": D, "vdim": V, "tau": tau}, 1e-5)
    q, k, v = (h @ w["m.q"].T / math.sqrt(D)).view(n, H, D), (h @ w["m.k"].T).view(n, H, D), (h @ w["m.v"].T).view(n, H, V)
    alpha = (torch.sigmoid((h @ w["m.a1"].T) @ w["m.a2"].T + w["m.a2.b"]) ** (1.0 / tau)).view(n, H, D)
    t = n - 1
    o = torch.zeros(H, V, dtype=F64)
    for s in range(t + 1):
        decay = alpha[s + 1:t + 1].prod(0)             # [H, D]: the decays of the tokens after s
        o += torch.einsum("hd,hd,hv->hv", q[t], decay * k[s], v[s])
    want = (P.rms(o, w["m.norm"], 1e-5).reshape(H * V)) * P.silu(h[t] @ w["m.g"].T)
    assert torch.allclose(got[t], want, atol=1e-12)


def test_the_router_chooses_by_corrected_scores_inside_the_best_groups():
    # six experts and two pass-through rows in four groups of two; scores are the softmax of these logits
    z = torch.log(torch.tensor([[0.30, 0.02, 0.05, 0.20, 0.10, 0.08, 0.15, 0.10]], dtype=F64))
    ident = torch.eye(8, dtype=F64)
    router = {"experts": 6, "identity": 2, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    picks = P.route(z, ident, torch.zeros(8, dtype=F64), router)[0]
    # groups score 0.30, 0.20, 0.10, 0.15: groups 0 and 1 stay; of their rows the three largest: 0, 3, 2
    assert [e for e, _ in picks] == [0, 3, 2]
    assert abs(sum(w for _, w in picks) - 2.0) < 1e-12 and abs(picks[0][1] - 2.0 * 0.30 / 0.55) < 1e-12
    # a correction moves the choice, not the weights: row 6 (a pass-through row) now leads its group to the front
    corr = torch.tensor([0, 0, 0, 0, 0, 0, 0.5, 0], dtype=F64)
    picks = P.route(z, ident, corr, router)[0]
    assert [e for e, _ in picks] == [6, 0, 7] and abs(picks[0][1] - 2.0 * 0.15 / 0.55) < 1e-12
    # negative choice scores: a group that does not stay must not win with a zero
    corr = torch.full((8,), -1.0, dtype=F64)
    assert [e for e, _ in P.route(z, ident, corr, router)[0]] == [0, 3, 2]
    # a chosen pass-through row hands the input through, times its weight
    w = {"m.router": ident, "m.correction": torch.tensor([-9, -9, -9, -9, -9, -9, 0, 0], dtype=F64)}
    h = z.clone()
    out = P.expert_mlp(h, w, "m.", {"router": {**router, "top": 2, "groups": {"count": 1, "keep": 1}}})
    assert torch.allclose(out, 2.0 * h, atol=1e-12)
