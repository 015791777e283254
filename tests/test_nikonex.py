"""The Nikonex configuration, its model description, the cache's shared key/value rows, and the plain
implementation's own mechanisms (no GPU)."""
import copy
import math

import numpy as np
import pytest
import torch

from odin_infer_b200.cache import CacheManager, KVRequest
from odin_infer_b200.config import ConfigError, NikonexConfig, config_from_dict, lookup_architecture
from odin_infer_b200.engine.model import DecoderModel
from odin_infer_b200.parts.base import PartSpec, Scaled, Several, build_part, split_update, update_factor
from tests.plain import nikonex_plain as P

F64 = torch.float64
RAMP = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
MOE = {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 6, "top": 2, "scale": 2.5, "groups": {"count": 3, "keep": 2}},
       "shared": {"ff": 56}}
RAW = {"architecture": "Nikonex", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.4,
       "layers": [{"type": "latent_attention",
                   "mixer": {"heads": 3, "dim": 24, "rot_dim": 8, "vdim": 20, "q_rank": 36, "kv_rank": 40, "scale": 0.21,
                             "rot": {"dims": 8, "base": 5000.0, "scaling": RAMP}, "mask": {"size": 37}},
                   "mlp": MOE},
                  {"type": "retention", "mixer": {"heads": 2, "dim": 24, "vdim": 40, "decay": [0.9, 0.995],
                                                  "rot": {"dims": 16, "base": 1000.0}},
                   "mlp": None}]}


def test_configuration_reads_and_writes_the_same_keys():
    cfg = config_from_dict(RAW)
    assert isinstance(cfg, NikonexConfig) and cfg.to_dict() == RAW
    assert config_from_dict(cfg.to_dict()) == cfg
    assert cfg.layers[0].rot_scaling == (4.0, 64.0, 8.0, 1.0) and cfg.layers[0].window == 37 and not cfg.layers[1].has_mlp
    assert (cfg.layers[0].groups, cfg.layers[0].keep, cfg.layers[0].route_scale) == (3, 2, 2.5)


def test_absent_keys_mean_absent_mechanisms():
    raw = {"architecture": "Nikonex", "vocab": 50, "width": 40, "norm": {"eps": 1e-6},
           "layers": [{"type": "latent_attention",
                       "mixer": {"heads": 2, "dim": 16, "rot_dim": 4, "vdim": 8, "q_rank": 12, "kv_rank": 20, "scale": 0.3,
                                 "rot": {"dims": 4, "base": 100.0}},
                       "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 1}}},
                      {"type": "retention", "mixer": {"heads": 1, "dim": 8, "vdim": 8, "decay": [0.5]}, "mlp": None}]}
    cfg = config_from_dict(raw)
    a, b = cfg.layers
    assert (a.window, a.rot_scaling, a.groups, a.keep, a.route_scale, a.shared_ff) == (0, None, 1, 1, 1.0, 0)
    assert b.rot_dims == 0 and cfg.residual_mult == 1.0
    spec = lookup_architecture("Nikonex").build_spec(cfg)
    assert len(spec.position_encodings) == 1                       # retention without "rot" turns nothing
    assert spec.layers[0].args["feed_forward"].args["shared_gate"] is False
    assert spec.layers[1].args["feed_forward"] is None and spec.tolerated_tensors == ("l1.norm2",)


def test_every_fault_of_a_configuration_in_one_error():
    bad = copy.deepcopy(RAW)
    bad["layers"][0]["mixer"]["rot"]["dims"] = 6
    bad["layers"][0]["mixer"]["kv_rank"] = 0
    bad["layers"][0]["mlp"]["router"]["groups"] = {"count": 4, "keep": 1}
    bad["layers"][1]["mixer"]["decay"] = [0.9]
    bad["layers"].append({"type": "attention", "mixer": {}, "mlp": None})
    bad["norm"] = {}
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    text = str(e.value)
    for part in ("rot_dim", "kv_rank", "groups", "decay", "type must be", "eps"):
        assert part in text, part


def test_the_model_description_names_every_tensor_once():
    cfg = config_from_dict(RAW)
    model = DecoderModel(lookup_architecture("Nikonex").build_spec(cfg))
    names = {p.name: p.shape for p in model.params() if not p.optional}
    assert names["l0.mix.dkv"] == (48, 96) and names["l0.mix.uq"] == (3 * 32, 36) and names["l0.mix.uk"] == (72, 40)
    assert names["l0.mlp.shared.sg"] == (1, 96) and names["l0.mlp.e5.down"] == (96, 40) and names["l1.mix.g"] == (80, 96)
    assert "l1.norm2" not in names and "l0.norm2" in names and "l0.mlp.e0.gate" not in names
    assert model.graph_safe
    lat, ret = model.layers[0].mixer, model.layers[1].mixer
    assert lat.cache_request() == KVRequest(1, 48, 37, 0, 0, True) and lat.state_bytes() == 0
    assert ret.cache_request() is None and ret.state_bytes() == 4 * 2 * 24 * 40
    assert lat.pe.layout == "pairs" and ret.pe.layout == "halves" and lat.pe.gain == pytest.approx(0.1 * math.log(4.0) + 1.0)


def test_shared_rows_have_one_storage_and_a_group_of_their_own():
    cache = CacheManager(max_tokens=768, max_seq_len=384)
    a = cache.add_entry(KVRequest(1, 48, 37, 0, 0, True), 0)
    b = cache.add_entry(KVRequest(1, 48, 37), 0)
    c = cache.add_entry(KVRequest(1, 48, 37, 0, 0, True), 128)
    assert cache.line_of[a][0] != cache.line_of[b][0] and cache.line_of[a][0] == cache.line_of[c][0]
    g = cache.groups[cache.line_of[a][0]]
    assert g.n_lines == 2 and g.bytes_per_token(2) == 2 * 48 * 2
    assert cache.groups[cache.line_of[b][0]].bytes_per_token(2) == 2 * 48 * 2   # keys and values of one line
    slot = cache.take_slot()
    cache.extend(slot, 200)
    cache.after_step(slot)
    assert g.pool.n_held == 2   # the next query (position 200) sees from 164 on: pages 2 and 3
    cache.give_back_slot(slot)
    cache.check()


def test_a_factor_travels_with_the_pending_updates():
    a, b = torch.ones(2, 3), torch.ones(2, 2, 3)
    pend = Scaled(Several([a, b]), 0.25)
    delta, bias = split_update(pend)
    assert delta == [a, b] and bias is None and update_factor(pend) == 0.25 and update_factor(Several([a])) == 1.0


def test_block_with_two_norms_builds_and_refuses_what_it_cannot_do():
    norm = PartSpec("rmsnorm", dict(width=8, eps=1e-5, weight="n1"))
    mixer = PartSpec("retention", dict(width=8, n_heads=1, head_dim=4, v_head_dim=4, decay=[0.5],
                                       names={k: k for k in "qkvgo"}))
    blk = build_part("block", PartSpec("parallel", dict(mixer=mixer, feed_forward=None, norm=norm, residual_mult=0.5)))
    assert blk.norm_ffn is None and blk.residual_mult == 0.5
    with pytest.raises(ValueError):
        build_part("mixer", PartSpec("retention", dict(width=8, n_heads=2, head_dim=4, v_head_dim=4, decay=[0.5],
                                                       names={k: k for k in "qkvgo"})))
    with pytest.raises(ValueError):
        build_part("feed_forward", PartSpec("routed_experts", dict(width=8, inner=4, n_experts=6, top=3, names={}, gated=False,
                                                                   activation="relu2", score="sigmoid_in_groups", groups=3, keep=1)))


# ------------------------------------------------------------------ the plain implementation's own mechanisms
def test_ramp_frequencies_branch_by_branch():
    freqs, gain = P.ramp_frequencies(16, 100.0, {"factor": 5.0, "original": 40, "fast": 4.0, "slow": 0.5})
    base = [100.0 ** (-2.0 * i / 16) for i in range(8)]
    # pair_of(4) = 16 ln(40 / 8 pi) / (2 ln 100) = 0.807 -> lo 0; pair_of(0.5) = 16 ln(40 / pi) / (2 ln 100) = 4.42 -> hi 5
    assert freqs[0] == pytest.approx(base[0]) and freqs[5] == pytest.approx(base[5] / 5.0) and freqs[7] == pytest.approx(base[7] / 5.0)
    assert freqs[2] == pytest.approx(base[2] * (1 - 0.4) + base[2] / 5.0 * 0.4)
    assert gain == pytest.approx(0.1 * math.log(5.0) + 1.0)
    assert P.ramp_frequencies(16, 100.0, None) == (base, 1.0)
    # a ramp whose two ends fall on one pair is a step
    freqs, _ = P.ramp_frequencies(8, 10.0, {"factor": 2.0, "original": 10, "fast": 1.0, "slow": 1.0})
    lo = max(math.floor(8 * math.log(10 / (2 * math.pi)) / (2 * math.log(10.0))), 0)
    assert freqs[lo] == pytest.approx(10.0 ** (-2.0 * lo / 8)) and freqs[3] == pytest.approx(10.0 ** (-6.0 / 8) / 2.0)


def test_the_rotation_knows_the_engine_s_tables():
    """The position encoding part's tables (host side) against the plain frequencies, gain included."""
    from odin_infer_b200.parts.position import RotaryEncoding

    class Rt:
        device = "cpu"
    scaling = {"factor": 3.0, "original": 50, "fast": 6.0, "slow": 0.7}
    pe = RotaryEncoding(12, 777.0, ramp=scaling, layout="pairs", exact_angles=True)
    pe.prepare(Rt(), 300)
    freqs, gain = P.ramp_frequencies(12, 777.0, scaling)
    want = np.array([[math.cos(p * f) * gain for f in freqs] for p in (0, 1, 299)])
    assert np.allclose(pe.cos[[0, 1, 299]].numpy(), want, atol=1e-6) and pe.sin.shape == (300, 6)
    assert abs(float(pe.sin[299, 0]) - math.sin(299.0) * gain) < 1e-6


@pytest.mark.parametrize("layout", ["pairs", "halves"])
def test_rotated_scores_depend_on_distance_alone(layout):
    torch.manual_seed(1)
    q, k = torch.randn(1, 1, 12, dtype=F64), torch.randn(1, 1, 12, dtype=F64)
    freqs, _ = P.ramp_frequencies(8, 50.0, None)
    def score(pq, pk):
        return float((P.rotate(q, [pq], freqs, 1.0, layout) * P.rotate(k, [pk], freqs, 1.0, layout)).sum())
    assert score(7, 3) == pytest.approx(score(104, 100)) and score(7, 3) != pytest.approx(score(8, 3))
    r = P.rotate(q, [5], freqs, 1.0, layout)
    assert torch.equal(r[..., 8:], q[..., 8:]) and float(r.norm()) == pytest.approx(float(q.norm()))
    # which elements turn together
    one = torch.zeros(1, 1, 12, dtype=F64)
    one[0, 0, 0] = 1.0
    moved = P.rotate(one, [1], freqs, 1.0, layout)[0, 0].nonzero().flatten().tolist()
    assert moved == ([0, 1] if layout == "pairs" else [0, 4])


def test_window_by_perturbation():
    torch.manual_seed(2)
    n, window = 12, 4
    q, k, v = (torch.randn(n, 2, 6, dtype=F64) for _ in range(3))
    ref = P.windowed_softmax_attention(q, k, v, 0.3, window)
    for j in range(n):
        v2 = v.clone()
        v2[j] += 1.0
        changed = (P.windowed_softmax_attention(q, k, v2, 0.3, window) - ref).abs().amax(dim=(1, 2)) > 1e-12
        assert changed.nonzero().flatten().tolist() == [i for i in range(n) if 0 <= i - j < window], j
    assert torch.allclose(P.windowed_softmax_attention(q, k, v, 0.3, 1), v)
    assert torch.allclose(P.windowed_softmax_attention(q, k, v, 0.3, 0), P.windowed_softmax_attention(q, k, v, 0.3, n))


def test_latent_attention_is_attention_over_expanded_keys():
    """The mixer against an assembly of its own pieces, and its window against a key pushed out of sight."""
    torch.manual_seed(3)
    mx = {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "q_rank": 7, "kv_rank": 9, "scale": 0.4, "mask": {"size": 3},
          "rot": {"dims": 4, "base": 30.0, "scaling": {"factor": 2.0, "original": 8, "fast": 2.0, "slow": 0.5}}}
    w = {"m.dq": torch.randn(7, 10, dtype=F64), "m.dq.norm": torch.rand(7, dtype=F64) + 0.5, "m.uq": torch.randn(20, 7, dtype=F64),
         "m.dkv": torch.randn(13, 10, dtype=F64), "m.dkv.norm": torch.rand(9, dtype=F64) + 0.5, "m.uk": torch.randn(12, 9, dtype=F64),
         "m.uv": torch.randn(10, 9, dtype=F64), "m.o": torch.randn(10, 10, dtype=F64)}
    h = torch.randn(6, 10, dtype=F64)
    out = P.latent_attention(h, w, "m.", mx, 1e-5)
    h2 = h.clone()
    h2[1] = torch.randn(10, dtype=F64)        # token 1 is seen by 1, 2, 3 and by nobody later
    diff = (P.latent_attention(h2, w, "m.", mx, 1e-5) - out).abs().amax(dim=1) > 1e-12
    assert diff.tolist() == [False, True, True, True, False, False]
    # the scale multiplies the whole score, rotated part included
    mx2 = dict(mx, scale=0.0)
    flat = P.latent_attention(h, w, "m.", mx2, 1e-5)
    c = P.rms(h @ w["m.dkv"].T[:, :9], w["m.dkv.norm"], 1e-5)
    v = (c @ w["m.uv"].T).view(6, 2, 5)
    want = torch.stack([v[max(0, i - 2):i + 1].mean(dim=0) for i in range(6)]).reshape(6, 10) @ w["m.o"].T
    assert torch.allclose(flat, want)


def test_retention_is_its_unrolled_sum_and_carries_its_state():
    torch.manual_seed(4)
    mx = {"heads": 2, "dim": 4, "vdim": 3, "decay": [0.5, 0.9], "rot": {"dims": 2, "base": 10.0}}
    w = {"m." + k: torch.randn(8 if k in "qk" else 6, 5, dtype=F64) for k in "qkvg"}
    w["m.o"] = torch.randn(5, 6, dtype=F64)
    h = torch.randn(7, 5, dtype=F64)
    out = P.retention(h, w, "m.", mx, 1e-5)
    # o_t = sum_{s <= t} decay^(t - s) (q_t . k_s) v_s with rotated q, k and k / sqrt(dim)
    freqs, _ = P.ramp_frequencies(2, 10.0, None)
    q = P.rotate((h @ w["m.q"].T).view(7, 2, 4), range(7), freqs, 1.0, "halves")
    k = P.rotate((h @ w["m.k"].T).view(7, 2, 4), range(7), freqs, 1.0, "halves") / 2.0
    v = (h @ w["m.v"].T).view(7, 2, 3)
    o = torch.zeros(7, 2, 3, dtype=F64)
    for t in range(7):
        for s in range(t + 1):
            for hd, d in enumerate(mx["decay"]):
                o[t, hd] += d ** (t - s) * float(q[t, hd] @ k[s, hd]) * v[s, hd]
    g = h @ w["m.g"].T
    want = (P.rms(o, None, 1e-5).reshape(7, 6) * g * torch.sigmoid(g)) @ w["m.o"].T
    assert torch.allclose(out, want)
    # in two portions, with the state handed on
    state = [torch.zeros(4, 3, dtype=F64) for _ in range(2)]
    a = P.retention(h[:3], w, "m.", mx, 1e-5, positions=range(3), state=state)
    b = P.retention(h[3:], w, "m.", mx, 1e-5, positions=range(3, 7), state=state)
    assert torch.allclose(torch.cat([a, b]), out)


def test_the_router_chooses_inside_the_best_groups():
    router = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    w = torch.eye(6, dtype=F64)
    # scores by expert: group 0 holds the single best expert, group 1 the best pair
    z = torch.tensor([[3.0, -4.0, 1.5, 1.4, 1.0, -1.0]], dtype=F64)
    ids, wts = P.route(z, w, router)
    assert ids == [[2, 3]]
    s = torch.sigmoid(z[0])
    assert torch.allclose(wts[0], torch.stack([s[2], s[3]]) / (s[2] + s[3]) * 2.0)
    ids, _ = P.route(z, w, dict(router, groups={"count": 3, "keep": 2}))
    assert ids == [[2, 3]]      # the group of the single best expert is only the third (0.97 against 1.62 and 1.0)
    ids, _ = P.route(z, w, dict(router, groups={"count": 3, "keep": 3}))
    assert ids == [[0, 2]]
    ids, wts = P.route(z, w, {"experts": 6, "top": 3})
    assert ids == [[0, 2, 3]] and float(wts.sum()) == pytest.approx(1.0)
    # ties go to the lower expert, and to the lower group
    ids, _ = P.route(torch.zeros(1, 6, dtype=F64), w, router)
    assert ids == [[0, 1]]


def test_the_shared_expert_is_gated_per_token():
    torch.manual_seed(5)
    mlp = {"kind": "moe", "expert": {"ff": 4}, "router": {"experts": 2, "top": 1}, "shared": {"ff": 3}}
    w = {"f.router": torch.randn(2, 5, dtype=F64), "f.shared.up": torch.randn(3, 5, dtype=F64),
         "f.shared.down": torch.randn(5, 3, dtype=F64), "f.shared.sg": torch.randn(1, 5, dtype=F64)}
    for e in range(2):
        w[f"f.e{e}.up"], w[f"f.e{e}.down"] = torch.randn(4, 5, dtype=F64), torch.randn(5, 4, dtype=F64)
    h = torch.randn(3, 5, dtype=F64)
    full = P.expert_mlp(h, w, "f.", mlp)
    bare = P.expert_mlp(h, w, "f.", {k: v for k, v in mlp.items() if k != "shared"})
    gate = torch.sigmoid(h @ w["f.shared.sg"].T)
    assert torch.allclose(full - bare, gate * (torch.relu(h @ w["f.shared.up"].T) ** 2 @ w["f.shared.down"].T))
    assert torch.allclose(P.relu2_mlp(-h.abs(), torch.eye(5, dtype=F64), torch.eye(5, dtype=F64)), torch.zeros(3, 5, dtype=F64))
