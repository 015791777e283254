"""Configuration of the Meropel decoder: token embeddings plus a hashed table of token pairs; blocks whose mixer and
feed-forward each stand between two norms (one on the sublayer's input, one on its output); mixers are two branches side
by side (softmax attention beside a state-space recurrence) or gated linear attention; feed-forwards are a gated one or
experts chosen among groups by corrected softmax scores, some of whose router rows hand the input through unchanged.

config.json keys: "architecture", "vocab", "width", "norm" {"eps"}, "logit_scale" (absent: 1), "embedding" {"bigram"
{"buckets", "mul_prev", "mul_cur"}} (absent: no pair table) and "layers": a list of

    {"type": "parallel" | "parallel_2" | "gla", "mixer": {...}, "mlp": null | {...}}

parallel:   mixer {left {heads, kv_heads, dim, vdim, scale, rot {dims, base} (absent: no rotation)}, left_scale,
            right {inner, state, dt_rank, conv}, right_scale}: attention with a sigmoid gate per head beside a selective scan.
parallel_2: mixer {left {as above}, right {heads, vdim, state, groups, norm_groups, conv}}: attention with biases and a norm
            over the whole q and k projections, rotation in pairs (2i, 2i+1), beside a scalar-decay recurrence per head.
gla:        mixer {heads, dim, vdim, tau}.
mlp: {"kind": "dense", "ff"} or {"kind": "moe", "expert" {"ff"}, "router" {"experts", "top", "scale" (absent: 1), "identity"
(absent: 0), "groups" {"count", "keep"} (absent: one group)}, "shared" {"ff"} (optional)}.
"""
from __future__ import annotations

import dataclasses

from .base import KeyReader, ModelConfig

LAYER_TYPES = ("parallel", "parallel_2", "gla")


@dataclasses.dataclass(frozen=True)
class MeropelAttention:
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 0.0
    rot_dims: int = 0
    rot_base: float = 10000.0

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return out


@dataclasses.dataclass(frozen=True)
class MeropelLayer:
    type: str
    left: MeropelAttention | None = None
    # parallel: the selective scan and the two factors
    inner: int = 0
    state: int = 0
    dt_rank: int = 0
    conv: int = 0
    left_scale: float = 1.0
    right_scale: float = 1.0
    # parallel_2: the recurrence over heads (state and conv as above)
    heads: int = 0
    vdim: int = 0
    groups: int = 1
    norm_groups: int = 1
    # gla (heads and vdim as above)
    dim: int = 0
    tau: float = 1.0
    # feed-forward
    mlp_kind: str | None = None       # None, "dense", "moe"
    ff: int = 0
    experts: int = 0
    top: int = 0
    identity: int = 0
    route_scale: float = 1.0
    expert_groups: int = 1
    keep: int = 1
    shared_ff: int = 0

    def mixer_dict(self) -> dict:
        if self.type == "gla":
            return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.type == "parallel":
            return {"left": self.left.to_dict(), "left_scale": self.left_scale,
                    "right": {"inner": self.inner, "state": self.state, "dt_rank": self.dt_rank, "conv": self.conv},
                    "right_scale": self.right_scale}
        return {"left": self.left.to_dict(),
                "right": {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                          "norm_groups": self.norm_groups, "conv": self.conv}}

    def mlp_dict(self):
        if self.mlp_kind is None:
            return None
        if self.mlp_kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top, "scale": self.route_scale, "identity": self.identity,
                  "groups": {"count": self.expert_groups, "keep": self.keep}}
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": router}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


def _sub(reader: KeyReader, key: str, where: str) -> KeyReader:
    raw = reader.raw.get(key)
    if not isinstance(raw, dict):
        reader.problems.append(f"missing key '{key}'")
        raw = {}
    return KeyReader(raw, where)


def _take(into: KeyReader, sub: KeyReader, label: str) -> None:
    into.problems += [f"{label}: {p}" for p in sub.problems]


@dataclasses.dataclass(frozen=True)
class MeropelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    logit_scale: float = 1.0
    bigram: tuple | None = None       # (buckets, mul_prev, mul_cur)
    layers: tuple[MeropelLayer, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "MeropelConfig":
        r = KeyReader(raw, where)
        vocab, width = r.get("vocab", int), r.get("width", int)
        norm = _sub(r, "norm", "norm")
        eps = norm.get("eps", float)
        _take(r, norm, "norm")
        logit_scale = r.get("logit_scale", float, 1.0)
        r.require(vocab > 0 and width > 0, f"'vocab' and 'width' must be positive, got {vocab} and {width}")
        r.require(eps > 0, f"norm eps must be positive, got {eps}")
        bigram = None
        emb = raw.get("embedding")
        if isinstance(emb, dict) and emb.get("bigram") is not None:
            b = _sub(KeyReader(emb, "embedding"), "bigram", "embedding bigram")
            bigram = (b.get("buckets", int), b.get("mul_prev", int), b.get("mul_cur", int))
            b.require(bigram[0] > 0, f"buckets must be positive, got {bigram[0]}")
            _take(r, b, "embedding bigram")
        raw_layers = raw.get("layers")
        if not (isinstance(raw_layers, list) and raw_layers):
            r.problems.append("key 'layers' must be a list with a layer in it")
            raw_layers = []
        layers = [cls._layer(r, i, e if isinstance(e, dict) else {}) for i, e in enumerate(raw_layers)]
        r.finish()
        return cls(architecture=str(raw.get("architecture", "Meropel")), vocab=vocab, width=width, norm_eps=eps,
                   logit_scale=logit_scale, bigram=bigram, layers=tuple(layers))

    @staticmethod
    def _attention(m: KeyReader, label: str) -> MeropelAttention:
        a = _sub(m, "left", label)
        heads, kv, dim, vdim = a.get("heads", int), a.get("kv_heads", int), a.get("dim", int), a.get("vdim", int)
        scale = a.get("scale", float)
        a.require(heads > 0 and kv > 0 and dim > 0 and vdim > 0 and heads % max(kv, 1) == 0,
                  f"needs positive heads, kv_heads, dim, vdim and heads a multiple of kv_heads, got {heads}, {kv}, {dim}, {vdim}")
        a.require(scale > 0, f"scale must be positive, got {scale}")
        dims, base = 0, 10000.0
        if a.raw.get("rot") is not None:
            rot = _sub(a, "rot", "rot")
            dims, base = rot.get("dims", int), rot.get("base", float)
            rot.require(dims >= 0 and dims % 2 == 0 and dims <= max(dim, 0), f"dims ({dims}) must be even and at most {dim}")
            rot.require(base > 0, f"base must be positive, got {base}")
            _take(a, rot, "rot")
        _take(m, a, "left")
        return MeropelAttention(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, rot_dims=dims, rot_base=base)

    @classmethod
    def _layer(cls, r: KeyReader, i: int, entry: dict) -> MeropelLayer:
        kind = entry.get("type")
        if kind not in LAYER_TYPES:
            r.problems.append(f"layer {i}: type must be one of {', '.join(LAYER_TYPES)}, got {kind!r}")
            return MeropelLayer(type="gla")
        m = KeyReader(entry.get("mixer") if isinstance(entry.get("mixer"), dict) else {}, f"layer {i} mixer")
        if kind == "gla":
            heads, dim, vdim, tau = m.get("heads", int), m.get("dim", int), m.get("vdim", int), m.get("tau", float)
            m.require(heads > 0 and dim > 0 and vdim > 0 and tau > 0, f"heads, dim, vdim and tau must be positive, got {heads}, {dim}, {vdim}, {tau}")
            layer = MeropelLayer(type=kind, heads=heads, dim=dim, vdim=vdim, tau=tau)
        elif kind == "parallel":
            left = cls._attention(m, "left")
            rg = _sub(m, "right", "right")
            inner, state, rank, conv = rg.get("inner", int), rg.get("state", int), rg.get("dt_rank", int), rg.get("conv", int)
            rg.require(min(inner, state, rank, conv) > 0, f"inner, state, dt_rank and conv must be positive, got {inner}, {state}, {rank}, {conv}")
            _take(m, rg, "right")
            layer = MeropelLayer(type=kind, left=left, inner=inner, state=state, dt_rank=rank, conv=conv,
                                 left_scale=m.get("left_scale", float, 1.0), right_scale=m.get("right_scale", float, 1.0))
        else:
            left = cls._attention(m, "left")
            rg = _sub(m, "right", "right")
            heads, vdim, state, conv = rg.get("heads", int), rg.get("vdim", int), rg.get("state", int), rg.get("conv", int)
            groups, ngroups = rg.get("groups", int, 1), rg.get("norm_groups", int, 1)
            rg.require(min(heads, vdim, state, conv, groups, ngroups) > 0 and heads % max(groups, 1) == 0
                       and (heads * vdim) % max(ngroups, 1) == 0,
                       f"needs positive sizes, heads a multiple of groups and heads * vdim a multiple of norm_groups, got heads {heads}, "
                       f"vdim {vdim}, state {state}, conv {conv}, groups {groups}, norm_groups {ngroups}")
            _take(m, rg, "right")
            layer = MeropelLayer(type=kind, left=left, heads=heads, vdim=vdim, state=state, conv=conv, groups=groups,
                                 norm_groups=ngroups)
        r.problems += [f"layer {i} mixer: {p}" for p in m.problems]
        mlp = entry.get("mlp")
        if mlp is not None:
            k = KeyReader(mlp if isinstance(mlp, dict) else {}, f"layer {i} mlp")
            mk = k.raw.get("kind")
            if mk == "dense":
                ff = k.get("ff", int)
                k.require(ff > 0, f"ff must be positive, got {ff}")
                layer = dataclasses.replace(layer, mlp_kind="dense", ff=ff)
            elif mk == "moe":
                ex, ro = _sub(k, "expert", "expert"), _sub(k, "router", "router")
                ff, n, top = ex.get("ff", int), ro.get("experts", int), ro.get("top", int)
                ident, rscale = ro.get("identity", int, 0), ro.get("scale", float, 1.0)
                groups, keep = 1, 1
                if ro.raw.get("groups") is not None:
                    gr = _sub(ro, "groups", "groups")
                    groups, keep = gr.get("count", int), gr.get("keep", int)
                    _take(ro, gr, "groups")
                shared_ff = 0
                if k.raw.get("shared") is not None:
                    sh = _sub(k, "shared", "shared")
                    shared_ff = sh.get("ff", int)
                    sh.require(shared_ff > 0, f"ff must be positive, got {shared_ff}")
                    _take(k, sh, "shared")
                _take(k, ex, "expert")
                _take(k, ro, "router")
                rows = n + ident
                k.require(ff > 0 and n > 0 and ident >= 0 and 0 < top <= max(rows, 1),
                          f"needs ff > 0, experts > 0 and 0 < top <= experts + identity, got ff {ff}, experts {n}, identity {ident}, top {top}")
                k.require(groups >= 1 and rows % max(groups, 1) == 0 and 1 <= keep <= max(groups, 1)
                          and keep * (rows // max(groups, 1)) >= top,
                          f"{rows} router rows in {groups} groups of which {keep} stay cannot give {top} experts a token")
                layer = dataclasses.replace(layer, mlp_kind="moe", ff=ff, experts=n, top=top, identity=ident, route_scale=rscale,
                                            expert_groups=groups, keep=keep, shared_ff=shared_ff)
            else:
                k.problems.append(f"kind must be 'dense' or 'moe', got {mk!r}")
            r.problems += [f"layer {i} mlp: {p}" for p in k.problems]
        return layer

    def to_dict(self) -> dict:
        layers = [{"type": l.type, "mixer": l.mixer_dict(), "mlp": l.mlp_dict()} for l in self.layers]
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "logit_scale": self.logit_scale, "layers": layers}
        if self.bigram is not None:
            out["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))}
        return out
