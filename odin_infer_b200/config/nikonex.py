"""Configuration of the Nikonex decoder: blocks whose mixer and feed-forward read two norms of the same residual
stream and whose updates are added times one factor; mixers are attention through latents (a query latent, one
key/value latent per token, a rotated key part shared by the heads, a sliding window) or retention (linear attention
with a fixed decay per head); feed-forwards are experts chosen by a sigmoid router inside the best groups of experts,
beside a shared expert behind a per-token gate.

config.json keys: "architecture", "vocab", "width", "norm" {"eps"}, "residual_mult" (absent: 1) and "layers": a list of

    {"type": "latent_attention" | "retention", "mixer": {...}, "mlp": null | {...}}

latent_attention mixer: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask {size} (absent: every earlier key),
rot {dims, base, scaling {factor, original, fast, slow} (optional)}.
retention mixer: heads, dim, vdim, decay [one per head], rot {dims, base} (absent: no rotation).
mlp: {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale" (absent: 1), "groups" {"count", "keep"}
(absent: one group)}, "shared": {"ff"} (optional)}.
"""
from __future__ import annotations

import dataclasses

from .base import KeyReader, ModelConfig

LAYER_TYPES = ("latent_attention", "retention")


@dataclasses.dataclass(frozen=True)
class NikonexLayer:
    type: str
    heads: int = 0
    dim: int = 0
    vdim: int = 0
    # latent attention
    rot_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    window: int = 0                   # 0: every earlier key
    # retention
    decay: tuple = ()
    # rotation (both)
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_scaling: tuple | None = None  # (factor, original, fast, slow)
    # feed-forward
    has_mlp: bool = False
    ff: int = 0
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0

    def mixer_dict(self) -> dict:
        rot = {"dims": self.rot_dims, "base": self.rot_base}
        if self.rot_scaling is not None:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.rot_scaling))
        if self.type == "retention":
            out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
            if self.rot_dims:
                out["rot"] = rot
            return out
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
               "kv_rank": self.kv_rank, "scale": self.scale, "rot": rot}
        if self.window:
            out["mask"] = {"size": self.window}
        return out

    def mlp_dict(self):
        if not self.has_mlp:
            return None
        router = {"experts": self.experts, "top": self.top, "scale": self.route_scale,
                  "groups": {"count": self.groups, "keep": self.keep}}
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": router}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


def _sub(reader: KeyReader, key: str, where: str) -> KeyReader:
    raw = reader.raw.get(key)
    return KeyReader(raw if isinstance(raw, dict) else {}, where)


@dataclasses.dataclass(frozen=True)
class NikonexConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    residual_mult: float = 1.0
    layers: tuple[NikonexLayer, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "NikonexConfig":
        r = KeyReader(raw, where)
        vocab, width = r.get("vocab", int), r.get("width", int)
        norm = _sub(r, "norm", where + " norm")
        eps = norm.get("eps", float)
        r.problems += norm.problems
        mult = r.get("residual_mult", float, 1.0)
        r.require(vocab > 0 and width > 0, f"'vocab' and 'width' must be positive, got {vocab} and {width}")
        r.require(eps > 0, f"norm eps must be positive, got {eps}")
        raw_layers = raw.get("layers")
        if not (isinstance(raw_layers, list) and raw_layers):
            r.problems.append("key 'layers' must be a list with a layer in it")
            raw_layers = []
        layers = [cls._layer(r, i, e if isinstance(e, dict) else {}) for i, e in enumerate(raw_layers)]
        r.finish()
        return cls(architecture=str(raw.get("architecture", "Nikonex")), vocab=vocab, width=width, norm_eps=eps,
                   residual_mult=mult, layers=tuple(layers))

    @staticmethod
    def _rot(m: KeyReader, i: int, limit: int, needed: bool):
        """(dims, base, scaling) of a mixer's "rot"."""
        if m.raw.get("rot") is None:
            if needed:
                m.problems.append("missing key 'rot'")
            return 0, 10000.0, None
        rot = _sub(m, "rot", f"layer {i} mixer rot")
        dims, base = rot.get("dims", int), rot.get("base", float)
        scaling = None
        if rot.raw.get("scaling") is not None:
            sc = _sub(rot, "scaling", f"layer {i} mixer rot scaling")
            scaling = tuple(sc.get(k, float) for k in ("factor", "original", "fast", "slow"))
            sc.require(all(v > 0 for v in scaling), f"factor, original, fast and slow must be positive, got {scaling}")
            rot.problems += [f"scaling: {p}" for p in sc.problems]
        rot.require(dims >= 0 and dims % 2 == 0 and dims <= limit, f"dims ({dims}) must be even and at most {limit}")
        rot.require(base > 0 and base != 1.0, f"base must be positive and not 1, got {base}")
        m.problems += [f"rot: {p}" for p in rot.problems]
        return dims, base, scaling

    @classmethod
    def _layer(cls, r: KeyReader, i: int, entry: dict) -> NikonexLayer:
        kind = entry.get("type")
        if kind not in LAYER_TYPES:
            r.problems.append(f"layer {i}: type must be one of {', '.join(LAYER_TYPES)}, got {kind!r}")
            return NikonexLayer(type="retention")
        m = KeyReader(entry.get("mixer") if isinstance(entry.get("mixer"), dict) else {}, f"layer {i} mixer")
        heads, dim, vdim = m.get("heads", int), m.get("dim", int), m.get("vdim", int)
        m.require(heads > 0 and dim > 0 and vdim > 0, f"heads, dim and vdim must be positive, got {heads}, {dim}, {vdim}")
        if kind == "latent_attention":
            rot_dim, q_rank, kv_rank = m.get("rot_dim", int), m.get("q_rank", int), m.get("kv_rank", int)
            scale = m.get("scale", float)
            window = 0
            if m.raw.get("mask") is not None:
                window = _sub(m, "mask", f"layer {i} mixer mask").get("size", int, 0)
            m.require(rot_dim >= 0 and rot_dim % 2 == 0, f"rot_dim must be even and not negative, got {rot_dim}")
            m.require(q_rank > 0 and kv_rank > 0, f"q_rank and kv_rank must be positive, got {q_rank} and {kv_rank}")
            m.require(scale > 0, f"scale must be positive, got {scale}")
            m.require(window >= 0, f"mask size must not be negative, got {window}")
            dims, base, scaling = cls._rot(m, i, max(rot_dim, 0), needed=rot_dim > 0)
            m.require(rot_dim == 0 or dims == rot_dim, f"rot dims ({dims}) must be rot_dim ({rot_dim}): the rotated part turns as a whole")
            layer = NikonexLayer(type=kind, heads=heads, dim=dim, vdim=vdim, rot_dim=rot_dim, q_rank=q_rank, kv_rank=kv_rank,
                                 scale=scale, window=window, rot_dims=dims, rot_base=base, rot_scaling=scaling)
        else:
            decay = m.raw.get("decay")
            ok = isinstance(decay, list) and len(decay) == heads and all(
                isinstance(d, (int, float)) and not isinstance(d, bool) and 0 <= d <= 1 for d in decay)
            m.require(ok, f"decay must list one number in [0, 1] per head ({heads}), got {decay!r}")
            dims, base, scaling = cls._rot(m, i, max(dim, 0), needed=False)
            m.require(scaling is None, "retention rotates without a frequency scaling")
            layer = NikonexLayer(type=kind, heads=heads, dim=dim, vdim=vdim, decay=tuple(float(d) for d in decay) if ok else (),
                                 rot_dims=dims, rot_base=base)
        r.problems += [f"layer {i} mixer: {p}" for p in m.problems]
        mlp = entry.get("mlp")
        if mlp is not None:
            k = KeyReader(mlp if isinstance(mlp, dict) else {}, f"layer {i} mlp")
            mk = k.raw.get("kind", "moe")
            if mk != "moe":
                k.problems.append(f"kind must be 'moe', got {mk!r}")
            ex, ro = _sub(k, "expert", "expert"), _sub(k, "router", "router")
            ff, n, top = ex.get("ff", int), ro.get("experts", int), ro.get("top", int)
            rscale = ro.get("scale", float, 1.0)
            groups, keep = 1, 1
            if ro.raw.get("groups") is not None:
                gr = _sub(ro, "groups", "groups")
                groups, keep = gr.get("count", int), gr.get("keep", int)
                ro.problems += [f"groups: {p}" for p in gr.problems]
            shared_ff = 0
            if k.raw.get("shared") is not None:
                sh = _sub(k, "shared", "shared")
                shared_ff = sh.get("ff", int)
                sh.require(shared_ff > 0, f"ff must be positive, got {shared_ff}")
                k.problems += [f"shared: {p}" for p in sh.problems]
            k.problems += [f"expert: {p}" for p in ex.problems] + [f"router: {p}" for p in ro.problems]
            k.require(ff > 0 and n > 0 and 0 < top <= max(n, 1), f"needs ff > 0 and 0 < top <= experts, got ff {ff}, top {top}, experts {n}")
            k.require(groups >= 1 and n % max(groups, 1) == 0 and 1 <= keep <= max(groups, 1)
                      and keep * (n // max(groups, 1)) >= top,
                      f"{n} experts in {groups} groups of which {keep} stay cannot give {top} experts a token")
            layer = dataclasses.replace(layer, has_mlp=True, ff=ff, experts=n, top=top, route_scale=rscale, groups=groups,
                                        keep=keep, shared_ff=shared_ff)
            r.problems += [f"layer {i} mlp: {p}" for p in k.problems]
        return layer

    def to_dict(self) -> dict:
        layers = [{"type": l.type, "mixer": l.mixer_dict(), "mlp": l.mlp_dict()} for l in self.layers]
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "layers": layers}
