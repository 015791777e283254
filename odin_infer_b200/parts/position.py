"""Position encodings."""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_part


@register_part("position_encoding", "rope")
class RotaryEncoding(PositionEncoding):
    """Half-split rotary encoding: pairs (i, i + rotary_dim/2), frequency
    1 / theta^(i / (rotary_dim/2)), angle = position * frequency, both formed in
    32-bit as the reference does (infer/forward.odin:67-70); cos and sin of that
    angle are tabulated on the host, so every kernel reads the same values.

    stretch = {"factor", "low", "high", "original"}: frequencies are stretched by their wavelength
    l = 2 pi / f: kept where l < original / high, divided by `factor` where l > original / low, and
    between the two blended, (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
    precise (always so with a stretch or a ramp): the frequencies are formed in double and rounded to 32-bit once,
    instead of by the reference's 32-bit power.

    ramp = {"factor", "original", "fast", "slow"}: frequencies are scaled down by the index of their pair.  With
    p(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), the pair whose wave turns t times in `original`
    positions, lo = max(floor(p(fast)), 0), hi = min(ceil(p(slow)), rotary_dim - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at f_i (1 - r_i) + f_i r_i / factor, and cos and
    sin are both multiplied by 0.1 ln(factor) + 1 (the tables hold the products).
    layout: which elements of a head form pair i: "halves" (i, i + rotary_dim / 2) or "pairs" (2i, 2i + 1); the
    tables are the same, the mixer's kernel reads the layout.
    exact_angles: position times frequency, cosine and sine are formed in double and rounded to 32-bit once (more
    than the 32-bit angle that the first architecture's reference forms)."""

    graph_safe = True

    def __init__(self, rotary_dim: int, theta: float, stretch: dict | None = None, precise: bool = False,
                 ramp: dict | None = None, layout: str = "halves", exact_angles: bool = False):
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim must be even, got {rotary_dim}")
        if layout not in ("halves", "pairs"):
            raise ValueError(f"a rotation's layout is 'halves' or 'pairs', got {layout!r}")
        self.rotary_dim, self.theta, self.precise = rotary_dim, float(theta), bool(precise)
        self.layout, self.exact_angles = layout, bool(exact_angles)
        self.ramp, self.gain = None, 1.0
        if ramp is not None:
            if stretch is not None:
                raise ValueError("a rotation takes a stretch by wavelength or a ramp by pair, not both")
            self.ramp = {k: float(ramp[k]) for k in ("factor", "original", "fast", "slow")}
            if not (self.ramp["factor"] > 0 and self.ramp["original"] > 0 and self.ramp["fast"] > 0 and self.ramp["slow"] > 0):
                raise ValueError(f"a frequency ramp needs positive factor, original, fast and slow, got {self.ramp}")
            self.gain = 0.1 * float(np.log(self.ramp["factor"])) + 1.0
        self.stretch = None
        if stretch is not None:
            self.stretch = {k: float(stretch[k]) for k in ("factor", "low", "high", "original")}
            if not (self.stretch["high"] > self.stretch["low"] and self.stretch["factor"] > 0):
                raise ValueError(f"frequency stretch needs high > low and a positive factor, got {self.stretch}")
        self.cos = self.sin = None

    def frequencies(self) -> np.ndarray:
        """The rotary_dim / 2 frequencies as 32-bit floats."""
        half = self.rotary_dim // 2
        i = np.arange(half, dtype=np.float32)
        if self.stretch is None and self.ramp is None and not self.precise:
            return (np.float32(1.0) / np.power(np.float32(self.theta), i / np.float32(max(half, 1)))).astype(np.float32)
        return self._frequencies64().astype(np.float32)

    def _frequencies64(self) -> np.ndarray:
        half = self.rotary_dim // 2
        f = np.power(np.float64(self.theta), -np.arange(half, dtype=np.float64) / max(half, 1))
        if self.ramp is not None:
            rp, dims = self.ramp, self.rotary_dim

            def pair_of(turns: float) -> float:
                return dims * np.log(rp["original"] / (2.0 * np.pi * turns)) / (2.0 * np.log(self.theta))
            lo = max(int(np.floor(pair_of(rp["fast"]))), 0)
            hi = min(int(np.ceil(pair_of(rp["slow"]))), dims - 1)
            r = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            return f / rp["factor"] * r + f * (1.0 - r)
        if self.stretch is None:
            return f
        st = self.stretch
        wavelength = 2.0 * np.pi / f
        s = (st["original"] / wavelength - st["low"]) / (st["high"] - st["low"])
        blended = (1.0 - s) * f / st["factor"] + s * f
        f = np.where(wavelength < st["original"] / st["high"], f,
                     np.where(wavelength > st["original"] / st["low"], f / st["factor"], blended))
        return f

    def prepare(self, rt, n_positions: int) -> None:
        if self.exact_angles:
            ang = np.arange(max(n_positions, 1), dtype=np.float64)[:, None] * self._frequencies64()[None, :]
        else:
            freq = self.frequencies()
            pos = np.arange(max(n_positions, 1), dtype=np.float32)[:, None]
            ang = (pos * freq[None, :]).astype(np.float32).astype(np.float64)
        self.cos = torch.from_numpy((np.cos(ang) * self.gain).astype(np.float32)).to(rt.device).contiguous()
        self.sin = torch.from_numpy((np.sin(ang) * self.gain).astype(np.float32)).to(rt.device).contiguous()

    def rotation(self):
        return self.cos, self.sin, self.rotary_dim


@register_part("position_encoding", "none")
class NoEncoding(PositionEncoding):
    """No position information beyond the causal mask."""

    graph_safe = True
