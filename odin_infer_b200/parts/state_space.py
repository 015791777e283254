"""State-space mixers, and a mixer of two branches that read the same input.

`selective_scan` keeps a state row per channel (inner x state), `state_space_dual` a matrix per head (state x head_dim)
with one decay per head and token; both keep the last taps - 1 inputs of their short causal convolution.  All of it
lives in 32-bit floats in the engine's per-sequence state area (zeroed when a slot is handed out) and is carried from
step to step; step sizes, decays, exponentials and the states are 32-bit whatever the element type of activations.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Combined, Mixer, ParamSpec, PartSpec, build_part, register_part
from .recurrent import _block_len, _f32_view


def _as_f32(*tensors):
    return [t.to(torch.float32).contiguous() for t in tensors]


@register_part("mixer", "selective_scan")
class SelectiveScan(Mixer):
    """W_in h = [x | z] (inner each).  x passes a causal convolution per channel (`taps` taps, the last one the current
    token's, a bias) and SiLU.  W_x x = [dt (dt_rank) | B (state) | C (state)]; step = softplus(W_dt dt + b_dt) per
    channel; A = -exp(A_log) (inner x state).  Per channel c and state index n:

        S[c, n] <- exp(step_c A[c, n]) S[c, n] + step_c x_c B_n          y_c = sum_n S[c, n] C_n + D_c x_c

    then y * silu(z) through W_o.  names: "in", "conv", "conv_bias", "x", "dt", "dt_bias", "A_log", "D", "o"."""

    graph_safe = True

    def __init__(self, width: int, inner: int, state: int, dt_rank: int, taps: int, names: dict):
        if min(width, inner, state, dt_rank, taps) < 1:
            raise ValueError("a selective scan needs positive sizes")
        self.width, self.inner, self.N, self.R, self.taps = width, inner, state, dt_rank, taps
        self.names = dict(names)

    def params(self):
        n = self.names
        return [ParamSpec(n["in"], (2 * self.inner, self.width)), ParamSpec(n["conv"], (self.inner, self.taps), init="near_zero"),
                ParamSpec(n["conv_bias"], (self.inner,), init="near_zero"),
                ParamSpec(n["x"], (self.R + 2 * self.N, self.inner)), ParamSpec(n["dt"], (self.inner, self.R), init="near_zero"),
                ParamSpec(n["dt_bias"], (self.inner,), init="decay"), ParamSpec(n["A_log"], (self.inner, self.N), init="near_zero"),
                ParamSpec(n["D"], (self.inner,), init="norm"), ParamSpec(n["o"], (self.width, self.inner))]

    def bind(self, tensors, rt):
        n = self.names
        self.w_in, self.w_o, self.w_dt = tensors[n["in"]], tensors[n["o"]], tensors[n["dt"]]
        wx = tensors.pop(n["x"])
        self.w_x_dt, self.w_x_bc = wx[:self.R].contiguous(), wx[self.R:].contiguous()
        self.conv_w, self.conv_b = tensors[n["conv"]].contiguous(), tensors[n["conv_bias"]].contiguous()
        self.dt_bias, self.A_log, self.D = _as_f32(tensors[n["dt_bias"]], tensors[n["A_log"]], tensors[n["D"]])

    def state_bytes(self) -> int:
        return 4 * (self.inner * self.N + (self.taps - 1) * self.inner)

    def kernel_groups(self):
        return {"state_space", "gemm_plain"}

    def forward(self, rt, step, h, entry):
        T, inner, N = h.shape[0], self.inner, self.N
        state = _f32_view(step.state(entry))
        S, window = state[:, :inner * N], state[:, inner * N:]
        xz = rt.linear(h, self.w_in)
        x = rt.empty(T, inner)
        ops.causal_conv(xz[:, :inner], self.conv_w, self.conv_b, True, window, step.tok_seq, step.seq_start, step.seq_slots,
                        step.n_seq_cap, x, single_rows=step.all_single)
        low = rt.linear(x, self.w_x_dt)
        bc = rt.linear(x, self.w_x_bc, out_dtype=torch.float32)
        dt = rt.linear(low, self.w_dt, out_dtype=torch.float32)
        y = rt.empty(T, inner)
        ops.selective_scan(x, dt, self.dt_bias, bc[:, :N], bc[:, N:], self.A_log, self.D, xz[:, inner:], S, y,
                           step.seq_start, step.seq_slots, step.n_seq_cap, block_len=_block_len(step), max_new=step.max_new)
        return rt.linear(y, self.w_o, out_dtype=torch.float32, may_split=True)


@register_part("mixer", "state_space_dual")
class StateSpaceDual(Mixer):
    """W_in h = [z (inner) | x (inner) | B (groups x state) | C (groups x state) | dt (heads)], inner = heads x head_dim.
    x, B and C together pass a causal convolution per channel and SiLU.  step = softplus(dt + dt_bias) per head; head h
    uses group h // (heads / groups).  Per head, with S (state x head_dim) zero at a sequence's start:

        S_t = exp(-exp(A_log_h) step) S_(t-1) + step B_t x_t^T          y_t = S_t^T C_t + D_h x_t

    y, heads side by side, times silu(z), then an RMSNorm in `norm_groups` equal consecutive parts of the row (each by
    its own root mean square) times the weight `norm`, through W_o.  The projection leaves its product as 32-bit: the
    step sizes and what the convolution hands to the recurrence are 32-bit.
    names: "in", "conv", "conv_bias", "dt_bias", "A_log", "D", "norm", "o"."""

    graph_safe = True

    def __init__(self, width: int, n_heads: int, head_dim: int, state: int, groups: int, norm_groups: int, taps: int,
                 names: dict, eps: float = 1e-5):
        if min(width, n_heads, head_dim, state, groups, norm_groups, taps) < 1:
            raise ValueError("a state-space mixer needs positive sizes")
        if n_heads % groups or (n_heads * head_dim) % norm_groups:
            raise ValueError(f"{n_heads} heads of {head_dim} do not split into {groups} groups and {norm_groups} norm groups")
        self.width, self.H, self.P, self.N, self.G = width, n_heads, head_dim, state, groups
        self.norm_groups, self.taps, self.eps, self.names = norm_groups, taps, float(eps), dict(names)
        self.inner = n_heads * head_dim
        self.channels = self.inner + 2 * groups * state

    def params(self):
        n = self.names
        return [ParamSpec(n["in"], (2 * self.inner + 2 * self.G * self.N + self.H, self.width)),
                ParamSpec(n["conv"], (self.channels, self.taps), init="near_zero"),
                ParamSpec(n["conv_bias"], (self.channels,), init="near_zero"), ParamSpec(n["dt_bias"], (self.H,), init="decay"),
                ParamSpec(n["A_log"], (self.H,), init="near_zero"), ParamSpec(n["D"], (self.H,), init="norm"),
                ParamSpec(n["norm"], (self.inner,), init="norm"), ParamSpec(n["o"], (self.width, self.inner))]

    def bind(self, tensors, rt):
        n = self.names
        self.w_in, self.w_o = tensors[n["in"]], tensors[n["o"]]
        self.conv_w, self.conv_b = tensors[n["conv"]].contiguous(), tensors[n["conv_bias"]].contiguous()
        self.dt_bias, self.A_log, self.D, self.norm_w = _as_f32(tensors[n["dt_bias"]], tensors[n["A_log"]], tensors[n["D"]],
                                                                tensors[n["norm"]])

    def state_bytes(self) -> int:
        return 4 * (self.H * self.N * self.P + (self.taps - 1) * self.channels)

    def kernel_groups(self):
        return {"state_space", "recurrent", "gemm_plain"}

    def forward(self, rt, step, h, entry):
        T, inner, GN = h.shape[0], self.inner, self.G * self.N
        state = _f32_view(step.state(entry))
        n_s = self.H * self.N * self.P
        S, window = state[:, :n_s], state[:, n_s:]
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)
        xbc = rt.empty(T, self.channels, dtype=torch.float32)
        ops.causal_conv(proj[:, inner:inner + self.channels], self.conv_w, self.conv_b, True, window, step.tok_seq,
                        step.seq_start, step.seq_slots, step.n_seq_cap, xbc, single_rows=step.all_single)
        x, B, C = xbc[:, :inner], xbc[:, inner:inner + GN], xbc[:, inner + GN:]
        o = rt.empty(T, inner, dtype=torch.float32)
        ops.linear_recurrence("ssd", C, B, proj[:, inner + self.channels:], x, self.A_log, self.dt_bias, o, S, step.seq_start,
                              step.seq_slots, step.n_seq_cap, self.H, self.N, self.P, block_len=_block_len(step),
                              max_new=step.max_new, heads_per_group=self.H // self.G)
        y = rt.empty(T, inner)
        ops.skip_gate_norm(o, x, self.D, self.P, proj[:, :inner], self.norm_w, self.norm_groups, self.eps, y)
        return rt.linear(y, self.w_o, out_dtype=torch.float32, may_split=True)


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    """Two mixers that read the same input; the update is left_scale * f_l(left) + right_scale * f_r(right), f the
    identity or, with `norms` = {"left": name, "right": name}, an RMSNorm over the width with that weight.  The sum is
    formed by whoever adds the update (the answer is `Combined`).  At most one branch keeps keys and values and at most
    one keeps fixed-size state: both are handed the block's own schedule entry."""

    def __init__(self, left: PartSpec, right: PartSpec, width: int, left_scale: float = 1.0, right_scale: float = 1.0,
                 norms: dict | None = None, eps: float = 1e-5):
        self.left, self.right = build_part("mixer", left), build_part("mixer", right)
        self.width, self.scales, self.eps = width, (float(left_scale), float(right_scale)), float(eps)
        self.norm_names = dict(norms) if norms else None
        self.norm_w = (None, None)
        if sum(m.cache_request() is not None for m in self._both()) > 1 or sum(m.state_bytes() > 0 for m in self._both()) > 1:
            raise ValueError("two mixers side by side: at most one keeps keys and values, at most one keeps state")
        if sum(getattr(m, "pe_name", None) is not None for m in self._both()) > 1:
            raise ValueError("two mixers side by side: at most one is rotated by a position encoding")

    def _both(self):
        return (self.left, self.right)

    def _rotated(self):
        return next((m for m in self._both() if getattr(m, "pe_name", None) is not None), None)

    @property
    def pe_name(self):
        m = self._rotated()
        return m.pe_name if m is not None else None

    @property
    def rope_layouts(self):
        return getattr(self._rotated(), "rope_layouts", ("halves",))

    @property
    def pe(self):
        m = self._rotated()
        return m.pe if m is not None else None

    @pe.setter
    def pe(self, value):
        self._rotated().pe = value

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self._both())

    def params(self):
        out = [p for m in self._both() for p in m.params()]
        if self.norm_names:
            out += [ParamSpec(self.norm_names[s], (self.width,), init="norm") for s in ("left", "right")]
        return out

    def bind(self, tensors, rt):
        for m in self._both():
            m.bind(tensors, rt)
        if self.norm_names:
            self.norm_w = tuple(tensors[self.norm_names[s]].contiguous() for s in ("left", "right"))

    def cache_request(self):
        return next((r for r in (m.cache_request() for m in self._both()) if r is not None), None)

    def state_bytes(self) -> int:
        return sum(m.state_bytes() for m in self._both())

    def kernel_groups(self):
        return {"rowwise"}.union(*(m.kernel_groups() for m in self._both()))

    def notes(self, rt):
        return [n for m in self._both() for n in m.notes(rt)]

    def forward(self, rt, step, h, entry):
        out = Combined()
        for m, scale, w in zip(self._both(), self.scales, self.norm_w):
            u = m.forward(rt, step, h, entry)
            if not torch.is_tensor(u):
                raise TypeError(f"{type(m).__name__} beside another mixer must answer a plain update, got {type(u).__name__}")
            out.append(ops.Term(u, scale, None, w, self.eps))
        return out
