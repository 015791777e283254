"""Mixers that keep a fixed-size state per sequence instead of keys and values.

Both rest on one recurrence over a matrix-valued state S (key channel x value channel) per head,
`ops.linear_recurrence`, held in 32-bit floats in the engine's per-sequence state area (zeroed
when a slot is handed out) and walked token by token; decays, gates and their exponentials are
32-bit whatever the element type of activations.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, ParamSpec, register_part


# A step in which a sequence brings this many tokens or more walks the recurrence in blocks of RECURRENCE_BLOCK
# tokens side by side (see ops.linear_recurrence); shorter steps, and every decode step, walk token by token.
RECURRENCE_BLOCK = 128
BLOCKS_FROM = 2 * RECURRENCE_BLOCK


def _block_len(step) -> int:
    return RECURRENCE_BLOCK if step.max_new >= BLOCKS_FROM else 0


def _f32_view(state_bytes: torch.Tensor) -> torch.Tensor:
    """The state rows (uint8 [slots, bytes], rows any distance apart) as float32 [slots, bytes / 4]."""
    return state_bytes.view(torch.float32)


@register_part("mixer", "wkv_token_shift")
class TokenShiftWKV(Mixer):
    """Time mixing with token shift and a data-dependent decay.

    With h' the row before in the sequence (zeros before its first token; carried in the state from
    step to step), five streams s in (r, k, v, g, w) read h + (h' - h) * mu_s.  r, k, v = W_r, W_k,
    W_v of their streams (heads x head_dim), gate = silu(W_g stream_g), and the decay per head and key
    channel is exp(-exp(W_w2 tanh(W_w1 stream_w) + w0)).  Per head:

        o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t          S_t = diag(decay_t) S_(t-1) + k_t v_t^T

    Each head's o is divided by its root mean square; the heads, side by side, are multiplied by the
    weight `norm` and the gate and go through W_o.  decay_rank (the inner size of the two-step decay
    projection) is taken from the tensors of a model folder; random weights need it given.
    """

    graph_safe = True
    takes_residual = True
    STREAMS = ("r", "k", "v", "g", "w")

    def __init__(self, width: int, n_heads: int, head_dim: int, names: dict, eps: float = 1e-5, decay_rank: int = 0):
        self.width, self.H, self.D, self.eps = width, n_heads, head_dim, float(eps)
        self.names, self.rank = dict(names), int(decay_rank)
        self.mu = self.w = None

    def params(self):
        n, inner = self.names, self.H * self.D
        rank = self.rank or -1
        fill = self.rank or max(8, self.width // 32 // 8 * 8)
        out = [ParamSpec(n["mu_" + s], (self.width,), init="unit") for s in self.STREAMS]
        out += [ParamSpec(n[s], (inner, self.width)) for s in ("r", "k", "v", "g")]
        out += [ParamSpec(n["w1"], (rank, self.width), shape_if_random=(fill, self.width)),
                ParamSpec(n["w2"], (inner, rank), shape_if_random=(inner, fill)),
                ParamSpec(n["w0"], (inner,), init="decay"), ParamSpec(n["u"], (self.H, self.D), init="unit"),
                ParamSpec(n["norm"], (inner,), init="norm"), ParamSpec(n["o"], (self.width, inner))]
        return out

    def bind(self, tensors, rt):
        n = self.names
        mus = [tensors.pop(n["mu_" + s]) for s in self.STREAMS]
        if len({t.dtype for t in mus}) > 1:
            mus = [t.float() for t in mus]
        self.mu = torch.stack(mus, dim=0).contiguous()
        self.w = {s: tensors[n[s]] for s in ("r", "k", "v", "g", "w1", "w2", "o", "norm")}
        w0, u = tensors[n["w0"]], tensors[n["u"]]
        if w0.dtype != u.dtype:
            w0, u = w0.float(), u.float()
        self.w0, self.u = w0.contiguous(), u.contiguous()

    def state_bytes(self) -> int:
        return 4 * (self.H * self.D * self.D + self.width)

    def kernel_groups(self):
        return {"recurrent", "rowwise", "gemm_plain"}

    def forward(self, rt, step, h, entry, residual=None):
        T, inner = h.shape[0], self.H * self.D
        state = _f32_view(step.state(entry))
        S, before = state[:, :inner * self.D], state[:, inner * self.D:]
        streams = rt.empty(len(self.STREAMS), T, self.width)
        ops.token_shift(h, before, self.mu, streams, step.tok_seq, step.seq_start, step.seq_slots)
        r, k, v, g = (rt.linear(streams[i], self.w[s], out_dtype=torch.float32) for i, s in enumerate("rkvg"))
        low = rt.linear(streams[4], self.w["w1"], out_dtype=torch.float32, may_split=True)
        bent = rt.empty(T, self.w["w1"].shape[0])
        ops.activation(low, "tanh", bent)
        raw = rt.linear(bent, self.w["w2"], out_dtype=torch.float32)
        o = rt.empty(T, inner, dtype=torch.float32)
        ops.linear_recurrence("bonus", r, k, raw, v, self.w0, self.u, o, S, step.seq_start, step.seq_slots,
                              step.n_seq_cap, self.H, self.D, self.D, shift_src=h, shift_state=before,
                              block_len=_block_len(step), max_new=step.max_new)
        y = rt.empty(T, inner)
        ops.head_unit_scale(o, self.w["norm"], True, g, self.eps, y, self.H, self.D)
        return rt.linear(y, self.w["o"], out_dtype=torch.float32, may_split=True, add_to=residual)


@register_part("mixer", "retention")
class Retention(Mixer):
    """Linear attention with one fixed decay per head, no softmax and no denominator.

    q = W_q h, k = W_k h (heads x head_dim), v = W_v h (heads x v_head_dim), no biases; q and k are rotated by the
    position (the encoding's first rotary_dim elements of a head, in its layout), then k is multiplied by
    head_dim^(-1/2).  Per head, with the state S (head_dim x v_head_dim) zero at a sequence's start:

        S_t = decay_h S_(t-1) + k_t v_t^T          o_t = S_t^T q_t

    Each head's o is divided by its root mean square (no weight); the heads, side by side, are multiplied by
    silu(W_g h) and go through W_o.  The four projections of h are fused into one at load and leave it as 32-bit;
    rotation, scaling, decay and state are 32-bit.  names: "q", "k", "v", "g", "o"."""

    graph_safe = True
    rope_layouts = ("halves", "pairs")

    def __init__(self, width: int, n_heads: int, head_dim: int, v_head_dim: int, decay, names: dict,
                 position_encoding: str | None = None, eps: float = 1e-5):
        decay = [float(d) for d in decay]
        if len(decay) != n_heads:
            raise ValueError(f"{n_heads} heads need as many decays, got {len(decay)}")
        self.width, self.H, self.D, self.V, self.eps = width, n_heads, head_dim, v_head_dim, float(eps)
        self.decay_values, self.names, self.pe_name = decay, dict(names), position_encoding
        self.pe = None

    def params(self):
        n, qk, vv = self.names, self.H * self.D, self.H * self.V
        return [ParamSpec(n["q"], (qk, self.width)), ParamSpec(n["k"], (qk, self.width)),
                ParamSpec(n["v"], (vv, self.width)), ParamSpec(n["g"], (vv, self.width)),
                ParamSpec(n["o"], (self.width, vv))]

    def bind(self, tensors, rt):
        n = self.names
        mats = [tensors.pop(n[s]) for s in ("q", "k", "v", "g")]
        if len({t.dtype for t in mats}) > 1:
            mats = [t.float() for t in mats]
        self.w_qkvg = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        # the heads' decays, rounded to 32-bit once
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).contiguous().to(rt.device)
        self._dummy = torch.zeros(1, 1, dtype=torch.float32, device=rt.device)

    def state_bytes(self) -> int:
        return 4 * self.H * self.D * self.V

    def kernel_groups(self):
        return {"recurrent", "latent", "gemm_plain"}

    def forward(self, rt, step, h, entry):
        T, qk, vv = h.shape[0], self.H * self.D, self.H * self.V
        qkvg = rt.linear(h, self.w_qkvg, out_dtype=torch.float32)
        rot = self.pe.rotation() if self.pe is not None else None
        cos, sin, rot_dim = rot if rot is not None else (self._dummy, self._dummy, 0)
        pairs = rot is not None and self.pe.layout == "pairs"
        # q and k are 2 H heads side by side: all are rotated in place, the k heads are scaled afterwards
        both = qkvg[:, :2 * qk]
        ops.rope_heads(both, self.D, both, self.D, 2 * self.H, self.D, rot_dim, pairs, cos, sin, step.tok_pos,
                       scale=float(self.D) ** -0.5, scale_from_head=self.H)
        o = rt.empty(T, vv, dtype=torch.float32)
        ops.linear_recurrence("fixed", qkvg[:, :qk], qkvg[:, qk:2 * qk], None, qkvg[:, 2 * qk:2 * qk + vv], self.decay,
                              self.decay, o, _f32_view(step.state(entry)), step.seq_start, step.seq_slots, step.n_seq_cap,
                              self.H, self.D, self.V, block_len=_block_len(step), max_new=step.max_new)
        y = rt.empty(T, vv)
        ops.head_unit_scale(o, None, False, qkvg[:, 2 * qk + vv:], self.eps, y, self.H, self.V)
        return rt.linear(y, self.w_o, out_dtype=torch.float32, may_split=True)


@register_part("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    """Linear attention whose forget gate also decides what is written (the HGRN2 form).

    q = silu(W_q h) (heads x head_dim), v = W_v h (heads x v_head_dim), and per head and channel
    f = l + (1 - l) * sigmoid(W_f h + b_f) with the lower bound l a tensor of the model.  Per head:

        S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T          o_t = S_t^T q_t

    Each head's o goes through an RMSNorm over v_head_dim with one weight shared by the heads, the heads
    side by side through W_o.  The three projections of h are fused into one at load.
    """

    graph_safe = True
    takes_residual = True

    def __init__(self, width: int, n_heads: int, head_dim: int, v_head_dim: int, names: dict, eps: float = 1e-5):
        self.width, self.H, self.D, self.V, self.eps = width, n_heads, head_dim, v_head_dim, float(eps)
        self.names = dict(names)

    def params(self):
        n, qk, vv = self.names, self.H * self.D, self.H * self.V
        return [ParamSpec(n["q"], (qk, self.width)), ParamSpec(n["f"], (qk, self.width)),
                ParamSpec(n["f_bias"], (qk,)), ParamSpec(n["lower"], (qk,), init="unit"),
                ParamSpec(n["v"], (vv, self.width)), ParamSpec(n["norm"], (self.V,), init="norm"),
                ParamSpec(n["o"], (self.width, vv))]

    def bind(self, tensors, rt):
        n = self.names
        q, f, v = tensors.pop(n["q"]), tensors.pop(n["f"]), tensors.pop(n["v"])
        if not (q.dtype == f.dtype == v.dtype):
            q, f, v = q.float(), f.float(), v.float()
        self.w_qfv = torch.cat([q, f, v], dim=0).contiguous()
        fb, low = tensors[n["f_bias"]], tensors[n["lower"]]
        if fb.dtype != low.dtype:
            fb, low = fb.float(), low.float()
        self.f_bias, self.lower = fb.contiguous(), low.contiguous()
        self.norm_w, self.w_o = tensors[n["norm"]], tensors[n["o"]]

    def state_bytes(self) -> int:
        return 4 * self.H * self.D * self.V

    def kernel_groups(self):
        return {"recurrent", "gemm_plain"}

    def forward(self, rt, step, h, entry, residual=None):
        T, qk, vv = h.shape[0], self.H * self.D, self.H * self.V
        qfv = rt.linear(h, self.w_qfv, out_dtype=torch.float32)
        o = rt.empty(T, vv, dtype=torch.float32)
        ops.linear_recurrence("gated", qfv[:, :qk], None, qfv[:, qk:2 * qk], qfv[:, 2 * qk:], self.f_bias, self.lower, o,
                              _f32_view(step.state(entry)), step.seq_start, step.seq_slots, step.n_seq_cap,
                              self.H, self.D, self.V, block_len=_block_len(step), max_new=step.max_new)
        y = rt.empty(T, vv)
        ops.head_unit_scale(o, self.norm_w, False, None, self.eps, y, self.H, self.V)
        return rt.linear(y, self.w_o, out_dtype=torch.float32, may_split=True, add_to=residual)


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    """Linear attention whose state decays per key channel by a gate of the input.

    q = W_q h * head_dim^(-1/2), k = W_k h (heads x head_dim), v = W_v h (heads x v_head_dim); the decay per head and key
    channel is a = sigmoid(W_a2 (W_a1 h) + b_a2)^(1 / tau), formed as exp(logsigmoid(.) / tau).  Per head:

        S_t = diag(a_t) S_(t-1) + k_t v_t^T          o_t = S_t^T q_t

    Each head's o goes through an RMSNorm over v_head_dim with one weight shared by the heads; the heads, side by side,
    are multiplied by silu(W_g h) and go through W_o.  q, k, v and g are one product that leaves its sums as 32-bit; the
    inner size of the decay's two-step projection is taken from the tensors of a model folder (random weights need it
    given).  names: "q", "k", "v", "g", "o", "norm", "a1", "a2", "a2_bias"."""

    graph_safe = True

    def __init__(self, width: int, n_heads: int, head_dim: int, v_head_dim: int, tau: float, names: dict, eps: float = 1e-5,
                 decay_rank: int = 0):
        if not tau > 0:
            raise ValueError(f"tau must be positive, got {tau}")
        self.width, self.H, self.D, self.V, self.eps = width, n_heads, head_dim, v_head_dim, float(eps)
        self.tau, self.names, self.rank = float(tau), dict(names), int(decay_rank)

    def params(self):
        n, qk, vv = self.names, self.H * self.D, self.H * self.V
        rank = self.rank or -1
        fill = self.rank or 16
        return [ParamSpec(n["q"], (qk, self.width)), ParamSpec(n["k"], (qk, self.width)),
                ParamSpec(n["v"], (vv, self.width)), ParamSpec(n["g"], (vv, self.width)),
                ParamSpec(n["o"], (self.width, vv)), ParamSpec(n["norm"], (self.V,), init="norm"),
                ParamSpec(n["a1"], (rank, self.width), shape_if_random=(fill, self.width)),
                ParamSpec(n["a2"], (qk, rank), shape_if_random=(qk, fill)),
                ParamSpec(n["a2_bias"], (qk,), init="logit")]

    def bind(self, tensors, rt):
        n = self.names
        mats = [tensors.pop(n[s]) for s in ("q", "k", "v", "g")]
        if len({t.dtype for t in mats}) > 1:
            mats = [t.float() for t in mats]
        self.w_qkvg = torch.cat(mats, dim=0).contiguous()
        self.w_a1, self.w_a2, self.w_o, self.norm_w = tensors[n["a1"]], tensors[n["a2"]], tensors[n["o"]], tensors[n["norm"]]
        self.a_bias = tensors[n["a2_bias"]].to(torch.float32).contiguous()
        # 1 / tau per key channel, rounded to 32-bit once
        self.inv_tau = torch.full((self.H * self.D,), 1.0 / self.tau, dtype=torch.float64).to(torch.float32).to(rt.device)

    def state_bytes(self) -> int:
        return 4 * self.H * self.D * self.V

    def kernel_groups(self):
        return {"recurrent", "gemm_plain"}

    def forward(self, rt, step, h, entry):
        T, qk, vv = h.shape[0], self.H * self.D, self.H * self.V
        qkvg = rt.linear(h, self.w_qkvg, out_dtype=torch.float32)
        low = rt.linear(h, self.w_a1)
        raw = rt.linear(low, self.w_a2, out_dtype=torch.float32)
        o = rt.empty(T, vv, dtype=torch.float32)
        ops.linear_recurrence("gla", qkvg[:, :qk], qkvg[:, qk:2 * qk], raw, qkvg[:, 2 * qk:2 * qk + vv], self.a_bias,
                              self.inv_tau, o, _f32_view(step.state(entry)), step.seq_start, step.seq_slots, step.n_seq_cap,
                              self.H, self.D, self.V, block_len=_block_len(step), max_new=step.max_new,
                              q_scale=float(self.D) ** -0.5)
        y = rt.empty(T, vv)
        ops.head_unit_scale(o, self.norm_w, False, qkvg[:, 2 * qk + vv:], self.eps, y, self.H, self.V)
        return rt.linear(y, self.w_o, out_dtype=torch.float32, may_split=True)
