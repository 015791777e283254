"""Attention whose keys and values come from one small latent per token."""
from __future__ import annotations

import torch

from ..cache import KVRequest
from ..csrc import ops
from .base import Mixer, ParamSpec, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Queries through a latent: c_q = RMSNorm(W_dq h) * w, q = W_uq c_q, per head [head_dim unrotated | rot_dim
    rotated].  Keys and values through ONE latent per token: W_dkv h = [c' | k_r], c = RMSNorm(c') * w (kv_rank wide),
    k_r (rot_dim wide, not normed) rotated by the position and shared by all heads; per head k = [W_uk c | k_r],
    v = W_uv c.  score = (q . k) * scale over the visible keys (window > 0: the last `window`), softmax, W_o on the
    heads side by side.

    The cache keeps one row [c | rotated k_r] per token (`KVRequest.shared_kv`), never a key or a value per head.
    Every head's unrotated query is carried over to the latent instead, q' = W_uk^T q (q . (W_uk c) = q' . c), so that
    attention is one kv head of kv_rank + rot_dim elements under all query heads with the cached rows as keys AND as
    values; the kernels' output over the row's first kv_rank elements goes through W_uv head by head.  Prompts,
    portions of prompts and decoding run the same way, through whichever attention kernel takes the row's size.

    names: "dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "o".  W_dq and W_dkv are fused into one product.
    The rotation's layout is the position encoding's (`pairs` or `halves`)."""

    graph_safe = True
    rope_layouts = ("halves", "pairs")

    def __init__(self, width: int, n_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, q_rank: int, kv_rank: int,
                 names: dict, position_encoding: str | None, eps: float, scale: float, window: int = 0):
        if min(width, n_heads, head_dim, v_head_dim, q_rank, kv_rank) <= 0 or rot_dim < 0 or rot_dim % 2:
            raise ValueError("latent attention needs positive sizes and an even rot_dim")
        if kv_rank + rot_dim > 512:
            raise ValueError(f"latent attention: a cached row of kv_rank + rot_dim = {kv_rank + rot_dim} elements is more than "
                             "the attention kernels take (512)")
        if rot_dim and position_encoding is None:
            raise ValueError("latent attention with a rotated part needs a position encoding")
        self.width, self.H, self.e, self.r, self.ev = width, n_heads, head_dim, rot_dim, v_head_dim
        self.q_rank, self.kv_rank, self.L = q_rank, kv_rank, kv_rank + rot_dim
        self.names, self.pe_name, self.eps = dict(names), position_encoding, float(eps)
        self.scale, self.window = float(scale), int(window)
        self.pe = None
        self._dummy = None

    def params(self):
        n, H = self.names, self.H
        return [ParamSpec(n["dq"], (self.q_rank, self.width)), ParamSpec(n["dq_norm"], (self.q_rank,), init="norm"),
                ParamSpec(n["uq"], (H * (self.e + self.r), self.q_rank)),
                ParamSpec(n["dkv"], (self.L, self.width)), ParamSpec(n["dkv_norm"], (self.kv_rank,), init="norm"),
                ParamSpec(n["uk"], (H * self.e, self.kv_rank)), ParamSpec(n["uv"], (H * self.ev, self.kv_rank)),
                ParamSpec(n["o"], (self.width, H * self.ev))]

    def bind(self, tensors, rt):
        n, H = self.names, self.H
        dq, dkv = tensors.pop(n["dq"]), tensors.pop(n["dkv"])
        if dq.dtype != dkv.dtype:
            dq, dkv = dq.float(), dkv.float()
        self.w_down = torch.cat([dq, dkv], dim=0).contiguous()
        self.q_norm, self.c_norm = tensors[n["dq_norm"]], tensors[n["dkv_norm"]]
        if self.q_norm.dtype != self.c_norm.dtype:
            self.q_norm, self.c_norm = self.q_norm.float(), self.c_norm.float()
        self.w_uq, self.w_o = tensors[n["uq"]], tensors[n["o"]]
        # per head, input channel before output channel: W_uk of a head as it is stored, W_uv of a head transposed
        self.w_uk = tensors.pop(n["uk"]).view(H, self.e, self.kv_rank).contiguous()
        self.w_uv = tensors.pop(n["uv"]).view(H, self.ev, self.kv_rank).transpose(1, 2).contiguous()
        self._dummy = torch.zeros(1, 1, dtype=torch.float32, device=rt.device)

    def cache_request(self):
        return KVRequest(1, self.L, self.window, 0, 0, shared_kv=True)

    def kernel_groups(self):
        return {"latent", "attention_plain", "gemm_plain"}

    def notes(self, rt):
        if rt.dtype != torch.bfloat16:
            return []
        out = []
        if not ops.attention_prefill_supported(self.L):
            out.append(f"latent attention: a cached row of {self.L} elements (kv_rank + rot_dim) is not 64 or 128: prompts "
                       "run the CUDA-core attention kernel (one warp per token and head)")
        if self.L not in (64, 128) or self.H > 16:
            out.append(f"latent attention: {self.H} heads over rows of {self.L}: decoding runs a CUDA-core attention kernel "
                       "(the tensor-core one takes rows of 64 or 128 and up to 16 heads)")
        return out

    def forward(self, rt, step, h, entry):
        T, H, e, r, L = h.shape[0], self.H, self.e, self.r, self.L
        down = rt.linear(h, self.w_down, may_split=True, beside_attention=True)
        line, _, block_table = step.kv(entry)
        rot = self.pe.rotation() if (self.pe is not None and r) else None
        cos, sin = (rot[0], rot[1]) if rot is not None else (self._dummy, self._dummy)
        pairs = rot is not None and self.pe.layout == "pairs"
        cq = rt.empty(T, self.q_rank)
        ops.latent_prep(down, self.q_rank, self.kv_rank, r, pairs, self.q_norm, self.c_norm, self.eps, cq, cos, sin,
                        step.tok_pos, step.tok_seq, block_table, line, write_cache=step.writes_cache(entry))
        q = rt.linear(cq, self.w_uq)
        qf = rt.empty(T, H * L)
        ops.heads_linear(q, e + r, self.w_uk, qf, L)
        if r:
            ops.rope_heads(q[:, e:], e + r, qf[:, self.kv_rank:], L, H, r, r, pairs, cos, sin, step.tok_pos)
        o = rt.empty(T, H * L)
        rt.attention(step, qf, o, H, 1, L, line, line, block_table, self.window, scale=self.scale)
        ov = rt.empty(T, H * self.ev)
        ops.heads_linear(o, L, self.w_uv, ov, self.ev)
        return rt.linear(ov, self.w_o, out_dtype=torch.float32, may_split=True, beside_attention=True)
