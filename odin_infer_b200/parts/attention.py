"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import torch

from ..cache import KVRequest
from ..csrc import ops
from .base import Biased, Mixer, ParamSpec, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    """q, k, v projections (no bias), optional per-head RMSNorm of q and k, rotation,
    causal attention of each query head h over kv head h // (n_q / n_kv), output
    projection.  Restates infer/forward.odin:53-117.

    window > 0 keeps only the last `window` keys visible; chunk > 0 only the keys of the query's own
    chunk of `chunk` positions (counted from the sequence's first position).  kv_shared: this mixer has
    no k and v of its own and reads the cache line its schedule entry names.
    The three projection matrices are fused into one at load time.

    qk_norm: True: RMSNorm with the weights `q_norm` / `k_norm` before the rotation; "unit_after":
    q and k heads divided by their root mean square after the rotation, no weight; "whole": one RMSNorm over the
    token's whole q projection (all heads at once, weight [n_q_heads * head_dim]) and one over its whole k projection,
    before the rotation; False: none.
    biases: names of bias vectors of the projections ({"q", "k", "v"} and optionally "o"), added in the projection.
    The rotation pairs elements as its position encoding's layout says ("halves": i with i + dims/2; "pairs": 2i with
    2i + 1).
    scale: factor on q . k (0: 1 / sqrt(head_dim)).  softcap > 0: scores become
    softcap * tanh(score / softcap) before the softmax.  v_head_dim: size of a value head (0: head_dim).
    sink: name of a tensor [n_q_heads]: a learned logit per query head whose exponential joins the softmax's
    denominator (no key, no value, not scaled).  gate: name of a matrix G; the heads' outputs are multiplied by
    sigmoid(G h) before the output projection, one factor per element (G: [n_q_heads * v_head_dim, width]) or,
    with gate_per_head, one per head (G: [n_q_heads, width]); G is fused with q, k and v into one product.
    """

    graph_safe = True
    rope_layouts = ("halves", "pairs")

    def __init__(self, width: int, n_q_heads: int, n_kv_heads: int, head_dim: int, names: dict,
                 position_encoding: str | None = None, qk_norm=True, eps: float = 1e-6,
                 window: int = 0, kv_shared: bool = False, chunk: int = 0, biases: dict | None = None,
                 scale: float = 0.0, softcap: float = 0.0, v_head_dim: int = 0, sink: str | None = None,
                 gate: str | None = None, gate_per_head: bool = False):
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} query heads are not a multiple of {n_kv_heads} kv heads")
        if qk_norm not in (True, False, "unit_after", "whole"):
            raise ValueError(f"qk_norm must be True, False, 'unit_after' or 'whole', got {qk_norm!r}")
        self.width, self.n_q, self.n_kv, self.hd = width, n_q_heads, n_kv_heads, head_dim
        self.vd = int(v_head_dim) or head_dim
        self.names, self.pe_name = dict(names), position_encoding
        self.qk_norm, self.eps, self.window, self.kv_shared = qk_norm in (True, "whole"), float(eps), int(window), kv_shared
        self.unit_after = qk_norm == "unit_after"
        self.whole_norm = qk_norm == "whole"
        self.chunk, self.scale, self.softcap = int(chunk), float(scale), float(softcap)
        self.bias_names = dict(biases) if biases else None
        # the heads as the first architecture has them: the fast kernels' ground
        self.sink_name, self.gate_name, self.gate_per_head = sink, gate, bool(gate_per_head)
        self.n_gate = 0 if gate is None else (self.n_q if self.gate_per_head else self.n_q * self.vd)
        self.plain_heads = (self.bias_names is None and not self.unit_after and not self.whole_norm and self.vd == self.hd
                            and self.chunk == 0 and self.scale == 0.0 and self.softcap == 0.0
                            and sink is None and gate is None)
        self.sink = None
        self.pe = None          # set by the model from pe_name
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.b_qkv = self.b_o = None
        self._dummy = None

    def params(self):
        n = self.names
        out = [ParamSpec(n["q"], (self.n_q * self.hd, self.width))]
        if not self.kv_shared:
            out += [ParamSpec(n["k"], (self.n_kv * self.hd, self.width)),
                    ParamSpec(n["v"], (self.n_kv * self.vd, self.width))]
        out.append(ParamSpec(n["o"], (self.width, self.n_q * self.vd)))
        if self.qk_norm:
            out.append(ParamSpec(n["q_norm"], (self.n_q * self.hd if self.whole_norm else self.hd,), init="norm"))
            if not self.kv_shared:
                out.append(ParamSpec(n["k_norm"], (self.n_kv * self.hd if self.whole_norm else self.hd,), init="norm"))
        if self.bias_names is not None:
            b = self.bias_names
            out.append(ParamSpec(b["q"], (self.n_q * self.hd,)))
            if not self.kv_shared:
                out += [ParamSpec(b["k"], (self.n_kv * self.hd,)), ParamSpec(b["v"], (self.n_kv * self.vd,))]
            if b.get("o"):
                out.append(ParamSpec(b["o"], (self.width,)))
        if self.sink_name is not None:
            out.append(ParamSpec(self.sink_name, (self.n_q,), init="logit"))
        if self.gate_name is not None:
            out.append(ParamSpec(self.gate_name, (self.n_gate, self.width)))
        return out

    def bind(self, tensors, rt):
        n = self.names
        if self.kv_shared and self.gate_name is None:
            self.w_qkv = tensors[n["q"]]
        else:
            mats = [tensors.pop(n["q"])] if not self.kv_shared else [tensors[n["q"]]]
            if not self.kv_shared:
                mats += [tensors.pop(n["k"]), tensors.pop(n["v"])]
            if self.gate_name is not None:
                mats.append(tensors.pop(self.gate_name))
            if len({t.dtype for t in mats}) > 1:
                mats = [t.to(torch.float32) for t in mats]
            self.w_qkv = torch.cat(mats, dim=0).contiguous()
        if self.sink_name is not None:
            self.sink = tensors[self.sink_name].to(torch.float32).contiguous()
        self.w_o = tensors[n["o"]]
        if self.qk_norm:
            self.q_norm = tensors[n["q_norm"]]
            self.k_norm = tensors[n["k_norm"]] if not self.kv_shared else self.q_norm
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        if self.bias_names is not None:
            b = self.bias_names
            parts = [tensors[b["q"]]] if self.kv_shared else [tensors.pop(b["q"]), tensors.pop(b["k"]), tensors.pop(b["v"])]
            if len({t.dtype for t in parts}) > 1:
                parts = [t.float() for t in parts]
            self.b_qkv = torch.cat(parts, dim=0).contiguous()
            self.b_o = tensors[b["o"]] if b.get("o") else None
        self._dummy = torch.zeros(1, 1, dtype=torch.float32, device=rt.device)

    def cache_request(self):
        return KVRequest(self.n_kv, self.hd, self.window, self.chunk, self.vd if self.vd != self.hd else 0)

    def kernel_groups(self):
        return {"head_prep", "attention_plain", "gemm_plain"} | ({"rowwise"} if self.gate_name is not None else set())

    def notes(self, rt):
        import torch
        if rt.dtype != torch.bfloat16:
            return []
        out, hd, group = [], self.hd, self.n_q // self.n_kv
        rot = self.pe.rotation() if self.pe is not None else None
        if self.vd != hd:
            out.append(f"attention: value heads of {self.vd} beside keys of {hd}: prompts and decoding run the CUDA-core "
                       "attention kernel (the tensor-core kernels take value heads of the keys' size)")
        elif not ops.attention_prefill_supported(hd):
            out.append(f"attention: head_dim {hd} is not 64 or 128: prompts run the CUDA-core attention kernel "
                       "(one warp per token and head), far slower than the tensor-core one")
        if not ops.attention_decode_supported(hd):
            out.append(f"attention: head_dim {hd} is no power of two from 16 to 256: decoding runs the CUDA-core "
                       "attention kernel without key splits")
        elif hd not in (64, 128) or group > 16:
            out.append(f"attention: head_dim {hd} with {group} query heads per kv head: decoding runs the CUDA-core "
                       "split-key kernel (the tensor-core one takes head_dim 64 or 128 and up to 16 query heads per kv head)")
        elif rot is not None and rot[2] != hd:
            out.append(f"attention: rotary_dim {rot[2]} < head_dim {hd}: head preparation runs as a kernel of its own "
                       "when decoding")
        for what, k in (("width", self.width), ("n_q_heads * head_dim", self.n_q * hd)):
            if k % 8:
                out.append(f"attention: {what} = {k} is no multiple of 8: its matrix products run on CUDA cores "
                           "(the tensor-core kernels read rows of whole 16 bytes)")
        return out

    takes_residual = True

    def forward(self, rt, step, h, entry, residual=None):
        T = h.shape[0]
        qkv = rt.linear(h, self.w_qkv, may_split=True, beside_attention=True)
        k_line, v_line, block_table = step.kv(entry)
        rot = self.pe.rotation() if self.pe is not None else None
        cos, sin, rot_dim = rot if rot is not None else (self._dummy, self._dummy, 0)
        writes = step.writes_cache(entry) and not self.kv_shared
        o = rt.empty(T, self.n_q * self.vd)
        pairs = rot is not None and getattr(self.pe, "layout", "halves") == "pairs"
        if not self.plain_heads or pairs:
            q_out = rt.empty(T, self.n_q * self.hd)
            q = ops.head_prep(qkv, self.n_q, 0 if self.kv_shared else self.n_kv, self.hd,
                              self.q_norm if self.qk_norm else None, self.k_norm if self.qk_norm else None, self.eps,
                              cos, sin, rot_dim, step.tok_pos, step.tok_seq, block_table, k_line, v_line,
                              write_kv=writes, q_out=q_out, bias=self.b_qkv, unit_norm_after=self.unit_after,
                              v_head_dim=self.vd, whole_norm=self.whole_norm, pairs=pairs)
            rt.attention(step, q, o, self.n_q, self.n_kv, self.hd, k_line, v_line, block_table, self.window,
                         chunk=self.chunk, scale=self.scale, softcap=self.softcap, v_head_dim=self.vd, sink=self.sink)
            if self.gate_name is not None:
                g0 = qkv.shape[-1] - self.n_gate
                ops.sigmoid_gate(o, qkv[..., g0:], self.n_q, self.vd, self.gate_per_head)
            out = rt.linear(o, self.w_o, out_dtype=torch.float32, may_split=True, beside_attention=True, add_to=residual)
            return out if self.b_o is None else Biased(out, self.b_o)
        # decoding: the attention kernel may prepare its heads itself
        if not self.kv_shared and rt.attention_with_head_prep(
                step, qkv, o, self.n_q, self.n_kv, self.hd, self.q_norm if self.qk_norm else None,
                self.k_norm if self.qk_norm else None, self.eps, cos, sin, rot_dim, k_line, v_line, block_table,
                self.window, writes):
            return rt.linear(o, self.w_o, out_dtype=torch.float32, may_split=True, beside_attention=True, add_to=residual)
        # a product of few tokens may come back as partial sums: they are added here
        q_out = rt.empty(T, self.n_q * self.hd) if qkv.dim() == 3 else None
        q = ops.head_prep(qkv, self.n_q, 0 if self.kv_shared else self.n_kv, self.hd,
                          self.q_norm if self.qk_norm else None, self.k_norm if self.qk_norm else None, self.eps,
                          cos, sin, rot_dim, step.tok_pos, step.tok_seq, block_table, k_line, v_line,
                          write_kv=writes, q_out=q_out)
        rt.attention(step, q, o, self.n_q, self.n_kv, self.hd, k_line, v_line, block_table, self.window)
        return rt.linear(o, self.w_o, out_dtype=torch.float32, may_split=True, beside_attention=True, add_to=residual)
