"""Token embedding and the output head."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Embedding, Head, ParamSpec, PartSpec, build_part, register_part


@register_part("embedding", "token_table")
class TokenEmbedding(Embedding):
    """x = E[token] (infer/forward.odin:43), times `scale` (a 32-bit product) where one is given.  norm: a norm
    (a PartSpec of a norm that can work in place) through which the embedded rows pass before they become the
    residual stream.

    pair = {"weight", "buckets", "mul_prev", "mul_cur"}: a second table of buckets + 1 rows is added, row
    (previous token * mul_prev + token * mul_cur) mod buckets, and its last row for a sequence's first token.  The previous
    token is per-sequence state (`state_bytes`; the model tells the part which state entry is its own, `state_entry`)."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, weight: str, norm: PartSpec | None = None, scale: float = 1.0,
                 pair: dict | None = None):
        self.vocab_size, self.width, self.weight_name, self.scale = vocab_size, width, weight, float(scale)
        self.norm = build_part("norm", norm) if norm is not None else None
        self.table = None
        self.pair = None
        if pair is not None:
            self.pair = {"weight": str(pair["weight"]), "buckets": int(pair["buckets"]), "mul_prev": int(pair["mul_prev"]),
                         "mul_cur": int(pair["mul_cur"])}
            if self.pair["buckets"] <= 0:
                raise ValueError(f"a table of token pairs needs buckets, got {self.pair['buckets']}")
        self.pair_table = None
        self.state_entry: int | None = None

    def params(self):
        out = [ParamSpec(self.weight_name, (self.vocab_size, self.width))]
        if self.pair is not None:
            out.append(ParamSpec(self.pair["weight"], (self.pair["buckets"] + 1, self.width)))
        return out + (self.norm.params() if self.norm else [])

    def state_bytes(self) -> int:
        """Bytes of per-sequence state: the token before (as token + 1; 0: none yet)."""
        return 4 if self.pair is not None else 0

    def bind(self, tensors, rt):
        self.table = tensors[self.weight_name]
        if self.pair is not None:
            self.pair_table = tensors[self.pair["weight"]]
            if self.pair_table.dtype != self.table.dtype:
                self.table, self.pair_table = self.table.float(), self.pair_table.float()
        if self.norm is not None:
            self.norm.bind(tensors, rt)

    def kernel_groups(self):
        return {"elementwise"} | (self.norm.kernel_groups() if self.norm else set())

    def forward(self, rt, step):
        x = rt.empty(step.n_rows, self.width, dtype=torch.float32)
        if self.pair is not None:
            before = step.state(self.state_entry).view(torch.int32)
            ops.embed_pair(self.table, self.pair_table, step.tok_ids, step.tok_seq, step.seq_start, step.seq_slots, before,
                           step.n_seq_cap, self.pair["buckets"], self.pair["mul_prev"], self.pair["mul_cur"], x, self.scale,
                           single_rows=step.all_single)
        else:
            ops.embed(self.table, step.tok_ids, x, self.scale)
        if self.norm is not None:
            self.norm.in_place(rt, x)
        return x


@register_part("head", "linear")
class LinearHead(Head):
    """logits = W h, 32-bit out; W is its own tensor or, when `tied_to` is given and
    the folder has no such tensor, the embedding table (infer/model.odin:150-158).
    softcap > 0: logits <- softcap * tanh(logits / softcap).  scale: a factor on the logits (a 32-bit product, after
    the cap)."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, weight: str, tied_to: str | None = None, softcap: float = 0.0,
                 scale: float = 1.0):
        self.vocab_size, self.width, self.weight_name, self.tied_to = vocab_size, width, weight, tied_to
        self.softcap, self.scale = float(softcap), float(scale)
        self.w = None

    def params(self):
        return [ParamSpec(self.weight_name, (self.vocab_size, self.width), alias_of=self.tied_to)]

    def bind(self, tensors, rt):
        self.w = tensors[self.weight_name]

    def kernel_groups(self):
        return {"gemm_plain"} | ({"rowwise"} if (self.softcap > 0 or self.scale != 1.0) else set())

    def forward(self, rt, step, h):
        logits = rt.linear(h, self.w, out_dtype=torch.float32)
        if self.softcap > 0 or self.scale != 1.0:
            ops.softcap(logits, self.softcap, self.scale)
        return logits
