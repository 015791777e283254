"""RMSNorm with a plain weight, fused with the residual add that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Combined, Norm, Normed, ParamSpec, Several, register_part


def terms_of(update) -> list:
    """The `ops.Term`s whose sum an update is."""
    if isinstance(update, Combined):
        return list(update)
    if isinstance(update, Several):
        return [ops.Term(u) for u in update if u is not None]
    if torch.is_tensor(update):
        return [ops.Term(update)]
    raise TypeError(f"an update of type {type(update).__name__} cannot be summed term by term")


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """o = w * (x / sqrt(mean(x^2) + eps)), in 32-bit (infer/ops.odin:7-19).

    groups > 1: the row is cut into that many equal consecutive parts and each part is divided
    by its own root mean square; the weight still spans the whole row.
    one_plus: the stored weight lies around zero and the factor is 1 + w (the sum is formed once at load,
    in 32-bit, and kept so)."""

    graph_safe = True
    takes_bias = True
    takes_several = True
    takes_scale = True
    takes_terms = True

    def __init__(self, width: int, eps: float, weight: str, groups: int = 1, one_plus: bool = False):
        if groups < 1 or width % groups:
            raise ValueError(f"a norm over {width} elements cannot be cut into {groups} equal groups")
        self.width, self.eps, self.weight_name, self.groups = width, float(eps), weight, int(groups)
        self.one_plus = bool(one_plus)
        self.weight: torch.Tensor | None = None

    def params(self):
        return [ParamSpec(self.weight_name, (self.width,), init="near_zero" if self.one_plus else "norm")]

    def bind(self, tensors, rt):
        self.weight = tensors[self.weight_name]
        if self.one_plus:
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()

    def kernel_groups(self):
        return {"elementwise", "rowwise"}

    def pairs_with(self, other) -> bool:
        """Whether `other` norms the same row by the same root mean square (another weight only), so that one kernel
        can write both outputs."""
        return (type(other) is type(self) and other.width == self.width and other.eps == self.eps
                and other.groups == self.groups)

    def forward(self, rt, x, delta, rows=None, bias=None, scale: float = 1.0, second=None):
        """second: a norm that `pairs_with` this one; both outputs of the one updated row come back, (out, out2)."""
        n = x.shape[0] if rows is None else rows.numel()
        out = rt.empty(n, self.width)
        if isinstance(delta, (Normed, Combined)):
            # a sum of terms, a norm of the update's own, the add and this norm: one kernel
            if self.groups != 1 or bias is not None or scale != 1.0 or second is not None:
                raise TypeError("an update of several terms or with a norm of its own meets a plain RMSNorm only")
            post_w, post_eps, inner = (delta.weight, delta.eps, delta.update) if isinstance(delta, Normed) else (None, 0.0, delta)
            ops.combine_add(x, terms_of(inner), post_w, post_eps, self.weight, self.eps, out, rows)
            return out
        if isinstance(delta, (list, tuple)) and len(delta) == 1:
            delta = delta[0]
        if delta is None and bias is None:
            scale = 1.0
        if second is not None:
            out2 = rt.empty(n, self.width)
            ops.row_update(x, delta, bias, self.weight, self.eps, self.groups, out, rows, scale=scale,
                           weight2=second.weight, out2=out2)
            return out, out2
        if self.groups == 1 and bias is None and scale == 1.0 and not isinstance(delta, (list, tuple)):
            ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        else:
            ops.row_update(x, delta, bias, self.weight, self.eps, self.groups, out, rows, scale=scale)
        return out

    def in_place(self, rt, x) -> None:
        """x (32-bit) <- its own norm."""
        ops.row_update(x, None, None, self.weight, self.eps, self.groups, x)
