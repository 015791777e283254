"""A feed-forward of experts chosen per token by a linear router."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Combined, FeedForward, ParamSpec, Several, register_part


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """`n_experts` gated feed-forwards W_down (act(W_gate h) * (W_up h)) of inner size `inner`, of which every
    token uses `top`: router logits z = W_r h + b in 32-bit, the `top` largest are chosen, their weights are
    the softmax over the chosen logits alone, and the update is the weighted sum of the chosen experts'
    outputs.  shared_inner > 0: one more expert of that inner size (tensor names under "shared_*") that every
    token uses with weight 1.

    names: "router", "router_bias" (None: no bias), "gate" / "up" / "down" with "{e}" for the expert's number,
    and "shared_gate" / "shared_up" / "shared_down".  The experts' matrices are stacked at load
    ([experts, 2 inner, width] gate rows before up rows, and [experts, width, inner]).  A shared expert whose
    inner size is a multiple of the experts' is cut into that many experts of the common size that every token
    uses with weight 1 (a gated feed-forward is a sum over its inner columns) and rides in the same launches;
    any other shared expert runs as a dense gated feed-forward beside them.

    gated=False: an expert is W_down act(W_up h) (no gate matrix; names "up" / "down", "shared_up" / "shared_down");
    activation may then also be "relu2", max(z, 0)^2.
    score: how the router chooses and weighs: "softmax_of_chosen" as above, or "sigmoid_in_groups": scores
    sigmoid(z) (no bias); the experts form `groups` equal groups of neighbours, a group's score is the sum of its
    two largest scores, only experts of the `keep` best groups can be chosen, the `top` largest scores among them
    are, and their weights are the scores divided by their sum (+ 1e-20), times `route_scale`.
    score "softmax_corrected_in_groups": scores softmax(z) over all rows of the router; the experts are chosen by score +
    correction (the tensor names["router_bias"], which the weights do not see), a group's score is its largest choice
    score, and the weights are the chosen scores / (their sum + 1e-20) * route_scale.
    n_pass: the router has that many rows more than there are experts; a token that chooses one of them gets its own input
    back, times the weight (they count as the last members of the groups; they have no tensors).
    shared_gate: the shared expert's output is multiplied by sigmoid(g . h), one number per token, g the tensor
    names["shared_token_gate"] ([1, width]); g rides as one more row of the router's matrix.

    The update of few tokens comes back as partial sums, one slice per choice, which the next norm adds in order;
    with many tokens the rows are sorted by expert and run as grouped tensor-core products (`Runtime.experts`)."""

    graph_safe = True

    def __init__(self, width: int, inner: int, n_experts: int, top: int, names: dict, activation: str = "silu",
                 shared_inner: int = 0, gated: bool = True, score: str = "softmax_of_chosen", groups: int = 1,
                 keep: int = 1, route_scale: float = 1.0, shared_gate: bool = False, n_pass: int = 0):
        n_rows = n_experts + int(n_pass)
        if not (0 < top <= n_rows) or n_pass < 0:
            raise ValueError(f"every token uses {top} of {n_rows} experts: not possible")
        if n_pass and score != "softmax_corrected_in_groups":
            raise ValueError("rows of the router without an expert go with the score 'softmax_corrected_in_groups'")
        if activation not in (("silu", "gelu_tanh") if gated else ("silu", "gelu_tanh", "relu2")):
            raise ValueError(f"an expert's activation is silu or gelu_tanh (or relu2 without a gate), got '{activation}'")
        if score not in ops.ROUTER_SCORES:
            raise ValueError(f"a router scores by one of {', '.join(ops.ROUTER_SCORES)}, got '{score}'")
        if groups < 1 or n_rows % groups or not (1 <= keep <= groups) or keep * (n_rows // groups) < top:
            raise ValueError(f"{n_rows} experts in {groups} groups of which {keep} stay cannot give {top} experts a token")
        if groups > 1 and score == "softmax_of_chosen":
            raise ValueError("groups of experts go with the scores 'sigmoid_in_groups' and 'softmax_corrected_in_groups'")
        if shared_gate and not shared_inner:
            raise ValueError("a gate on the shared expert needs a shared expert")
        if shared_gate and gated:
            raise ValueError("a gate on the shared expert is built for experts without a gate matrix")
        self.width, self.inner, self.n_experts, self.top = width, inner, n_experts, top
        self.names, self.activation, self.shared_inner = dict(names), activation, int(shared_inner)
        self.gated, self.score, self.groups, self.keep = bool(gated), score, int(groups), int(keep)
        self.route_scale, self.shared_gate, self.n_pass = float(route_scale), bool(shared_gate), int(n_pass)
        # the shared expert as experts of the common size that every token uses
        self.shared_as_experts = self.shared_inner // inner if (self.shared_inner and self.shared_inner % inner == 0) else 0
        self.w_router = self.b_router = self.w_gate_up = self.w_down = self.ws_gate_up = self.ws_down = None

    def _expert_names(self, e: int):
        n = self.names
        if not self.gated:
            return n["up"].format(e=e), n["down"].format(e=e)
        return n["gate"].format(e=e), n["up"].format(e=e), n["down"].format(e=e)

    def params(self):
        n = self.names
        out = [ParamSpec(n["router"], (self.n_experts + self.n_pass, self.width))]
        if n.get("router_bias"):
            out.append(ParamSpec(n["router_bias"], (self.n_experts + self.n_pass,), init="near_zero"))
        for e in range(self.n_experts):
            *ups, d = self._expert_names(e)
            out += [ParamSpec(u, (self.inner, self.width)) for u in ups] + [ParamSpec(d, (self.width, self.inner))]
        if self.shared_inner:
            if self.gated:
                out.append(ParamSpec(n["shared_gate"], (self.shared_inner, self.width)))
            out += [ParamSpec(n["shared_up"], (self.shared_inner, self.width)),
                    ParamSpec(n["shared_down"], (self.width, self.shared_inner))]
            if self.shared_gate:
                out.append(ParamSpec(n["shared_token_gate"], (1, self.width)))
        return out

    def bind(self, tensors, rt):
        n = self.names
        self.w_router = tensors[n["router"]].contiguous()
        if self.shared_gate:
            sg = tensors.pop(n["shared_token_gate"]).reshape(1, self.width)
            wr = self.w_router
            if sg.dtype != wr.dtype:
                sg, wr = sg.float(), wr.float()
            self.w_router = torch.cat([wr, sg], dim=0).contiguous()   # the gate's vector as the row after the experts'
        self.b_router = tensors[n["router_bias"]].to(torch.float32).contiguous() if n.get("router_bias") else None
        gate_up, down = [], []
        for e in range(self.n_experts):
            *ups, d = (tensors.pop(k) for k in self._expert_names(e))
            gate_up.append(torch.cat(ups, dim=0) if self.gated else ups[0])
            down.append(d)
        if self.shared_inner:
            g = tensors.pop(n["shared_gate"]) if self.gated else None
            u, d = tensors.pop(n["shared_up"]), tensors.pop(n["shared_down"])
            if self.shared_as_experts:
                f = self.inner
                for p in range(self.shared_as_experts):
                    rows = [t[p * f:(p + 1) * f] for t in ((g, u) if self.gated else (u,))]
                    gate_up.append(torch.cat(rows, dim=0) if self.gated else rows[0])
                    down.append(d[:, p * f:(p + 1) * f])
            elif not self.gated:
                self.ws_gate_up, self.ws_down = u.contiguous(), d
            else:
                if g.dtype != u.dtype:
                    g, u = g.float(), u.float()
                self.ws_gate_up, self.ws_down = torch.cat([g, u], dim=0).contiguous(), d
        if len({t.dtype for t in gate_up + down}) > 1:
            gate_up, down = [t.float() for t in gate_up], [t.float() for t in down]
        self.w_gate_up = torch.stack(gate_up).contiguous()
        self.w_down = torch.stack([t.contiguous() for t in down]).contiguous()

    def kernel_groups(self):
        return {"moe", "moe_tc", "elementwise", "rowwise", "gemm_plain"}

    def forward(self, rt, step, h, residual=None):
        T = h.shape[0]
        per = self.top + self.shared_as_experts
        ids = rt.empty(T, per, dtype=torch.int32)
        wts = rt.empty(T, per, dtype=torch.float32)
        logits = None
        if T > 64 and rt.dtype == torch.bfloat16 and ops.gemm_tc_supported(h, self.w_router):
            # many tokens: the logits as a tensor-core product (bfloat16 factors, 32-bit sums); the 32-bit engine keeps
            # the one kernel whatever the number of tokens, so that a token's logits are the same bits in every cut
            logits = rt.linear(h, self.w_router, out_dtype=torch.float32)
        beside = self.ws_gate_up is not None   # a shared expert that runs as a dense feed-forward beside the experts
        gate = rt.empty(T, dtype=torch.float32) if (self.shared_gate and beside) else None
        passed = rt.empty(T, dtype=torch.float32) if self.n_pass else None
        ops.moe_router(h, self.w_router, self.b_router, self.top, self.shared_as_experts, step.tok_seq, ids, wts, logits,
                       score=self.score, groups=self.groups, keep=self.keep, route_scale=self.route_scale,
                       gate_row=self.shared_gate, gate_out=gate, n_real=self.n_experts, pass_out=passed)
        y = rt.experts(h, self.w_gate_up, self.w_down, ids, wts, self.activation, gated=self.gated)
        if self.n_pass:
            # the input itself, times the summed weight of the chosen rows that have no expert, is one more term
            terms = Combined([ops.Term(y)])
            if beside:
                act = rt.gated_linear(h, self.ws_gate_up, self.shared_inner, self.activation)
                terms.append(ops.Term(rt.linear(act, self.ws_down, out_dtype=torch.float32, may_split=True)))
            terms.append(ops.Term(h, 1.0, passed))
            return terms
        if not beside:
            return y
        if self.gated:
            act = rt.gated_linear(h, self.ws_gate_up, self.shared_inner, self.activation)
        else:
            # act(W_up h), every row times its token's gate: W_down (s a) = s (W_down a)
            act = rt.empty(T, self.shared_inner)
            ops.activation(rt.linear(h, self.ws_gate_up, may_split=True), self.activation, act, row_scale=gate)
        return Several([y, rt.linear(act, self.ws_down, out_dtype=torch.float32, may_split=True)])
