"""A feed-forward of experts chosen per token by a linear router."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, ParamSpec, Several, register_part


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

    The update of few tokens comes back as partial sums, one slice per choice, which the next norm adds in order;
    with many tokens the rows are sorted by expert and run as grouped tensor-core products (`Runtime.experts`)."""

    graph_safe = True

    def __init__(self, width: int, inner: int, n_experts: int, top: int, names: dict, activation: str = "silu",
                 shared_inner: int = 0):
        if not (0 < top <= n_experts):
            raise ValueError(f"every token uses {top} of {n_experts} experts: not possible")
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"an expert's activation is silu or gelu_tanh, got '{activation}'")
        self.width, self.inner, self.n_experts, self.top = width, inner, n_experts, top
        self.names, self.activation, self.shared_inner = dict(names), activation, int(shared_inner)
        # the shared expert as experts of the common size that every token uses
        self.shared_as_experts = self.shared_inner // inner if (self.shared_inner and self.shared_inner % inner == 0) else 0
        self.w_router = self.b_router = self.w_gate_up = self.w_down = self.ws_gate_up = self.ws_down = None

    def _expert_names(self, e: int):
        n = self.names
        return n["gate"].format(e=e), n["up"].format(e=e), n["down"].format(e=e)

    def params(self):
        n = self.names
        out = [ParamSpec(n["router"], (self.n_experts, self.width))]
        if n.get("router_bias"):
            out.append(ParamSpec(n["router_bias"], (self.n_experts,), init="near_zero"))
        for e in range(self.n_experts):
            g, u, d = self._expert_names(e)
            out += [ParamSpec(g, (self.inner, self.width)), ParamSpec(u, (self.inner, self.width)),
                    ParamSpec(d, (self.width, self.inner))]
        if self.shared_inner:
            out += [ParamSpec(n["shared_gate"], (self.shared_inner, self.width)),
                    ParamSpec(n["shared_up"], (self.shared_inner, self.width)),
                    ParamSpec(n["shared_down"], (self.width, self.shared_inner))]
        return out

    def bind(self, tensors, rt):
        n = self.names
        self.w_router = tensors[n["router"]].contiguous()
        self.b_router = tensors[n["router_bias"]].to(torch.float32).contiguous() if n.get("router_bias") else None
        gate_up, down = [], []
        for e in range(self.n_experts):
            g, u, d = (tensors.pop(k) for k in self._expert_names(e))
            gate_up.append(torch.cat([g, u], dim=0))
            down.append(d)
        if self.shared_inner:
            g, u, d = tensors.pop(n["shared_gate"]), tensors.pop(n["shared_up"]), tensors.pop(n["shared_down"])
            if self.shared_as_experts:
                f = self.inner
                for p in range(self.shared_as_experts):
                    gate_up.append(torch.cat([g[p * f:(p + 1) * f], u[p * f:(p + 1) * f]], dim=0))
                    down.append(d[:, p * f:(p + 1) * f])
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
        ops.moe_router(h, self.w_router, self.b_router, self.top, self.shared_as_experts, step.tok_seq, ids, wts, logits)
        y = rt.experts(h, self.w_gate_up, self.w_down, ids, wts, self.activation)
        if self.ws_gate_up is None:
            return y
        act = rt.gated_linear(h, self.ws_gate_up, self.shared_inner, self.activation)
        return Several([y, rt.linear(act, self.ws_down, out_dtype=torch.float32, may_split=True)])
