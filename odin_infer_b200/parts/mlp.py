"""Dense feed-forward parts."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, ParamSpec, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """down( silu(gate(x)) * up(x) ), no bias (infer/forward.odin:125-135).  The gate
    and up matrices are fused into one at load time.  activation: "silu", or "gelu_tanh" for
    down( gelu_tanh(gate(x)) * up(x) )."""

    graph_safe = True

    def __init__(self, width: int, inner: int, names: dict, activation: str = "silu"):
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"a gated feed-forward takes silu or gelu_tanh, got '{activation}'")
        self.width, self.inner, self.names, self.activation = width, inner, dict(names), activation
        self.w_gate_up = self.w_down = None

    def params(self):
        n = self.names
        return [ParamSpec(n["gate"], (self.inner, self.width)), ParamSpec(n["up"], (self.inner, self.width)),
                ParamSpec(n["down"], (self.width, self.inner))]

    def bind(self, tensors, rt):
        n = self.names
        g, u = tensors.pop(n["gate"]), tensors.pop(n["up"])
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[n["down"]]

    def kernel_groups(self):
        return {"elementwise", "gemm_plain"} | ({"rowwise"} if self.activation != "silu" else set())

    def notes(self, rt):
        if rt.dtype != torch.bfloat16:
            return []
        return [f"feed-forward: {what} = {k} is no multiple of 8: its matrix products run on CUDA cores "
                "(the tensor-core kernels read rows of whole 16 bytes)"
                for what, k in (("width", self.width), ("inner", self.inner)) if k % 8]

    takes_residual = True

    def forward(self, rt, step, h, residual=None):
        act = rt.gated_linear(h, self.w_gate_up, self.inner, self.activation)
        return rt.linear(act, self.w_down, out_dtype=torch.float32, may_split=True, add_to=residual)


@register_part("feed_forward", "activated")
class ActivatedMLP(FeedForward):
    """down( act( up(x) ) ), no gate and no bias.  activation: one of `ops.ACTIVATIONS`; "xielu" reads its
    two numbers (p, q) from the tensor `names["act"]`:
    z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""

    graph_safe = True
    takes_residual = True

    def __init__(self, width: int, inner: int, names: dict, activation: str = "xielu"):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation '{activation}' (known: {', '.join(ops.ACTIVATIONS)})")
        self.width, self.inner, self.names, self.activation = width, inner, dict(names), activation
        self.w_up = self.w_down = self.act_params = None

    def params(self):
        n = self.names
        out = [ParamSpec(n["up"], (self.inner, self.width)), ParamSpec(n["down"], (self.width, self.inner))]
        if self.activation == "xielu":
            out.append(ParamSpec(n["act"], (2,), init="unit"))
        return out

    def bind(self, tensors, rt):
        n = self.names
        self.w_up, self.w_down = tensors[n["up"]], tensors[n["down"]]
        if self.activation == "xielu":
            self.act_params = tensors[n["act"]]

    def kernel_groups(self):
        return {"rowwise", "gemm_plain"}

    def forward(self, rt, step, h, residual=None):
        up = rt.linear(h, self.w_up, may_split=True)
        act = rt.empty(h.shape[0], self.inner)
        ops.activation(up, self.activation, act, self.act_params)
        return rt.linear(act, self.w_down, out_dtype=torch.float32, may_split=True, add_to=residual)
