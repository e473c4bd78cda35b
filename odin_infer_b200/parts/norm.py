"""RMSNorm with a plain weight, fused with the residual add that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, ParamSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """o = w * (x / sqrt(mean(x^2) + eps)), in 32-bit (infer/ops.odin:7-19).

    groups > 1: the row is cut into that many equal consecutive parts and each part is divided
    by its own root mean square; the weight still spans the whole row."""

    graph_safe = True
    takes_bias = True

    def __init__(self, width: int, eps: float, weight: str, groups: int = 1):
        if groups < 1 or width % groups:
            raise ValueError(f"a norm over {width} elements cannot be cut into {groups} equal groups")
        self.width, self.eps, self.weight_name, self.groups = width, float(eps), weight, int(groups)
        self.weight: torch.Tensor | None = None

    def params(self):
        return [ParamSpec(self.weight_name, (self.width,), init="norm")]

    def bind(self, tensors, rt):
        self.weight = tensors[self.weight_name]

    def kernel_groups(self):
        return {"elementwise", "rowwise"}

    def forward(self, rt, x, delta, rows=None, bias=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = rt.empty(n, self.width)
        if self.groups == 1 and bias is None:
            ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        else:
            ops.row_update(x, delta, bias, self.weight, self.eps, self.groups, out, rows)
        return out

    def in_place(self, rt, x) -> None:
        """x (32-bit) <- its own norm."""
        ops.row_update(x, None, None, self.weight, self.eps, self.groups, x)
