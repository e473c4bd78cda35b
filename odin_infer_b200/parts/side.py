"""Extras of a block: what it does to the residual stream after its mixer and feed-forward."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import BlockExtra, ParamSpec, register_part, split_update


@register_part("block_extra", "token_side_input")
class TokenSideInput(BlockExtra):
    """A per-layer input from the tokens themselves: a second embedding table (shared by the layers, one
    slice of `dim` columns per layer) is gated by the residual stream and projected back into it,

        e = T[token, first_column : first_column + dim]      g = gelu_tanh(G x) * e
        y = P g                                               x += w * y / sqrt(mean(y^2) + eps)

    (the last norm is a plain RMSNorm over the width, whatever norm the model uses elsewhere)."""

    graph_safe = True

    def __init__(self, width: int, dim: int, vocab_size: int, table_width: int, first_column: int, names: dict,
                 eps: float = 1e-5):
        if not (0 <= first_column and first_column + dim <= table_width):
            raise ValueError(f"columns {first_column}..{first_column + dim} lie outside a table of {table_width}")
        self.width, self.dim, self.vocab_size, self.table_width = width, dim, vocab_size, table_width
        self.first_column, self.names, self.eps = first_column, dict(names), float(eps)

    def params(self):
        n = self.names
        return [ParamSpec(n["table"], (self.vocab_size, self.table_width)), ParamSpec(n["gate"], (self.dim, self.width)),
                ParamSpec(n["proj"], (self.width, self.dim)), ParamSpec(n["norm"], (self.width,), init="norm")]

    def bind(self, tensors, rt):
        n = self.names
        self.table, self.w_gate, self.w_proj, self.norm_w = (tensors[n[k]] for k in ("table", "gate", "proj", "norm"))

    def kernel_groups(self):
        return {"rowwise", "gemm_plain"}

    def forward(self, rt, step, x, pending):
        xa = rt.settle(x, *split_update(pending))
        gate = rt.linear(xa, self.w_gate, out_dtype=torch.float32, may_split=True)
        g = rt.empty(x.shape[0], self.dim)
        ops.gated_lookup(gate, "gelu_tanh", self.table, self.first_column, step.tok_ids, g)
        y = rt.linear(g, self.w_proj, out_dtype=torch.float32, may_split=True)
        ops.normed_add(x, y, self.norm_w, self.eps, step.tok_seq)
        return x, None
