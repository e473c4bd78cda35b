"""Token embedding and the output head."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Embedding, Head, ParamSpec, PartSpec, build_part, register_part


@register_part("embedding", "token_table")
class TokenEmbedding(Embedding):
    """x = E[token] (infer/forward.odin:43), times `scale` (a 32-bit product) where one is given.  norm: a norm
    (a PartSpec of a norm that can work in place) through which the embedded rows pass before they become the
    residual stream."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, weight: str, norm: PartSpec | None = None, scale: float = 1.0):
        self.vocab_size, self.width, self.weight_name, self.scale = vocab_size, width, weight, float(scale)
        self.norm = build_part("norm", norm) if norm is not None else None
        self.table = None

    def params(self):
        return [ParamSpec(self.weight_name, (self.vocab_size, self.width))] + (self.norm.params() if self.norm else [])

    def bind(self, tensors, rt):
        self.table = tensors[self.weight_name]
        if self.norm is not None:
            self.norm.bind(tensors, rt)

    def kernel_groups(self):
        return {"elementwise"} | (self.norm.kernel_groups() if self.norm else set())

    def forward(self, rt, step):
        x = rt.empty(step.n_rows, self.width, dtype=torch.float32)
        ops.embed(self.table, step.tok_ids, x, self.scale)
        if self.norm is not None:
            self.norm.in_place(rt, x)
        return x


@register_part("head", "linear")
class LinearHead(Head):
    """logits = W h, 32-bit out; W is its own tensor or, when `tied_to` is given and
    the folder has no such tensor, the embedding table (infer/model.odin:150-158).
    softcap > 0: logits <- softcap * tanh(logits / softcap)."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, weight: str, tied_to: str | None = None, softcap: float = 0.0):
        self.vocab_size, self.width, self.weight_name, self.tied_to = vocab_size, width, weight, tied_to
        self.softcap = float(softcap)
        self.w = None

    def params(self):
        return [ParamSpec(self.weight_name, (self.vocab_size, self.width), alias_of=self.tied_to)]

    def bind(self, tensors, rt):
        self.w = tensors[self.weight_name]

    def kernel_groups(self):
        return {"gemm_plain"} | ({"rowwise"} if self.softcap > 0 else set())

    def forward(self, rt, step, h):
        logits = rt.linear(h, self.w, out_dtype=torch.float32)
        if self.softcap > 0:
            ops.softcap(logits, self.softcap)
        return logits
