"""A per-layer input from the token itself, added to the stream after the layer:

    e = table[token, col0 : col0 + dim]      (one table for all layers, a slice of columns per layer)
    y = Wproj (gelu_tanh(Wgate x) * e)       (x: the stream)
    delta = y / sqrt(mean(y^2) + eps) * norm

The norm is float32; the delta is handed back for the stream's next reader to add.
"""
from __future__ import annotations

from typing import List

import torch

from .base import TokenInput
from .registry import register_part
from .spec import TensorNeed, TokenSideSpec


class GatedTokenSide(TokenInput):
    def __init__(self, spec: TokenSideSpec, env):
        super().__init__(spec, env)
        if spec.col0 < 0 or spec.col0 + spec.dim > spec.table_width:
            raise ValueError("token side input: the layer's columns lie outside the table")
        self.table = self.w_gate = self.w_proj = self.norm = None

    @staticmethod
    def tensor_needs(spec: TokenSideSpec) -> List[TensorNeed]:
        return [TensorNeed(spec.table, (spec.vocab_size, spec.table_width)),
                TensorNeed(spec.gate_weight, (spec.dim, spec.hidden)),
                TensorNeed(spec.proj_weight, (spec.hidden, spec.dim)),
                TensorNeed(spec.norm_weight, (spec.hidden,), "float32", init="around_one")]

    def load(self, tensors) -> None:
        s = self.spec
        self.table, self.w_gate, self.w_proj, self.norm = (tensors[s.table], tensors[s.gate_weight], tensors[s.proj_weight],
                                                           tensors[s.norm_weight])

    def forward(self, x, ctx) -> torch.Tensor:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        z = ctx.ws.get("side.z", (n, s.dim), dt)
        ops.gemm(x[:n], self.w_gate, z)
        g = ctx.ws.get("side.g", (n, s.dim), dt)
        ops.token_gate(z, self.table, s.col0, ctx.token_ids, g)
        y = ctx.ws.get("side.y", (n, s.hidden), torch.float32)
        ops.gemm(g, self.w_proj, y)
        delta = ctx.ws.get("side.delta", (n, s.hidden), torch.float32)
        return ops.rmsnorm(y, self.norm, s.eps, delta)


register_part("token_input", "gated_side", GatedTokenSide)
