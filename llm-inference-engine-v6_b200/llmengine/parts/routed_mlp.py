"""Routed feed-forward (mixture of experts): every token goes through `top` of `experts` small feed-forward
layers, chosen by a linear router, and the results are added with the router's weights.

    z = Wr x + b  (float32);  chosen = the `top` largest z;  g = softmax(z[chosen])
    out = sum_e g_e * Wdown_e act(Wup_e x),  act = the exact (erf) gelu, no biases

The step's (token, choice) pairs are sorted by expert on the device into tiles of rows of one expert; the
per-expert products run over those tiles (all experts in one launch) and write each pair's row at the
pair's own index, so the weighted sum is a fixed-order sum over a token's `top` rows. All shapes depend on
the number of tokens alone: nothing is read back, and a decode step can be recorded as a CUDA graph.
"""
from __future__ import annotations

from typing import List

import torch

from .base import FeedForward, NormalizedRows
from .registry import register_part
from .spec import RoutedMLPSpec, TensorNeed


class RoutedMLP(FeedForward):
    def __init__(self, spec: RoutedMLPSpec, env):
        super().__init__(spec, env)
        if spec.activation != "gelu":
            raise ValueError(f"routed feed-forward: activation '{spec.activation}' is not implemented (gelu is)")
        if not (1 <= spec.top <= spec.experts):
            raise ValueError(f"routed feed-forward: cannot choose {spec.top} of {spec.experts} experts")
        if len(spec.up_weights) != spec.experts or len(spec.down_weights) != spec.experts:
            raise ValueError("routed feed-forward: one up and one down matrix per expert")
        self.router = self.bias = self.w_up = self.w_down = None

    @staticmethod
    def tensor_needs(spec: RoutedMLPSpec) -> List[TensorNeed]:
        out = [TensorNeed(spec.router_weight, (spec.experts, spec.hidden))]
        if spec.router_bias:
            out.append(TensorNeed(spec.router_bias, (spec.experts,), "float32", init="zeros"))
        for up, down in zip(spec.up_weights, spec.down_weights):
            out += [TensorNeed(up, (spec.intermediate, spec.hidden)), TensorNeed(down, (spec.hidden, spec.intermediate))]
        return out

    def kernel_notes(self):
        s = self.spec
        if self.env.dtype == torch.bfloat16 and (s.hidden % 8 or s.intermediate % 8):
            return [f"routed feed-forward: sizes {s.hidden} and {s.intermediate} are not both multiples of 8: the per-expert "
                    "products run on CUDA cores"]
        return []

    def load(self, tensors) -> None:
        s = self.spec
        self.router = tensors[s.router_weight]
        self.bias = tensors[s.router_bias] if s.router_bias else None
        self.w_up = torch.stack([tensors[n] for n in s.up_weights]).contiguous()      # [E, ff, hidden]
        self.w_down = torch.stack([tensors[n] for n in s.down_weights]).contiguous()  # [E, hidden, ff]

    def forward(self, x, ctx) -> torch.Tensor:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        x = x[:n]
        idx = ctx.ws.get("routed.idx", (n, s.top), torch.int32)
        share = ctx.ws.get("routed.share", (n, s.top), torch.float32)
        ops.route(x, self.router, self.bias, s.top, idx, share)
        tile = ops.routed_tile_rows(n, dt, (s.hidden, s.intermediate), n * s.top / s.experts)
        tile_expert, tile_rows = ops.routed_group(idx, s.experts, tile, ctx.ws, "routed")
        act = ctx.ws.get("routed.act", (n * s.top, s.intermediate), dt)
        ops.routed_product(x, s.top, self.w_up, tile_expert, tile_rows, act, "gelu")
        y = ctx.ws.get("routed.y", (n * s.top, s.hidden), torch.float32)
        ops.routed_product(act, 1, self.w_down, tile_expert, tile_rows, y, "share", share=share.view(-1))
        out = ctx.ws.get("routed.delta", (n, s.hidden), torch.float32)
        return ops.routed_combine(y, out, s.top)


register_part("feed_forward", "routed_mlp", RoutedMLP)
