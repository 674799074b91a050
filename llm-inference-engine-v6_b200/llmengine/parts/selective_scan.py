"""Selective scan: a recurrent mixer whose decay, input and output maps depend on the token (SelectiveScanSpec).

With h the mixer's input, per token (C channels, N state numbers a channel, K taps):
    [x | z] = W_in h
    x_c <- silu(bias_c + sum_j conv[c, j] * x_c(t - (K - 1) + j))      causal, zeros before the sequence
    [dt_low | B | Cm] = W_x x;  dt = softplus(W_dt dt_low + dt_bias)   one step size a channel
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,  A = -exp(a_log)
    y_c = sum_n S[c, n] Cm_n + skip_c x_c;   out = W_o (y * silu(z))
What a request keeps between steps is of fixed size and lives in its state slot: S (float32 [C, N]) and the last K - 1
inputs of the convolution (float32 [K - 1, C]); both start at zero. Step sizes, decays, B, Cm and the state are float32
in both engine precisions. With up to 8 tokens, and always in the 32-bit engine, the W_x product is written out in float32 and the
step-size map runs on CUDA cores from it; with more tokens in bfloat16 the low-rank rows are a product of their own, rounded to
bfloat16 as the operand of the step-size map on the tensor cores (a projection, like W_x itself), whose float32 sums the scan
turns into step sizes. The convolution's result is rounded to the engine precision once, as the operand of W_x.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .attention import add_into_stream_or_partials
from .base import LayerCache, Mixer, NormalizedRows, StateNeed
from .registry import register_part
from .spec import SelectiveScanSpec, TensorNeed


class SelectiveScan(Mixer):
    def __init__(self, spec: SelectiveScanSpec, env):
        super().__init__(spec, env)
        for name in ("inner", "state", "taps", "dt_rank"):
            if getattr(spec, name) <= 0:
                raise ValueError(f"selective scan: {name} must be >= 1")
        self.w_in = self.w_conv = self.conv_bias = self.w_x = self.w_dt_t = self.dt_bias = self.a_log = self.skip = self.w_o = None

    @staticmethod
    def tensor_needs(spec: SelectiveScanSpec) -> List[TensorNeed]:
        C, N, R = spec.inner, spec.state, spec.dt_rank
        return [TensorNeed(spec.in_weight, (2 * C, spec.hidden)), TensorNeed(spec.conv_weight, (C, spec.taps)),
                TensorNeed(spec.conv_bias, (C,), "float32", init="zeros"), TensorNeed(spec.x_weight, (R + 2 * N, C)),
                TensorNeed(spec.dt_weight, (C, R)), TensorNeed(spec.dt_bias, (C,), "float32"),
                TensorNeed(spec.a_log, (C, N), "float32"), TensorNeed(spec.skip, (C,), "float32", init="around_one"),
                TensorNeed(spec.o_weight, (spec.hidden, C))]

    def cache_needs(self):
        s = self.spec
        return (StateNeed("scan", (s.inner, s.state)), StateNeed("conv", (s.taps - 1, s.inner)))

    def load(self, tensors) -> None:
        s = self.spec
        self.w_in, self.w_conv, self.conv_bias = tensors[s.in_weight], tensors[s.conv_weight], tensors[s.conv_bias]
        self.w_x = tensors[s.x_weight]
        # for steps of many tokens in bfloat16: the low-rank rows and [B | C] as products of their own, so that the low-rank rows
        # come out in bfloat16 as the operand of the step-size product on the tensor cores
        self.w_x_low = self.w_x[:s.dt_rank].contiguous()
        self.w_x_bc = self.w_x[s.dt_rank:].contiguous()
        self.w_dt = tensors[s.dt_weight]
        self.w_dt_t = tensors[s.dt_weight].t().contiguous()  # [rank, channels]: neighbouring channels read neighbouring words
        self.dt_bias, self.a_log, self.skip, self.w_o = tensors[s.dt_bias], tensors[s.a_log], tensors[s.skip], tensors[s.o_weight]

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        C, N, R = s.inner, s.state, s.dt_rank
        if n <= 64:
            xz = ops.gemm_partials(x[:n], self.w_in, ctx.ws, "scan.in_parts")
        else:
            xz = ctx.ws.get("scan.in_parts", (1, n, 2 * C), torch.float32)
            ops.gemm(x[:n], self.w_in, xz[0])
        xc = ctx.ws.get("scan.xc", (n, C), dt)
        ops.conv_silu(xz, 0, C, self.w_conv, self.conv_bias, cache.states["conv"], ctx, xc)
        step = ctx.ws.get("scan.dt", (n, C), torch.float32)
        y = ctx.ws.get("scan.y", (n, C), dt)
        if dt == torch.bfloat16 and n > 8 and R % 8 == 0 and C % 8 == 0:
            # more than a handful of tokens: the step-size map is a tensor-core product of the low-rank rows (rounded to bfloat16 as its operand);
            # bias and softplus are applied where the scan reads the sums
            low = ctx.ws.get("scan.low", (n, R), dt)
            ops.gemm(xc, self.w_x_low, low, ctx.ws)
            proj = ctx.ws.get("scan.proj", (n, 2 * N), torch.float32)
            ops.gemm(xc, self.w_x_bc, proj, ctx.ws)
            ops.gemm(low, self.w_dt, step, ctx.ws)
            ops.selective_scan(xc, step, proj, 0, N, N, xz, C, self.a_log, self.skip, cache.states["scan"], ctx, y,
                               dt_bias=self.dt_bias, dt_raw=True)
        else:
            proj = ctx.ws.get("scan.proj", (n, R + 2 * N), torch.float32)
            ops.gemm(xc, self.w_x, proj, ctx.ws)
            ops.dt_softplus(proj, R, self.w_dt_t, self.dt_bias, step, n)
            ops.selective_scan(xc, step, proj, R, R + N, N, xz, C, self.a_log, self.skip, cache.states["scan"], ctx, y)
        return add_into_stream_or_partials(ops, y, self.w_o, ctx, False, "scan.delta")


register_part("mixer", "selective_scan", SelectiveScan)
