"""Latent attention: causal softmax attention whose keys and values are linear maps of ONE cached
latent per token.

With h the mixer's input, per token:
    cq = rmsnorm(Wdq h) * dq_norm,  q = Wuq cq        (per head: `dim` unrotated numbers, then `rot_dim` rotated)
    [c' | kr'] = Wdkv h,  c = rmsnorm(c') * dkv_norm,  kr = rot(kr')  (one rotated key part for all heads)
    k_a = [Wuk_a c | kr],  v_a = Wuv_a c,  score_a(i, j) = (q_a(i) . k_a(j)) * scale,  j <= i
    out = Wo ((heads' outputs side by side) * sigmoid(Wg h))
Only [c | kr] is kept per token (a page tensor [pages, 1, page, kv_rank + rot_dim], no value tensor).
The products with Wuk and Wuv are moved to the query and to the result:
    q_a . Wuk_a c = (Wuk_a^T q_a) . c,    sum_j p_j Wuv_a c_j = Wuv_a (sum_j p_j c_j)
so attention itself runs over the cached rows, as one key/value head of size kv_rank + rot_dim shared
by all heads, with values = the first kv_rank numbers of the rows. Norms, rotation, scores and softmax
are float32 in both engine precisions. The first three products read the same h and run as one product
against [Wdq; Wdkv; Wg]; its float32 sums feed the norms, the rotation and the gate directly.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .attention import add_into_stream_or_partials
from .base import KVNeed, LayerCache, Mixer, NormalizedRows
from .registry import build_part, part_class, register_part
from .spec import LatentAttentionSpec, TensorNeed


class LatentAttention(Mixer):
    def __init__(self, spec: LatentAttentionSpec, env):
        super().__init__(spec, env)
        for name in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
            if getattr(spec, name) <= 0:
                raise ValueError(f"latent attention: {name} must be >= 1")
        if spec.rot_dim < 0 or spec.window < 0:
            raise ValueError("latent attention: rot_dim and window must be >= 0")
        self.position = build_part("position", spec.position, env)
        tables = self.position.rotation_tables()
        if tables is None:
            raise ValueError("latent attention needs a position encoding with rotation tables")
        self.cos, self.sin = tables
        self.rot_dims = 0 if self.cos is None else 2 * self.cos.shape[1]
        if self.rot_dims > spec.rot_dim:
            raise ValueError(f"latent attention: {self.rot_dims} rotated dimensions do not fit a part of {spec.rot_dim}")
        self.w_in = self.w_uq = self.w_ukt = self.w_uv = self.w_o = self.dq_norm = self.dkv_norm = None

    @staticmethod
    def tensor_needs(spec: LatentAttentionSpec) -> List[TensorNeed]:
        H = spec.heads
        return [TensorNeed(spec.dq_weight, (spec.q_rank, spec.hidden)),
                TensorNeed(spec.dq_norm, (spec.q_rank,), "float32", init="around_one"),
                TensorNeed(spec.uq_weight, (H * (spec.dim + spec.rot_dim), spec.q_rank)),
                TensorNeed(spec.dkv_weight, (spec.kv_rank + spec.rot_dim, spec.hidden)),
                TensorNeed(spec.dkv_norm, (spec.kv_rank,), "float32", init="around_one"),
                TensorNeed(spec.uk_weight, (H * spec.dim, spec.kv_rank)),
                TensorNeed(spec.uv_weight, (H * spec.vdim, spec.kv_rank)),
                TensorNeed(spec.gate_weight, (H * spec.vdim, spec.hidden)),
                TensorNeed(spec.o_weight, (spec.hidden, H * spec.vdim))] + \
            list(part_class("position", spec.position.kind).tensor_needs(spec.position))

    def subparts(self):
        return (self.position,)

    def cache_needs(self):
        s = self.spec
        return (KVNeed(1, s.kv_rank + s.rot_dim, s.window, value_dim=0),)

    def kernel_notes(self):
        s, notes, ops = self.spec, [], self.env.ops
        if self.env.dtype == torch.bfloat16 and hasattr(ops, "latent_attention_kernel"):
            kernel = ops.latent_attention_kernel(s.heads, s.kv_rank, s.rot_dim, self.env.page_size)
            if kernel != "tensor cores":
                notes.append(f"latent attention with a latent of {s.kv_rank} + {s.rot_dim} numbers and pages of "
                             f"{self.env.page_size}: runs on {kernel}")
        return notes

    def load(self, tensors) -> None:
        s = self.spec
        # one product for everything that reads the mixer's input: columns [query latent | key/value latent, part to rotate | gate]
        self.w_in = torch.cat([tensors[s.dq_weight], tensors[s.dkv_weight], tensors[s.gate_weight]], dim=0).contiguous()
        self.w_uq = tensors[s.uq_weight]
        # the heads' key maps transposed, [H, kv_rank, dim]: applied to the unrotated part of the query
        self.w_ukt = tensors[s.uk_weight].view(s.heads, s.dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[s.uv_weight].view(s.heads, s.vdim, s.kv_rank).contiguous()
        self.w_o = tensors[s.o_weight]
        self.dq_norm, self.dkv_norm = tensors[s.dq_norm], tensors[s.dkv_norm]
        self.position.load(tensors)

    def forward(self, x, ctx, cache: LayerCache) -> Optional[torch.Tensor]:
        s, ops, n, dt = self.spec, self.env.ops, ctx.n_tokens, self.env.dtype
        if isinstance(x, NormalizedRows):
            x = x.dense(ctx)
        H, Dk = s.heads, s.kv_rank + s.rot_dim
        kv_off, g_off = s.q_rank, s.q_rank + Dk
        # the first product as float32 sums (in parts when few tokens stream the weights)
        if n <= 64:
            parts = ops.gemm_partials(x[:n], self.w_in, ctx.ws, "latent.in_parts")
        else:
            parts = ctx.ws.get("latent.in_parts", (1, n, self.w_in.shape[0]), torch.float32)
            ops.gemm(x[:n], self.w_in, parts[0])
        cq = ctx.ws.get("latent.cq", (n, s.q_rank), dt)
        writes = cache.writes and cache.k is not None
        ops.latent_prep(parts, 0, s.q_rank, kv_off, s.kv_rank, s.rot_dim, self.rot_dims, self.dq_norm, self.dkv_norm, s.eps,
                        self.cos, self.sin, ctx, ctx.block_tables[cache.group], cq, cache.k if writes else None)
        q = ctx.ws.get("latent.q", (n, H * (s.dim + s.rot_dim)), dt)
        ops.gemm(cq, self.w_uq, q, ctx.ws)
        ql = ctx.ws.get("latent.ql", (n, H, Dk), dt)
        many = n > 32 and hasattr(ops, "gemm_heads")
        if many and ops.gemm_heads(q.view(n, H, s.dim + s.rot_dim)[:, :, :s.dim], self.w_ukt, ql[:, :, :s.kv_rank]):
            # more than a few tokens: the heads' key maps as one tensor-core launch over tiles of tokens
            ops.latent_query(q, None, ql, H, s.dim, s.rot_dim, s.kv_rank, self.rot_dims, self.cos, self.sin, ctx.positions, absorb=False)
        else:
            ops.latent_query(q, self.w_ukt, ql, H, s.dim, s.rot_dim, s.kv_rank, self.rot_dims, self.cos, self.sin, ctx.positions)
        ol = ctx.ws.get("latent.ol", (n, H, s.kv_rank), dt)
        ops.latent_attention(ql, cache.k, ctx, ctx.block_tables[cache.group], ol, s.kv_rank, s.scale, s.window)
        att = ctx.ws.get("latent.out", (n, H * s.vdim), dt)
        if many and ops.gemm_heads(ol, self.w_uv, att.view(n, H, s.vdim), gate=parts, gate_off=g_off):
            pass  # the heads' value maps and the output gate in one tensor-core launch
        else:
            ops.heads_product(ol, self.w_uv, att.view(n, H, s.vdim), gate=parts, gate_off=g_off)
        return add_into_stream_or_partials(ops, att, self.w_o, ctx, False, "latent.delta")


register_part("mixer", "latent_attention", LatentAttention)
