"""The latent attention and routed-product kernels alone, tensor-core and CUDA-core forms, against float64 formulas:
geometries with every accumulator width, more heads than a row tile holds, prompt portions beside single tokens,
single tokens whose key range is cut into splits, a window, pages scattered over the pool."""
import numpy as np
import pytest
import torch

from gpu_helpers import DEV, Harness
from llmengine.ops import get_ops

pytestmark = pytest.mark.gpu


def reference_attention(ql, cache, ctx, table, R, scale, window):
    n, page = ctx.n_tokens, cache.shape[2]
    pos, seq = ctx.positions[:n].cpu().tolist(), ctx.token_seq[:n].cpu().tolist()
    table, rows_all, q = table.cpu(), cache.double().cpu(), ql.double().cpu()
    out = torch.zeros(n, ql.shape[1], R, dtype=torch.float64)
    for t in range(n):
        lo = max(0, pos[t] - window + 1) if window else 0
        idx = torch.arange(lo, pos[t] + 1)
        rows = rows_all[table[seq[t]][idx // page].long(), 0, idx % page]
        p = torch.softmax((q[t] @ rows.T) * scale, dim=-1)
        out[t] = p @ rows[:, :R]
    return out


@pytest.mark.parametrize("H,R,dr,page", [(3, 64, 16, 4), (16, 128, 32, 16), (40, 192, 16, 16), (5, 320, 48, 8), (8, 512, 64, 32)])
@pytest.mark.parametrize("window", [0, 45])
def test_latent_attention_tensor_cores_and_cuda_cores(H, R, dr, page, window):
    ops = get_ops()
    h = Harness(torch.bfloat16, page=page, pages=1200 // page + 8, windows=(0,), nkv=1, hd=R + dr)
    g = torch.Generator().manual_seed(H * R + dr)
    h.cache.k.copy_((torch.randn(h.cache.k.shape, generator=g) * 0.7).to(torch.bfloat16))
    scale = 0.9 / (R + dr) ** 0.5 * 4
    steps = [[(1, 3, []), (2, 70, [])],                # first tokens, a portion
             [(1, 600, []), (2, 1, []), (3, 130, [])],  # a long portion beside a single token and a new request
             [(1, 1, []), (2, 1, []), (3, 1, [])],      # single tokens: the long request's keys are cut into splits
             [(3, 2, []), (1, 1, [])]]                  # a portion of two
    for batch in steps:
        ctx = h.ctx(batch)
        n = ctx.n_tokens
        ql = (torch.randn(n, H, R + dr, generator=g)).to(torch.bfloat16).to(DEV)
        want = reference_attention(ql, h.cache.k, ctx, ctx.block_tables[0], R, scale, window)
        for tensor_cores in (True, False):
            ops.latent_tensor_cores = tensor_cores
            try:
                out = torch.zeros(n, H, R, dtype=torch.bfloat16, device=DEV)
                ops.latent_attention(ql, h.cache.k, ctx, ctx.block_tables[0], out, R, scale, window)
            finally:
                ops.latent_tensor_cores = True
            err = (out.double().cpu() - want).abs().max().item()
            assert err < 2.5e-2, f"{'tensor' if tensor_cores else 'CUDA'} cores, step {batch}: {err:.3e}"
    assert ops.latent_attention_kernel(H, R, dr, page) == "tensor cores"


@pytest.mark.parametrize("E,N,K,pairs_per_token,n", [(5, 72, 40, 2, 37), (16, 200, 128, 4, 300), (3, 64, 264, 1, 5), (4, 328, 200, 2, 700)])
def test_routed_products_tensor_cores_against_cuda_cores_and_formula(E, N, K, pairs_per_token, n):
    ops = get_ops()
    from llmengine.engine.context import Workspace
    ws = Workspace(DEV)
    g = torch.Generator().manual_seed(E + N)
    x = torch.randn(n, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(E, N, K, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    idx = torch.stack([torch.randperm(E, generator=g)[:pairs_per_token] for _ in range(n)]).to(torch.int32).to(DEV)
    share = torch.rand(n * pairs_per_token, generator=g).to(DEV)
    full = torch.einsum("tk,enk->ten", x.double().cpu(), w.double().cpu())  # every expert for every token
    picked = torch.stack([full[t, idx[t, j].item()] for t in range(n) for j in range(pairs_per_token)])
    # tiles of the tensor-core kernel (128 rows where an expert gets many, else 64) and of the CUDA-core kernel
    for tile in (ops.routed_tile_rows(n, torch.bfloat16, (K,), n * pairs_per_token / E), ops.routed_tile_rows(n, torch.float32)):
        te, tr = ops.routed_group(idx, E, tile, ws, f"t{tile}")
        seen = sorted(p for p in tr.cpu().reshape(-1).tolist() if p >= 0)
        assert seen == list(range(n * pairs_per_token)), "every pair lies in exactly one tile"
        for e, rows in zip(te.cpu().tolist(), tr.cpu().tolist()):
            assert all(p < 0 or idx.reshape(-1)[p].item() == e for p in rows), "a tile holds rows of one expert"
        act = torch.zeros(n * pairs_per_token, N, dtype=torch.bfloat16, device=DEV)
        ops.routed_product(x, pairs_per_token, w, te, tr, act, "gelu")
        want = 0.5 * picked * (1 + torch.erf(picked / 2 ** 0.5))
        assert (act.double().cpu() - want).abs().max() < 3e-2 * max(1.0, want.abs().max().item())
        y = torch.zeros(n * pairs_per_token, N, dtype=torch.float32, device=DEV)
        ops.routed_product(x.repeat_interleave(pairs_per_token, 0).contiguous(), 1, w, te, tr, y, "share", share=share)
        want = picked * share.double().cpu()[:, None]
        assert (y.double().cpu() - want).abs().max() < 1e-3 * max(1.0, want.abs().max().item())
