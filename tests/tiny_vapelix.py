"""Tiny Vapelix configurations for the tests. They differ from one another in every size and option, and
no two sizes that could be mixed up are equal within one of them (query latent != key/value latent,
unrotated != rotated != value size, loop not starting at layer 0, one expert chosen, a layer without a
feed-forward, rotation with and without a frequency ramp)."""
from __future__ import annotations


def _mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling=None, dims=None):
    rot = {"dims": rot_dim if dims is None else dims, "base": base}
    if scaling:
        rot["scaling"] = scaling
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "rot": rot}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


RAMP_A = {"factor": 8.0, "original": 48, "fast": 16.0, "slow": 2.0}
MIX_A = _mixer(3, 16, 8, 24, 40, 24, 0.21, 10000.0, RAMP_A)
# A: 4 layers (dense, routed 2 of 5, no feed-forward, routed 1 of 3); layers 1..2 run three times; token input of 6;
#    width 72; vocab 301; pages of 4.
VAPELIX_A = {"architecture": "Vapelix", "vocab": 301, "width": 72, "norm": {"eps": 1e-5}, "max_positions": 512,
             "layers": [{"type": "latent_attention", "mixer": MIX_A, "mlp": {"kind": "dense", "ff": 100}},
                        {"type": "latent_attention", "mixer": MIX_A, "mlp": _moe(36, 5, 2)},
                        {"type": "latent_attention", "mixer": MIX_A, "mlp": None},
                        {"type": "latent_attention", "mixer": MIX_A, "mlp": _moe(20, 3, 1)}],
             "loop": {"start": 1, "stop": 3, "times": 3}, "token_side": {"dim": 6}}
# B: 2 layers with different mixers, no loop, no token input, no frequency ramp, rotation over a part of the
#    rotated numbers in the second; width 96; vocab 257; pages of 16.
VAPELIX_B = {"architecture": "Vapelix", "vocab": 257, "width": 96, "norm": {"eps": 1e-6}, "max_positions": 600,
             "layers": [{"type": "latent_attention", "mixer": _mixer(2, 8, 16, 12, 64, 32, 0.3, 50000.0), "mlp": _moe(48, 6, 3)},
                        {"type": "latent_attention", "mixer": _mixer(5, 24, 12, 8, 36, 20, 0.15, 1000.0, dims=8),
                         "mlp": {"kind": "dense", "ff": 128}}]}
# C: sizes the tensor-core kernels take (latents and head sizes multiples of 16, feed-forward multiples of 128):
#    3 layers, the first runs twice; width 128; vocab 512; pages of 16.
MIX_C = _mixer(4, 32, 16, 48, 64, 96, 0.18, 250000.0, {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0})
VAPELIX_C = {"architecture": "Vapelix", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "max_positions": 1024,
             "layers": [{"type": "latent_attention", "mixer": MIX_C, "mlp": {"kind": "dense", "ff": 256}},
                        {"type": "latent_attention", "mixer": MIX_C, "mlp": _moe(128, 8, 2)},
                        {"type": "latent_attention", "mixer": MIX_C, "mlp": _moe(64, 4, 4)}],
             "loop": {"start": 0, "stop": 1, "times": 2}, "token_side": {"dim": 16}}

VAPELIX = {"va": (VAPELIX_A, 4), "vb": (VAPELIX_B, 16), "vc": (VAPELIX_C, 16)}  # name -> (config.json, page size)
