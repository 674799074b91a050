"""Tiny Zulopel configurations and their weights for the tests. The configurations differ from one another in every
size and option, and no two sizes that could be mixed up are equal within one of them (query heads != key/value heads,
key size != value size, rotated part != key size, state != taps != step-size rank, groups kept != groups, one layer
without a feed-forward, one feed-forward without a shared expert, one without groups).

The weights are made here by rules of the test's own (not the package's random-weights mode), so that every tensor
matters: sinks and corrections away from zero, step sizes between a thousandth and a tenth, decays from fast to very
slow (a state that is lost or reset shows hundreds of tokens later), a value-mixing weight well inside (0, 1).
`sharp=True` scales the query norm's weight so that the softmax of most heads rests on one or two keys, wherever they
are: a key that is lost, shifted, read from a wrong page or let through a chunk's edge moves the logits."""
from __future__ import annotations

import json
import math
import os

import torch


def _att(heads, kv_heads, dim, vdim, scale, dims, base, chunk=None, v_mix=False, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = scaling
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot, "v_mix": v_mix}
    if chunk:
        m["mask"] = {"size": chunk}
    return m


def _scan(inner, state, conv, dt_rank):
    return {"inner": inner, "state": state, "conv": conv, "dt_rank": dt_rank}


def _moe(ff, experts, top, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    f = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        f["shared"] = {"ff": shared}
    return f


RAMP_A = {"factor": 8.0, "original": 48, "fast": 16.0, "slow": 2.0}
# A: scan, attention (first of the value mixers), attention (mixes), scan without a feed-forward, attention that does not
#    mix; chunks of 20 and 12 and none; 6 / 4 / 3 query heads on 2 / 2 / 3 key-value heads; pages of 4; nothing a multiple of 8
ZULOPEL_A = {"architecture": "Zulopel", "vocab": 301, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5}, "max_positions": 512,
             "layers": [{"type": "mamba1", "mixer": _scan(40, 5, 3, 7), "mlp": _moe(36, 6, 2, (3, 2), 20)},
                        {"type": "attention", "mixer": _att(6, 2, 24, 10, 0.21, 10, 10000.0, 20, True, RAMP_A), "mlp": _moe(20, 5, 1)},
                        {"type": "attention", "mixer": _att(4, 2, 12, 10, 0.3, 12, 777.0, 12, True), "mlp": _moe(28, 4, 4, (2, 2), 44)},
                        {"type": "mamba1", "mixer": _scan(52, 9, 2, 3), "mlp": None},
                        {"type": "attention", "mixer": _att(3, 3, 14, 18, 0.25, 6, 50000.0), "mlp": _moe(12, 9, 3, (3, 1))}]}
# B: sizes the tensor-core products take (multiples of 16, feed-forwards multiples of 128 or 64); attention first; one mixer of
#    values only (its mixing weight is never used); as many query as key/value heads; taps 5; pages of 16
ZULOPEL_B = {"architecture": "Zulopel", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "max_positions": 1024,
             "layers": [{"type": "attention", "mixer": _att(4, 4, 32, 64, 0.18, 32, 250000.0, 48, True), "mlp": _moe(128, 8, 2, None, 256)},
                        {"type": "mamba1", "mixer": _scan(256, 16, 5, 8), "mlp": _moe(64, 4, 2, (4, 2), 128)},
                        {"type": "mamba1", "mixer": _scan(128, 32, 4, 16), "mlp": _moe(64, 16, 4, (4, 3))}]}
# C: one key/value head for five query heads, a chunk of one page, a single tap, one expert chosen of one kept group; pages of 8
ZULOPEL_C = {"architecture": "Zulopel", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 6.9}, "max_positions": 400,
             "layers": [{"type": "mamba1", "mixer": _scan(24, 3, 1, 2), "mlp": _moe(16, 6, 1, (2, 1), 8)},
                        {"type": "attention", "mixer": _att(5, 1, 16, 6, 0.4, 16, 300.0, 8, False, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}),
                         "mlp": _moe(24, 3, 2)}]}

ZULOPEL = {"za": (ZULOPEL_A, 4), "zb": (ZULOPEL_B, 16), "zc": (ZULOPEL_C, 8)}  # name -> (config.json, page size)


def make_tensors(cfg, seed, dtype, sharp=False):
    """name -> tensor, as a checkpoint stores them (matrices in `dtype`; the same for vectors: the reader widens)."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    t = {}

    def lin(name, out, inp, gain=1.0):
        t[name] = torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def near_one(name, n):
        t[name] = 1.0 + 0.2 * torch.randn(n, generator=g)

    t["embed"] = torch.randn(V, D, generator=g) * 0.5
    lin("head", V, D)
    near_one("final.norm", D)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        near_one(p + "norm1", D)
        near_one(p + "ls1", D)
        if l["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            lin(p + "mix.q", H * dk, D); lin(p + "mix.k", G * dk, D); lin(p + "mix.v", G * dv, D); lin(p + "mix.g", H * dv, D)
            lin(p + "mix.o", D, H * dv)
            near_one(p + "mix.q.norm", dk); near_one(p + "mix.k.norm", dk)
            if sharp:
                t[p + "mix.q.norm"] *= 6.0 / (m["scale"] * math.sqrt(dk))  # scores with a spread of about 6
            t[p + "mix.sink"] = torch.randn(H, generator=g) + 1.0
            if m.get("v_mix"):
                t[p + "mix.vmix"] = torch.tensor(0.3 + 0.05 * i)
        else:
            C, N, K, R = m["inner"], m["state"], m["conv"], m["dt_rank"]
            lin(p + "mix.in", 2 * C, D)
            t[p + "mix.conv"] = torch.randn(C, K, generator=g) * 0.5
            t[p + "mix.conv.b"] = torch.randn(C, generator=g) * 0.1
            lin(p + "mix.x", R + 2 * N, C); lin(p + "mix.dt", C, R)
            step = torch.exp(torch.rand(C, generator=g) * math.log(100.0) + math.log(1e-3))  # 0.001 .. 0.1
            t[p + "mix.dt.b"] = torch.log(torch.expm1(step))
            t[p + "mix.A_log"] = torch.log(torch.exp(torch.rand(C, N, generator=g) * math.log(800.0) + math.log(0.01)))  # A 0.01 .. 8
            near_one(p + "mix.D", C)
            lin(p + "mix.o", D, C)
        f = l.get("mlp")
        if f:
            near_one(p + "norm2", D)
            near_one(p + "ls2", D)
            E = f["router"]["experts"]
            lin(p + "mlp.router", E, D, gain=2.0)
            t[p + "mlp.correction"] = torch.randn(E, generator=g) * (0.5 / E)
            for k in range(E):
                lin(f"{p}mlp.e{k}.gate", f["expert"]["ff"], D); lin(f"{p}mlp.e{k}.up", f["expert"]["ff"], D)
                lin(f"{p}mlp.e{k}.down", D, f["expert"]["ff"])
            if f.get("shared"):
                s = f["shared"]["ff"]
                lin(p + "mlp.shared.gate", s, D); lin(p + "mlp.shared.up", s, D); lin(p + "mlp.shared.down", D, s)
    return {k: v.to(dtype).contiguous() for k, v in t.items()}


def write_model(path, cfg, dtype, seed=11, sharp=False):
    from llmengine.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), make_tensors(cfg, seed, dtype, sharp))
    return path
