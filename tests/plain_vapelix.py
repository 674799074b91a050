"""A plain, slow implementation of the Vapelix decoder, one function per mechanism, in float64 (or any
torch dtype) on the CPU. It shares no code with the package: it reads config.json and the tensors by
name and loops over tokens, heads and experts. The engine's tests compare against it.

Notation: T tokens, D width, H heads, dn / dr unrotated / rotated query-key sizes of a head, dv value
size of a head, R latent size of keys and values, Rq latent size of queries.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# ---------------------------------------------------------------------------- files
def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        base = 8 + n
        out = {}
        for name, info in head.items():
            if name == "__metadata__":
                continue
            lo, hi = info["data_offsets"]
            f.seek(base + lo)
            raw = f.read(hi - lo)
            dt = info["dtype"]
            if dt == "BF16":
                a = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
                t = torch.from_numpy(a.view(np.float32).copy())
            elif dt == "F32":
                t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
            elif dt == "I32":
                t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
            else:
                raise ValueError(f"{name}: dtype {dt}")
            out[name] = t.reshape(info["shape"])
    return out


def read_model(model_dir, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}


# ---------------------------------------------------------------------------- small pieces
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotary_frequencies(rot):
    """-> (frequency of each pair [dims/2], factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, pos, rot):
    """x [..., dims] at position pos: pair (i, i + dims/2) turned by pos * f_i; dims beyond rot.dims pass."""
    dims = int(rot["dims"])
    half = dims // 2
    f, m = rotary_frequencies(rot)
    ang = torch.tensor([pos * fi for fi in f], dtype=torch.float64)
    c, s = (torch.cos(ang) * m).to(x.dtype), (torch.sin(ang) * m).to(x.dtype)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------- mixer
def latent_attention(w, p, m, eps, h, pos0, past):
    """h [T, D]: the mixer's input for positions pos0 .. pos0+T-1. past: {"c": [S, R], "kr": [S, dr]} of the
    earlier positions (or None). -> (output [T, D], the cache with the new positions appended)."""
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, dn + dr)
    kv = h @ w[p + "dkv"].T
    c = rms_norm(kv[:, :R], w[p + "dkv.norm"], eps)
    kr = torch.stack([rotate(kv[t, R:], pos0 + t, m["rot"]) for t in range(T)])
    if past is not None:
        c, kr = torch.cat([past["c"], c]), torch.cat([past["kr"], kr])
    kn = (c @ w[p + "uk"].T).view(-1, H, dn)
    val = (c @ w[p + "uv"].T).view(-1, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        pos = pos0 + t
        for a in range(H):
            qr = rotate(q[t, a, dn:], pos, m["rot"])
            s = (kn[:pos + 1, a] @ q[t, a, :dn] + kr[:pos + 1] @ qr) * m["scale"]
            out[t, a] = torch.softmax(s, dim=0) @ val[:pos + 1, a]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T, {"c": c, "kr": kr}


# ---------------------------------------------------------------------------- feed-forward
def dense_ff(w, p, h):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(w, p, f, h):
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.argsort(z[t], descending=True, stable=True)[:top]
        share = torch.softmax(z[t, chosen], dim=0)
        for e, g in zip(chosen.tolist(), share):
            out[t] += g * (gelu_erf(h[t] @ w[p + f"e{e}.up"].T) @ w[p + f"e{e}.down"].T)
    return out


def token_side(w, cfg, i, tokens, x):
    """The per-layer token input of layer i: -> what is added to x."""
    d = cfg["token_side"]["dim"]
    e = w["side.embed"][torch.tensor(tokens)][:, i * d:(i + 1) * d]
    y = (gelu_tanh(x @ w[f"l{i}.side.gate"].T) * e) @ w[f"l{i}.side.proj"].T
    return rms_norm(y, w[f"l{i}.side.norm"], cfg["norm"]["eps"])


# ---------------------------------------------------------------------------- model
def run_order(cfg):
    """-> [(layer index, first of a repeated pass?)] in execution order."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(L)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for k in range(times):
        order += [(i, k > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, L)]


def forward(cfg, w, tokens, pos0=0, cache=None, layer_outputs=None):
    """tokens at positions pos0.. of one sequence -> (logits [T, V], cache). cache: one entry per layer run."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.tensor(tokens)]
    x = x0.clone()
    order = run_order(cfg)
    cache = cache if cache is not None else [None] * len(order)
    for r, (i, again) in enumerate(order):
        if again:
            x = x + x0
        layer = cfg["layers"][i]
        assert layer["type"] == "latent_attention"
        mix, cache[r] = latent_attention(w, f"l{i}.mix.", layer["mixer"], eps, rms_norm(x, w[f"l{i}.norm1"], eps), pos0, cache[r])
        f = layer.get("mlp")
        if f:
            h2 = rms_norm(x, w[f"l{i}.norm2"], eps)
            mix = mix + (dense_ff(w, f"l{i}.mlp.", h2) if f["kind"] == "dense" else routed_ff(w, f"l{i}.mlp.", f, h2))
        x = x + mix
        if cfg.get("token_side"):
            x = x + token_side(w, cfg, i, tokens, x)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T, cache


def generate(cfg, w, prompt, n_new):
    logits, cache = forward(cfg, w, prompt)
    out = list(prompt)
    for _ in range(n_new):
        nxt = int(torch.argmax(logits[-1]))
        out.append(nxt)
        logits, cache = forward(cfg, w, [nxt], len(out) - 1, cache)
    return out
