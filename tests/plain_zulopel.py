"""A plain, slow implementation of the Zulopel decoder, one function per mechanism, in float64 (or any
torch dtype) on the CPU. It shares no code with the package: it reads config.json and the tensors by
name and loops over tokens, heads, channels and experts. The engine's tests compare against it.

Notation: T tokens, D width, H query heads, G key/value heads, dk query/key size of a head, dv value size of a
head, C channels of a recurrent mixer, N its state size, K its convolution taps, E experts.

A layer:  x += ls1 * rmsnorm1(mixer(x));  x += ls2 * rmsnorm2(ff(x))   (the sublayers read x itself).
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
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotary_frequencies(rot):
    """-> (frequency of each pair [dims/2], factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(vec, pos, rot):
    """vec [..., d] of one token at position pos: the first rot.dims numbers are turned in pairs (i, i + dims/2)."""
    dims = int(rot["dims"])
    if dims == 0:
        return vec
    f, m = rotary_frequencies(rot)
    half = dims // 2
    out = vec.clone()
    for i in range(half):
        a = pos * f[i]
        c, s = math.cos(a) * m, math.sin(a) * m
        u, v = vec[..., i], vec[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


# ---------------------------------------------------------------------------- attention mixer
def attention_mixer(h, w, p, m, eps, start, state, shared):
    """h [T, D]: the tokens at positions start .. start + T - 1 of one sequence. state: {"k": [..], "v": [..]} rows of
    all earlier positions (extended here). shared: a dict that lives for one pass over the layers; the first layer
    with value mixing leaves its values there."""
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, G, dk)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    for t in range(T):
        q[t] = rotate(q[t], start + t, m["rot"])
        k[t] = rotate(k[t], start + t, m["rot"])
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v.clone()
        else:
            lam = w[p + "vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
    state.setdefault("k", []).extend(k[t] for t in range(T))
    state.setdefault("v", []).extend(v[t] for t in range(T))
    chunk = int(m["mask"]["size"]) if m.get("mask") else 0
    scale = float(m["scale"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        i = start + t
        lo = (i // chunk) * chunk if chunk > 0 else 0
        keys, vals = torch.stack(state["k"][lo:i + 1]), torch.stack(state["v"][lo:i + 1])  # [n, G, dk], [n, G, dv]
        for a in range(H):
            g = a // (H // G)
            s = (keys[:, g] @ q[t, a]) * scale
            sink = w[p + "sink"][a]
            top = torch.maximum(s.max(), sink)
            e = torch.exp(s - top)
            denom = e.sum() + torch.exp(sink - top)  # the sink: one more term below the line, nothing above it
            out[t, a] = (e / denom) @ vals[:, g]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


# ---------------------------------------------------------------------------- recurrent mixer
def mamba_mixer(h, w, p, m, state):
    """Selective scan. state: {"conv": [K - 1, C] the last inputs of the convolution, "ssm": [C, N]} (made here at zero)."""
    T = h.shape[0]
    C, N, K, R = int(m["inner"]), int(m["state"]), int(m["conv"]), int(m["dt_rank"])
    xz = h @ w[p + "in"].T
    x, z = xz[:, :C], xz[:, C:]
    if "conv" not in state:
        state["conv"] = torch.zeros(K - 1, C, dtype=h.dtype)
        state["ssm"] = torch.zeros(C, N, dtype=h.dtype)
    padded = torch.cat([state["conv"], x], dim=0)  # row t .. t + K - 1 are the taps of token t, the last one its own
    state["conv"] = padded[padded.shape[0] - (K - 1):].clone()
    xc = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        acc = w[p + "conv.b"].clone()
        for j in range(K):
            acc = acc + w[p + "conv"][:, j] * padded[t + j]
        xc[t] = silu(acc)
    proj = xc @ w[p + "x"].T
    dt = softplus(proj[:, :R] @ w[p + "dt"].T + w[p + "dt.b"])
    B, Cm = proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    A = -torch.exp(w[p + "A_log"])
    S = state["ssm"]
    y = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * xc[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + w[p + "D"] * xc[t]
    state["ssm"] = S
    return (y * silu(z)) @ w[p + "o"].T


# ---------------------------------------------------------------------------- feed-forward
def gated_expert(x, w, p):
    return (silu(x @ w[p + "gate"].T) * (x @ w[p + "up"].T)) @ w[p + "down"].T


def route(z, correction, top, groups, keep):
    """z [E] router logits of one token -> (chosen experts, their weights)."""
    E = z.shape[0]
    s = torch.softmax(z, dim=0)
    choice = s + correction
    per = E // groups
    best = torch.stack([choice[g * per:(g + 1) * per].max() for g in range(groups)])
    order = sorted(range(groups), key=lambda g: (-float(best[g]), g))
    allowed = set(order[:keep])
    cand = [e for e in range(E) if e // per in allowed]
    cand.sort(key=lambda e: (-float(choice[e]), e))
    chosen = cand[:top]
    wts = torch.stack([s[e] for e in chosen])
    return chosen, wts / (wts.sum() + 1e-20)


def moe(h, w, p, f):
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    g = r.get("groups") or {"count": 1, "keep": 1}
    out = torch.zeros_like(h)
    zs = h @ w[p + "router"].T
    corr = w[p + "correction"] if p + "correction" in w else torch.zeros(E, dtype=h.dtype)
    for t in range(h.shape[0]):
        chosen, wts = route(zs[t], corr, top, int(g["count"]), int(g["keep"]))
        for e, a in zip(chosen, wts):
            out[t] += a * gated_expert(h[t], w, f"{p}e{e}.")
    if f.get("shared"):
        out = out + gated_expert(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------------------- the model
class PlainZulopel:
    """forward(tokens, state) runs the next tokens of ONE sequence; `state` (a dict, empty at first) carries the
    keys, values and recurrent states, so a prompt may be fed whole, in portions or token by token."""

    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, weights

    def forward(self, tokens, state, layers_out=None):
        cfg, w = self.cfg, self.w
        eps = float(cfg["norm"]["eps"])
        start = state.get("len", 0)
        x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
        shared = {}
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            st = state.setdefault(i, {})
            if layer["type"] == "attention":
                a = attention_mixer(x, w, p + "mix.", layer["mixer"], eps, start, st, shared)
            elif layer["type"] == "mamba1":
                a = mamba_mixer(x, w, p + "mix.", layer["mixer"], st)
            else:
                raise ValueError(layer["type"])
            x = x + rms_norm(a, w[p + "norm1"], eps) * w[p + "ls1"]
            if layer.get("mlp"):
                b = moe(x, w, p + "mlp.", layer["mlp"])
                x = x + rms_norm(b, w[p + "norm2"], eps) * w[p + "ls2"]
            if layers_out is not None:
                layers_out.append(x.clone())
        state["len"] = start + len(tokens)
        return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def forward(cfg, w, tokens):
    """Logits [T, vocab] of one whole sequence."""
    return PlainZulopel(cfg, w).forward(tokens, {})


def generate(cfg, w, prompt, n_new):
    """Greedy: the first index of the largest logit, token by token through the carried state."""
    m, state = PlainZulopel(cfg, w), {}
    out = list(prompt)
    logits = m.forward(out, state)
    for _ in range(n_new):
        out.append(int(torch.argmax(logits[-1])))
        logits = m.forward(out[-1:], state)
    return out
