"""Plain, slow Lotirax decoder: whole sequences, no cache, one function per mechanism, all float64.

The oracle of the Lotirax tests.  It shares no code with the product package: its own reading of the
configuration (a dict as config.json holds it) and its own arithmetic.  A sequence is run whole.

Notation: h is a part's input [T, width]; W[name] a weight [out, in] applied as h @ W^T; positions count
from 0; `unit(x)` is x over its root mean square (eps under the root).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight lies around zero: unit(x) * (1 + w)."""
    return unit(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def rotary_frequencies(rot):
    """Per pair i < dims/2: base^(-2i/dims), stretched by the YaRN rule when rot has 'scaling'; and the
    factor both cosine and sine are multiplied by."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn(t):            # the (fractional) pair index whose wave makes t turns over the original length
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_half(x, pos, rot):
    """x [T, ..., n]: entry i < dims/2 is paired with entry i + dims/2; entries from dims on pass."""
    if not rot:
        return x
    dims = int(rot["dims"])
    freq, mag = rotary_frequencies(rot)
    out = x.clone()
    half = dims // 2
    for i in range(half):
        ang = pos.to(F64) * freq[i]
        shape = [-1] + [1] * (x.dim() - 2)
        c, s = (torch.cos(ang) * mag).reshape(shape), (torch.sin(ang) * mag).reshape(shape)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def softmax_window(q, k, v, scale, window):
    """One attention map: q [T, n], k [T, n], v [T, m]; token i sees j with 0 <= i - j < window (all j <= i
    when window is 0)."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1) if window else 0
        p = torch.softmax((k[lo: i + 1] @ q[i]) * scale, dim=0)
        out[i] = p @ v[lo: i + 1]
    return out


def differential_attention(h, W, m, eps):
    """Two softmax maps per head over the same values, o = a1 - lam * a2, unit-normed per head and scaled by
    (1 - diff).  W holds the mixer's tensors by their short names ('q', 'q.b', 'q.norm', 'lq1', ...)."""
    T = h.shape[0]
    H, G, n, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    window = int((m.get("mask") or {}).get("size", 0))
    pos = torch.arange(T)
    q = (h @ W["q"].T + W["q.b"]).reshape(T, H, 2, n)
    k = (h @ W["k"].T + W["k.b"]).reshape(T, G, 2, n)
    v = (h @ W["v"].T + W["v.b"]).reshape(T, G, dv)
    q = rotate_half(unit(q, eps) * W["q.norm"], pos, m.get("rot"))
    k = rotate_half(unit(k, eps) * W["k.norm"], pos, m.get("rot"))
    lam = math.exp(float((W["lq1"] * W["lk1"]).sum())) - math.exp(float((W["lq2"] * W["lk2"]).sum())) + diff
    heads = []
    for a in range(H):
        g = a // (H // G)
        a1 = softmax_window(q[:, a, 0], k[:, g, 0], v[:, g], float(m["scale"]), window)
        a2 = softmax_window(q[:, a, 1], k[:, g, 1], v[:, g], float(m["scale"]), window)
        heads.append(unit(a1 - lam * a2, eps) * (1.0 - diff))
    return torch.cat(heads, dim=1) @ W["o"].T


def dense_feed_forward(h, W):
    return (silu(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def small_expert(h, up, down):
    return relu_squared(h @ up.T) @ down.T


def table_experts(h, tokens, W, f):
    """Each token's experts are listed in a table row chosen by its token id; equal weights."""
    top = int(f["router"]["top"])
    out = torch.zeros_like(h)
    for t, tok in enumerate(tokens):
        for e in W["table"][tok].tolist():
            out[t] += small_expert(h[t: t + 1], W[f"e{int(e)}.up"], W[f"e{int(e)}.down"])[0] / top
    if f.get("shared"):
        out = out + small_expert(h, W["shared.up"], W["shared.down"])
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(x, tokens, i, cfg, weights):
    """x + m * (ls1 * mixer(h) + ls2 * feed_forward(h)) with the one normed input h."""
    L, eps = cfg["layers"][i], float(cfg["norm"]["eps"])
    p = f"l{i}."
    h = norm_one_plus(x, weights[p + "norm1"], eps)
    if L["type"] != "attention":
        raise ValueError(f"unknown mixer {L['type']!r}")
    y = differential_attention(h, sub(weights, p + "mix."), L["mixer"], eps) * weights[p + "ls1"]
    f = L.get("mlp")
    if f is not None:
        W = sub(weights, p + "mlp.")
        z = dense_feed_forward(h, W) if f["kind"] == "dense" else table_experts(h, tokens, W, f)
        y = y + z * weights[p + "ls2"]
    return x + float(cfg.get("residual_mult", 1.0)) * y


def run_order(cfg):
    """(layer, pass or None, first of its pass) in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    out = [(i, None, False) for i in range(a)]
    for t in range(times):
        out += [(i, t, i == a) for i in range(a, b)]
    return out + [(i, None, False) for i in range(b, n)]


def forward(cfg, weights, tokens, streams=None):
    """Logits [T, vocab] of a whole sequence.  weights: name -> float64 tensor (integer tables as they are).
    streams: a list that receives the residual stream after every layer run."""
    x0 = weights["embed"][torch.tensor(tokens)]
    x = x0
    for i, t, first in run_order(cfg):
        if first:
            x = torch.cat([x, x0], dim=1) @ weights["loop.in"].T + weights["loop.step"][t]
        x = layer(x, tokens, i, cfg, weights)
        if streams is not None:
            streams.append(x)
    return norm_one_plus(x, weights["final.norm"], float(cfg["norm"]["eps"])) @ weights["embed"].T
