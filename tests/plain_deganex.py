"""Plain, slow Deganex decoder: whole sequences, no cache, one function per mechanism.

The oracle of the Deganex tests.  It shares no code with the product package: its own
reading of config.json, its own safetensors reader (plain_llama's) and its own arithmetic,
all float64.  A sequence is run whole, token by token where the mechanism is a recurrence.

Notation: h is a mixer's or feed-forward's input [T, width]; W[name] a weight [out, in]
applied as h @ W^T; positions count from 0.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x over its root mean square along the last axis (eps under the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def embed_bigram(tokens, embed, bigram, buckets, mul_prev, mul_cur):
    """Token row plus the row of a hashed (previous, current) pair; the first token of a
    sequence takes the table's last row."""
    out = []
    for t, tok in enumerate(tokens):
        row = buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets
        out.append(embed[tok] + bigram[row])
    return torch.stack(out)


def rotate_pairs(x, pos, dims, base):
    """Rotary encoding on the first `dims` entries of the last axis, entry 2i paired with 2i+1:
    (a, b) -> (a cos - b sin, b cos + a sin), angle pos * base^(-2i/dims).  x: [T, ..., n]."""
    out = x.clone()
    for i in range(dims // 2):
        ang = pos.to(F64) * (float(base) ** (-2.0 * i / dims))
        shape = [-1] + [1] * (x.dim() - 2)
        c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def latent_attention(h, W, m, eps, window=0):
    """Attention whose keys and values are expanded from a shared low-rank latent; one rotated
    key part is shared by all heads.  Causal, softmax over all visible keys, sigmoid output gate."""
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ W["q"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], pos, m["rot"]["dims"], m["rot"]["base"])
    down = h @ W["dkv"].T
    latent = rms_norm(down[:, :rank], W["dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, rank:].reshape(T, 1, dr), pos, m["rot"]["dims"], m["rot"]["base"])[:, 0]
    k_plain = (latent @ W["uk"].T).reshape(T, H, dn)
    val = (latent @ W["uv"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hd in range(H):
            lo = max(0, t - window + 1) if window else 0           # a window keeps the last `window` keys (the model itself has none)
            s = (k_plain[lo: t + 1, hd] @ q_plain[t, hd] + k_rot[lo: t + 1] @ q_rot[t, hd]) * m["scale"]
            p = torch.softmax(s, dim=0)
            out[t, hd] = p @ val[lo: t + 1, hd]
    gated = out.reshape(T, H * dv) * torch.sigmoid(h @ W["g"].T)
    return gated @ W["o"].T


def mlstm(h, W, m, eps):
    """Matrix-memory recurrence with exponential gates stabilised by a running maximum that starts at 0."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ W["q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ W["k"].T).reshape(T, H, dk)
    v = (h @ W["v"].T).reshape(T, H, dv)
    log_i = cap * torch.tanh((h @ W["i"].T + W["i.b"]) / cap)                       # [T, H]
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W["f"].T + W["f.b"]) / cap))
    S = torch.zeros(H, dk, dv, dtype=F64)
    n = torch.zeros(H, dk, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        new_mx = torch.maximum(log_f[t] + mx, log_i[t])
        keep = torch.exp(log_f[t] + mx - new_mx)
        take = torch.exp(log_i[t] - new_mx)
        S = keep[:, None, None] * S + take[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new_mx
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    y = rms_unit(out, eps).reshape(T, H * dv) * W["norm"] * torch.sigmoid(h @ W["g"].T)
    return y @ W["o"].T


def mamba2(h, W, m, eps):
    """Selective state space with a scalar decay per head; short causal convolution ahead of it,
    gate before a grouped norm behind it."""
    T = h.shape[0]
    H, P, N, G, taps, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner = H * P
    proj = h @ W["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=F64), xbc])
    conv = torch.stack([(padded[t: t + taps] * W["conv"].T).sum(0) for t in range(T)]) + W["conv.b"]
    conv = silu(conv)
    x = conv[:, :inner].reshape(T, H, P)
    B = conv[:, inner: inner + G * N].reshape(T, G, N)
    C = conv[:, inner + G * N:].reshape(T, G, N)
    step = torch.nn.functional.softplus(dt + W["dt_bias"])                          # [T, H]
    rate = torch.exp(W["A_log"])
    S = torch.zeros(H, N, P, dtype=F64)
    y = torch.zeros(T, H, P, dtype=F64)
    per = H // G
    for t in range(T):
        for hd in range(H):
            g = hd // per
            S[hd] = torch.exp(-rate[hd] * step[t, hd]) * S[hd] + step[t, hd] * B[t, g][:, None] * x[t, hd][None, :]
            y[t, hd] = S[hd].T @ C[t, g] + W["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def moe(h, W, f):
    """Top-k routed experts, weights = softmax over the chosen logits; plus a shared expert scaled
    by a sigmoid of one number per token."""
    E, top = f["router"]["experts"], f["router"]["top"]
    logits = h @ W["router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(logits[t], top).indices
        w = torch.softmax(logits[t, chosen], dim=0)
        for j, e in enumerate(chosen.tolist()):
            out[t] += w[j] * gated_ff(h[t: t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    if f.get("shared"):
        shared = gated_ff(h, W["shared.gate"], W["shared.up"], W["shared.down"])
        out = out + torch.sigmoid(h @ W["shared.sg"].T) * shared
    return out


MIXERS = {"latent_attention": latent_attention, "mlstm": mlstm, "mamba2": mamba2}


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def owner(layers, i):
    while layers[i].get("weights_of") is not None:
        i = layers[i]["weights_of"]
    return i


def forward(cfg, weights, tokens, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = embed_bigram(list(tokens), w["embed"], w["bigram"], bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    else:
        x = w["embed"][list(tokens)]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner(cfg['layers'], i)}."
        delta = MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), sub(w, p + "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            delta = delta + moe(rms_norm(x, w[p + "norm2"], eps), sub(w, p + "mlp."), layer["mlp"])
        x = x + delta
        streams.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if keep_layers else logits


def greedy(cfg, weights, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(cfg, weights, seq)[-1].argmax()))
    return seq[len(prompt):]


def read_model_dir(model_dir):
    from plain_llama import read_safetensors
    d = Path(model_dir)
    return json.loads((d / "config.json").read_text()), read_safetensors(d / "model.safetensors")
