"""Small Lotirax configurations with weights drawn for the tests: matrices scaled so that activations are of order
one and attention is peaked (scale = sharp / sqrt(dim) on unit-normed maps), which is what makes a lost key, a window
that is one token off or another request's page show in the logits.  Sizes differ from layer to layer on purpose:
grouped and ungrouped heads, value sizes that are not twice the map size, rotations over part of a map, with and
without stretching, with and without a window, feed-forwards of every kind and none."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch

from qorvix_b200.weights import write_safetensors


def attn(heads=4, kv_heads=2, dim=24, vdim=40, sharp=3.0, diff=0.25, window=23, rot_dims=16, base=3000.0, scaling="yes"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": sharp / dim ** 0.5, "diff": diff}
    if window:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling == "yes":
            m["rot"]["scaling"] = {"factor": 3.0, "original": 48, "fast": 6.0, "slow": 1.5}
        elif scaling:
            m["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": m}


def dense(ff=88):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=3, ff=24, shared=40):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(layers, vocab=211, width=72, eps=2e-5, mult=0.5, loop=None):
    cfg = {"architecture": "Lotirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# A: grouped heads, partial stretched rotation, every kind of feed-forward, the two middle layers run twice
CONFIG_A = config([layer(attn(), dense()), layer(attn(heads=3, kv_heads=3, dim=20, vdim=12, window=9, rot_dims=20, scaling=None), moe()),
                   layer(attn(heads=2, kv_heads=1, dim=16, vdim=56, window=40, rot_dims=4), None),
                   layer(attn(heads=6, kv_heads=2, dim=8, vdim=8, window=0, rot_dims=8, diff=0.6), moe(experts=3, top=1, ff=16, shared=0))],
                  loop=(1, 3, 2))
# B: no stretch of layers runs again, multiplier one, a layer without rotation, one head, many experts of which all but a few idle
CONFIG_B = config([layer(attn(heads=1, kv_heads=1, dim=36, vdim=24, window=17, rot_dims=0), moe(experts=37, top=2, ff=8, shared=24)),
                   layer(attn(heads=5, kv_heads=5, dim=12, vdim=28, window=64, rot_dims=12,
                              scaling={"factor": 8.0, "original": 16, "fast": 4.0, "slow": 0.5}), dense(ff=50)),
                   layer(attn(heads=2, kv_heads=2, dim=12, vdim=28, window=0, rot_dims=6, scaling=None), moe(experts=4, top=4, ff=40, shared=8))],
                  vocab=150, width=48, eps=1e-6, mult=1.0)
# C: the whole model runs three times from its first layer on; sizes in multiples of 16 and 32
CONFIG_C = config([layer(attn(heads=4, kv_heads=2, dim=32, vdim=64, window=33, rot_dims=32), moe(experts=6, top=2, ff=32, shared=16)),
                   layer(attn(heads=4, kv_heads=4, dim=16, vdim=32, window=48, rot_dims=16), dense(ff=96))],
                  vocab=190, width=64, eps=4e-6, mult=0.35, loop=(0, 2, 3))
# D: sizes that are multiples of neither 8 nor 16 anywhere (width, maps, values, feed-forwards, vocabulary), three query
# heads on one key/value head, a stretch of one layer that runs once
CONFIG_D = config([layer(attn(heads=3, kv_heads=1, dim=10, vdim=14, window=11, rot_dims=6), dense(ff=30)),
                   layer(attn(heads=2, kv_heads=2, dim=6, vdim=22, window=29, rot_dims=2, scaling=None), moe(experts=7, top=2, ff=12, shared=10))],
                  vocab=97, width=44, eps=3e-5, mult=0.7, loop=(1, 2, 1))


def _rnd(g, *shape):
    return torch.randn(*shape, generator=g)


def mixer_weights(m, width, g):
    """Weights of one differential-attention mixer by their short names, float32 values that bfloat16 holds exactly."""
    H, G, n, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    fan = width ** -0.5
    w = {"q": _rnd(g, H * 2 * n, width) * fan, "q.b": 0.3 * _rnd(g, H * 2 * n), "k": _rnd(g, G * 2 * n, width) * fan,
         "k.b": 0.3 * _rnd(g, G * 2 * n), "v": _rnd(g, G * dv, width) * fan, "v.b": 0.3 * _rnd(g, G * dv),
         "q.norm": 1 + 0.2 * _rnd(g, n), "k.norm": 1 + 0.2 * _rnd(g, n), "o": _rnd(g, width, H * dv) * (H * dv) ** -0.5}
    for name in ("lq1", "lk1", "lq2", "lk2"):
        w[name] = 0.25 * _rnd(g, n)
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def mlp_weights(f, width, vocab, g):
    fan = width ** -0.5
    if f["kind"] == "dense":
        ff = f["ff"]
        w = {"gate": _rnd(g, ff, width) * fan * 1.5, "up": _rnd(g, ff, width) * fan * 1.5, "down": _rnd(g, width, ff) * ff ** -0.5}
        return {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    E, top, ff = f["router"]["experts"], f["router"]["top"], f["expert"]["ff"]
    w = {}
    for e in range(E):
        w[f"e{e}.up"] = _rnd(g, ff, width) * fan * 1.5
        w[f"e{e}.down"] = _rnd(g, width, ff) * ff ** -0.5
    if f.get("shared"):
        sf = f["shared"]["ff"]
        w["shared.up"] = _rnd(g, sf, width) * fan * 1.5
        w["shared.down"] = _rnd(g, width, sf) * sf ** -0.5
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    w["table"] = torch.argsort(torch.rand(vocab, E, generator=g), dim=1)[:, :top].to(torch.int32).contiguous()
    return w


def model_weights(cfg, seed):
    """name -> tensor as a checkpoint stores it (bfloat16, the tables int32)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    w = {"embed": _rnd(g, vocab, width), "final.norm": 0.1 * _rnd(g, width)}
    if cfg.get("loop"):
        w["loop.in"] = _rnd(g, width, 2 * width) * (2 * width) ** -0.5 * 1.4
        w["loop.step"] = 0.3 * _rnd(g, cfg["loop"]["times"], width)
    for i, l in enumerate(cfg["layers"]):
        w[f"l{i}.norm1"] = 0.1 * _rnd(g, width)
        w[f"l{i}.ls1"] = 1 + 0.2 * _rnd(g, width)
        for k, v in mixer_weights(l["mixer"], width, g).items():
            w[f"l{i}.mix.{k}"] = v
        if l.get("mlp") is not None:
            w[f"l{i}.ls2"] = 1 + 0.2 * _rnd(g, width)
            for k, v in mlp_weights(l["mlp"], width, vocab, g).items():
                w[f"l{i}.mlp.{k}"] = v
    return {k: (v if v.dtype == torch.int32 else v.to(torch.bfloat16)) for k, v in w.items()}


def as_float64(weights):
    return {k: (v.clone() if v.dtype == torch.int32 else v.double()) for k, v in weights.items()}


def make_model_dir(cfg, seed) -> Path:
    d = Path(tempfile.mkdtemp(prefix="qv_lotirax_"))
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(d / "model.safetensors", model_weights(cfg, seed).items())
    return d
