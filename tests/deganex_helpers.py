"""Small Deganex configurations with weights drawn for the tests: matrices scaled so that activations are of
order one, attention is peaked and the recurrences' gates move, which is what makes a lost key, a stale state
or a wrong slot show in the logits.  Sizes differ from mechanism to mechanism on purpose (no two of head size,
rotated size, value size, rank, state size are equal; several are no multiple of 16 or 32)."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch

from qorvix_b200.weights import write_safetensors


def attn(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, scale=0.21, base=500.0):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "scale": scale, "rot": {"base": base, "dims": rot_dim}}}


def mlstm(heads=3, dim=20, vdim=40, gate_cap=6.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}}


def mamba(heads=6, vdim=24, state=20, groups=3, conv=3, norm_groups=4):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def moe(experts=5, top=3, ff=24, shared=40):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def layer(mixer, mlp, weights_of=None):
    out = dict(mixer, mlp=mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config(layers, vocab=211, width=72, eps=2e-5, softcap=9.0, bigram=(53, 7, 13)):
    cfg = {"architecture": "Deganex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if softcap:
        cfg["logit_softcap"] = softcap
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return cfg


# two models that share no size; B has what A lacks: one group, one chosen expert, no shared expert, a layer
# without feed-forward, heads == groups, a filter of two taps, no bigram table and no cap on the logits
CONFIG_A = config([layer(attn(), moe()), layer(mlstm(), moe()), layer(mamba(), moe()),
                   layer(attn(), moe(), weights_of=0), layer(mlstm(), moe(), weights_of=1), layer(mamba(), moe(), weights_of=2)])
CONFIG_B = config([layer(mamba(heads=2, vdim=40, state=12, groups=2, conv=2, norm_groups=1), moe(experts=3, top=1, ff=16, shared=0)),
                   layer(attn(heads=1, dim=8, rot_dim=16, vdim=36, kv_rank=24, scale=0.3, base=10000.0), None),
                   layer(mlstm(heads=1, dim=33, vdim=16, gate_cap=3.0), moe(experts=4, top=4, ff=40, shared=8)),
                   layer(attn(heads=1, dim=8, rot_dim=16, vdim=36, kv_rank=24, scale=0.3, base=10000.0), None, weights_of=1),
                   layer(mamba(heads=4, vdim=16, state=36, groups=1, conv=5, norm_groups=2), moe(experts=6, top=2, ff=8, shared=24))],
                  vocab=150, width=48, eps=1e-6, softcap=0.0, bigram=None)


# sizes the tensor-core kernels take (latent of 64, rotated part of 16, inner sizes that are multiples of 8), sixteen
# heads so that a tile of rows spans two tokens, and sizes that differ between the mixers
_ATTN_C = dict(heads=16, dim=8, rot_dim=16, vdim=24, kv_rank=64, scale=0.25, base=3000.0)
CONFIG_C = config([layer(attn(**_ATTN_C), moe(experts=6, top=2, ff=32, shared=16)), layer(mamba(heads=4, vdim=32, state=16, groups=2, conv=4, norm_groups=2), moe(experts=6, top=2, ff=32, shared=16)),
                   layer(mlstm(heads=2, dim=16, vdim=32, gate_cap=8.0), moe(experts=6, top=2, ff=32, shared=16)),
                   layer(attn(**_ATTN_C), moe(experts=6, top=2, ff=32, shared=16), weights_of=0)],
                  vocab=190, width=64, eps=1e-5, softcap=12.0, bigram=(31, 3, 5))


def _rnd(g, *shape):
    return torch.randn(*shape, generator=g)


def mixer_weights(kind, m, width, g, sharp=1.0):
    """Weights of one mixer by their short names ('q', 'dkv.norm', ...), float32 values that bfloat16 holds exactly."""
    w = {}
    fan = width ** -0.5
    if kind == "latent_attention":
        H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        w["q"] = _rnd(g, H * (dn + dr), width) * fan * sharp
        w["dkv"] = _rnd(g, rank + dr, width) * fan * sharp
        w["dkv.norm"] = 1 + 0.2 * _rnd(g, rank)
        w["uk"] = _rnd(g, H * dn, rank) * rank ** -0.5 * 2.0
        w["uv"] = _rnd(g, H * dv, rank) * rank ** -0.5
        w["g"] = _rnd(g, H * dv, width) * fan * 2.0
        w["o"] = _rnd(g, width, H * dv) * (H * dv) ** -0.5
    elif kind == "mlstm":
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        w["q"] = _rnd(g, H * dk, width) * fan * 2.0
        w["k"] = _rnd(g, H * dk, width) * fan * 2.0
        w["v"] = _rnd(g, H * dv, width) * fan
        w["g"] = _rnd(g, H * dv, width) * fan * 2.0
        w["o"] = _rnd(g, width, H * dv) * (H * dv) ** -0.5
        w["norm"] = 1 + 0.2 * _rnd(g, H * dv)
        w["i"] = _rnd(g, H, width) * fan * 3.0
        w["i.b"] = _rnd(g, H)
        w["f"] = _rnd(g, H, width) * fan * 3.0
        w["f.b"] = 1.0 + _rnd(g, H)
    else:
        H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
        inner, ch = H * P, H * P + 2 * G * N
        w["in"] = _rnd(g, inner + ch + H, width) * fan * 1.5
        w["conv"] = _rnd(g, ch, taps) * 0.6
        w["conv.b"] = 0.2 * _rnd(g, ch)
        w["dt_bias"] = -0.5 + _rnd(g, H)
        w["A_log"] = 0.7 * _rnd(g, H)
        w["D"] = 1 + 0.3 * _rnd(g, H)
        w["norm"] = 1 + 0.2 * _rnd(g, inner)
        w["o"] = _rnd(g, width, inner) * inner ** -0.5
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def moe_weights(f, width, g):
    w = {"router": _rnd(g, f["router"]["experts"], width) * width ** -0.5 * 3.0}
    ff = f["expert"]["ff"]
    for e in range(f["router"]["experts"]):
        w[f"e{e}.gate"] = _rnd(g, ff, width) * width ** -0.5 * 1.5
        w[f"e{e}.up"] = _rnd(g, ff, width) * width ** -0.5 * 1.5
        w[f"e{e}.down"] = _rnd(g, width, ff) * ff ** -0.5
    if f.get("shared"):
        sf = f["shared"]["ff"]
        w["shared.gate"] = _rnd(g, sf, width) * width ** -0.5 * 1.5
        w["shared.up"] = _rnd(g, sf, width) * width ** -0.5 * 1.5
        w["shared.down"] = _rnd(g, width, sf) * sf ** -0.5
        w["shared.sg"] = _rnd(g, 1, width) * width ** -0.5 * 2.0
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def model_weights(cfg, seed, sharp=1.0):
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    w = {"embed": _rnd(g, vocab, width), "final.norm": 1 + 0.1 * _rnd(g, width), "head": _rnd(g, vocab, width) * width ** -0.5 * 2.0}
    if cfg.get("embedding", {}).get("bigram"):
        w["bigram"] = _rnd(g, cfg["embedding"]["bigram"]["buckets"] + 1, width)
    for i, l in enumerate(cfg["layers"]):
        if l.get("weights_of") is not None:
            continue
        w[f"l{i}.norm1"] = 1 + 0.1 * _rnd(g, width)
        for k, v in mixer_weights(l["type"], l["mixer"], width, g, sharp).items():
            w[f"l{i}.mix.{k}"] = v * (0.7 if k == "o" else 1.0)
        if l.get("mlp") is not None:
            w[f"l{i}.norm2"] = 1 + 0.1 * _rnd(g, width)
            for k, v in moe_weights(l["mlp"], width, g).items():
                w[f"l{i}.mlp.{k}"] = v * (0.7 if k.endswith("down") else 1.0)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def make_model_dir(cfg, seed, sharp=1.0) -> Path:
    d = Path(tempfile.mkdtemp(prefix="qv_deganex_"))
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(d / "model.safetensors", model_weights(cfg, seed, sharp).items())
    return d
