"""The Lotirax decoder as data: LotiraxConfig -> ModelSpec.

Every layer is a parallel block with ONE norm (weight stored around zero) whose output both parts read: a
differential-attention mixer (two softmax maps per head, biases, per-map query/key norm, partial rotation with
YaRN stretching, sliding window) beside a dense gated feed-forward, small experts chosen by a table over token
ids, or nothing.  Each part's output has a per-feature factor and the block's sum a multiplier.  A stretch of
layers may run several times with the same weights: its layers become repeated entries of the execution order
(parts built once, a cache per run) and the stream re-enters each pass through a product with the embedding's
output.  The head is the embedding table.
Tensor names: embed, loop.in, loop.step, l<i>.norm1, l<i>.mix.*, l<i>.mlp.*, l<i>.ls1, l<i>.ls2, final.norm.
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.lotirax_config import LotiraxConfig
from ..parts.spec import (ActMLPSpec, DiffAttentionSpec, LayerSpec, LoopSpec, ModelSpec, RMSNormSpec, RotarySpec, SwiGLUSpec,
                          TableMoESpec, YarnScaling)


def _mixer_spec(kind: str, m: dict, p: str, width: int, eps: float):
    if kind != "attention":
        raise ValueError(f"unknown mixer '{kind}'")
    position = None
    rot = m.get("rot")
    if rot is not None:
        sc = rot.get("scaling")
        scaling = YarnScaling(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None
        position = RotarySpec(head_dim=m["dim"], rotary_dim=rot["dims"], theta=float(rot["base"]), scaling=scaling)
    return DiffAttentionSpec(
        hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
        scale=float(m["scale"]), diff=float(m["diff"]), eps=eps, q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", q_norm=p + "q.norm",
        k_norm=p + "k.norm", lam_q1=p + "lq1", lam_k1=p + "lk1", lam_q2=p + "lq2", lam_k2=p + "lk2", o_proj=p + "o",
        position=position, window=int((m.get("mask") or {}).get("size", 0)))


def _feed_forward_spec(f, p: str, width: int, vocab: int):
    if f is None:
        return None
    if f["kind"] == "dense":
        return SwiGLUSpec(width, f["ff"], p + "gate", p + "up", p + "down")
    shared = None
    if f.get("shared") is not None:
        shared = ActMLPSpec(width, f["shared"]["ff"], p + "shared.up", p + "shared.down")
    return TableMoESpec(hidden_size=width, vocab_size=vocab, experts=f["router"]["experts"], top=f["router"]["top"],
                        expert_ff=f["expert"]["ff"], table=p + "table", expert_prefix=p + "e", shared=shared)


def lotirax_spec(cfg: LotiraxConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps
    layers, optional = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ff = _feed_forward_spec(layer.get("mlp"), p + "mlp.", width, cfg.vocab_size)
        layers.append(LayerSpec(
            mixer_norm=RMSNormSpec(width, eps, p + "norm1", one_plus=True), mixer=_mixer_spec(layer["type"], layer["mixer"], p + "mix.", width, eps),
            ffn_norm=None, feed_forward=ff, block="parallel", mixer_scale=p + "ls1", ffn_scale=p + "ls2" if ff is not None else None,
            residual_mult=cfg.residual_mult))
        if ff is None:
            optional.append(p + "ls2")           # a factor for a feed-forward the layer has not: passed over if stored
    runs = cfg.run_order()
    loop = None
    if cfg.loop is not None:
        start = cfg.loop[0]
        first_runs = tuple(r for r, (i, t) in enumerate(runs) if t is not None and i == start)
        loop = LoopSpec(first_runs=first_runs, in_proj="loop.in", step="loop.step", hidden_size=width)
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=width, embedding="embed", layers=layers,
                     order=[i for i, _ in runs], final_norm=RMSNormSpec(width, eps, "final.norm", one_plus=True), lm_head=None, loop=loop,
                     optional_tensors=tuple(optional))


register_architecture("Lotirax", LotiraxConfig.from_dict, lotirax_spec)
