"""The Deganex decoder as data: DeganexConfig -> ModelSpec.

Every layer is a parallel block (mixer and routed feed-forward both read the stream as it enters, each
through an RMS norm of its own) whose mixer is latent attention, a matrix-memory LSTM or a selective state
space, as config.json says layer by layer.  Layers that use another layer's weights become repeated
entries of the execution order: the parts are built once and every run keeps a cache or state of its own.
Tensor names: embed, bigram, l<i>.norm1/.norm2, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.deganex_config import DeganexConfig
from ..parts.spec import (BigramEmbeddingSpec, LatentAttentionSpec, LayerSpec, Mamba2Spec, MLSTMSpec, ModelSpec, MoESpec, RMSNormSpec,
                          RotarySpec, SwiGLUSpec)


def _mixer_spec(kind: str, m: dict, p: str, width: int, eps: float):
    if kind == "latent_attention":
        rot = m["rot"]
        return LatentAttentionSpec(
            hidden_size=width, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"],
            kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=eps,
            position=RotarySpec(head_dim=m["rot_dim"], rotary_dim=rot["dims"], theta=float(rot["base"]), pairing="interleaved"),
            q_proj=p + "q", kv_down=p + "dkv", kv_norm=p + "dkv.norm", k_up=p + "uk", v_up=p + "uv", gate_proj=p + "g", o_proj=p + "o")
    if kind == "mlstm":
        return MLSTMSpec(hidden_size=width, num_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"], gate_cap=float(m["gate_cap"]),
                         eps=eps, q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", gate_proj=p + "g", i_proj=p + "i", i_bias=p + "i.b",
                         f_proj=p + "f", f_bias=p + "f.b", norm=p + "norm", o_proj=p + "o")
    if kind == "mamba2":
        return Mamba2Spec(hidden_size=width, num_heads=m["heads"], value_dim=m["vdim"], state_dim=m["state"], groups=m["groups"],
                          conv_taps=m["conv"], norm_groups=m["norm_groups"], eps=eps, in_proj=p + "in", conv_weight=p + "conv",
                          conv_bias=p + "conv.b", dt_bias=p + "dt_bias", a_log=p + "A_log", skip=p + "D", norm=p + "norm", o_proj=p + "o")
    raise ValueError(f"unknown mixer '{kind}'")


def _feed_forward_spec(f, p: str, width: int):
    if f is None:
        return None
    shared = None
    if f.get("shared") is not None:
        shared = SwiGLUSpec(width, f["shared"]["ff"], p + "shared.gate", p + "shared.up", p + "shared.down")
    return MoESpec(hidden_size=width, experts=f["router"]["experts"], top=f["router"]["top"], expert_ff=f["expert"]["ff"],
                   router=p + "router", expert_prefix=p + "e", shared=shared, shared_gate=p + "shared.sg" if shared else None)


def deganex_spec(cfg: DeganexConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps
    layers, index_of, order = [], {}, []
    for i, layer in enumerate(cfg.layers):
        o = cfg.owner(i)
        if o not in index_of:
            src = cfg.layers[o]
            p = f"l{o}."
            ff = _feed_forward_spec(src.get("mlp"), p + "mlp.", width)
            index_of[o] = len(layers)
            layers.append(LayerSpec(
                mixer_norm=RMSNormSpec(width, eps, p + "norm1"), mixer=_mixer_spec(src["type"], src["mixer"], p + "mix.", width, eps),
                ffn_norm=RMSNormSpec(width, eps, p + "norm2") if ff is not None else None, feed_forward=ff, block="parallel"))
        order.append(index_of[o])
    if cfg.bigram is not None:
        embedding = BigramEmbeddingSpec(cfg.vocab_size, width, "embed", "bigram", *cfg.bigram)
    else:
        embedding = "embed"
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=width, embedding=embedding,
                     layers=layers, order=order, final_norm=RMSNormSpec(width, eps, "final.norm"), lm_head="head",
                     logit_softcap=cfg.logit_softcap)


register_architecture("Deganex", DeganexConfig.from_dict, deganex_spec)
