"""Configuration of the Deganex decoder, read from its own config.json keys.

A Deganex model is a list of layers, each with one mixer (latent attention, a matrix-memory LSTM or a
selective state space) beside a routed feed-forward; config.json gives every size and constant, layer
by layer, so nothing about a layer is assumed from another.  A layer may name another layer whose
weights it uses (`weights_of`) while keeping a cache or state of its own.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .model_config import ConfigError, ModelConfig

MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
    "mlstm": ("heads", "dim", "vdim", "gate_cap"),
    "mamba2": ("heads", "vdim", "state", "groups", "conv", "norm_groups"),
}


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{where}.{key}' is missing")
    return d[key]


def _positive_int(d: dict, key: str, where: str) -> int:
    v = _need(d, key, where)
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: '{where}.{key}' = {v!r} must be a positive integer")
    return v


@dataclass(frozen=True)
class DeganexConfig(ModelConfig):
    """Field names follow config.json; `layers` keeps each layer's entry as it is written there."""
    vocab_size: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    logit_softcap: float = 0.0                    # 0: none
    bigram: Optional[Tuple[int, int, int]] = None  # (buckets, mul_prev, mul_cur)
    layers: Tuple[dict, ...] = field(default_factory=tuple)

    @staticmethod
    def from_dict(d: dict) -> "DeganexConfig":
        layers = _need(d, "layers", "config")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        bg = (d.get("embedding") or {}).get("bigram")
        bigram = None
        if bg is not None:
            bigram = (_positive_int(bg, "buckets", "embedding.bigram"), int(_need(bg, "mul_prev", "embedding.bigram")),
                      int(_need(bg, "mul_cur", "embedding.bigram")))
        cfg = DeganexConfig(
            architecture=str(d.get("architecture") or (d.get("architectures") or ["Deganex"])[0]),
            vocab_size=_positive_int(d, "vocab", "config"), width=_positive_int(d, "width", "config"),
            norm_eps=float(_need(_need(d, "norm", "config"), "eps", "norm")),
            logit_softcap=float(d.get("logit_softcap") or 0.0), bigram=bigram,
            layers=tuple(copy.deepcopy(l) for l in layers), eos_token_id=d.get("eos_token_id"))
        cfg.validate()
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself unless it names another)."""
        seen = set()
        while self.layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of runs in a circle")
            seen.add(i)
            i = int(self.layers[i]["weights_of"])
        return i

    def validate(self) -> None:
        if self.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a known mixer (known: {', '.join(sorted(MIXER_KEYS))})")
            m = _need(layer, "mixer", where)
            for key in MIXER_KEYS[kind]:
                _need(m, key, where + ".mixer")
            for key in ("heads", "dim", "vdim", "kv_rank", "rot_dim", "state", "groups", "conv", "norm_groups"):
                if key in MIXER_KEYS[kind]:
                    _positive_int(m, key, where + ".mixer")
            if kind == "latent_attention":
                rot = m["rot"]
                dims = _positive_int(rot, "dims", where + ".mixer.rot")
                _need(rot, "base", where + ".mixer.rot")
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims {dims} must be even and at most rot_dim {m['rot_dim']}")
            if kind == "mamba2":
                if m["heads"] % m["groups"]:
                    raise ConfigError(f"config.json: {where}.mixer.heads {m['heads']} is not a multiple of groups {m['groups']}")
                if (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise ConfigError(f"config.json: {where}.mixer: heads * vdim is not a multiple of norm_groups {m['norm_groups']}")
            w = layer.get("weights_of")
            if w is not None:
                if not isinstance(w, int) or not 0 <= w < len(self.layers) or w == i:
                    raise ConfigError(f"config.json: {where}.weights_of = {w!r} names no other layer")
                o = self.layers[self.owner(i)]
                if o.get("type") != kind or o.get("mixer") != m or o.get("mlp") != layer.get("mlp"):
                    raise ConfigError(f"config.json: {where} uses the weights of layer {w} but differs from it")
            f = layer.get("mlp")
            if f is not None:
                if f.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{f.get('kind')}' is not known (known: moe)")
                _positive_int(_need(f, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                r = _need(f, "router", where + ".mlp")
                e, top = _positive_int(r, "experts", where + ".mlp.router"), _positive_int(r, "top", where + ".mlp.router")
                if top > e:
                    raise ConfigError(f"config.json: {where}.mlp.router.top {top} exceeds experts {e}")
                if f.get("shared") is not None:
                    _positive_int(f["shared"], "ff", where + ".mlp.shared")

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "layers": [copy.deepcopy(l) for l in self.layers]}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.bigram is not None:
            d["embedding"] = {"bigram": {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
