"""Configuration of the Lotirax decoder, read from its own config.json keys.

A Lotirax model is a list of layers, each a differential-attention mixer beside an optional feed-forward
(dense gated, or small experts chosen by a table over token ids) that reads the same normed input; a
stretch of layers may run several times in a row with the same weights (`loop`).  config.json gives every
size and constant layer by layer, so nothing about a layer is assumed from another.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .deganex_config import _need, _positive_int
from .model_config import ConfigError, ModelConfig

MIXER_KEYS = {"attention": ("heads", "kv_heads", "dim", "vdim", "scale", "diff")}
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class LotiraxConfig(ModelConfig):
    """Field names follow config.json; `layers` keeps each layer's entry as it is written there."""
    vocab_size: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    residual_mult: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times): layers start..stop-1 run `times` times
    layers: Tuple[dict, ...] = field(default_factory=tuple)

    @staticmethod
    def from_dict(d: dict) -> "LotiraxConfig":
        layers = _need(d, "layers", "config")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = (int(_need(lp, "start", "loop")), int(_need(lp, "stop", "loop")), _positive_int(lp, "times", "loop"))
        cfg = LotiraxConfig(
            architecture=str(d.get("architecture") or (d.get("architectures") or ["Lotirax"])[0]),
            vocab_size=_positive_int(d, "vocab", "config"), width=_positive_int(d, "width", "config"),
            norm_eps=float(_need(_need(d, "norm", "config"), "eps", "norm")),
            residual_mult=float(d.get("residual_mult", 1.0)), loop=loop,
            layers=tuple(copy.deepcopy(l) for l in layers), eos_token_id=d.get("eos_token_id"))
        cfg.validate()
        return cfg

    def run_order(self):
        """(layer, pass number or None) in execution order; a pass's first entry is where the stream re-enters."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop
        out = [(i, None) for i in range(a)]
        for t in range(times):
            out += [(i, t) for i in range(a, b)]
        return out + [(i, None) for i in range(b, n)]

    def validate(self) -> None:
        if self.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if self.loop is not None:
            a, b, _ = self.loop
            if not 0 <= a < b <= len(self.layers):
                raise ConfigError(f"config.json: loop.start {a} and loop.stop {b} name no stretch of the {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a known mixer (known: {', '.join(sorted(MIXER_KEYS))})")
            m = _need(layer, "mixer", where)
            for key in MIXER_KEYS[kind]:
                _need(m, key, where + ".mixer")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _positive_int(m, key, where + ".mixer")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: {where}.mixer.heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
            rot = m.get("rot")
            if rot is not None:
                dims = _positive_int(rot, "dims", where + ".mixer.rot")
                _need(rot, "base", where + ".mixer.rot")
                if dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims {dims} must be even and at most dim {m['dim']}")
                sc = rot.get("scaling")
                if sc is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        _need(sc, key, where + ".mixer.rot.scaling")
            mask = m.get("mask")
            if mask is not None:
                _positive_int(mask, "size", where + ".mixer.mask")
            f = layer.get("mlp")
            if f is None:
                continue
            fk = _need(f, "kind", where + ".mlp")
            if fk not in MLP_KINDS:
                raise ConfigError(f"config.json: {where}.mlp.kind '{fk}' is not known (known: {', '.join(MLP_KINDS)})")
            if fk == "dense":
                _positive_int(f, "ff", where + ".mlp")
            else:
                _positive_int(_need(f, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                r = _need(f, "router", where + ".mlp")
                e, top = _positive_int(r, "experts", where + ".mlp.router"), _positive_int(r, "top", where + ".mlp.router")
                if top > e:
                    raise ConfigError(f"config.json: {where}.mlp.router.top {top} exceeds experts {e}")
                if f.get("shared") is not None:
                    _positive_int(f["shared"], "ff", where + ".mlp.shared")

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                             "layers": [copy.deepcopy(l) for l in self.layers]}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
