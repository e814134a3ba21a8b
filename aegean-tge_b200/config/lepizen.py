"""Typed configuration of the Lepizen decoder, read from config.json.

A Lepizen model is a list of layers, each with an attention mixer and an
optional dense feed-forward that read one shared norm (a parallel block).
Everything that may differ between two models of the design is in
config.json::

    architecture        "Lepizen"
    vocab, width        vocabulary and residual width
    norm.eps            epsilon of every RMS norm (the layers', the final one, and the q/k norms)
    residual_mult       m in  x <- x + m * (mixer(h) + mlp(h))
    logit_scale         multiplies the head's output
    logit_softcap       c in  logits <- c * tanh(logits / c)
    layers[i].type      "attention"
    layers[i].mixer     heads, kv_heads, dim (query/key size per head), vdim (value size per head),
                        scale (multiplies q . k), v_mix (whether the layer takes part in value mixing)
    layers[i].mlp       null, or {"kind": "dense", "ff": inner width}

The design has no position encoding, hence no longest sequence; the engine's
``context`` alone bounds a request.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .common import ConfigError

ARCHITECTURE = "Lepizen"


def _int(where: str, raw: Dict[str, Any], key: str, minimum: int = 1) -> int:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: {where}'{key}' must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be >= {minimum}, got {value}")
    return value


def _number(where: str, raw: Dict[str, Any], key: str, positive: bool = True) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)):
        raise ConfigError(f"config.json: {where}'{key}' must be a finite number, got {value!r}")
    if positive and not float(value) > 0.0:
        raise ConfigError(f"config.json: {where}'{key}' must be positive, got {value}")
    return float(value)


@dataclass(frozen=True)
class LepizenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    v_mix: bool


@dataclass(frozen=True)
class LepizenLayer:
    mixer: LepizenAttention
    ff: Optional[int]            # inner width of the dense feed-forward, None: the layer has none


@dataclass(frozen=True)
class LepizenConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_scale: float
    logit_softcap: float
    layers: Tuple[LepizenLayer, ...]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "LepizenConfig":
        vocab = _int("", raw, "vocab")
        if vocab >= 2 ** 31:
            raise ConfigError(f"config.json: vocab {vocab} does not fit 32-bit token ids")
        width = _int("", raw, "width")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: missing object 'norm' (with 'eps')")
        eps = _number("norm.", norm, "eps")
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        mixing: Optional[Tuple[int, int]] = None
        for index, entry in enumerate(listed):
            where = f"layers[{index}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{index}] must be an object")
            if entry.get("type") != "attention":
                raise ConfigError(f"config.json: {where}'type' must be 'attention', got {entry.get('type')!r}")
            m = entry.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: missing object {where}'mixer'")
            heads, kv_heads = _int(where + "mixer.", m, "heads"), _int(where + "mixer.", m, "kv_heads")
            if heads % kv_heads:
                raise ConfigError(f"config.json: {where}mixer: {heads} heads are not a multiple of {kv_heads} kv_heads")
            v_mix = m.get("v_mix", False)
            if not isinstance(v_mix, bool):
                raise ConfigError(f"config.json: {where}mixer.'v_mix' must be true or false, got {v_mix!r}")
            mixer = LepizenAttention(heads=heads, kv_heads=kv_heads, dim=_int(where + "mixer.", m, "dim"),
                                     vdim=_int(where + "mixer.", m, "vdim"),
                                     scale=_number(where + "mixer.", m, "scale"), v_mix=v_mix)
            if v_mix:
                if mixing is None:
                    mixing = (kv_heads, mixer.vdim)
                elif mixing != (kv_heads, mixer.vdim):
                    raise ConfigError(f"config.json: {where}mixer mixes its values with those of the first mixing layer, "
                                      f"which have {mixing[0]} kv_heads of vdim {mixing[1]}, not {kv_heads} of {mixer.vdim}")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}'mlp' must be null or of kind 'dense', got {mlp!r}")
                ff = _int(where + "mlp.", mlp, "ff")
            layers.append(LepizenLayer(mixer=mixer, ff=ff))
        return LepizenConfig(vocab=vocab, width=width, eps=eps,
                             residual_mult=_number("", raw, "residual_mult", positive=False),
                             logit_scale=_number("", raw, "logit_scale", positive=False),
                             logit_softcap=_number("", raw, "logit_softcap"), layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        return {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
            "residual_mult": self.residual_mult, "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap,
            "layers": [{"type": "attention",
                        "mixer": {"heads": l.mixer.heads, "kv_heads": l.mixer.kv_heads, "dim": l.mixer.dim,
                                  "vdim": l.mixer.vdim, "scale": l.mixer.scale, "v_mix": l.mixer.v_mix},
                        "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}} for l in self.layers],
        }
