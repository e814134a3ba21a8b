"""Typed configuration of the Mozepel decoder, read from config.json.

A Mozepel model is a list of layers that normalise after each sum
(x <- norm(alpha x + sublayer(x))).  A layer's mixer is one of two kinds, and
a layer may borrow all its weights from an earlier one while keeping a state
and cache of its own.  Everything that may differ between two models of the
design is in config.json::

    architecture        "Mozepel"
    vocab, width        vocabulary and residual width
    norm.eps            epsilon of every RMS norm
    postln_alpha        alpha in  x <- norm(alpha x + sublayer(x))
    layers[i].type      "retention" or "parallel"
    layers[i].weights_of  (optional) index of the layer whose tensors this one uses
    layers[i].mlp       null, or {"kind": "dense", "ff": inner width}  (a gated SiLU feed-forward)
    layers[i].mixer     retention: heads, dim, vdim, decay [heads], rot {base, dims}
                        parallel:  left_scale, right_scale,
                                   left  {heads, kv_heads, dim, vdim, scale, conv (taps), mask {size, pool},
                                          rot {base, dims, scaling {factor, low, high, original}}}
                                   right {heads, dim, vdim, decay [heads]}

The design states no longest sequence: the engine's ``context`` alone bounds a request.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .common import ConfigError
from .lepizen import _int, _number

ARCHITECTURE = "Mozepel"


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, low, high, original

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return out


@dataclass(frozen=True)
class DecayMixer:
    """Linear attention with a decay per head: the retention mixer, and the right branch of the parallel one."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[Rotation] = None

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class WindowAttention:
    """The left branch of the parallel mixer: softmax attention over a window and pooled blocks."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int                    # taps of the short convolution, 0: none
    window: int
    pool: int                    # tokens per pooled block, 0: none
    rot: Optional[Rotation]

    def to_dict(self) -> Dict[str, Any]:
        mask: Dict[str, Any] = {"size": self.window}
        if self.pool:
            mask["pool"] = self.pool
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale, "mask": mask}
        if self.conv:
            out["conv"] = self.conv
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class ParallelMixer:
    left: WindowAttention
    right: DecayMixer
    left_scale: float
    right_scale: float

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class MozepelLayer:
    kind: str                                   # "retention" or "parallel"
    mixer: Any                                  # DecayMixer or ParallelMixer
    ff: Optional[int]                           # inner width of the feed-forward, None: the layer has none
    weights_of: Optional[int] = None


def _rotation(where: str, raw: Any, dim: int) -> Optional[Rotation]:
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where}'rot' must be an object")
    dims = _int(where + "rot.", raw, "dims", minimum=2)
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most the head size {dim}")
    scaling = raw.get("scaling")
    values = None
    if scaling is not None:
        if not isinstance(scaling, dict):
            raise ConfigError(f"config.json: {where}rot.'scaling' must be an object")
        values = tuple(_number(where + "rot.scaling.", scaling, key, positive=key in ("factor", "original"))
                       for key in ("factor", "low", "high", "original"))
        if not values[2] > values[1] >= 0.0:
            raise ConfigError(f"config.json: {where}rot.scaling needs high > low >= 0")
    return Rotation(base=_number(where + "rot.", raw, "base"), dims=dims, scaling=values)


def _decay_mixer(where: str, m: Dict[str, Any]) -> DecayMixer:
    heads, dim = _int(where, m, "heads"), _int(where, m, "dim")
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads:
        raise ConfigError(f"config.json: {where}'decay' must list one factor per head ({heads})")
    values = []
    for value in decay:
        if isinstance(value, bool) or not isinstance(value, (int, float)) or not 0.0 < float(value) <= 1.0:
            raise ConfigError(f"config.json: {where}'decay' holds {value!r}; factors lie in (0, 1]")
        values.append(float(value))
    return DecayMixer(heads=heads, dim=dim, vdim=_int(where, m, "vdim"), decay=tuple(values),
                      rot=_rotation(where, m.get("rot"), dim))


def _window_attention(where: str, m: Dict[str, Any]) -> WindowAttention:
    heads, kv_heads, dim = _int(where, m, "heads"), _int(where, m, "kv_heads"), _int(where, m, "dim")
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv_heads} kv_heads")
    mask = m.get("mask")
    if not isinstance(mask, dict):
        raise ConfigError(f"config.json: missing object {where}'mask' (with 'size')")
    conv = 0 if m.get("conv") is None else _int(where, m, "conv", minimum=0)
    if conv > 16:
        raise ConfigError(f"config.json: {where}'conv' has {conv} taps; at most 16")
    pool = 0 if mask.get("pool") is None else _int(where + "mask.", mask, "pool", minimum=0)
    return WindowAttention(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_int(where, m, "vdim"),
                           scale=_number(where, m, "scale"), conv=conv, window=_int(where + "mask.", mask, "size"),
                           pool=pool, rot=_rotation(where, m.get("rot"), dim))


@dataclass(frozen=True)
class MozepelConfig:
    vocab: int
    width: int
    eps: float
    alpha: float
    layers: Tuple[MozepelLayer, ...]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "MozepelConfig":
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
        for index, entry in enumerate(listed):
            where = f"layers[{index}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{index}] must be an object")
            kind = entry.get("type")
            m = entry.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: missing object {where}'mixer'")
            if kind == "retention":
                mixer: Any = _decay_mixer(where + "mixer.", m)
            elif kind == "parallel":
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    raise ConfigError(f"config.json: {where}mixer needs objects 'left' and 'right'")
                mixer = ParallelMixer(left=_window_attention(where + "mixer.left.", left),
                                      right=_decay_mixer(where + "mixer.right.", right),
                                      left_scale=_number(where + "mixer.", m, "left_scale", positive=False),
                                      right_scale=_number(where + "mixer.", m, "right_scale", positive=False))
            else:
                raise ConfigError(f"config.json: {where}'type' must be 'retention' or 'parallel', got {kind!r}")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}'mlp' must be null or of kind 'dense', got {mlp!r}")
                ff = _int(where + "mlp.", mlp, "ff")
            source = entry.get("weights_of")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < index:
                    raise ConfigError(f"config.json: {where}'weights_of' must name an earlier layer, got {source!r}")
                other = layers[source]
                if other.weights_of is not None:
                    raise ConfigError(f"config.json: {where}'weights_of' names layer {source}, which has no tensors of its own")
                if (other.kind, other.mixer, other.ff) != (kind, mixer, ff):
                    raise ConfigError(f"config.json: layer {index} uses the weights of layer {source} but is described differently")
            layers.append(MozepelLayer(kind=kind, mixer=mixer, ff=ff, weights_of=source))
        return MozepelConfig(vocab=vocab, width=width, eps=eps, alpha=_number("", raw, "postln_alpha", positive=False),
                             layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            entry: Dict[str, Any] = {"type": layer.kind, "mixer": layer.mixer.to_dict(),
                                     "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "postln_alpha": self.alpha, "layers": layers}
