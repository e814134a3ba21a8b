"""The Mozepel decoder as a ModelSpec, and its random weights.

Every layer normalises after its sums: x <- rms(a x + mixer(x)) g1, then x <- rms(a x + mlp(x)) g2, the
sublayers reading the stream itself (block ``post_norm``).  A "retention" layer's mixer is linear attention with
a decay per head (``decay_linear_attention``: rotated q and k, k times dim^-1/2, each head's readout over its
own root mean square, a SiLU gate).  A "parallel" layer's mixer is the sum (``mixer_sum``) of a softmax
attention over a sliding window and pooled blocks, its projections passed through a short convolution, q and k
normalised per head and rotated with wavelength-rescaled frequencies (``gqa_attention`` with ``short_conv``,
``pool``), and a second decayed linear attention with SiLU on q, k and v, one norm over all heads and a
logistic gate.  The feed-forward is SwiGLU.  A layer with ``weights_of`` runs an earlier layer's parts with a
cache and state of its own (``LayerSpec.weights_from``).

Checkpoint tensor names: ``embed``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mlp.{gate,up,down}`` (a layer without feed-forward has neither these nor, as a rule, ``norm2``); retention ``l<i>.mix.{q,k,v,g,o}``; parallel ``l<i>.mix.left.{q,k,v,o}``,
``l<i>.mix.left.{q,k}.norm``, ``l<i>.mix.left.{q,k,v}.conv``, ``l<i>.mix.right.{q,k,v,g,o,norm}``.
"""
from __future__ import annotations

from typing import Dict, Iterator, Optional, Tuple

from ..config.model_spec import LayerSpec, ModelSpec, PartSpec
from ..config.mozepel import ARCHITECTURE, DecayMixer, MozepelConfig, Rotation, WindowAttention
from ..registry import Architecture, register_architecture
from ..weights.draws import Draw, normal, uniform

NO_POSITION_LIMIT = 2 ** 31 - 1      # the design states no longest sequence; the rotation's tables follow the engine's context


def _position(rot: Optional[Rotation], dim: int) -> PartSpec:
    if rot is None:
        return PartSpec("none")
    params = {"head_dim": dim, "theta": rot.base, "rotary_dim": rot.dims, "precise": True}
    if rot.scaling is not None:
        params["scaling"] = dict(zip(("factor", "low", "high", "original"), rot.scaling))
    return PartSpec("rope_neox", params)


def _decay_part(m: DecayMixer, width: int, eps: float, prefix: str, *, retention: bool) -> Tuple[PartSpec, Dict[str, str]]:
    """The two decayed linear attentions of the design differ only in what surrounds the recurrence."""
    params = {"hidden_size": width, "heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "decay": tuple(m.decay),
              "eps": eps, "position": _position(m.rot, m.dim)}
    weights = {f"{t}.weight": prefix + t for t in ("q", "k", "v", "g", "o")}
    if retention:
        params.update(k_scale=m.dim ** -0.5, activation="none", out_norm="head", out_norm_weight=False, gate="silu")
    else:
        params.update(k_scale=1.0, activation="silu", out_norm="all", out_norm_weight=True, gate="sigmoid")
        weights["norm.weight"] = prefix + "norm"
    return PartSpec("decay_linear_attention", params, weights), weights


def _window_part(m: WindowAttention, width: int, eps: float, prefix: str) -> Tuple[PartSpec, Dict[str, str]]:
    weights = {"q.weight": prefix + "q", "k.weight": prefix + "k", "v.weight": prefix + "v", "o.weight": prefix + "o",
               "q_norm.weight": prefix + "q.norm", "k_norm.weight": prefix + "k.norm"}
    if m.conv:
        weights.update({f"{t}.conv.weight": f"{prefix}{t}.conv" for t in ("q", "k", "v")})
    params = {"hidden_size": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
              "scale": m.scale, "qkv_bias": False, "o_bias": False, "window": m.window, "pool": m.pool or None,
              "short_conv": m.conv or None, "prepare_in_one_kernel": True, "position": _position(m.rot, m.dim), "qk_norm": {"scope": "head", "eps": eps}}
    return PartSpec("gqa_attention", params, weights), weights


def build_spec(config: MozepelConfig) -> ModelSpec:
    width, eps = config.width, config.eps
    layers = []
    for n, layer in enumerate(config.layers):
        source = n if layer.weights_of is None else layer.weights_of
        prefix = f"l{source}."
        if layer.kind == "retention":
            mixer, _ = _decay_part(layer.mixer, width, eps, prefix + "mix.", retention=True)
        else:
            left, left_w = _window_part(layer.mixer.left, width, eps, prefix + "mix.left.")
            right, right_w = _decay_part(layer.mixer.right, width, eps, prefix + "mix.right.", retention=False)
            weights = {f"left.{k}": v for k, v in left_w.items()}
            weights.update({f"right.{k}": v for k, v in right_w.items()})
            mixer = PartSpec("mixer_sum", {"branches": (("left", left, layer.mixer.left_scale),
                                                        ("right", right, layer.mixer.right_scale))}, weights)
        ffn = None
        # a layer without feed-forward has no second sum to normalise; should a checkpoint hold a second norm for it
        # all the same, it is applied to the scaled stream alone
        norm2 = PartSpec("rmsnorm", {"size": width, "eps": eps, "optional": True}, {"weight": prefix + "norm2"})
        if layer.ff is not None:
            ffn = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": layer.ff},
                           {"gate.weight": prefix + "mlp.gate", "up.weight": prefix + "mlp.up",
                            "down.weight": prefix + "mlp.down"})
            norm2 = PartSpec("rmsnorm", {"size": width, "eps": eps}, {"weight": prefix + "norm2"})
        norm1 = PartSpec("rmsnorm", {"size": width, "eps": eps}, {"weight": prefix + "norm1"})
        layers.append(LayerSpec("post_norm", mixer, ffn, norm1, norm2, block_params={"alpha": config.alpha},
                                weights_from=layer.weights_of))
    sizes = {"vocab_size": config.vocab, "hidden_size": width}
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=config.vocab, max_positions=NO_POSITION_LIMIT,
        layers=tuple(layers), schedule=tuple(range(len(layers))),
        embedding=PartSpec("token_embedding", sizes, {"weight": "embed"}),
        final_norm=PartSpec("rmsnorm", {"size": width, "eps": eps}, {"weight": "final.norm"}),
        head=PartSpec("linear_head", sizes, {"weight": "head"}))


def random_plan(config: MozepelConfig) -> Iterator[Tuple[str, Tuple[int, ...], str, Draw]]:
    """(name, shape, role, draw) of every checkpoint tensor.  Projections N(0, 1/sqrt(fan-in)), norm weights
    1 + U(-0.1, 0.1), convolution taps U(-0.5, 0.5)."""
    w = config.width
    yield "embed", (config.vocab, w), "matrix", normal(1.0)
    for n, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{n}."
        yield p + "norm1", (w,), "vector", uniform(0.9, 1.1)
        if layer.ff is not None:
            yield p + "norm2", (w,), "vector", uniform(0.9, 1.1)
        if layer.kind == "retention":
            m = layer.mixer
            for t, rows in (("q", m.heads * m.dim), ("k", m.heads * m.dim), ("v", m.heads * m.vdim), ("g", m.heads * m.vdim)):
                yield f"{p}mix.{t}", (rows, w), "matrix", normal(w ** -0.5)
            yield p + "mix.o", (w, m.heads * m.vdim), "matrix", normal((m.heads * m.vdim) ** -0.5)
        else:
            a, r = layer.mixer.left, layer.mixer.right
            for t, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
                yield f"{p}mix.left.{t}", (rows, w), "matrix", normal(w ** -0.5)
                if a.conv:
                    yield f"{p}mix.left.{t}.conv", (rows, a.conv), "vector", uniform(-0.5, 0.5)
            yield p + "mix.left.q.norm", (a.dim,), "vector", uniform(0.9, 1.1)
            yield p + "mix.left.k.norm", (a.dim,), "vector", uniform(0.9, 1.1)
            yield p + "mix.left.o", (w, a.heads * a.vdim), "matrix", normal((a.heads * a.vdim) ** -0.5)
            for t, rows in (("q", r.heads * r.dim), ("k", r.heads * r.dim), ("v", r.heads * r.vdim), ("g", r.heads * r.vdim)):
                yield f"{p}mix.right.{t}", (rows, w), "matrix", normal(w ** -0.5)
            yield p + "mix.right.norm", (r.heads * r.vdim,), "vector", uniform(0.9, 1.1)
            yield p + "mix.right.o", (w, r.heads * r.vdim), "matrix", normal((r.heads * r.vdim) ** -0.5)
        if layer.ff is not None:
            yield p + "mlp.gate", (layer.ff, w), "matrix", normal(w ** -0.5)
            yield p + "mlp.up", (layer.ff, w), "matrix", normal(w ** -0.5)
            yield p + "mlp.down", (w, layer.ff), "matrix", normal(layer.ff ** -0.5)
    yield "final.norm", (w,), "vector", uniform(0.9, 1.1)
    yield "head", (config.vocab, w), "matrix", normal(w ** -0.5)


register_architecture(Architecture(name=ARCHITECTURE, parse_config=MozepelConfig.from_dict, build_spec=build_spec,
                                   random_plan=random_plan))
