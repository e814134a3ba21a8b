"""The Lepizen decoder as a ModelSpec, and its random weights.

Every layer is a parallel block: h = rms(x) g, x <- x + m (attention(h) + mlp(h)), the feed-forward
optional.  The attention has no position encoding; q and k are RMS-normalised over their whole
projections, the softmax has one sink per head, values have a size of their own, and the layers that
mix values blend theirs with the values the first such layer computed for the same token.  The
feed-forward is Wdown gelu(Wup h) with the erf GELU.  The head multiplies by ``logit_scale`` and caps
the logits with tanh.  All of it is built from the engine's shared parts with these options switched on.

Checkpoint tensor names: ``embed``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1``,
``l<i>.mix.{q,k,v,o}``, ``l<i>.mix.{q,k}.norm``, ``l<i>.mix.sink``, ``l<i>.mix.vmix`` (a scalar; in the
first mixing layer present and unused), ``l<i>.mlp.{up,down}``.
"""
from __future__ import annotations

from typing import Iterator, Tuple

from ..config.lepizen import ARCHITECTURE, LepizenConfig
from ..config.model_spec import LayerSpec, ModelSpec, PartSpec
from ..registry import Architecture, register_architecture
from ..weights.draws import Draw, normal, uniform

NO_POSITION_LIMIT = 2 ** 31 - 1      # nothing in the design depends on a position


def build_spec(config: LepizenConfig) -> ModelSpec:
    width = config.width
    layers = []
    seen_mixing = False
    for n, layer in enumerate(config.layers):
        prefix = f"l{n}."
        m = layer.mixer
        weights = {"q.weight": prefix + "mix.q", "k.weight": prefix + "mix.k", "v.weight": prefix + "mix.v",
                   "o.weight": prefix + "mix.o", "q_norm.weight": prefix + "mix.q.norm",
                   "k_norm.weight": prefix + "mix.k.norm", "sink": prefix + "mix.sink",
                   "value_mix.weight": prefix + "mix.vmix"}        # used by blending layers, optional in the others
        value_mix = None
        if m.v_mix:
            value_mix = "blend" if seen_mixing else "first"
            seen_mixing = True
        mixer = PartSpec(
            "gqa_attention",
            {"hidden_size": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
             "scale": m.scale, "qkv_bias": False, "o_bias": False, "window": None, "position": PartSpec("none"),
             "qk_norm": {"scope": "projection", "eps": config.eps}, "sinks": True, "value_mix": value_mix},
            weights)
        ffn = None
        if layer.ff is not None:
            ffn = PartSpec("dense_mlp", {"hidden_size": width, "intermediate_size": layer.ff, "activation": "gelu"},
                           {"up.weight": prefix + "mlp.up", "down.weight": prefix + "mlp.down"})
        norm = PartSpec("rmsnorm", {"size": width, "eps": config.eps}, {"weight": prefix + "norm1"})
        layers.append(LayerSpec("parallel", mixer, ffn, norm, None, block_params={"residual_mult": config.residual_mult}))
    sizes = {"vocab_size": config.vocab, "hidden_size": width}
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=config.vocab, max_positions=NO_POSITION_LIMIT,
        layers=tuple(layers), schedule=tuple(range(len(layers))),
        embedding=PartSpec("token_embedding", sizes, {"weight": "embed"}),
        final_norm=PartSpec("rmsnorm", {"size": width, "eps": config.eps}, {"weight": "final.norm"}),
        head=PartSpec("linear_head", {**sizes, "logit_scale": config.logit_scale, "soft_cap": config.logit_softcap},
                      {"weight": "head"}))


def random_plan(config: LepizenConfig) -> Iterator[Tuple[str, Tuple[int, ...], str, Draw]]:
    """(name, shape, role, draw) of every checkpoint tensor.  Projections N(0, 1/sqrt(fan-in)) so that activations
    keep their size through the layers, norm weights 1 + U(-0.1, 0.1), sinks U(0, 2), blend weights U(0.2, 0.8)."""
    w = config.width
    yield "embed", (config.vocab, w), "matrix", normal(1.0)
    for n, layer in enumerate(config.layers):
        p, m = f"l{n}.", layer.mixer
        yield p + "norm1", (w,), "vector", uniform(0.9, 1.1)
        yield p + "mix.q", (m.heads * m.dim, w), "matrix", normal(w ** -0.5)
        yield p + "mix.k", (m.kv_heads * m.dim, w), "matrix", normal(w ** -0.5)
        yield p + "mix.v", (m.kv_heads * m.vdim, w), "matrix", normal(w ** -0.5)
        yield p + "mix.q.norm", (m.heads * m.dim,), "vector", uniform(0.9, 1.1)
        yield p + "mix.k.norm", (m.kv_heads * m.dim,), "vector", uniform(0.9, 1.1)
        if m.v_mix:
            yield p + "mix.vmix", (), "vector", uniform(0.2, 0.8)
        yield p + "mix.sink", (m.heads,), "vector", uniform(0.0, 2.0)
        yield p + "mix.o", (w, m.heads * m.vdim), "matrix", normal((m.heads * m.vdim) ** -0.5)
        if layer.ff is not None:
            yield p + "mlp.up", (layer.ff, w), "matrix", normal(w ** -0.5)
            yield p + "mlp.down", (w, layer.ff), "matrix", normal(layer.ff ** -0.5)
    yield "final.norm", (w,), "vector", uniform(0.9, 1.1)
    yield "head", (config.vocab, w), "matrix", normal(w ** -0.5)


register_architecture(Architecture(name=ARCHITECTURE, parse_config=LepizenConfig.from_dict, build_spec=build_spec,
                                   random_plan=random_plan))
