"""What the Lepizen design needs no GPU for: its configuration, its model spec and tensor names, random weights on the
host, the planner, and the plain implementation's own properties."""
import copy
import json
import math

import numpy as np
import pytest
import torch

from plain import lepizen_plain as plain
from test_cli import _run


def _layer(heads, kv_heads, dim, vdim, scale, v_mix, ff):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "scale": scale, "v_mix": v_mix},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIG = {"architecture": "Lepizen", "vocab": 120, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
          "logit_scale": 4.0, "logit_softcap": 9.0,
          "layers": [_layer(4, 2, 8, 12, 0.3, False, 40), _layer(6, 3, 16, 4, 0.2, True, None),
                     _layer(3, 3, 8, 4, 0.25, True, 24)]}


def _weights(config, seed=0):
    from aegean_tge_b200.weights.random_init import random_tensors
    return {name: tensor.numpy().astype(np.float64)
            for name, tensor in random_tensors(config, seed, torch.float32, torch.device("cpu"))}


def test_the_registry_finds_the_design_by_its_own_key():
    from aegean_tge_b200.config.common import ConfigError
    from aegean_tge_b200.registry import architecture_of, registered_architectures
    assert "Lepizen" in registered_architectures()
    arch = architecture_of(CONFIG)
    config = arch.parse_config(CONFIG)
    assert config.to_dict() == CONFIG
    with pytest.raises(ConfigError, match="not registered"):
        architecture_of({"architecture": "Nobody"})
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({"vocab": 3})


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.update(width=0), "width"),
    (lambda c: c.update(norm={}), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c["layers"][0].update(type="recurrent"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(scale=-1.0), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "dense"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "first mixing layer"),
    (lambda c: c.update(logit_softcap=0.0), "logit_softcap"),
    (lambda c: c["layers"][1]["mixer"].update(v_mix=1), "v_mix"),
])
def test_a_config_that_cannot_be_a_model_is_refused(change, message):
    from aegean_tge_b200.config.common import ConfigError
    from aegean_tge_b200.config.lepizen import LepizenConfig
    raw = copy.deepcopy(CONFIG)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        LepizenConfig.from_dict(raw)


def test_the_spec_names_every_tensor_once_and_marks_the_mixing_layers():
    from aegean_tge_b200.config.model_spec import expected_tensors
    from aegean_tge_b200.registry import architecture_of
    arch = architecture_of(CONFIG)
    config = arch.parse_config(CONFIG)
    spec = arch.build_spec(config)
    spec.validate()
    assert [layer.mixer.params["value_mix"] for layer in spec.layers] == [None, "first", "blend"]
    assert [layer.feed_forward is None for layer in spec.layers] == [False, True, False]
    assert all(layer.block == "parallel" and layer.ffn_norm is None for layer in spec.layers)
    planned = {name: tuple(shape) for name, shape, _role, _draw in arch.random_plan(config)}
    assert set(planned) == set(expected_tensors(spec)) - {"l0.mix.vmix"}     # a layer that does not mix may lack it
    assert planned["l1.mix.q"] == (96, 48) and planned["l1.mix.v"] == (12, 48) and planned["l1.mix.o"] == (48, 24)
    assert planned["l1.mix.q.norm"] == (96,) and planned["l1.mix.vmix"] == () and "l0.mix.vmix" not in planned
    assert "l1.mlp.up" not in planned and planned["l2.mlp.down"] == (48, 24)


def test_the_model_on_paper_and_the_planner(tmp_path):
    from aegean_tge_b200.models.decoder import DecoderModel
    from aegean_tge_b200.parts.base import BuildEnv
    from aegean_tge_b200.registry import architecture_of
    arch = architecture_of(CONFIG)
    spec = arch.build_spec(arch.parse_config(CONFIG))
    model = DecoderModel(spec, BuildEnv(dtype=torch.bfloat16, device=torch.device("cpu"), hidden_size=48,
                                        max_positions=256, page_size=64, ops=None))
    assert model.graph_safe
    # per token: layer 0 keeps 2 x (8 + 12), layer 1 3 x (16 + 4), layer 2 3 x (8 + 4) elements of two bytes
    assert model.cache_bytes_per_token() == 2 * (2 * 20 + 3 * 20 + 3 * 12)
    manifest = model.manifest()
    assert manifest["l2.mix.vmix"][0].shape == () and not manifest["l2.mix.vmix"][0].optional
    assert manifest["l1.mix.vmix"][0].optional                    # present in a checkpoint, unused by the first mixing layer
    assert manifest["l0.mix.vmix"][0].optional                    # a layer that does not mix: taken if present
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIG))
    out = _run("make-random", "--config", str(config), "--out", str(tmp_path / "m"), "--seed", "3")
    assert out.returncode == 0, out.stderr
    out = _run("plan", "--model", str(tmp_path / "m"), "--context", "256", "--sessions", "2")
    assert out.returncode == 0, out.stderr
    assert f"kv       : {model.cache_bytes_per_token()} bytes per token" in out.stdout


def test_plain_attention_is_causal_and_the_sink_only_shrinks():
    rng = np.random.default_rng(0)
    q, k, v = rng.normal(size=(9, 4, 8)), rng.normal(size=(9, 2, 8)), rng.normal(size=(9, 2, 5))
    sink = rng.normal(size=4)
    full = plain.sink_attention(q, k, v, sink, 0.4)
    k2, v2 = k.copy(), v.copy()
    k2[6:], v2[6:] = 100.0, -100.0                                   # the future changes nothing before it
    assert np.allclose(plain.sink_attention(q, k2, v2, sink, 0.4)[:6], full[:6], rtol=0, atol=1e-12)
    assert np.allclose(plain.sink_attention(q[5:], k, v, sink, 0.4, start=5), full[5:], rtol=0, atol=1e-12)
    # without a sink (minus infinity) it is the plain softmax; the first row then returns its own value
    none = plain.sink_attention(q, k, v, np.full(4, -np.inf), 0.4)
    assert np.allclose(none[0, 0], v[0, 0]) and np.allclose(none[0, 3], v[0, 1])
    # the sink takes exp(sink) / (exp(sink) + sum exp(s)) of the weight away, whatever the values are
    s = 0.4 * (k[:1, 0] @ q[0, 0])
    share = math.exp(sink[0]) / (math.exp(sink[0]) + math.exp(float(s[0])))
    assert np.allclose(full[0, 0], (1.0 - share) * v[0, 0])


def test_plain_model_mixes_values_of_the_same_token_only():
    w = _weights(CONFIG, seed=4)
    tokens = [5, 17, 3, 99, 41, 7, 0, 64]
    streams = []
    logits = plain.forward(CONFIG, w, tokens, streams)
    assert logits.shape == (8, 120) and len(streams) == 3 and float(np.abs(logits).max()) < 9.0
    shorter = plain.forward(CONFIG, w, tokens[:5])
    assert np.allclose(shorter, logits[:5], rtol=0, atol=1e-10)       # a prefix's logits do not depend on what follows
    other = copy.deepcopy(CONFIG)
    other["layers"][2]["mixer"]["v_mix"] = False
    assert np.abs(plain.forward(other, w, tokens) - logits).max() > 1e-3
    # with a blend weight of zero the last layer keeps its own values: the same as not mixing at all
    w0 = dict(w)
    w0["l2.mix.vmix"] = np.zeros(())
    assert np.allclose(plain.forward(CONFIG, w0, tokens), plain.forward(other, w, tokens), rtol=0, atol=1e-10)


def test_gelu_forms():
    z = np.linspace(-6.0, 6.0, 25)
    assert np.allclose(plain.gelu_erf(z)[12], 0.0) and np.allclose(plain.gelu_erf(np.array([1.0])), 0.8413447460685429)
    assert np.allclose(plain.gelu_erf(z) - plain.gelu_erf(-z), z)
