"""Plain float64 implementation of the Lepizen decoder: the oracle of the tests.

Whole sequences, no cache, no batching, one function per mechanism, numpy only; it shares no
code with the package.  ``weights`` maps tensor names to arrays, ``config`` is the parsed
config.json.  In the notation used here a layer is

    h = rms(x) * g                                  (one norm per layer)
    x <- x + m * (attention(h) + mlp(h))            (both sublayers read the same h)

with attention(h): q = Wq h, k = Wk h, v = Wv h; q and k are each normalised over their WHOLE
projection (all heads at once) and scaled by a weight of that size; query head i reads key/value
head i // (heads / kv_heads); score(i, j) = scale * <q_i, k_j> for j <= i, no positional term;
weights p_ij = exp(s_ij) / (exp(sink) + sum_j' exp(s_ij')) with one learned sink per head; the
values of every value-mixing layer after the first are blended with the first such layer's values
of the same token, v <- (1 - lam) v + lam v_first.  mlp(h) = Wdown gelu_erf(Wup h).  The logits are
cap * tanh(logit_scale * (Whead rms(x) g_final) / cap).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import numpy as np

F = np.float64


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    x = x.astype(F)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * weight.astype(F)


def gelu_erf(z: np.ndarray) -> np.ndarray:
    erf = np.vectorize(math.erf, otypes=[F])
    return 0.5 * z * (1.0 + erf(z / math.sqrt(2.0)))


def dense_mlp(h: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    return gelu_erf(h @ up.astype(F).T) @ down.astype(F).T


def blend_values(v: np.ndarray, v_first: Optional[np.ndarray], lam: float) -> np.ndarray:
    return v if v_first is None else (1.0 - lam) * v + lam * v_first


def sink_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, sink: np.ndarray, scale: float,
                   start: int = 0) -> np.ndarray:
    """q [T, H, d], k [S, G, d], v [S, G, dv] with S = start + T: query t sits at position start + t and
    sees keys 0..start + t.  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    for head in range(H):
        g = head // (H // G)
        for t in range(T):
            last = start + t
            s = scale * (k[:last + 1, g] @ q[t, head])
            top = max(float(s.max()), float(sink[head]))
            e = np.exp(s - top)
            out[t, head] = (e @ v[:last + 1, g]) / (e.sum() + math.exp(float(sink[head]) - top))
    return out


def attention_mixer(h: np.ndarray, w: Dict[str, np.ndarray], prefix: str, mixer: dict, eps: float,
                    v_first: Optional[np.ndarray], blends: bool) -> Tuple[np.ndarray, np.ndarray]:
    """Returns (the mixer's output [T, width], the values this layer attends over [T, G, dv])."""
    H, G, d, dv = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    q = rms_norm(h @ w[prefix + "q"].astype(F).T, w[prefix + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(h @ w[prefix + "k"].astype(F).T, w[prefix + "k.norm"], eps).reshape(T, G, d)
    v = (h @ w[prefix + "v"].astype(F).T).reshape(T, G, dv)
    if blends:
        v = blend_values(v, v_first, float(w[prefix + "vmix"]))
    a = sink_attention(q, k, v, w[prefix + "sink"].astype(F), float(mixer["scale"]))
    return a.reshape(T, H * dv) @ w[prefix + "o"].astype(F).T, v


def soft_cap(z: np.ndarray, cap: float) -> np.ndarray:
    return cap * np.tanh(z / cap)


def forward(config: dict, w: Dict[str, np.ndarray], tokens: List[int],
            streams: Optional[list] = None) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence; ``streams`` collects the residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    m = float(config["residual_mult"])
    x = w["embed"].astype(F)[np.asarray(tokens)]
    v_first = None
    for index, layer in enumerate(config["layers"]):
        if layer["type"] != "attention":
            raise ValueError(f"layer {index}: unknown type {layer['type']}")
        p = f"l{index}."
        h = rms_norm(x, w[p + "norm1"], eps)
        blends = bool(layer["mixer"].get("v_mix", False))
        a, v = attention_mixer(h, w, p + "mix.", layer["mixer"], eps, v_first, blends)
        if blends and v_first is None:
            v_first = v
        f = 0.0
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"layer {index}: unknown feed-forward {layer['mlp']['kind']}")
            f = dense_mlp(h, w[p + "mlp.up"], w[p + "mlp.down"])
        x = x + m * (a + f)
        if streams is not None:
            streams.append(x.copy())
    z = rms_norm(x, w["final.norm"], eps) @ w["head"].astype(F).T * float(config["logit_scale"])
    return soft_cap(z, float(config["logit_softcap"]))
