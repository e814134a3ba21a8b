"""Plain float64 implementation of the Mozepel decoder: the oracle of the tests.

Whole sequences, no cache, no batching, one function per mechanism, numpy only; it shares no code
with the package.  ``weights`` maps tensor names to arrays, ``config`` is the parsed config.json.

A layer normalises AFTER each sum and its sublayers read the stream itself:

    x <- rms(a x + mixer(x)) g1,    x <- rms(a x + mlp(x)) g2        (a = postln_alpha)

Mixer "retention": q, k, v, gate = Wq x, Wk x, Wv x, Wg x; q and k rotated; k scaled by dim^-1/2;
per head S_t = c S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; each head's o divided by its root mean
square; out = Wo (o * silu(gate)).

Mixer "parallel": left_scale * left(x) + right_scale * right(x).
  left  - q, k, v projected, each channel passed through a short causal convolution over time, q and
          k normalised per head and rotated (frequencies rescaled by wavelength), then softmax
          attention in which query i sees the last ``size`` tokens and, for every block of ``pool``
          tokens that lies wholly before them, the mean key and the mean value of the block;
  right - q, k, v = silu of their projections; S_t = c S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; all
          heads normalised together, times sigmoid(Wg x), projected.
mlp(x) = Wdown (silu(Wgate x) * (Wup x)).  Logits = Whead (rms(x) g_final).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np

F = np.float64


def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    return unit_rms(x.astype(F), eps) * weight.astype(F)


def silu(z: np.ndarray) -> np.ndarray:
    return z / (1.0 + np.exp(-z))


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def frequencies(dims: int, base: float, scaling: Optional[dict] = None) -> np.ndarray:
    """f_i = base^(-2i/dims); with ``scaling`` long wavelengths are slowed down by ``factor``, short ones
    kept, and those between blended linearly in original/wavelength."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    if scaling is None:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.copy()
    for i, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            continue
        if wavelength > original / low:
            out[i] = fi / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x: np.ndarray, positions: np.ndarray, dims: int, freq: np.ndarray) -> np.ndarray:
    """x [T, heads, d]: element i < dims/2 is paired with element i + dims/2; the rest passes."""
    half = dims // 2
    angle = positions.astype(F)[:, None] * freq[None, :]
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    return np.concatenate([lo * cos - hi * sin, hi * cos + lo * sin, x[..., dims:]], axis=-1)


def short_conv(u: np.ndarray, w: np.ndarray) -> np.ndarray:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F), u.astype(F)], axis=0)
    y = np.zeros((T, C), dtype=F)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j].astype(F)[None, :]
    return y


def decayed_state_readout(q: np.ndarray, k: np.ndarray, v: np.ndarray, decay: List[float]) -> np.ndarray:
    """q, k [T, H, d], v [T, H, dv] -> o [T, H, dv] with S_t = c_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, d = q.shape
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    for h in range(H):
        S = np.zeros((d, v.shape[2]), dtype=F)
        for t in range(T):
            S = float(decay[h]) * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def retention(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str, m: dict, eps: float) -> np.ndarray:
    T = x.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (x @ w[prefix + "q"].astype(F).T).reshape(T, H, d)
    k = (x @ w[prefix + "k"].astype(F).T).reshape(T, H, d)
    v = (x @ w[prefix + "v"].astype(F).T).reshape(T, H, dv)
    gate = x @ w[prefix + "g"].astype(F).T
    if m.get("rot"):
        freq = frequencies(m["rot"]["dims"], m["rot"]["base"])
        q = rotate(q, np.arange(T), m["rot"]["dims"], freq)
        k = rotate(k, np.arange(T), m["rot"]["dims"], freq)
    k = k * d ** -0.5
    o = unit_rms(decayed_state_readout(q, k, v, m["decay"]), eps).reshape(T, H * dv)
    return (o * silu(gate)) @ w[prefix + "o"].astype(F).T


def window_pool_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, size: int, pool: int) -> np.ndarray:
    """q [T, H, d], k [T, G, d], v [T, G, dv].  Query i sees tokens j with 0 <= i - j < size and block b
    (positions b pool .. b pool + pool - 1, by its mean key and mean value) if b pool + pool - 1 <= i - size."""
    T, H, _ = q.shape
    G = k.shape[1]
    blocks = T // pool if pool else 0
    kp = np.stack([k[b * pool:(b + 1) * pool].mean(axis=0) for b in range(blocks)]) if blocks else np.zeros((0,) + k.shape[1:])
    vp = np.stack([v[b * pool:(b + 1) * pool].mean(axis=0) for b in range(blocks)]) if blocks else np.zeros((0,) + v.shape[1:])
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            first = max(i - size + 1, 0)
            seen = max((i - size + 1) // pool, 0) if pool else 0     # blocks whose last position is <= i - size
            keys = np.concatenate([kp[:seen, g], k[first:i + 1, g]], axis=0)
            vals = np.concatenate([vp[:seen, g], v[first:i + 1, g]], axis=0)
            s = scale * (keys @ q[i, h])
            e = np.exp(s - s.max())
            out[i, h] = (e @ vals) / e.sum()
    return out


def left_branch(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str, m: dict, eps: float) -> np.ndarray:
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (x @ w[prefix + name].astype(F).T for name in ("q", "k", "v"))
    if m.get("conv"):
        q, k, v = (short_conv(u, w[f"{prefix}{name}.conv"]) for u, name in ((q, "q"), (k, "k"), (v, "v")))
    q = rms_norm(q.reshape(T, H, d), w[prefix + "q.norm"], eps)
    k = rms_norm(k.reshape(T, G, d), w[prefix + "k.norm"], eps)
    v = v.reshape(T, G, dv)
    if m.get("rot"):
        freq = frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
        q = rotate(q, np.arange(T), m["rot"]["dims"], freq)
        k = rotate(k, np.arange(T), m["rot"]["dims"], freq)
    a = window_pool_attention(q, k, v, m["scale"], m["mask"]["size"], m["mask"].get("pool") or 0)
    return a.reshape(T, H * dv) @ w[prefix + "o"].astype(F).T


def right_branch(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str, m: dict, eps: float) -> np.ndarray:
    T = x.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(x @ w[prefix + "q"].astype(F).T).reshape(T, H, d)
    k = silu(x @ w[prefix + "k"].astype(F).T).reshape(T, H, d)
    v = silu(x @ w[prefix + "v"].astype(F).T).reshape(T, H, dv)
    o = decayed_state_readout(q, k, v, m["decay"]).reshape(T, H * dv)
    o = rms_norm(o, w[prefix + "norm"], eps) * sigmoid(x @ w[prefix + "g"].astype(F).T)
    return o @ w[prefix + "o"].astype(F).T


def parallel(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str, m: dict, eps: float) -> np.ndarray:
    return (m["left_scale"] * left_branch(x, w, prefix + "left.", m["left"], eps)
            + m["right_scale"] * right_branch(x, w, prefix + "right.", m["right"], eps))


def gated_mlp(x: np.ndarray, gate: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    return (silu(x @ gate.astype(F).T) * (x @ up.astype(F).T)) @ down.astype(F).T


def layer_forward(x: np.ndarray, w: Dict[str, np.ndarray], config: dict, index: int) -> np.ndarray:
    entry = config["layers"][index]
    source = entry.get("weights_of", index)
    p = f"l{source}."
    eps, alpha = config["norm"]["eps"], config["postln_alpha"]
    mix = {"retention": retention, "parallel": parallel}[entry["type"]]
    x = rms_norm(alpha * x + mix(x, w, p + "mix.", entry["mixer"], eps), w[p + "norm1"], eps)
    if entry.get("mlp") is not None:
        x = rms_norm(alpha * x + gated_mlp(x, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"]), w[p + "norm2"], eps)
    elif p + "norm2" in w:           # a second norm kept for a layer without feed-forward: of the scaled stream alone
        x = rms_norm(alpha * x, w[p + "norm2"], eps)
    return x


def forward(config: dict, w: Dict[str, np.ndarray], tokens: List[int], layers_out: Optional[list] = None) -> np.ndarray:
    """Logits [T, vocab] of the whole sequence; ``layers_out`` collects the stream after every layer."""
    x = w["embed"].astype(F)[np.asarray(tokens)]
    for index in range(len(config["layers"])):
        x = layer_forward(x, w, config, index)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, w["final.norm"], config["norm"]["eps"]) @ w["head"].astype(F).T


def greedy(config: dict, w: Dict[str, np.ndarray], prompt: List[int], n: int) -> List[int]:
    tokens, out = list(prompt), []
    for _ in range(n):
        nxt = int(np.argmax(forward(config, w, tokens)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out
