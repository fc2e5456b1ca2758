"""The plain Sebilorn: every mechanism as a slow function of its own, in 64-bit numpy, over one whole sequence.

It shares nothing with the engine: it reads a configuration dictionary (the keys of config.json) and a dictionary of
arrays by tensor name, and runs the sequence position by position where a mechanism is recurrent and as dense
[T, T] tables where it is attention. The tests hold the engine's parts and whole models to it.

Notation: n is a normed row, W is stored [out, in] and applied as W n, T tokens at positions 0..T-1.
"""

from __future__ import annotations

import math

import numpy as np

DECAY_RATE = math.exp(-0.5)       # the delta rule's decay is exp(-DECAY_RATE * sigmoid(.))
UNIT_KEY_EPS = 1e-6               # added to the sum of a key's squares before the root


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def layer_norm(x, w, b, eps):
    mean = x.mean(-1, keepdims=True)
    var = ((x - mean) ** 2).mean(-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rotary_frequencies(base: float, dims: int, scaling: dict | None = None) -> np.ndarray:
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` = {factor, low, high, original} long wavelengths are slowed:
    wavelength l = 2 pi / f; l < original/high: kept; l > original/low: f / factor; between them a blend."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.copy()
    for i, fi in enumerate(f):
        l = 2.0 * math.pi / fi
        if l < orig / high:
            continue
        if l > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / l - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_halves(x: np.ndarray, positions: np.ndarray, freqs: np.ndarray, sign: float = 1.0) -> np.ndarray:
    """x [T, heads, D]: entry i and entry i + d/2 (d = 2 len(freqs) <= D) are a pair that turns by sign * p * f_i; the
    entries from d on pass."""
    half = len(freqs)
    a = sign * positions[:, None, None].astype(np.float64) * freqs[None, None, :]
    c, s = np.cos(a), np.sin(a)
    out = x.copy()
    u, v = x[..., :half], x[..., half:2 * half]
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


def visible(T: int, window: int | None, keep_first: int) -> np.ndarray:
    """[T, T] booleans: row i sees key j when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok &= (i - j < window) | (j < keep_first)
    return ok


def softmax_attention(q, k, v, scale: float, softcap: float | None, see: np.ndarray) -> np.ndarray:
    """q [T, H, D], k [T, G, D], v [T, G, VD] -> [T, H, VD]; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        s = np.where(see, s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def attention_keys_values(n, m: dict, w: dict, pre: str):
    """The keys (rotated) and the values (rotated over all their entries) as the layer's cache holds them."""
    T = n.shape[0]
    G, D, VD = m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    rot = m["rot"]
    k = (n @ w[pre + "k"].T).reshape(T, G, D)
    v = (n @ w[pre + "v"].T).reshape(T, G, VD)
    k = rotate_halves(k, pos, rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling")))
    v = rotate_halves(v, pos, rotary_frequencies(rot["base"], VD))
    return k, v


def mixer_attention(n, m: dict, w: dict, pre: str, kv) -> np.ndarray:
    """Sliding-window attention with kept first tokens, capped scores and values that turn with their position; `kv`: the
    (keys, values) of the layer this one borrows them from, or None for its own."""
    T = n.shape[0]
    H, D, VD = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    rot = m["rot"]
    q = (n @ w[pre + "q"].T).reshape(T, H, D)
    q = rotate_halves(q, pos, rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling")))
    k, v = kv if kv is not None else attention_keys_values(n, m, w, pre)
    mask = m.get("mask")
    see = visible(T, mask["size"] if mask else None, mask.get("keep_first", 0) if mask else 0)
    o = softmax_attention(q, k, v, m["scale"], m.get("softcap"), see)
    o = rotate_halves(o, pos, rotary_frequencies(rot["base"], VD), sign=-1.0)     # turned back by the row's own position
    return o.reshape(T, H * VD) @ w[pre + "o"].T


def mixer_gated_attention(n, m: dict, w: dict, pre: str) -> np.ndarray:
    """Causal attention over all keys, rotary on q and k, the concatenated heads times sigmoid(W_g n) entry by entry."""
    T = n.shape[0]
    H, G, D, VD = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    f = rotary_frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    q = rotate_halves((n @ w[pre + "q"].T).reshape(T, H, D), pos, f)
    k = rotate_halves((n @ w[pre + "k"].T).reshape(T, G, D), pos, f)
    v = (n @ w[pre + "v"].T).reshape(T, G, VD)
    o = softmax_attention(q, k, v, m["scale"], None, visible(T, None, 0)).reshape(T, H * VD)
    return (o * sigmoid(n @ w[pre + "g"].T)) @ w[pre + "o"].T


def delta_rule_decay(n, w: dict, pre: str) -> np.ndarray:
    return np.exp(-DECAY_RATE * sigmoid(np.tanh(n @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"]))


def mixer_delta_rule(n, m: dict, w: dict, pre: str, eps: float, state=None, return_state: bool = False):
    """S <- diag(w) S - (a u)(u^T S) + k v^T with both terms reading the old S; o = S^T r; per head [dim, dim]."""
    T = n.shape[0]
    H, D = m["heads"], m["dim"]
    r = (n @ w[pre + "r"].T).reshape(T, H, D)
    k = (n @ w[pre + "k"].T).reshape(T, H, D)
    v = (n @ w[pre + "v"].T).reshape(T, H, D)
    decay = delta_rule_decay(n, w, pre).reshape(T, H, D)
    a = sigmoid(n @ w[pre + "a"].T + w[pre + "a.b"]).reshape(T, H, D)
    u = k / np.sqrt((k * k).sum(-1, keepdims=True) + UNIT_KEY_EPS)
    S = np.zeros((H, D, D)) if state is None else state.copy()
    o = np.zeros((T, H, D))
    for t in range(T):
        for h in range(H):
            old = S[h]
            S[h] = decay[t, h][:, None] * old - np.outer(a[t, h] * u[t, h], u[t, h] @ old) + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ r[t, h]
    o = unit_rms(o, eps).reshape(T, H * D) * w[pre + "norm"] * sigmoid(n @ w[pre + "g"].T)
    out = o @ w[pre + "o"].T
    return (out, S) if return_state else out


def mixer_parallel(n, m: dict, w: dict, pre: str, eps: float) -> np.ndarray:
    left = mixer_gated_attention(n, m["left"], w, pre + "left.")
    right = mixer_delta_rule(n, m["right"], w, pre + "right.", eps)
    return m["left_scale"] * left + m["right_scale"] * right


def mixer_lightning(n, m: dict, w: dict, pre: str, eps: float, state=None, return_state: bool = False):
    """S <- decay_h S + k v^T, o = S^T q, with q, k, v behind a SiLU; all heads normed together."""
    T = n.shape[0]
    H, D, VD = m["heads"], m["dim"], m["vdim"]
    q = silu(n @ w[pre + "q"].T).reshape(T, H, D)
    k = silu(n @ w[pre + "k"].T).reshape(T, H, D)
    v = silu(n @ w[pre + "v"].T).reshape(T, H, VD)
    S = np.zeros((H, D, VD)) if state is None else state.copy()
    o = np.zeros((T, H, VD))
    for t in range(T):
        for h in range(H):
            S[h] = m["decay"][h] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    o = unit_rms(o.reshape(T, H * VD), eps) * w[pre + "norm"] * sigmoid(n @ w[pre + "g"].T)
    out = o @ w[pre + "o"].T
    return (out, S) if return_state else out


def dense_relu2(n, w: dict, pre: str) -> np.ndarray:
    z = np.maximum(n @ w[pre + "up"].T, 0.0)
    return (z * z) @ w[pre + "down"].T


def forward(config: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of the whole sequence (and, with `return_layers`, the stream after every layer)."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)] * float(config["embedding"]["scale"])
    kept, streams = {}, []
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]
        n = layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps)
        kind = layer["type"]
        if kind == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(n, m, w, pre + "mix.")
            x = x + mixer_attention(n, m, w, pre + "mix.", kept[i if src is None else src])
        elif kind == "parallel":
            x = x + mixer_parallel(n, m, w, pre + "mix.", eps)
        elif kind == "lightning":
            x = x + mixer_lightning(n, m, w, pre + "mix.", eps)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            x = x + dense_relu2(layer_norm(x, w[pre + "norm2"], w[pre + "norm2.b"], eps), w, pre + "mlp.")
        streams.append(x.copy())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = x @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(streams)) if return_layers else logits
