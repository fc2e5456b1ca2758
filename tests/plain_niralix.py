"""The plain Niralix: every mechanism as a slow function of its own, in 64-bit numpy, over one whole sequence.

It shares nothing with the engine: it reads a configuration dictionary (the keys of config.json) and a dictionary of
arrays by tensor name, and runs the sequence position by position where a mechanism is recurrent and as dense
[T, T] tables where it is attention. The tests hold the engine's parts and whole models to it.

Notation: n is a normed row, W is stored [out, in] and applied as W n, T tokens at positions 0..T-1.
"""

from __future__ import annotations

import math

import numpy as np

RAMP_MAGNITUDE_SLOPE = 0.1        # cosines and sines of a stretched rotation are multiplied by 1 + slope * ln(factor)
RAMP_MIN_WIDTH = 0.001


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def softmax(z):
    e = np.exp(z - z.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def offset_norm(x, w, eps):
    """The layers' and the model's norm: the weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    return unit_rms(x, eps) * w


# ---- rotations ----

def stretched_frequencies(base: float, dims: int, scaling: dict | None) -> tuple[np.ndarray, float]:
    """(f_i for i < dims / 2, the factor on cosines and sines). f_i = base^(-2i/dims); with `scaling` = {factor, original,
    fast, slow}: d(t) = dims ln(original / (2 pi t)) / (2 ln base); pairs below d(fast) keep f_i, pairs above d(slow) turn
    `factor` times slower, and a ramp blends in between."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def d(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(scaling["fast"]))), 0)
    hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
    out = f.copy()
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, RAMP_MIN_WIDTH), 0.0), 1.0)
        out[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
    return out, RAMP_MAGNITUDE_SLOPE * math.log(factor) + 1.0


def rotate_halves(x: np.ndarray, positions: np.ndarray, freqs: np.ndarray, magnitude: float = 1.0) -> np.ndarray:
    """x [T, heads, D]: entry i and entry i + d/2 (d = 2 len(freqs) <= D) are a pair that turns by p * f_i; entries from d on pass."""
    half = len(freqs)
    a = positions[:, None, None].astype(np.float64) * freqs[None, None, :]
    c, s = np.cos(a) * magnitude, np.sin(a) * magnitude
    out = x.copy()
    u, v = x[..., :half], x[..., half:2 * half]
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


def rotate_neighbours(x: np.ndarray, positions: np.ndarray, freqs: np.ndarray) -> np.ndarray:
    """x [T, heads, D]: entries 2i and 2i + 1 (i < len(freqs)) are a pair that turns by p * f_i; the rest pass."""
    n = len(freqs)
    a = positions[:, None, None].astype(np.float64) * freqs[None, None, :]
    c, s = np.cos(a), np.sin(a)
    out = x.copy()
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


# ---- mixers ----

def gla_decay(n, m: dict, w: dict, pre: str) -> np.ndarray:
    """[T, heads, dim]: sigmoid(z)^(1 / tau), z from two small products and a bias."""
    z = (n @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    return (sigmoid(z) ** (1.0 / float(m["tau"]))).reshape(n.shape[0], int(m["heads"]), int(m["dim"]))


def mixer_gla(n, m: dict, w: dict, pre: str, eps: float, state=None, return_state: bool = False):
    T = n.shape[0]
    H, D, VD = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (n @ w[pre + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (n @ w[pre + "k"].T).reshape(T, H, D)
    v = (n @ w[pre + "v"].T).reshape(T, H, VD)
    alpha = gla_decay(n, m, w, pre)
    S = np.zeros((H, D, VD)) if state is None else state.copy()
    o = np.zeros((T, H, VD))
    for t in range(T):
        for h in range(H):
            S[h] = alpha[t, h][:, None] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    o = plain_norm(o, w[pre + "norm"], eps).reshape(T, H * VD)
    out = (o * silu(n @ w[pre + "g"].T)) @ w[pre + "o"].T
    return (out, S) if return_state else out


def attention_values(n, m: dict, w: dict, pre: str) -> np.ndarray:
    """[T, kv_heads, vdim]: what the v matrix and its bias make of the rows, before any mixing."""
    return (n @ w[pre + "v"].T + w[pre + "v.b"]).reshape(n.shape[0], int(m["kv_heads"]), int(m["vdim"]))


def mixer_attention(n, m: dict, w: dict, pre: str, v_first=None) -> np.ndarray:
    """`v_first`: the values of the first value-mixing layer for the same tokens; None in that layer itself and in layers
    that do not mix."""
    T = n.shape[0]
    H, G, D, VD = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = np.arange(T)
    q = (n @ w[pre + "q"].T + w[pre + "q.b"]).reshape(T, H, D)
    k = (n @ w[pre + "k"].T + w[pre + "k.b"]).reshape(T, G, D)
    v = attention_values(n, m, w, pre)
    if v_first is not None:
        lam = float(w[pre + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    rot = m.get("rot")
    if rot:
        f, mag = stretched_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"))
        q, k = rotate_halves(q, pos, f, mag), rotate_halves(k, pos, f, mag)
    out = np.zeros((T, H, VD))
    causal = pos[None, :] <= pos[:, None]
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * float(m["scale"])
        s = np.where(causal, s, -np.inf)
        out[:, h] = softmax(s) @ v[:, g]
    return out.reshape(T, H * VD) @ w[pre + "o"].T + w[pre + "o.b"]


def mixer_latent_attention(n, m: dict, w: dict, pre: str, eps: float) -> np.ndarray:
    T = n.shape[0]
    H, D, R, VD, L = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = np.arange(T)
    rot = m["rot"]
    f = np.array([float(rot["base"]) ** (-2.0 * i / int(rot["dims"])) for i in range(int(rot["dims"]) // 2)])
    cq = plain_norm(n @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
    q = (cq @ w[pre + "uq"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_neighbours(q[..., D:], pos, f)
    down = n @ w[pre + "dkv"].T
    c = plain_norm(down[:, :L], w[pre + "dkv.norm"], eps)
    k_rot = rotate_neighbours(down[:, None, L:], pos, f)[:, 0]
    k_plain = (c @ w[pre + "uk"].T).reshape(T, H, D)
    v = (c @ w[pre + "uv"].T).reshape(T, H, VD)
    out = np.zeros((T, H, VD))
    causal = pos[None, :] <= pos[:, None]
    for h in range(H):
        s = (q_plain[:, h] @ k_plain[:, h].T + q_rot[:, h] @ k_rot.T) * float(m["scale"])
        s = np.where(causal, s, -np.inf)
        sink = float(w[pre + "sink"][h])
        top = np.maximum(s.max(-1, keepdims=True), sink)
        e = np.exp(s - top)
        p = e / (e.sum(-1, keepdims=True) + np.exp(sink - top))      # the sink counts once, has no key and no value
        out[:, h] = p @ v[:, h]
    gate = sigmoid(n @ w[pre + "g"].T)
    return (out.reshape(T, H * VD) * gate) @ w[pre + "o"].T


# ---- feed-forwards ----

def dense_gated(n, w: dict, pre: str) -> np.ndarray:
    return (silu(n @ w[pre + "gate"].T) * (n @ w[pre + "up"].T)) @ w[pre + "down"].T


def routed_experts(n, mlp: dict, w: dict, pre: str, return_choice: bool = False):
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    s = softmax(n @ w[pre + "router"].T)
    out = np.zeros((n.shape[0], w[pre + "e0.down"].shape[0]))
    choice = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    for t in range(n.shape[0]):
        for e in choice[t]:
            out[t] += s[t, e] * dense_gated(n[t:t + 1], w, f"{pre}e{e}.")[0]      # the scores as they are, not renormalized
    return (out, choice) if return_choice else out


def feed_forward(n, mlp: dict, w: dict, pre: str) -> np.ndarray:
    return dense_gated(n, w, pre) if mlp["kind"] == "dense" else routed_experts(n, mlp, w, pre)


# ---- the stream ----

def hyper_read(streams: np.ndarray, w_in: np.ndarray) -> np.ndarray:
    """streams [S, T, W] -> what a sublayer's norm reads: the streams weighed and summed."""
    return np.tensordot(w_in, streams, axes=(0, 0))


def hyper_write(streams: np.ndarray, y: np.ndarray, mix: np.ndarray, w_out: np.ndarray) -> np.ndarray:
    """All streams at once from the old ones: new_t = sum_s mix[s, t] old_s + w_out[t] y."""
    return np.einsum("st,snw->tnw", mix, streams) + w_out[:, None, None] * y[None]


def forward(config: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence; with `return_layers` also the stream (the sum of the streams) after every layer."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    S = config.get("streams")
    x = w["embed"][np.asarray(tokens)]
    streams = np.stack([x] * int(S)) if S else None
    layers, v_first = [], None
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]

        def mixer(n):
            nonlocal v_first
            if layer["type"] == "gla":
                return mixer_gla(n, m, w, pre + "mix.", eps)
            if layer["type"] == "latent_attention":
                return mixer_latent_attention(n, m, w, pre + "mix.", eps)
            if layer["type"] != "attention":
                raise ValueError(layer["type"])
            if m.get("v_mix") and v_first is None:
                v_first = attention_values(n, m, w, pre + "mix.")
                return mixer_attention(n, m, w, pre + "mix.")
            return mixer_attention(n, m, w, pre + "mix.", v_first if m.get("v_mix") else None)

        subs = [("1", mixer)]
        if layer.get("mlp"):
            subs.append(("2", lambda n: feed_forward(n, layer["mlp"], w, pre + "mlp.")))
        for q, fn in subs:
            if streams is None:
                x = x + fn(offset_norm(x, w[f"{pre}norm{q}"], eps))
            else:
                u = hyper_read(streams, w[f"{pre}hc{q}.in"])
                y = fn(offset_norm(u, w[f"{pre}norm{q}"], eps))
                streams = hyper_write(streams, y, w[f"{pre}hc{q}.mix"], w[f"{pre}hc{q}.out"])
        if streams is not None:
            x = streams.sum(0)
        layers.append(x.copy())
    logits = offset_norm(x, w["final.norm"], eps) @ w["embed"].T * float(config.get("logit_scale", 1.0))
    return (logits, np.stack(layers)) if return_layers else logits
