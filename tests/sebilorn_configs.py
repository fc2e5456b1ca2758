"""Tiny Sebilorn configurations of the tests (config.json dictionaries), their random weights and prompts.

b1: sizes no kernel is tuned for (an odd vocabulary, a width that is no multiple of 8): an attention layer whose values are
    narrower than its keys, half of a head rotated, a window of 5 that keeps 2 first tokens; a layer that borrows its keys
    and values through a wider window that keeps 3; a parallel layer whose left values are wider than its keys and whose
    delta rule has heads of 24; a lightning layer without a feed-forward; a second owner of keys with one KV head.
b2: sizes the tensor-core kernels take (multiples of 8, heads of 64 and 32), windows of 70 and 48, a borrower two layers
    behind its owner, a lightning layer first.
b3: what another model makes equal or absent: as many KV heads as heads, no kept first tokens, no cap on scores or logits,
    no frequency scaling, an attention layer without a mask at all, an embedding scale of 1, one head, rot.dims below dim
    in the left mixer, weights of 1 on both sides of the parallel layer.
b4: large heads: keys of 128 with values of 256, a delta rule of 160 keys a head (more than a warp's lanes hold in 16s,
    filled up to the next power of two), a lightning layer of 40 keys and 72 values, a window of exactly four pages.
The decay's inner size is no key of the configuration: the stored `w1` says it (RANKS).
"""

from __future__ import annotations

import json
import math
import os

import torch


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def _mlp(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def _attn(heads, kv, dim, vdim, scale, rot, mask=None, softcap=None, kv_from=None, ff=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if mask:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if softcap:
        m["softcap"] = softcap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": _mlp(ff)}


def _parallel(left, right, ls, rs, ff=None):
    l = {"heads": left[0], "kv_heads": left[1], "dim": left[2], "vdim": left[3], "scale": left[4], "rot": left[5]}
    return {"type": "parallel", "mixer": {"left": l, "right": {"heads": right[0], "dim": right[1]}, "left_scale": ls,
                                          "right_scale": rs}, "mlp": _mlp(ff)}


def _lightning(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": _mlp(ff)}


B1 = {"architecture": "Sebilorn", "vocab": 97, "width": 44, "norm": {"eps": 1e-4}, "embedding": {"scale": 3.5},
      "logit_softcap": 9.0,
      "layers": [_attn(4, 2, 16, 8, 0.31, _rot(10000.0, 8, (4.0, 1.0, 3.0, 64)), (5, 2), 7.0, ff=80),
                 _attn(4, 2, 16, 8, 0.2, _rot(10000.0, 8, (4.0, 1.0, 3.0, 64)), (9, 3), 11.0, kv_from=0, ff=None),
                 _parallel((3, 3, 12, 20, 0.4, _rot(500.0, 4)), (2, 24), 1.3, 0.4, ff=52),
                 _lightning(3, 8, 24, [0.5, 0.9, 0.97]),
                 _attn(6, 1, 8, 6, 0.5, _rot(77.0, 8), (1, 0), 30.0, ff=36)]}
B2 = {"architecture": "Sebilorn", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.3},
      "logit_softcap": 20.0,
      "layers": [_lightning(2, 64, 64, [0.8, 0.995], ff=192),
                 _attn(4, 2, 64, 64, 0.12, _rot(100000.0, 64, (8.0, 1.0, 4.0, 256)), (70, 4), 40.0, ff=256),
                 _parallel((8, 4, 32, 32, 0.17, _rot(10000.0, 32)), (2, 64), 0.7, 0.6, ff=128),
                 _attn(4, 2, 64, 64, 0.1, _rot(100000.0, 64, (8.0, 1.0, 4.0, 256)), (48, 17), 25.0, kv_from=1, ff=128)]}
B3 = {"architecture": "Sebilorn", "vocab": 130, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
      "layers": [_parallel((2, 2, 32, 32, 0.2, _rot(1000.0, 16)), (1, 32), 1.0, 1.0, ff=96),
                 _attn(2, 2, 32, 16, 0.15, _rot(300.0, 32), None, None, ff=72),
                 _attn(1, 1, 64, 64, 0.1, _rot(5000.0, 32), (33, 0), None, ff=None),
                 _lightning(1, 16, 16, [0.93], ff=40)]}
B4 = {"architecture": "Sebilorn", "vocab": 211, "width": 96, "norm": {"eps": 3e-6}, "embedding": {"scale": 6.0},
      "logit_softcap": 30.0,
      "layers": [_attn(2, 1, 128, 256, 0.07, _rot(50000.0, 96, (2.0, 1.0, 2.0, 128)), (64, 5), 15.0, ff=120),
                 _parallel((4, 2, 64, 128, 0.11, _rot(2000.0, 64)), (2, 160), 0.9, 1.1, ff=None),
                 _lightning(3, 40, 72, [0.7, 0.95, 0.999], ff=88)]}
CONFIGS = {"b1": B1, "b2": B2, "b3": B3, "b4": B4}
SEEDS = {"b1": 21, "b2": 22, "b3": 23, "b4": 24}
RANKS = {"b1": 5, "b2": 16, "b3": 8, "b4": 12}


def tensor_shapes(cfg: dict, rank: int) -> dict[str, tuple]:
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "head": (cfg["vocab"], cfg["width"])}

    def norm(name):
        out[name], out[name + ".b"] = (W,), (W,)

    def attention(p, m, gated):
        out[p + "q"] = (m["heads"] * m["dim"], W)
        if m.get("kv_from") is None:
            out[p + "k"] = (m["kv_heads"] * m["dim"], W)
            out[p + "v"] = (m["kv_heads"] * m["vdim"], W)
        if gated:
            out[p + "g"] = (m["heads"] * m["vdim"], W)
        out[p + "o"] = (W, m["heads"] * m["vdim"])

    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        norm(p + "norm1")
        if layer["type"] == "attention":
            attention(p + "mix.", m, False)
        elif layer["type"] == "parallel":
            attention(p + "mix.left.", m["left"], True)
            I, q = m["right"]["heads"] * m["right"]["dim"], p + "mix.right."
            for x in ("r", "k", "v", "a", "g"):
                out[q + x] = (I, W)
            out[q + "a.b"], out[q + "w0"], out[q + "norm"] = (I,), (I,), (I,)
            out[q + "w1"], out[q + "w2"], out[q + "o"] = (rank, W), (I, rank), (W, I)
        else:
            out[p + "mix.q"] = out[p + "mix.k"] = (m["heads"] * m["dim"], W)
            out[p + "mix.v"] = out[p + "mix.g"] = (m["heads"] * m["vdim"], W)
            out[p + "mix.norm"] = (m["heads"] * m["vdim"],)
            out[p + "mix.o"] = (W, m["heads"] * m["vdim"])
        if layer["mlp"] is not None:
            norm(p + "norm2")
            out[p + "mlp.up"] = (layer["mlp"]["ff"], W)
            out[p + "mlp.down"] = (W, layer["mlp"]["ff"])
    norm("final.norm")
    return out


def random_weights(cfg: dict, rank: int, seed: int, bf16_exact: bool = True) -> dict[str, torch.Tensor]:
    """32-bit random weights by stored name; with `bf16_exact` every value is a bfloat16 value, so that the engine in
    either precision and the plain model read the same numbers."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for key, shape in tensor_shapes(cfg, rank).items():
        t = torch.randn(shape, generator=g)
        if key == "embed":
            t = t * (0.8 / float(cfg["embedding"]["scale"]))
        elif key.endswith(".b") or key.endswith(".w0"):
            t = 0.3 * t
        elif "norm" in key:
            t = 1.0 + 0.2 * t
        elif key.endswith(".w2"):
            t = t * 0.5
        else:
            t = t * (shape[1] ** -0.5)
        out[key] = t.to(torch.bfloat16).float() if bf16_exact else t
    return out


def weights(name: str, bf16_exact: bool = True) -> dict[str, torch.Tensor]:
    return random_weights(CONFIGS[name], RANKS[name], SEEDS[name], bf16_exact)


def tokens(name: str, n: int, seed: int = 0) -> list[int]:
    g = torch.Generator().manual_seed(seed * 7919 + n)
    return torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist()


def write_folder(folder: str, name: str) -> str:
    """config.json and model.safetensors (bfloat16, as the design stores them) of the tiny model `name`."""
    from tandemllm_b200.weights.safetensors_io import write_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(CONFIGS[name], f)
    write_file(os.path.join(folder, "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in weights(name).items()})
    return folder


def random_config(seed: int) -> tuple[dict, int]:
    """A model drawn at random: layer order, sizes from a few numbers up, with and without masks, caps, scalings, kept
    first tokens, borrowed keys and feed-forwards. Returns (config, the decay's inner size)."""
    import random
    r = random.Random(seed)
    W = r.choice([24, 40, 64, 72])
    layers, owners = [], []
    for i in range(r.randint(2, 5)):
        kind = r.choice(["attention", "attention", "parallel", "lightning"])
        ff = r.choice([None, 16, 40, 64])
        if kind == "attention":
            if owners and r.random() < 0.4:
                j = r.choice(owners)
                src = layers[j]["mixer"]
                mask = r.choice([None, (r.randint(1, 40), r.randint(0, 6))])
                layers.append(_attn(src["heads"], src["kv_heads"], src["dim"], src["vdim"], r.uniform(0.05, 0.4), src["rot"], mask,
                                    r.choice([None, 5.0, 50.0]), kv_from=j, ff=ff))
                continue
            kv = r.choice([1, 2, 3])
            dim, vdim = r.choice([8, 16, 24, 32, 64]), r.choice([4, 8, 16, 32, 48])
            scaling = r.choice([None, (r.choice([2.0, 8.0]), 1.0, r.choice([2.0, 4.0]), r.choice([32, 128]))])
            mask = r.choice([None, (r.randint(1, 40), r.randint(0, 6))])
            owners.append(i)
            layers.append(_attn(kv * r.choice([1, 2, 4]), kv, dim, vdim, r.uniform(0.05, 0.4),
                                _rot(r.choice([100.0, 10000.0]), r.choice([d for d in (2, 4, 8, 16, 32, 64) if d <= dim]), scaling),
                                mask, r.choice([None, 5.0, 50.0]), ff=ff))
        elif kind == "parallel":
            kv = r.choice([1, 2])
            dim = r.choice([8, 16, 32])
            layers.append(_parallel((kv * r.choice([1, 2]), kv, dim, r.choice([8, 16, 24]), r.uniform(0.05, 0.4),
                                     _rot(r.choice([100.0, 10000.0]), r.choice([d for d in (2, 8, 16, 32) if d <= dim]))),
                                    (r.choice([1, 2, 3]), r.choice([4, 16, 20, 64])), r.uniform(0.3, 1.5), r.uniform(0.3, 1.5), ff=ff))
        else:
            H = r.choice([1, 2, 4])
            layers.append(_lightning(H, r.choice([4, 16, 24, 64]), r.choice([8, 16, 40]),
                                     [math.exp(-r.uniform(0.001, 0.7)) for _ in range(H)], ff=ff))
    cfg = {"architecture": "Sebilorn", "vocab": r.choice([50, 97, 128]), "width": W, "norm": {"eps": r.choice([1e-5, 1e-4])},
           "embedding": {"scale": r.choice([1.0, 4.0])}, "layers": layers}
    if r.random() < 0.6:
        cfg["logit_softcap"] = r.choice([8.0, 30.0])
    return cfg, r.choice([3, 8, 16])
