"""Tiny Niralix configurations of the tests (config.json dictionaries), their random weights and prompts.

n1: sizes no kernel is tuned for (an odd vocabulary, a width that is no multiple of 8, three streams): a gla layer with values
    narrower than its keys, an attention layer with half a head rotated and values of 8 under keys of 16 that is the first
    value-mixing layer, a latent-attention layer, a routed feed-forward with top 2 of 5, a second value-mixing layer without
    a feed-forward.
n2: sizes the tensor-core kernels take (heads of 64, a latent of 64), two streams, routed experts top 3 of 8, attention
    first and last with value mixing, a gla layer of 64 x 64.
n3: what another model makes equal, 1 or absent: no `streams` key (one plain residual), as many KV heads as heads, one head,
    no frequency stretch, no rotation at all in one attention layer, no value mixing, top 1 of 2 experts, a logit scale of 1,
    a latent layer whose unrotated part is smaller than its rotated part, tau 1.
n4: large heads and one stream with hyper-connection weights: keys of 128 with values of 64, a gla layer of 40 keys and 72 values
    (filled up to the next power of two), rot.dims equal to dim, a stretch whose ramp covers every pair, three value-mixing
    layers.
The decay's inner size is no key of the configuration: the stored `a1` says it (RANKS).
"""

from __future__ import annotations

import json
import os

import torch


def _mlp(ff):
    if ff is None:
        return None
    if isinstance(ff, tuple):
        return {"kind": "moe", "router": {"experts": ff[0], "top": ff[1]}, "expert": {"ff": ff[2]}}
    return {"kind": "dense", "ff": ff}


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _gla(heads, dim, vdim, tau, ff=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": _mlp(ff)}


def _attn(heads, kv, dim, vdim, scale, rot, v_mix=False, ff=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = rot
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m, "mlp": _mlp(ff)}


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, ff=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim}}, "mlp": _mlp(ff)}


N1 = {"architecture": "Niralix", "vocab": 97, "width": 44, "norm": {"eps": 1e-4}, "logit_scale": 0.7, "streams": 3,
      "layers": [_gla(3, 8, 6, 4.0, ff=80),
                 _attn(4, 2, 16, 8, 0.31, _rot(10000.0, 8, (4.0, 64, 8.0, 2.0)), v_mix=True, ff=(5, 2, 24)),
                 _latent(3, 12, 4, 10, 20, 14, 0.2, 300.0, ff=52),
                 _attn(2, 2, 8, 8, 0.4, _rot(77.0, 8), v_mix=True, ff=None)]}
N2 = {"architecture": "Niralix", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.25, "streams": 2,
      "layers": [_attn(4, 2, 64, 64, 0.12, _rot(100000.0, 64, (8.0, 256, 16.0, 1.0)), v_mix=True, ff=256),
                 _gla(2, 64, 64, 16.0, ff=(8, 3, 64)),
                 _latent(4, 64, 32, 64, 64, 48, 0.1, 10000.0, ff=192),
                 _attn(8, 2, 64, 64, 0.1, _rot(100000.0, 32, (8.0, 256, 16.0, 1.0)), v_mix=True, ff=(8, 3, 64))]}
N3 = {"architecture": "Niralix", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
      "layers": [_latent(1, 8, 16, 24, 16, 8, 0.2, 1000.0, ff=(2, 1, 40)),
                 _attn(2, 2, 32, 16, 0.15, _rot(300.0, 16), ff=72),
                 _gla(1, 16, 16, 1.0, ff=None),
                 _attn(1, 1, 64, 64, 0.1, None, ff=40)]}
N4 = {"architecture": "Niralix", "vocab": 211, "width": 96, "norm": {"eps": 3e-6}, "logit_scale": 1.5, "streams": 1,
      "layers": [_attn(2, 1, 128, 64, 0.07, _rot(50000.0, 128, (2.0, 128, 1e9, 1e-9)), v_mix=True, ff=120),
                 _gla(3, 40, 72, 8.0, ff=88),
                 _attn(4, 1, 32, 64, 0.2, _rot(2000.0, 32), v_mix=True, ff=None),
                 _attn(1, 1, 16, 64, 0.3, _rot(2000.0, 2), v_mix=True, ff=(4, 4, 16))]}
CONFIGS = {"n1": N1, "n2": N2, "n3": N3, "n4": N4}
SEEDS = {"n1": 31, "n2": 32, "n3": 33, "n4": 34}
RANKS = {"n1": 5, "n2": 16, "n3": 8, "n4": 12}


def tensor_shapes(cfg: dict, rank: int) -> dict[str, tuple]:
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],)}
    S = cfg.get("streams")
    first_mix_seen = False
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        out[f"l{i}.norm1"] = (W,)
        subs = [1]
        if layer["type"] == "gla":
            I = m["heads"] * m["dim"]
            out[p + "q"] = out[p + "k"] = (I, W)
            out[p + "v"] = out[p + "g"] = (m["heads"] * m["vdim"], W)
            out[p + "o"] = (W, m["heads"] * m["vdim"])
            out[p + "norm"] = (m["vdim"],)
            out[p + "a1"], out[p + "a2"], out[p + "a2.b"] = (rank, W), (I, rank), (I,)
        elif layer["type"] == "attention":
            sizes = {"q": m["heads"] * m["dim"], "k": m["kv_heads"] * m["dim"], "v": m["kv_heads"] * m["vdim"]}
            for x, n in sizes.items():
                out[p + x], out[p + x + ".b"] = (n, W), (n,)
            out[p + "o"], out[p + "o.b"] = (W, m["heads"] * m["vdim"]), (W,)
            if m.get("v_mix"):
                out[p + "vmix"] = ()
        else:
            H, L = m["heads"], m["kv_rank"]
            out[p + "dq"], out[p + "dq.norm"] = (m["q_rank"], W), (m["q_rank"],)
            out[p + "uq"] = (H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            out[p + "dkv"], out[p + "dkv.norm"] = (L + m["rot_dim"], W), (L,)
            out[p + "uk"], out[p + "uv"] = (H * m["dim"], L), (H * m["vdim"], L)
            out[p + "sink"] = (H,)
            out[p + "g"], out[p + "o"] = (H * m["vdim"], W), (W, H * m["vdim"])
        mlp = layer["mlp"]
        if mlp is not None:
            subs.append(2)
            out[f"l{i}.norm2"] = (W,)
            q = f"l{i}.mlp."
            if mlp["kind"] == "dense":
                out[q + "gate"] = out[q + "up"] = (mlp["ff"], W)
                out[q + "down"] = (W, mlp["ff"])
            else:
                out[q + "router"] = (mlp["router"]["experts"], W)
                for e in range(mlp["router"]["experts"]):
                    out[f"{q}e{e}.gate"] = out[f"{q}e{e}.up"] = (mlp["expert"]["ff"], W)
                    out[f"{q}e{e}.down"] = (W, mlp["expert"]["ff"])
        if S:
            for s in subs:
                out[f"l{i}.hc{s}.in"], out[f"l{i}.hc{s}.out"], out[f"l{i}.hc{s}.mix"] = (S,), (S,), (S, S)
    return out


def random_weights(cfg: dict, rank: int, seed: int, bf16_exact: bool = True) -> dict[str, torch.Tensor]:
    """32-bit random weights by stored name; with `bf16_exact` every value is a bfloat16 value, so that the engine in
    either precision and the plain model read the same numbers."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for key, shape in tensor_shapes(cfg, rank).items():
        t = torch.randn(shape, generator=g)
        last = key.rsplit(".", 1)[-1]
        if key == "embed":
            t = t * 0.8
        elif key.endswith(".mix.norm") or key.endswith("dq.norm") or key.endswith("dkv.norm"):
            t = 1.0 + 0.2 * t                   # plain weights
        elif "norm" in last:
            t = 0.2 * t                         # stored around zero
        elif ".hc" in key:
            if last == "mix":
                t = torch.eye(shape[0]) + 0.25 * t
            elif last == "in":
                t = 1.0 / shape[0] + 0.3 * t
            else:
                t = 0.8 + 0.3 * t
        elif last == "vmix":
            t = torch.sigmoid(t)
        elif last == "sink":
            t = 1.5 * t
        elif last == "b":
            t = 0.3 * t + (1.5 if key.endswith("a2.b") else 0.0)       # decays mostly near one, some far from it
        elif last == "a2":
            t = t * 0.8
        elif last == "router":
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
    """A model drawn at random: layer order, sizes from a few numbers up, with and without streams, stretches, value mixing
    and feed-forwards. Returns (config, the decay's inner size)."""
    import random
    r = random.Random(seed)
    W = r.choice([24, 36, 40, 50, 64, 72, 100])
    mixing = None          # (kv heads, vdim) that every value-mixing layer shares
    layers = []
    for _ in range(r.randint(2, 5)):
        kind = r.choice(["attention", "attention", "gla", "latent_attention"])
        ff = r.choice([None, 16, 40, 64, (r.choice([2, 3, 6]), 1, 16), (4, r.choice([2, 4]), 24)])
        if kind == "attention":
            kv, vdim = r.choice([1, 2, 3]), r.choice([4, 8, 16, 32, 48])
            v_mix = r.random() < 0.6
            if v_mix:
                mixing = mixing or (kv, vdim)
                kv, vdim = mixing
            dim = r.choice([8, 16, 24, 32, 64])
            dims = r.choice([d for d in (2, 4, 8, 16, 32, 64) if d <= dim])
            scaling = r.choice([None, (r.choice([2.0, 8.0]), r.choice([32, 128]), r.choice([4.0, 32.0]), r.choice([0.5, 1.0]))])
            rot = r.choice([None, _rot(r.choice([100.0, 10000.0]), dims, scaling), _rot(r.choice([100.0, 10000.0]), dims, scaling)])
            layers.append(_attn(kv * r.choice([1, 2, 4]), kv, dim, vdim, r.uniform(0.05, 0.4), rot, v_mix, ff))
        elif kind == "gla":
            layers.append(_gla(r.choice([1, 2, 4]), r.choice([4, 16, 24, 64]), r.choice([8, 16, 40]), r.choice([1.0, 4.0, 16.0]), ff))
        else:
            rot_dim = r.choice([2, 4, 8, 16])
            layers.append(_latent(r.choice([1, 2, 3]), r.choice([4, 8, 12, 32]), rot_dim, r.choice([8, 16, 24]),
                                  r.choice([8, 20, 32, 64]), r.choice([6, 16, 24]), r.uniform(0.05, 0.4),
                                  r.choice([100.0, 10000.0]), ff))
    cfg = {"architecture": "Niralix", "vocab": r.choice([50, 131, 256]), "width": W, "norm": {"eps": r.choice([1e-6, 1e-4])},
           "logit_scale": r.choice([1.0, 0.3, 2.0]), "layers": layers}
    streams = r.choice([None, 1, 2, 4])
    if streams:
        cfg["streams"] = streams
    return cfg, r.choice([3, 8, 16])
