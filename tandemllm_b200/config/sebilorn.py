"""The Sebilorn configuration (`"architecture": "Sebilorn"`), typed.

A decoder whose layers are listed one by one in config.json; an entry names its mixer's type, the mixer's sizes and
constants and its feed-forward (or none). Everything that can differ between models of the design is read here and
nowhere else; `to_spec()` turns it into the architecture-neutral `ModelSpec`. A key this reader does not know stops the
load with its name.

  config.json   vocab, width, norm: {eps}, embedding: {scale}, logit_softcap, layers: [{type, mixer, mlp | null}, ...]
  attention     {heads, kv_heads, dim, vdim, scale, softcap, rot: {base, dims, scaling: {factor, low, high, original}},
                mask: {size, keep_first}, kv_from}: grouped-query attention, rotary on the first `rot.dims` entries of a head
                (halves layout) with the long wavelengths slowed, values turned by their position over all their entries and
                the output turned back, capped scores, a sliding window that also keeps the first tokens; with `kv_from`
                the layer has no key and value matrices and reads the named layer's cache. Tensors l<i>.mix.{q,k,v,o}
  parallel      {left, right, left_scale, right_scale}: left a causal attention over all keys with an entry-wise sigmoid
                gate (l<i>.mix.left.{q,k,v,g,o}), right the generalized delta rule (l<i>.mix.right.{r,k,v,a,a.b,w1,w2,w0,
                g,norm,o}); the two outputs are weighed and summed
  lightning     {heads, dim, vdim, decay: [a number a head]}: linear attention with a fixed decay a head
                (l<i>.mix.{q,k,v,g,norm,o})
  mlp           {kind: dense, ff}: down(relu(up n)^2), tensors l<i>.mlp.{up,down}
  norms         layer norms with weight and bias: l<i>.norm1, l<i>.norm2, final.norm, each with `.b`
  head          its own matrix `head`; the logits are capped by logit_softcap
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

from .spec import LayerSpec, ModelSpec, PartSpec, Site

ARCHITECTURES = ("Sebilorn",)
MODEL_TYPES = ("sebilorn",)

DELTA_DECAY_RATE = math.exp(-0.5)   # the delta rule's decay a channel is exp(-DELTA_DECAY_RATE * sigmoid(.))
UNIT_KEY_EPS = 1e-6                 # added to the sum of a key's squares before the root

TOP_KEYS = {"architecture", "architectures", "model_type", "layers", "norm", "vocab", "width", "embedding", "logit_softcap"}
LAYER_KEYS = {"type", "mixer", "mlp"}
ROT_KEYS = {"base", "dims", "scaling"}
SCALING_KEYS = {"factor", "low", "high", "original"}
ATTENTION_KEYS = {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot", "mask", "kv_from"}
LEFT_KEYS = {"heads", "kv_heads", "dim", "vdim", "scale", "rot"}
RIGHT_KEYS = {"heads", "dim"}
PARALLEL_KEYS = {"left", "right", "left_scale", "right_scale"}
LIGHTNING_KEYS = {"heads", "dim", "vdim", "decay"}
MLP_KEYS = {"kind", "ff"}


def _only(d: dict, known: set, where: str) -> None:
    unknown = sorted(set(d) - known)
    if unknown:
        raise ValueError(f"Sebilorn config: {where} has key(s) this engine does not know: {', '.join(unknown)}")


def _need(d: dict, keys, where: str) -> None:
    for k in keys:
        if k not in d:
            raise ValueError(f"Sebilorn config: {where} lacks the required key {k!r}")


def _check_rot(rot, where: str) -> None:
    if rot is None:
        return
    _only(rot, ROT_KEYS, where)
    _need(rot, ("base", "dims"), where)
    if rot.get("scaling") is not None:
        _only(rot["scaling"], SCALING_KEYS, where + ".scaling")
        _need(rot["scaling"], sorted(SCALING_KEYS), where + ".scaling")


def _position(rot, dim: int) -> PartSpec:
    if not rot or int(rot["dims"]) == 0:
        return PartSpec("none", {})
    s = rot.get("scaling")
    scaling = {k: float(s[k]) for k in SCALING_KEYS} if s else None
    return PartSpec("rope_neox", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "scaling": scaling,
                                  "precise": True})


@dataclass
class SebilornLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass
class SebilornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    logit_softcap: float | None = None
    layers: list[SebilornLayer] = field(default_factory=list)
    path: str = ""

    @classmethod
    def from_dict(cls, raw: dict, path: str = "", generation: dict | None = None) -> "SebilornConfig":
        _only(raw, TOP_KEYS, "the top level")
        _need(raw, ("layers", "norm", "vocab", "width"), "the top level")
        _only(raw["norm"], {"eps"}, "norm")
        _need(raw["norm"], ("eps",), "norm")
        emb = raw.get("embedding") or {}
        _only(emb, {"scale"}, "embedding")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _only(entry, LAYER_KEYS, where)
            _need(entry, ("type", "mixer"), where)
            kind = str(entry["type"])
            m = dict(entry["mixer"])
            at = where + ".mixer"
            if kind == "attention":
                _only(m, ATTENTION_KEYS, at)
                _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), at)
                _check_rot(m.get("rot"), at + ".rot")
                if m.get("mask") is not None:
                    _only(m["mask"], {"size", "keep_first"}, at + ".mask")
                    _need(m["mask"], ("size",), at + ".mask")
            elif kind == "parallel":
                _only(m, PARALLEL_KEYS, at)
                _need(m, ("left", "right"), at)
                _only(m["left"], LEFT_KEYS, at + ".left")
                _need(m["left"], ("heads", "kv_heads", "dim", "vdim", "scale"), at + ".left")
                _check_rot(m["left"].get("rot"), at + ".left.rot")
                _only(m["right"], RIGHT_KEYS, at + ".right")
                _need(m["right"], ("heads", "dim"), at + ".right")
            elif kind == "lightning":
                _only(m, LIGHTNING_KEYS, at)
                _need(m, ("heads", "dim", "vdim", "decay"), at)
            else:
                raise ValueError(f"Sebilorn config: {where}.type {kind!r}: attention, parallel and lightning are implemented")
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                _only(mlp, MLP_KEYS, where + ".mlp")
                _need(mlp, ("kind", "ff"), where + ".mlp")
                if mlp["kind"] != "dense":
                    raise ValueError(f"Sebilorn config: {where}.mlp.kind {mlp['kind']!r}: dense is implemented")
            layers.append(SebilornLayer(kind, m, mlp))
        cap = raw.get("logit_softcap")
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                  embedding_scale=float(emb.get("scale", 1.0)), logit_softcap=float(cap) if cap else None, layers=layers,
                  path=path)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("Sebilorn config: vocab, width and the number of layers must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "attention":
                src = m.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not 0 <= src < i or self.layers[src].type != "attention" or self.layers[src].mixer.get("kv_from") is not None:
                        raise ValueError(f"Sebilorn config: layers[{i}].mixer.kv_from {src}: an earlier attention layer with "
                                         "keys and values of its own")
                    o = self.layers[src].mixer
                    if any(int(o[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
                        raise ValueError(f"Sebilorn config: layers[{i}] reads layer {src}'s keys and values, whose sizes differ")
            heads = [m] if layer.type != "parallel" else [m["left"], m["right"]]
            for h in heads:
                H, G = int(h["heads"]), int(h.get("kv_heads", h["heads"]))
                if H <= 0 or G <= 0 or H % G or int(h["dim"]) <= 0:
                    raise ValueError(f"Sebilorn config: layers[{i}]: {H} heads over {G} kv_heads of size {h['dim']}")
            if layer.type == "lightning" and len(m["decay"]) != int(m["heads"]):
                raise ValueError(f"Sebilorn config: layers[{i}]: {len(m['decay'])} decays for {m['heads']} heads")
            if layer.mlp is not None and int(layer.mlp["ff"]) <= 0:
                raise ValueError(f"Sebilorn config: layers[{i}]: mlp.ff must be positive")

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURES[0], "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale},
               "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out

    def to_spec(self) -> ModelSpec:
        eps = self.norm_eps

        def norm(name, optional=False):
            return PartSpec("layernorm", {"eps": eps, "name": name, "optional": optional})

        def kept_by(i: int) -> tuple[int | None, int]:
            """What layer i's pages must keep readable: the widest window and the most first tokens among the layer and
            the layers that read its keys and values (no window at all if one of them has none)."""
            masks = [l.mixer.get("mask") for j, l in enumerate(self.layers)
                     if l.type == "attention" and (j == i or l.mixer.get("kv_from") == i)]
            if any(k is None for k in masks):
                return None, 0
            return max(int(k["size"]) for k in masks), max(int(k.get("keep_first", 0)) for k in masks)

        def softmax_attention(m: dict, pre: str, gated: bool, rotated_values: bool, kept=None) -> PartSpec:
            rot = m.get("rot")
            mask = m.get("mask")
            names = {"q": pre + "q", "out": pre + "o"}
            shared = m.get("kv_from") is not None
            if not shared:
                names.update({"k": pre + "k", "v": pre + "v"})
            return PartSpec("attention", {
                "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
                "value_dim": int(m["vdim"]), "qk_norm": None, "position": _position(rot, int(m["dim"])),
                "scale": float(m["scale"]), "softcap": float(m["softcap"]) if m.get("softcap") else None,
                "window": int(mask["size"]) if mask else None, "keep_first": int(mask.get("keep_first", 0)) if mask else 0,
                "value_rotation": float(rot["base"]) if (rotated_values and rot) else None,
                "cache_window": kept[0] if kept else (int(mask["size"]) if mask else None),
                "cache_keep_first": kept[1] if kept else (int(mask.get("keep_first", 0)) if mask else 0),
                "entry_gate": pre + "g" if gated else None, "borrows_keys": shared,
                "weight_suffix": "", "names": names})

        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "attention":
                mixer = softmax_attention(m, "mix.", gated=False, rotated_values=True, kept=kept_by(i))
            elif layer.type == "parallel":
                r = m["right"]
                right = PartSpec("delta_rule", {
                    "heads": int(r["heads"]), "head_dim": int(r["dim"]), "eps": eps, "decay_rate": DELTA_DECAY_RATE,
                    "key_eps": UNIT_KEY_EPS,
                    "names": {k: "mix.right." + v for k, v in {
                        "r": "r", "k": "k", "v": "v", "a": "a", "a_bias": "a.b", "w1": "w1", "w2": "w2", "w0": "w0", "gate": "g",
                        "norm": "norm", "out": "o"}.items()}})
                left = softmax_attention(m["left"], "mix.left.", gated=True, rotated_values=False)
                mixer = PartSpec("weighted_sum", {"mixers": (left, right),
                                                  "weights": (float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))})
            else:
                mixer = PartSpec("decayed_linear_attention", {
                    "heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
                    "decay": tuple(float(d) for d in m["decay"]), "activation": "silu", "eps": eps,
                    "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "gate": "mix.g", "norm": "mix.norm", "out": "mix.o"}})
            if layer.mlp is None:
                ff = PartSpec("none", {})
            else:
                ff = PartSpec("dense_act", {"intermediate_size": int(layer.mlp["ff"]), "activation": "relu2",
                                            "names": {"up": "mlp.up", "down": "mlp.down"}})
            layers.append(LayerSpec(prefix=f"l{i}.", mixer=mixer, feed_forward=ff, mixer_norm=norm("norm1"),
                                    feed_forward_norm=norm("norm2") if layer.mlp is not None else None))
        sites = tuple(Site(i, cache_of=(int(l.mixer["kv_from"]) if l.type == "attention" and l.mixer.get("kv_from") is not None
                                        else None)) for i, l in enumerate(self.layers))
        return ModelSpec(
            architecture=ARCHITECTURES[0], hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers), schedule=sites,
            final_norm=PartSpec("layernorm", {"eps": eps}), embedding_name="embed", final_norm_prefix="final.norm.",
            head_name="head", embedding_scale=self.embedding_scale, logit_softcap=self.logit_softcap, name_prefixes=())
