"""The Niralix configuration (`"architecture": "Niralix"`), typed.

A decoder whose layers are listed one by one in config.json; an entry names its mixer's type, the mixer's sizes and
constants and its feed-forward (or none). Everything that can differ between models of the design is read here and
nowhere else; `to_spec()` turns it into the architecture-neutral `ModelSpec`. A key this reader does not know stops the
load with its name.

  config.json       vocab, width, norm: {eps}, logit_scale, streams, layers: [{type, mixer, mlp | null}, ...]
  stream            with `streams` = S the residual is S streams that all start as the embedded row; sublayer q of a layer
                    (1: mixer, 2: feed-forward) reads u = sum_s in[s] x_s, and its output y rewrites all streams at once,
                    x_t <- sum_s mix[s, t] x_s + out[t] y, with the tensors l<i>.hc<q>.{in,out,mix}; the last norm reads the
                    sum of the streams. Without the key: one residual, x <- x + y
  norms             RMS norms whose stored weight is the distance from one (out = (1 + w) x / rms(x)): l<i>.norm1, l<i>.norm2,
                    final.norm
  gla               mixer {heads, dim, vdim, tau}: gated linear attention with a decay a key channel, sigmoid(z)^(1 / tau),
                    z = a2 (a1 n) + a2.b; a norm a head and a silu gate; tensors l<i>.mix.{q,k,v,g,o,norm,a1,a2,a2.b}
  attention         mixer {heads, kv_heads, dim, vdim, scale, rot: {base, dims, scaling: {factor, original, fast, slow}}, v_mix}:
                    grouped-query attention over all earlier keys, biases on q, k, v and o (`.b`), rotary on the first
                    `rot.dims` entries of a head (halves layout) stretched by a ramp over the pairs; with `v_mix` every such
                    layer but the first blends its values with the first one's, (1 - l) v + l v_first, l = l<i>.mix.vmix;
                    tensors l<i>.mix.{q,k,v,o}
  latent_attention  mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims}}: attention over a cached
                    latent with interleaved rotary positions on the rot_dim part, a sink a head in the softmax and an
                    entry-wise sigmoid gate on the heads; tensors l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o}
  mlp               {kind: dense, ff}: down(silu(gate n) * up n), tensors l<i>.mlp.{gate,up,down};
                    {kind: moe, router: {experts, top}, expert: {ff}}: the `top` experts with the largest softmax scores over
                    all experts, weighed by those scores as they are; tensors l<i>.mlp.{router,e<j>.{gate,up,down}}
  head              the embedding table `embed`, times logit_scale
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .spec import LayerSpec, ModelSpec, PartSpec, plain_schedule

ARCHITECTURES = ("Niralix",)
MODEL_TYPES = ("niralix",)

NORM_WEIGHT_OFFSET = 1.0        # the design stores its norms' weights as their distance from one

TOP_KEYS = {"architecture", "architectures", "model_type", "layers", "norm", "vocab", "width", "logit_scale", "streams"}
LAYER_KEYS = {"type", "mixer", "mlp"}
GLA_KEYS = {"heads", "dim", "vdim", "tau"}
ATTENTION_KEYS = {"heads", "kv_heads", "dim", "vdim", "scale", "rot", "v_mix"}
LATENT_KEYS = {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"}
ROT_KEYS = {"base", "dims", "scaling"}
SCALING_KEYS = {"factor", "original", "fast", "slow"}
MLP_KEYS = {"kind", "ff", "router", "expert"}
CARRY_KEY = "values of the first value-mixing layer"


def _only(d: dict, known: set, where: str) -> None:
    unknown = sorted(set(d) - known)
    if unknown:
        raise ValueError(f"Niralix config: {where} has key(s) this engine does not know: {', '.join(unknown)}")


def _need(d: dict, keys, where: str) -> None:
    for k in keys:
        if k not in d:
            raise ValueError(f"Niralix config: {where} lacks the required key {k!r}")


def _check_rot(rot, where: str, scaling_allowed: bool) -> None:
    if rot is None:
        return
    _only(rot, ROT_KEYS if scaling_allowed else ROT_KEYS - {"scaling"}, where)
    _need(rot, ("base", "dims"), where)
    if rot.get("scaling") is not None:
        _only(rot["scaling"], SCALING_KEYS, where + ".scaling")
        _need(rot["scaling"], sorted(SCALING_KEYS), where + ".scaling")


@dataclass
class NiralixLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass
class NiralixConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float = 1.0
    streams: int | None = None
    layers: list[NiralixLayer] = field(default_factory=list)
    path: str = ""

    @classmethod
    def from_dict(cls, raw: dict, path: str = "", generation: dict | None = None) -> "NiralixConfig":
        _only(raw, TOP_KEYS, "the top level")
        _need(raw, ("layers", "norm", "vocab", "width"), "the top level")
        _only(raw["norm"], {"eps"}, "norm")
        _need(raw["norm"], ("eps",), "norm")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _only(entry, LAYER_KEYS, where)
            _need(entry, ("type", "mixer"), where)
            kind = str(entry["type"])
            m = dict(entry["mixer"])
            at = where + ".mixer"
            if kind == "gla":
                _only(m, GLA_KEYS, at)
                _need(m, ("heads", "dim", "vdim", "tau"), at)
            elif kind == "attention":
                _only(m, ATTENTION_KEYS, at)
                _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), at)
                _check_rot(m.get("rot"), at + ".rot", True)
            elif kind == "latent_attention":
                _only(m, LATENT_KEYS, at)
                _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"), at)
                _check_rot(m.get("rot"), at + ".rot", False)
            else:
                raise ValueError(f"Niralix config: {where}.type {kind!r}: gla, attention and latent_attention are implemented")
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                _only(mlp, MLP_KEYS, where + ".mlp")
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] == "dense":
                    _need(mlp, ("ff",), where + ".mlp")
                elif mlp["kind"] == "moe":
                    _need(mlp, ("router", "expert"), where + ".mlp")
                    _only(mlp["router"], {"experts", "top"}, where + ".mlp.router")
                    _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
                    _only(mlp["expert"], {"ff"}, where + ".mlp.expert")
                    _need(mlp["expert"], ("ff",), where + ".mlp.expert")
                else:
                    raise ValueError(f"Niralix config: {where}.mlp.kind {mlp['kind']!r}: dense and moe are implemented")
            layers.append(NiralixLayer(kind, m, mlp))
        streams = raw.get("streams")
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                  logit_scale=float(raw.get("logit_scale", 1.0)), streams=int(streams) if streams is not None else None,
                  layers=layers, path=path)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("Niralix config: vocab, width and the number of layers must be positive")
        if self.streams is not None and not 1 <= self.streams <= 8:
            raise ValueError(f"Niralix config: streams {self.streams}: 1 to 8 are implemented")
        carried = None
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            H, G = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
            if H <= 0 or G <= 0 or H % G or int(m["dim"]) < 0 or int(m["vdim"]) <= 0:
                raise ValueError(f"Niralix config: layers[{i}]: {H} heads over {G} kv_heads of sizes {m['dim']} and {m['vdim']}")
            if layer.type == "gla" and not float(m["tau"]) > 0.0:
                raise ValueError(f"Niralix config: layers[{i}].mixer.tau must be positive")
            if layer.type == "attention":
                rot = m.get("rot")
                if rot and (int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(m["dim"])):
                    raise ValueError(f"Niralix config: layers[{i}]: {rot['dims']} rotated entries of a head of {m['dim']}")
                if m.get("v_mix"):
                    sizes = (G, int(m["vdim"]))
                    if carried is not None and carried != sizes:
                        raise ValueError(f"Niralix config: layers[{i}] mixes its values with the first such layer's, whose "
                                         f"sizes differ: {sizes} against {carried}")
                    carried = carried or sizes
            if layer.type == "latent_attention":
                rot = m.get("rot")
                if rot and int(rot["dims"]) != int(m["rot_dim"]):
                    raise ValueError(f"Niralix config: layers[{i}]: rot.dims {rot['dims']} is not rot_dim {m['rot_dim']}")
            mlp = layer.mlp
            if mlp is not None and mlp["kind"] == "moe":
                E, k = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
                if not 0 < k <= E or int(mlp["expert"]["ff"]) <= 0:
                    raise ValueError(f"Niralix config: layers[{i}]: top {k} of {E} experts of {mlp['expert']['ff']}")
            elif mlp is not None and int(mlp["ff"]) <= 0:
                raise ValueError(f"Niralix config: layers[{i}]: mlp.ff must be positive")

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURES[0], "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "logit_scale": self.logit_scale,
               "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    def to_spec(self) -> ModelSpec:
        eps = self.norm_eps

        def norm(tensor: str) -> PartSpec:
            return PartSpec("rmsnorm", {"eps": eps, "tensor": tensor, "offset": NORM_WEIGHT_OFFSET})

        layers, ignored, first_mix = [], [], None
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "gla":
                mixer = PartSpec("gated_linear_attention", {
                    "heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "tau": float(m["tau"]),
                    "eps": eps,
                    "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "gate": "mix.g", "norm": "mix.norm", "a1": "mix.a1",
                              "a2": "mix.a2", "a_bias": "mix.a2.b", "out": "mix.o"}})
            elif layer.type == "attention":
                rot = m.get("rot")
                if rot and int(rot["dims"]) > 0:
                    s = rot.get("scaling")
                    position = PartSpec("rope_neox", {
                        "theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "precise": True,
                        "scaling": {k: float(s[k]) for k in SCALING_KEYS} if s else None})
                else:
                    position = PartSpec("none", {})
                carry = None
                if not m.get("v_mix"):
                    ignored.append(f"l{i}.mix.vmix")      # a blend weight stored for a layer that does not blend: never read
                if m.get("v_mix"):
                    # the first such layer's own blend weight is stored and never used
                    carry = {"key": CARRY_KEY, "blend": "mix.vmix" if first_mix is not None else None}
                    if first_mix is None:
                        first_mix = i
                        ignored.append(f"l{i}.mix.vmix")
                mixer = PartSpec("attention", {
                    "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
                    "value_dim": int(m["vdim"]), "qk_norm": None, "position": position, "scale": float(m["scale"]),
                    "bias": True, "bias_suffix": ".b", "value_carry": carry, "weight_suffix": "",
                    "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "out": "mix.o"}})
            else:
                rot = m.get("rot")
                mixer = PartSpec("latent_attention", {
                    "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
                    "value_dim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]),
                    "scale": float(m["scale"]), "window": None, "eps": eps,
                    "position": PartSpec("rope_pairs", {"theta": float(rot["base"]) if rot else 1.0,
                                                        "rotary_dim": int(rot["dims"]) if rot else 0}),
                    "names": {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq", "dkv": "mix.dkv",
                              "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "sink": "mix.sink", "gate": "mix.g",
                              "out": "mix.o"}})
            mlp = layer.mlp
            if mlp is None:
                ff = PartSpec("none", {})
                # what a folder may still hold for the sublayer that is not there
                ignored += [f"l{i}.norm2"] + [f"l{i}.hc2.{x}" for x in ("in", "out", "mix")]
            elif mlp["kind"] == "dense":
                ff = PartSpec("swiglu", {"intermediate_size": int(mlp["ff"]), "activation": "silu", "weight_suffix": "",
                                         "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
            else:
                ff = PartSpec("sigmoid_topk_experts", {
                    "num_experts": int(mlp["router"]["experts"]), "top_k": int(mlp["router"]["top"]),
                    "intermediate_size": int(mlp["expert"]["ff"]), "expert_bias": False, "normalize": False, "scale": 1.0,
                    "scoring": "softmax", "activation": "silu", "weight_suffix": "", "expert_separator": "",
                    "names": {"router": "mlp.router", "experts": "mlp.e", "gate": "gate", "up": "up", "down": "down"}})
            hyper = None
            if self.streams is not None:
                hyper = {"streams": self.streams, "feed_forward": mlp is not None,
                         "names": {"in": "in", "out": "out", "mix": "mix"}}
            layers.append(LayerSpec(prefix=f"l{i}.", mixer=mixer, feed_forward=ff, mixer_norm=norm("norm1"),
                                    feed_forward_norm=norm("norm2") if mlp is not None else None,
                                    arrangement="hyper_connections" if hyper else "prenorm_residual", arrangement_params=hyper))
        return ModelSpec(
            architecture=ARCHITECTURES[0], hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            schedule=plain_schedule(len(layers)), final_norm=norm("norm"), embedding_name="embed", final_norm_prefix="final.",
            head_name=None, logit_scale=self.logit_scale, streams=self.streams or 0, ignored_names=tuple(ignored),
            name_prefixes=())
