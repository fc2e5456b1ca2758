"""How a layer's parts are arranged, and a layer built from a `LayerSpec`.

`prenorm_residual` is the pre-norm block with two residual adds (engine/models/lfm2_moe/ref.py:231-239):

    n = norm_m(h);  h = h + mixer(n);  n = norm_f(h);  h = h + feed_forward(n)

A residual add is fused with the norm that follows it, so a layer receives the previous branch's output as
`pending` (not yet added to the residual stream), and returns its own feed-forward output the same way.

`sandwich_norm_residual` norms every sublayer before and after:

    h = h + norm_mb(mixer(norm_m(h)));  h = h + norm_fb(feed_forward(norm_f(h)))

The norm behind a branch, the residual add and the norm in front of the next sublayer are one kernel where the next
sublayer is in the same layer (`add_normed(..., then=next norm)`); a layer hands nothing pending to the next one, so
that whatever a run order adds to the stream between two layers meets a complete residual.

`hyper_connections` carries several residual streams x_1 .. x_S [S, rows, hidden] instead of one. Sublayer q of a layer
(1: mixer, 2: feed-forward) has three small tensors, `<prefix>hc<q>.in` [S], `.out` [S] and `.mix` [S, S] (indexed [from, to]):

    u = sum_s in[s] x_s;  y = sublayer(norm(u));  x_t <- sum_s mix[s, t] x_s + out[t] y   (all streams at once from the old ones)

What a sublayer leaves is not added by itself here either: it goes on as an `ops.StreamUpdate` (y with its `mix` and `out`),
and the norm kernel of the next sublayer rewrites the streams, forms the next u with its own `in` and norms it, all in one
pass over the row. The model starts every stream from the embedded row and sums the streams in front of its last norm.
"""

from __future__ import annotations

from ..config.spec import LayerSpec, PartSpec
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import ARRANGEMENTS, make_part, register_part


@register_part("arrangement", "prenorm_residual")
class PreNormResidual:
    def run(self, layer: "Layer", residual, pending, step, cache, writes_cache: bool = True):
        n = layer.mixer_norm.add_norm(residual, pending)
        d = layer.mixer.forward(n, step, cache, writes_cache=writes_cache)
        ff = layer.feed_forward
        if hasattr(ff, "forward_from"):
            return ff.forward_from(layer.feed_forward_norm, residual, d, step)
        return ff.forward(layer.feed_forward_norm.add_norm(residual, d), step)


@register_part("arrangement", "sandwich_norm_residual")
class SandwichNormResidual:
    def run(self, layer: "Layer", residual, pending, step, cache, writes_cache: bool = True):
        n = layer.mixer_norm.add_norm(residual, pending)
        d = layer.mixer.forward(n, step, cache, writes_cache=writes_cache)
        ff = layer.feed_forward
        if getattr(ff, "absent", False):
            layer.mixer_post_norm.add_normed(residual, d)
            return None
        if hasattr(ff, "router_args"):
            # the norm in front of a routed feed-forward runs its router too: the add first, then that kernel
            layer.mixer_post_norm.add_normed(residual, d)
            out = ff.forward_from(layer.feed_forward_norm, residual, None, step)
        else:
            out = ff.forward(layer.mixer_post_norm.add_normed(residual, d, then=layer.feed_forward_norm), step)
        if isinstance(out, ops.GatedSum):       # a dense part, its gate a row, a routed part: added by the norm's kernel
            layer.feed_forward_post_norm.add_normed(residual, out.dense, gate=out.gate, experts=out.experts)
        else:
            layer.feed_forward_post_norm.add_normed(residual, out)
        return None


class _Reading:
    """A norm seen by a feed-forward that runs it itself: whatever the feed-forward asks of it, the streams are read with the
    sublayer's own weights."""

    def __init__(self, norm, read):
        self.norm, self.read = norm, read

    def add_norm(self, residual, delta, **kw):
        return self.norm.add_norm(residual, delta.reading(self.read), **kw)


@register_part("arrangement", "hyper_connections")
class HyperConnections:
    """See the module's text. `params`: `streams` and `names` (in, out, mix: the tensors' names behind `<prefix>hc<q>.`)."""
    graph_safe = True

    def __init__(self, params=None, prefix: str = ""):
        params = params or {}
        self.streams = int(params["streams"])
        if not 1 <= self.streams <= 8:
            raise ValueError(f"{self.streams} residual streams: 1 to 8 are implemented")
        names = params.get("names") or {"in": "in", "out": "out", "mix": "mix"}
        self.n = {(q, k): f"{prefix}hc{q}.{v}" for q in (1, 2) for k, v in names.items()}
        self.has_second = bool(params.get("feed_forward", True))
        self.w = {}

    def weight_specs(self, present=None):
        S, out = self.streams, []
        for q in (1, 2) if self.has_second else (1,):
            out += [TensorSpec(self.n[q, "in"], (S,), "vector", "ones"), TensorSpec(self.n[q, "out"], (S,), "vector", "ones"),
                    TensorSpec(self.n[q, "mix"], (S, S), "vector", "mix")]
        return out

    def bind(self, read, runtime):
        self.w = {key: runtime.vector(read(name)) for key, name in self.n.items() if self.has_second or key[0] == 1}

    def step_bytes(self, elem: int, **_) -> int:
        return sum(4 * t.numel() for t in self.w.values())

    def run(self, layer: "Layer", residual, pending, step, cache, writes_cache: bool = True):
        w = self.w
        if pending is None:
            pending = ops.StreamUpdate(None, None, None)
        n = layer.mixer_norm.add_norm(residual, pending.reading(w[1, "in"]))
        d = ops.StreamUpdate(layer.mixer.forward(n, step, cache, writes_cache=writes_cache), w[1, "mix"], w[1, "out"])
        ff = layer.feed_forward
        if getattr(ff, "absent", False):
            return d
        norm = _Reading(layer.feed_forward_norm, w[2, "in"])
        if hasattr(ff, "forward_from"):
            out = ff.forward_from(norm, residual, d, step)
        else:
            out = ff.forward(norm.add_norm(residual, d), step)
        return ops.StreamUpdate(out, w[2, "mix"], w[2, "out"])


class Layer:
    """One layer's parts, built from its spec. The layer knows its parts; no part knows the layer."""

    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.spec = spec
        p = spec.prefix

        def norm(ps: PartSpec):
            name = ps.get("name")
            return make_part("norm", ps, prefix=p + (name + "." if name else ""), size=hidden_size)

        self.mixer_norm = norm(spec.mixer_norm)
        self.feed_forward_norm = norm(spec.feed_forward_norm) if spec.feed_forward_norm else None
        self.mixer_post_norm = norm(spec.mixer_post_norm) if spec.mixer_post_norm else None
        self.feed_forward_post_norm = norm(spec.feed_forward_post_norm) if spec.feed_forward_post_norm else None
        self.mixer = make_part("mixer", spec.mixer, prefix=p, hidden_size=hidden_size)
        self.feed_forward = make_part("feed_forward", spec.feed_forward, prefix=p, hidden_size=hidden_size)
        if spec.arrangement not in ARRANGEMENTS:
            raise ValueError(f"unknown arrangement {spec.arrangement!r}; registered: {', '.join(sorted(ARRANGEMENTS))}")
        cls = ARRANGEMENTS[spec.arrangement]
        self.arrangement = cls(spec.arrangement_params, prefix=p) if spec.arrangement_params is not None else cls()

    @property
    def parts(self):
        """The layer's parts that have tensors and a say in whether a step may be captured (an arrangement with tensors of its
        own is one of them)."""
        own = (self.arrangement,) if hasattr(self.arrangement, "weight_specs") else ()
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm,
                                 self.feed_forward, self.feed_forward_post_norm) if p is not None) + own

    def weight_specs(self, present=None):
        out = []
        for part in self.parts:
            out += part.weight_specs(present)
        return out

    def bind(self, read, runtime):
        for part in self.parts:
            part.bind(read, runtime)

    def run(self, residual, pending, step, cache, writes_cache: bool = True):
        return self.arrangement.run(self, residual, pending, step, cache, writes_cache)
