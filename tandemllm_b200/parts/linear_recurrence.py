"""Mixers that carry a matrix state a head, S [keys, values] in 32-bit, from token to token in a request's slot, and the
mixer that runs several mixers side by side on the same rows.

`decayed_linear_attention`: q = act(W_q n), k = act(W_k n) (heads x head_dim), v = act(W_v n) (heads x value_dim);
    a head: S <- c_h S + k v^T, o = S^T q with the new S, c_h a fixed number a head (`decay`); the concatenated heads are
    brought to unit root mean square together, times the weight `norm`, times sigmoid(W_g n), and projected by W_o.

`delta_rule`: r, k, v = W_r n, W_k n, W_v n (heads x head_dim each). A decay a key channel d = exp(-decay_rate *
    sigmoid(W_w2 tanh(W_w1 n) + w0)), a removal rate a key channel a = sigmoid(W_a n + a_b), the unit key
    u = k / sqrt(sum k^2 + key_eps) a head: S <- diag(d) S - (a * u)(u^T S) + k v^T, both terms reading the old S; o = S^T r;
    every head's o is brought to unit root mean square on its own, times `norm`, times sigmoid(W_g n), and projected by W_o.

`gated_linear_attention`: q = W_q n * head_dim^(-1/2), k = W_k n (heads x head_dim), v = W_v n (heads x value_dim). A decay a key
    channel and token, alpha = sigmoid(z)^(1 / tau) with z = W_a2 (W_a1 n) + b (two small products through an inner size that the
    stored `a1` says): S <- diag(alpha) S + k v^T, o = S^T q with the new S; every head's o is brought to unit root mean square
    on its own, times the weight `norm` (one head's size, shared by the heads), times silu(W_g n), and projected by W_o.

`weighted_sum`: out = sum_i weight_i mixer_i(n). Each mixer keeps what it needs (pages, a slot) for itself; the weights ride
    in the kernels that form the mixers' concatenated heads, and the out projections are one product over all of them.

Everything that enters a recurrence is 32-bit in both precisions: the projections' results are kept unrounded, the
activations, decays, unit keys, the state and the outputs are 32-bit (csrc/recurrence.cu). A portion of any length starts
from the slot and leaves it as the next portion needs it; a new request's slot is zero.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, SlotNeed, make_part, register_part
from .linear import linear


def _stack(mats: list[tuple[str, torch.Tensor]]) -> tuple[torch.Tensor, dict[str, int]]:
    """Matrices one below the other for a single product, each beginning at a multiple of 8 rows; where each begins."""
    rows, col, at = [], {}, 0
    for name, m in mats:
        col[name] = at
        pad = -m.shape[0] % 8
        rows += [m, torch.zeros(pad, m.shape[1], dtype=m.dtype, device=m.device)] if pad else [m]
        at += m.shape[0] + pad
    return torch.cat(rows).contiguous(), col


@register_part("mixer", "decayed_linear_attention")
class DecayedLinearAttention(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.heads, self.head_dim = int(spec["heads"]), int(spec["head_dim"])
        self.value_dim = int(spec.get("value_dim") or self.head_dim)
        self.decay = tuple(float(d) for d in spec["decay"])
        if len(self.decay) != self.heads:
            raise ValueError(f"{len(self.decay)} decays for {self.heads} heads")
        if not 1 <= self.head_dim <= 512:
            raise ValueError(f"a state of {self.head_dim} keys a head: 1 to 512 are implemented")
        self.activation = str(spec.get("activation", "silu"))
        if self.activation not in ("silu", "identity"):
            raise ValueError(f"activation {self.activation!r} on q, k, v: silu or identity")
        self.eps = float(spec["eps"])
        self.n = {k: prefix + v for k, v in spec["names"].items()}

    @property
    def out_dim(self) -> int:
        return self.heads * self.value_dim

    def weight_specs(self, present=None):
        n, W, H, D, VD = self.n, self.hidden_size, self.heads, self.head_dim, self.value_dim
        return [TensorSpec(n["q"], (H * D, W)), TensorSpec(n["k"], (H * D, W)), TensorSpec(n["v"], (H * VD, W)),
                TensorSpec(n["gate"], (H * VD, W)), TensorSpec(n["norm"], (H * VD,), "vector", "ones"),
                TensorSpec(n["out"], (W, H * VD))]

    def bind(self, read, runtime):
        self.runtime = runtime
        n = self.n
        self.w_in, self.col = _stack([(x, runtime.matrix(read(n[x]))) for x in ("q", "k", "v", "gate")])
        self.w_norm = runtime.vector(read(n["norm"]))
        self.w_out = runtime.matrix(read(n["out"]))
        self.head_decay = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def cache_need(self):
        return SlotNeed((self.heads, self.head_dim, self.value_dim), torch.float32)

    def forward_inner(self, x, step, cache, writes_cache: bool, out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
        R, dev = x.shape[0], x.device
        proj = linear(self.runtime, x, self.w_in, out_dtype=torch.float32)
        y = torch.empty(R, self.out_dim, dtype=torch.float32, device=dev)
        ops.recurrence_scan(proj, self.col["q"], self.col["k"], self.col["v"], cache.state, step.state_slot, step.row_start,
                            step.n_requests, y, self.heads, self.head_dim, self.value_dim, head_decay=self.head_decay,
                            silu_inputs=self.activation == "silu", write_state=writes_cache,
                            max_rows=step.max_rows_per_request)
        return ops.group_norm_gate(y, proj[:, self.col["gate"]:], proj.stride(0), self.w_norm, self.eps, 1, out_scale, out)

    def forward(self, x, step, cache, writes_cache: bool = True):
        o = torch.empty(x.shape[0], self.out_dim, dtype=x.dtype, device=x.device)
        self.forward_inner(x, step, cache, writes_cache, o)
        return linear(self.runtime, o, self.w_out, out_dtype=torch.float32, defer=True)


@register_part("mixer", "delta_rule")
class DeltaRuleMixer(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.heads, self.head_dim = int(spec["heads"]), int(spec["head_dim"])
        if not 1 <= self.head_dim <= 512:
            raise ValueError(f"a state of {self.head_dim} keys a head: 1 to 512 are implemented")
        self.eps = float(spec["eps"])
        self.decay_rate = float(spec["decay_rate"])
        self.key_eps = float(spec["key_eps"])
        self.n = {k: prefix + v for k, v in spec["names"].items()}
        self.rank = None        # the inner size of the decay's two products: the shape of `w1` says it

    @property
    def out_dim(self) -> int:
        return self.heads * self.head_dim

    def weight_specs(self, present=None):
        n, W, I = self.n, self.hidden_size, self.heads * self.head_dim
        rank = self.rank if self.rank is not None else max(8, I // 16)
        return [TensorSpec(n["r"], (I, W)), TensorSpec(n["k"], (I, W)), TensorSpec(n["v"], (I, W)), TensorSpec(n["a"], (I, W)),
                TensorSpec(n["a_bias"], (I,), "vector", "bias"), TensorSpec(n["w1"], (rank, W)), TensorSpec(n["w2"], (I, rank)),
                TensorSpec(n["w0"], (I,), "vector", "bias"), TensorSpec(n["gate"], (I, W)),
                TensorSpec(n["norm"], (I,), "vector", "ones"), TensorSpec(n["out"], (W, I))]

    def shapes_from(self, shape_of) -> None:
        """The decay's inner size is no key of the configuration: the stored `w1` says it."""
        shape = shape_of(self.n["w1"])
        if shape is not None:
            self.rank = int(shape[0])

    def bind(self, read, runtime):
        self.runtime = runtime
        n = self.n
        self.w_in, self.col = _stack([(x, runtime.matrix(read(n[x]))) for x in ("r", "k", "v", "a", "gate")])
        w1 = runtime.matrix(read(n["w1"]))
        w2 = runtime.matrix(read(n["w2"]))
        # the inner size is filled up with zero rows and columns to a multiple of 8 (16-byte rows for the products)
        pad = -w1.shape[0] % 8
        if pad:
            w1 = torch.cat([w1, torch.zeros(pad, w1.shape[1], dtype=w1.dtype, device=w1.device)]).contiguous()
            w2 = torch.cat([w2, torch.zeros(w2.shape[0], pad, dtype=w2.dtype, device=w2.device)], dim=1).contiguous()
        self.w1, self.w2 = w1, w2
        self.w0 = runtime.vector(read(n["w0"]))
        self.a_bias = runtime.vector(read(n["a_bias"]))
        self.w_norm = runtime.vector(read(n["norm"]))
        self.w_out = runtime.matrix(read(n["out"]))

    def cache_need(self):
        return SlotNeed((self.heads, self.head_dim, self.head_dim), torch.float32)

    def forward_inner(self, x, step, cache, writes_cache: bool, out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
        R, dev = x.shape[0], x.device
        proj = linear(self.runtime, x, self.w_in, out_dtype=torch.float32)
        inner = linear(self.runtime, x, self.w1)
        ops.activation(inner, inner, ops.ACTIVATIONS["tanh"])
        w = linear(self.runtime, inner, self.w2, out_dtype=torch.float32)
        y = torch.empty(R, self.out_dim, dtype=torch.float32, device=dev)
        ops.recurrence_scan(proj, self.col["r"], self.col["k"], self.col["v"], cache.state, step.state_slot, step.row_start,
                            step.n_requests, y, self.heads, self.head_dim, self.head_dim, a_col=self.col["a"], w=w, w0=self.w0,
                            a_bias=self.a_bias, rate=self.decay_rate, key_eps=self.key_eps, write_state=writes_cache,
                            max_rows=step.max_rows_per_request)
        return ops.group_norm_gate(y, proj[:, self.col["gate"]:], proj.stride(0), self.w_norm, self.eps, self.heads, out_scale,
                                   out)

    def forward(self, x, step, cache, writes_cache: bool = True):
        o = torch.empty(x.shape[0], self.out_dim, dtype=x.dtype, device=x.device)
        self.forward_inner(x, step, cache, writes_cache, o)
        return linear(self.runtime, o, self.w_out, out_dtype=torch.float32, defer=True)


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.heads, self.head_dim = int(spec["heads"]), int(spec["head_dim"])
        self.value_dim = int(spec.get("value_dim") or self.head_dim)
        if not 1 <= self.head_dim <= 512:
            raise ValueError(f"a state of {self.head_dim} keys a head: 1 to 512 are implemented")
        self.eps = float(spec["eps"])
        self.tau = float(spec["tau"])
        if not self.tau > 0.0:
            raise ValueError(f"a decay's root tau = {self.tau}: a positive number")
        self.n = {k: prefix + v for k, v in spec["names"].items()}
        self.rank = None        # the inner size of the decay's two products: the shape of `a1` says it

    @property
    def out_dim(self) -> int:
        return self.heads * self.value_dim

    def weight_specs(self, present=None):
        n, W, H, D, VD = self.n, self.hidden_size, self.heads, self.head_dim, self.value_dim
        rank = self.rank if self.rank is not None else max(8, H * D // 16)
        return [TensorSpec(n["q"], (H * D, W)), TensorSpec(n["k"], (H * D, W)), TensorSpec(n["v"], (H * VD, W)),
                TensorSpec(n["gate"], (H * VD, W)), TensorSpec(n["norm"], (VD,), "vector", "ones"),
                TensorSpec(n["a1"], (rank, W)), TensorSpec(n["a2"], (H * D, rank)),
                TensorSpec(n["a_bias"], (H * D,), "vector", "bias"), TensorSpec(n["out"], (W, H * VD))]

    def shapes_from(self, shape_of) -> None:
        shape = shape_of(self.n["a1"])
        if shape is not None:
            self.rank = int(shape[0])

    def bind(self, read, runtime):
        self.runtime = runtime
        n = self.n
        # q, k, v and the gate read the same rows: one product whose result stays 32-bit
        self.w_in, self.col = _stack([(x, runtime.matrix(read(n[x]))) for x in ("q", "k", "v", "gate")])
        a1, a2 = runtime.matrix(read(n["a1"])), runtime.matrix(read(n["a2"]))
        # the inner size is filled up with zero rows and columns to a multiple of 8 (16-byte rows for the products)
        pad = -a1.shape[0] % 8
        if pad:
            a1 = torch.cat([a1, torch.zeros(pad, a1.shape[1], dtype=a1.dtype, device=a1.device)]).contiguous()
            a2 = torch.cat([a2, torch.zeros(a2.shape[0], pad, dtype=a2.dtype, device=a2.device)], dim=1).contiguous()
        self.w_a1, self.w_a2 = a1, a2
        self.a_bias = runtime.vector(read(n["a_bias"]))
        self.w_norm = runtime.vector(read(n["norm"]))
        self.w_out = runtime.matrix(read(n["out"]))

    def cache_need(self):
        return SlotNeed((self.heads, self.head_dim, self.value_dim), torch.float32)

    def forward_inner(self, x, step, cache, writes_cache: bool, out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
        R, dev = x.shape[0], x.device
        proj = linear(self.runtime, x, self.w_in, out_dtype=torch.float32)
        # the decay's logits: the inner rows in the compute dtype as the second product's operand, the result 32-bit
        z = linear(self.runtime, linear(self.runtime, x, self.w_a1), self.w_a2, out_dtype=torch.float32)
        y = torch.empty(R, self.out_dim, dtype=torch.float32, device=dev)
        ops.recurrence_scan(proj, self.col["q"], self.col["k"], self.col["v"], cache.state, step.state_slot, step.row_start,
                            step.n_requests, y, self.heads, self.head_dim, self.value_dim, w=z, w0=self.a_bias,
                            rate=1.0 / self.tau, write_state=writes_cache, max_rows=step.max_rows_per_request,
                            q_scale=self.head_dim ** -0.5)
        return ops.group_norm_gate(y, proj[:, self.col["gate"]:], proj.stride(0), self.w_norm, self.eps, self.heads, out_scale,
                                   out, gate_activation="silu")

    def forward(self, x, step, cache, writes_cache: bool = True):
        o = torch.empty(x.shape[0], self.out_dim, dtype=x.dtype, device=x.device)
        self.forward_inner(x, step, cache, writes_cache, o)
        return linear(self.runtime, o, self.w_out, out_dtype=torch.float32, defer=True)


@register_part("mixer", "weighted_sum")
class WeightedSumMixer(Part):
    """Several mixers on the same rows, their outputs weighed and summed. Every mixer must hand out its concatenated
    heads (`forward_inner`, `out_dim`, `w_out`); the site's cache is the tuple of the mixers' own."""

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.mixers = [make_part("mixer", ps, prefix=prefix, hidden_size=hidden_size) for ps in spec["mixers"]]
        self.weights = tuple(float(w) for w in spec["weights"])
        if len(self.weights) != len(self.mixers) or not self.mixers:
            raise ValueError(f"{len(self.weights)} weights for {len(self.mixers)} mixers")
        for m in self.mixers:
            if not hasattr(m, "forward_inner"):
                raise ValueError(f"a {type(m).__name__} does not hand out its concatenated heads")

    @property
    def graph_safe(self) -> bool:
        return all(m.graph_safe for m in self.mixers)

    def weight_specs(self, present=None):
        return [s for m in self.mixers for s in m.weight_specs(present)]

    def shapes_from(self, shape_of) -> None:
        for m in self.mixers:
            if hasattr(m, "shapes_from"):
                m.shapes_from(shape_of)

    def bind(self, read, runtime):
        self.runtime = runtime
        for m in self.mixers:
            m.bind(read, runtime)
        # one out projection over the concatenated heads of all mixers, each part beginning at a multiple of 8 columns
        self.at, cols, at = [], [], 0
        for m in self.mixers:
            self.at.append(at)
            pad = -m.w_out.shape[1] % 8
            cols.append(m.w_out)
            if pad:
                cols.append(torch.zeros(m.w_out.shape[0], pad, dtype=m.w_out.dtype, device=m.w_out.device))
            at += m.w_out.shape[1] + pad
        self.inner = at
        self.padded = any(-m.w_out.shape[1] % 8 for m in self.mixers)
        self.w_out = torch.cat(cols, dim=1).contiguous()
        for m in self.mixers:
            m.w_out = None          # the single matrices are not kept twice

    def cache_need(self):
        return tuple(m.cache_need() for m in self.mixers)

    def step_bytes(self, elem: int, **kw) -> int:
        return sum(m.step_bytes(elem, **kw) for m in self.mixers)

    def forward(self, x, step, cache, writes_cache: bool = True):
        R = x.shape[0]
        make = torch.zeros if self.padded else torch.empty
        o = make(R, self.inner, dtype=x.dtype, device=x.device)
        for m, w, at, c in zip(self.mixers, self.weights, self.at, cache):
            m.forward_inner(x, step, c, writes_cache, o[:, at:at + m.out_dim], w)
        return linear(self.runtime, o, self.w_out, out_dtype=torch.float32, defer=True)
