"""Norms fused with the residual add in front of them: RMS norm, Dynamic Tanh, and the weightless unit-RMS norm of q and k.

  y = x * rsqrt(mean(x^2) + eps);  out = w * y      plain w, not 1 + w  (engine/models/lfm2_moe/ref.py:105-109)

A design whose norm weights are stored as their distance from a number (out = (offset + w) * y) names it as `offset` in
the norm's spec; the sum is formed once at bind time, in 32-bit.

Over a residual of several streams the norm takes an `ops.StreamUpdate` as what is added (see `parts/block.py`,
`hyper_connections`): the same kernel rewrites the streams and norms their weighed sum.

The residual stream is 32-bit; mean, rsqrt and the scale are 32-bit and the result is rounded once to the
compute dtype. The reference fuses the same pair (`add_rms`, engine/models/lfm2_moe/kernels.py:90-107).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", size: int = 0, **_):
        super().__init__(spec, prefix)
        self.size = size
        self.eps = float(spec["eps"])
        self.name = prefix + str(spec.get("tensor") or "weight")     # `tensor`: the weight's own name behind the prefix
        self.offset = float(spec.get("offset") or 0.0)               # the stored weight is the distance from this number
        self.weight = None

    def weight_specs(self, present=None):
        return [TensorSpec(self.name, (self.size,), role="vector", init="bias" if self.offset else "ones")]

    def bind(self, read, runtime):
        self.runtime = runtime
        self.weight = runtime.vector(read(self.name))
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()

    def add_norm(self, residual: torch.Tensor, delta, out: torch.Tensor | None = None,
                 gather: torch.Tensor | None = None, n_out: int | None = None, want32: bool = False,
                 route: dict | None = None):
        """residual += delta (32-bit; a tensor or a branch output in one of the deferred forms of `kernels.ops`);
        returns the normed rows in the compute dtype, and with `want32` the pair (normed, the same rows unrounded
        in 32-bit). `route` (see `ops.add_rmsnorm`) also runs a router on the unrounded rows in the same kernel."""
        rows = residual.shape[-2] if gather is None else (n_out if n_out is not None else gather.shape[0])
        if out is None:
            out = torch.empty(rows, self.size, dtype=self.runtime.dtype, device=residual.device)
        if not want32:
            return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, gather, None, route)
        if out.dtype == torch.float32:
            ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, gather, None, route)
            return out, out
        out32 = torch.empty(rows, self.size, dtype=torch.float32, device=residual.device)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, gather, out32, route)
        return out, out32


    def add_normed(self, residual: torch.Tensor, delta, gate: torch.Tensor | None = None, experts=None, then=None,
                   gather: torch.Tensor | None = None, n_out: int | None = None):
        """This norm behind a branch: residual += weight * d / rms(d), d the branch output `delta` (a tensor or a deferred
        form; times sigmoid(gate[r]) with `gate`; plus the weighed rows of `experts`). `then`: the RMS norm in front of
        the next sublayer, whose rows of the new residual are returned (the same kernel makes them; with `gather` only
        of those rows, and the residual stays as it was)."""
        if then is None:
            ops.add_normed(residual, delta, self.weight, self.eps, gate, experts)
            return None
        rows = residual.shape[0] if gather is None else (n_out if n_out is not None else gather.shape[0])
        out = torch.empty(rows, self.size, dtype=self.runtime.dtype, device=residual.device)
        g = gather[:rows] if gather is not None else None
        return ops.add_normed(residual, delta, self.weight, self.eps, gate, experts, (then.weight, then.eps, out, g))


@register_part("norm", "dyt")
class DynamicTanh(Part):
    """Dynamic Tanh: out = tanh(alpha * x) * w + b, element by element, alpha one scalar a norm; no mean and no variance
    are computed. Tensors: `<name>` (w), `<name>.b`, `<name>.alpha`, where `<name>` is the prefix without its last dot.
    With `optional` in the spec the norm reads its tensors only when the folder holds them (a layer whose feed-forward
    is absent has no use for the norm in front of it)."""
    graph_safe = True

    def __init__(self, spec, prefix: str = "", size: int = 0, **_):
        super().__init__(spec, prefix)
        self.size = size
        self.eps = float(spec.get("eps", 0.0))          # carried for the mixers that ask their layer's eps; unused here
        self.name = prefix[:-1] if prefix.endswith(".") else prefix
        self.optional = bool(spec.get("optional", False))
        self.weight = self.bias = self.alpha = None

    def weight_specs(self, present=None):
        if self.optional and (present is None or self.name not in present):
            return []
        return [TensorSpec(self.name, (self.size,), role="vector", init="ones"),
                TensorSpec(self.name + ".b", (self.size,), role="vector", init="bias"),
                TensorSpec(self.name + ".alpha", (), role="vector", init="ones")]

    def bind(self, read, runtime):
        self.runtime = runtime
        if self.optional:
            try:
                read(self.name)
            except KeyError:
                return
        self.weight = runtime.vector(read(self.name))
        self.bias = runtime.vector(read(self.name + ".b"))
        self.alpha = runtime.vector(read(self.name + ".alpha")).reshape(1)

    def add_norm(self, residual: torch.Tensor, delta, out: torch.Tensor | None = None,
                 gather: torch.Tensor | None = None, n_out: int | None = None, want32: bool = False,
                 route: dict | None = None):
        if route is not None:
            raise NotImplementedError("a router inside the Dynamic Tanh kernel")
        rows = residual.shape[0] if gather is None else (n_out if n_out is not None else gather.shape[0])
        if out is None:
            out = torch.empty(rows, self.size, dtype=self.runtime.dtype, device=residual.device)
        g = gather[:rows] if gather is not None else None
        ops.add_dyt(residual, delta, self.weight, self.bias, self.alpha, out, g)
        if not want32:
            return out
        if out.dtype == torch.float32:
            return out, out
        out32 = torch.empty(rows, self.size, dtype=torch.float32, device=residual.device)
        # the residual already holds the sum (or, with `gather`, the delta is added once more from its source)
        ops.add_dyt(residual, delta if gather is not None else None, self.weight, self.bias, self.alpha, out32, g)
        return out, out32


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """Layer norm with weight and bias: out = (x - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations,
    all in 32-bit. Tensors: `<name>` (w) and `<name>.b`, where `<name>` is the prefix without its last dot."""
    graph_safe = True

    def __init__(self, spec, prefix: str = "", size: int = 0, **_):
        super().__init__(spec, prefix)
        self.size = size
        self.eps = float(spec["eps"])
        self.name = prefix[:-1] if prefix.endswith(".") else prefix
        self.weight = self.bias = None

    def weight_specs(self, present=None):
        return [TensorSpec(self.name, (self.size,), role="vector", init="ones"),
                TensorSpec(self.name + ".b", (self.size,), role="vector", init="bias")]

    def bind(self, read, runtime):
        self.runtime = runtime
        self.weight = runtime.vector(read(self.name))
        self.bias = runtime.vector(read(self.name + ".b"))

    def add_norm(self, residual: torch.Tensor, delta, out: torch.Tensor | None = None,
                 gather: torch.Tensor | None = None, n_out: int | None = None, want32: bool = False,
                 route: dict | None = None):
        if route is not None or want32:
            raise NotImplementedError("a router or unrounded rows from the layer norm kernel")
        rows = residual.shape[0] if gather is None else (n_out if n_out is not None else gather.shape[0])
        if out is None:
            out = torch.empty(rows, self.size, dtype=self.runtime.dtype, device=residual.device)
        g = gather[:rows] if gather is not None else None
        return ops.add_layernorm(residual, delta, self.weight, self.bias, self.eps, out, g)


@register_part("norm", "unit_rms")
class UnitRMS(Part):
    """x / sqrt(mean(x^2) + eps) without a weight: what a mixer names for q and k that are only brought to unit root
    mean square. It has no tensors; the mixer's q/k kernel does the arithmetic."""
    graph_safe = True
    weight = None

    def __init__(self, spec, prefix: str = "", size: int = 0, **_):
        super().__init__(spec, prefix)
        self.size = size
        self.eps = float(spec["eps"])
