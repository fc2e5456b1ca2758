"""Position encodings applied to q and k inside a mixer.

`rope_neox`: inv_freq_i = theta^(-2i/d), angle = position * inv_freq_i (32-bit), the two halves of the
rotated part share a frequency: x' = x cos + rotate_half(x) sin with rotate_half(x) = cat(-x[d/2:], x[:d/2])
(engine/models/lfm2_moe/ref.py:84, 111-120). The frequencies are computed here once, in 32-bit, by the
reference's expression; the angles, sines and cosines are computed in the kernel in 32-bit per row.

With `scaling` = {factor, low, high, original} the long wavelengths are slowed (the Llama 3.1 rule): with wavelength
l = 2 pi / f, f stays where l < original / high, becomes f / factor where l > original / low, and between the two is
(1 - s) f / factor + s f with s = (original / l - low) / (high - low). With `precise` (or a scaling) the frequencies are
formed in 64-bit and rounded once.

With `scaling` = {factor, original, fast, slow} (`fast` in the place of `low`) the stretch is a ramp over the pairs instead:
d(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta) is the pair that makes t turns over `original` positions; with
lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
pair i turns at f_i (1 - ramp_i) + f_i / factor ramp_i, and the sines and cosines are multiplied by `magnitude` =
0.1 ln(factor) + 1, which the mixer hands to its q/k kernel.

`rope_pairs`: the interleaved layout: entries 2i and 2i + 1 of the rotated part are a pair, (u, v) at position p becomes
(u cos a - v sin a, v cos a + u sin a) with a = p * theta^(-2i/d), for the first d = `rotary_dim` entries (the rest pass).
The frequencies are formed once in 64-bit and rounded to 32-bit; angles, sines and cosines are 32-bit in the kernel. A
mixer whose kernel turns pairs asks `fused_rotary_pairs()`.

`none`: q and k are left as they are.

An encoding either hands the fused q/k kernel its table (`fused_rotary`), or is applied by the mixer
through `apply(q, k, positions)` between the norm and the cache write.
"""

from __future__ import annotations

import math

import torch

from .base import Part, register_part


RAMP_MAGNITUDE_SLOPE = 0.1      # a ramped stretch multiplies sines and cosines by 1 + slope * ln(factor)
RAMP_MIN_WIDTH = 0.001


@register_part("position_encoding", "rope_neox")
class RotaryNeox(Part):
    graph_safe = True

    def __init__(self, spec, head_dim: int = 0, **_):
        super().__init__(spec)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec.get("rotary_dim") or head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} for head size {head_dim}: an even size up to the head size")
        self.scaling = spec.get("scaling")
        self.precise = bool(spec.get("precise", False)) or self.scaling is not None
        self.inv_freq = None
        self.ramped = bool(self.scaling) and "fast" in self.scaling
        self.magnitude = RAMP_MAGNITUDE_SLOPE * math.log(float(self.scaling["factor"])) + 1.0 if self.ramped else 1.0

    def frequencies(self) -> torch.Tensor:
        d = self.rotary_dim
        if not self.precise:
            return 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        f = self.theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
        if self.ramped:
            s = self.scaling
            factor, orig = float(s["factor"]), float(s["original"])

            def pair_of(turns: float) -> float:
                return d * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(pair_of(float(s["fast"]))), 0)
            hi = min(math.ceil(pair_of(float(s["slow"]))), d - 1)
            ramp = ((torch.arange(d // 2, dtype=torch.float64) - lo) / max(hi - lo, RAMP_MIN_WIDTH)).clamp(0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
        elif self.scaling:
            s = self.scaling
            factor, low, high, orig = (float(s[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            blend = (orig / wavelength - low) / (high - low)
            mid = (1.0 - blend) * f / factor + blend * f
            f = torch.where(wavelength < orig / high, f, torch.where(wavelength > orig / low, f / factor, mid))
        return f.to(torch.float32)

    def bind(self, read, runtime):
        self.runtime = runtime
        self.inv_freq = self.frequencies().to(runtime.device)

    def fused_rotary(self):
        return self.inv_freq, self.rotary_dim

    def apply(self, q, k, positions):
        raise NotImplementedError("rope_neox is applied by the fused q/k kernel")


@register_part("position_encoding", "rope_pairs")
class RotaryPairs(Part):
    graph_safe = True

    def __init__(self, spec, head_dim: int = 0, **_):
        super().__init__(spec)
        self.theta = float(spec["theta"])
        d = spec.get("rotary_dim")
        self.rotary_dim = int(head_dim if d is None else d)
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} for a rotated part of {head_dim}: an even size up to it")
        self.inv_freq = None

    def bind(self, read, runtime):
        self.runtime = runtime
        d = self.rotary_dim
        inv = self.theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / max(d, 1))
        self.inv_freq = inv.to(torch.float32).to(runtime.device)

    def fused_rotary(self):
        return None

    def fused_rotary_pairs(self):
        return self.inv_freq, self.rotary_dim

    def apply(self, q, k, positions):
        raise NotImplementedError("rope_pairs is applied by the mixer's own kernel")


@register_part("position_encoding", "none")
class NoPosition(Part):
    graph_safe = True

    def __init__(self, spec, head_dim: int = 0, **_):
        super().__init__(spec)

    def fused_rotary(self):
        return None, 0

    def apply(self, q, k, positions):
        return None
