"""The latent-attention mixer: keys and values of all heads come from one small latent a token, which is all the cache holds.

  c_q = norm(dq n) * w_dq;  q = uq c_q                      per head [dim unrotated | rot_dim rotated]
  [c | k_r] = dkv n;  c = norm(c) * w_dkv (the latent, `kv_rank` numbers);  k_r: one rotated key part for all heads
  head h: key = [uk_h c | rot(k_r)], value = uv_h c;  score = (q_unrotated . uk_h c + rot(q_rotated) . rot(k_r)) * scale
  softmax over the visible keys (0 <= i - j < window, or all); out = o(concatenated heads)
  with a `sink` tensor named ([heads]): a head's softmax denominator also holds exp(sink_h), which has no key and no value, is
  not scaled and counts once; with a `gate` matrix named ([heads * value_dim, hidden]): the concatenated heads are multiplied
  entry by entry by sigmoid(gate n), n the mixer's input, before the out projection

The position encoding is a part of its own (a kind with `fused_rotary_pairs()`); it turns the rotated parts only. What is
stored a token is c and rot(k_r): one row of kv_rank + rot_dim numbers (`PagedNeed(1, kv_rank + rot_dim, window,
values=False)`). The products with uk and uv are regrouped so that no key or value of a head is ever formed (csrc/
attention_latent.cu): q'_h = uk_h^T q_unrotated, scores against the cached rows, the weighted sum of the latents, then uv_h.
uk is transposed a head once at bind time for that.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import PagedNeed, Part, make_part, register_part
from .linear import linear


@register_part("mixer", "latent_attention")
class LatentAttentionMixer(Part):
    @property
    def graph_safe(self) -> bool:
        return self.position.graph_safe

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.heads, self.dim, self.rot_dim = int(spec["num_heads"]), int(spec["head_dim"]), int(spec["rot_dim"])
        self.vdim, self.kv_rank, self.q_rank = int(spec["value_dim"]), int(spec["kv_rank"]), int(spec["q_rank"])
        self.scale = float(spec.get("scale") or (self.dim + self.rot_dim) ** -0.5)
        self.window = spec.get("window")
        self.eps = float(spec["eps"])
        if min(self.heads, self.vdim, self.kv_rank, self.q_rank) <= 0 or self.dim < 0 or self.rot_dim < 0 \
                or self.dim + self.rot_dim <= 0:
            raise ValueError("latent attention: heads, ranks and head sizes must be positive")
        if self.kv_rank > 512:
            raise ValueError(f"a latent of {self.kv_rank} numbers: up to 512 are implemented")
        self.position = make_part("position_encoding", spec["position"], head_dim=self.rot_dim)
        self.n = {k: prefix + v for k, v in spec["names"].items()}
        self.has_sink, self.has_gate = "sink" in self.n, "gate" in self.n
        self.sinks = None

    def weight_specs(self, present=None):
        n, W, H = self.n, self.hidden_size, self.heads
        more = [TensorSpec(n["sink"], (H,), "vector", "bias")] if self.has_sink else []
        if self.has_gate:
            more.append(TensorSpec(n["gate"], (H * self.vdim, W)))
        return more + [TensorSpec(n["dq"], (self.q_rank, W)), TensorSpec(n["dq_norm"], (self.q_rank,), "vector", "ones"),
                TensorSpec(n["uq"], (H * (self.dim + self.rot_dim), self.q_rank)),
                TensorSpec(n["dkv"], (self.kv_rank + self.rot_dim, W)),
                TensorSpec(n["dkv_norm"], (self.kv_rank,), "vector", "ones"),
                TensorSpec(n["uk"], (H * self.dim, self.kv_rank)), TensorSpec(n["uv"], (H * self.vdim, self.kv_rank)),
                TensorSpec(n["out"], (W, H * self.vdim))]

    def bind(self, read, runtime):
        self.runtime = runtime
        n, H = self.n, self.heads
        # the two down-projections (and an output gate) read the same rows: one product, the query's latent first; padded
        # with zero rows so that every part begins at a multiple of 8 columns
        dq, dkv = runtime.matrix(read(n["dq"])), runtime.matrix(read(n["dkv"]))
        self.kv_at = -(-self.q_rank // 8) * 8
        pad = torch.zeros(self.kv_at - self.q_rank, dq.shape[1], dtype=dq.dtype, device=dq.device)
        parts = [dq, pad, dkv]
        if self.has_gate:
            self.gate_at = self.kv_at + -(-dkv.shape[0] // 8) * 8
            parts += [torch.zeros(self.gate_at - self.kv_at - dkv.shape[0], dq.shape[1], dtype=dq.dtype, device=dq.device),
                      runtime.matrix(read(n["gate"]))]
        self.w_down = torch.cat(parts).contiguous()
        if self.has_sink:
            self.sinks = runtime.vector(read(n["sink"]))
        self.w_dq_norm = runtime.vector(read(n["dq_norm"]))
        self.w_dkv_norm = runtime.vector(read(n["dkv_norm"]))
        self.w_uq = runtime.matrix(read(n["uq"]))
        # uk [H dim, rank] -> a head's [rank, dim]: the query's unrotated part goes through it into the latent's space
        self.w_uk_t = runtime.matrix(read(n["uk"])).view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = runtime.matrix(read(n["uv"])).view(H, self.vdim, self.kv_rank).contiguous()
        self.w_out = runtime.matrix(read(n["out"]))
        self.position.bind(read, runtime)

    def cache_need(self):
        return PagedNeed(1, self.kv_rank + self.rot_dim, self.window, values=False)

    def forward(self, x, step, cache, writes_cache: bool = True):
        if not writes_cache:
            raise NotImplementedError("latent attention over another site's cache")
        rt = self.runtime
        R, dt, dev = x.shape[0], x.dtype, x.device
        H, D, Rr, L = self.heads, self.dim, self.rot_dim, self.kv_rank
        Dk = L + Rr
        down = linear(rt, x, self.w_down)                       # [R, q_rank .. | kv_rank + rot_dim]
        cq = torch.empty(R, self.q_rank, dtype=dt, device=dev)
        ops.rmsnorm_rows(down, self.q_rank, self.w_dq_norm, self.eps, cq)
        q = linear(rt, cq, self.w_uq)                           # [R, H (D + Rr)]
        kv = down[:, self.kv_at:self.kv_at + Dk]
        gate = down[:, self.gate_at:] if self.has_gate else None
        table = step.block_tables[cache.group]
        inv_freq, rot_dims = self.position.fused_rotary_pairs()
        qa = torch.empty(R, H, Dk, dtype=torch.float32, device=dev)
        ops.latent_prepare(q, kv, self.w_dkv_norm, self.eps, inv_freq, rot_dims, step.positions, step.req_of_row, table,
                           cache.page_size, cache.k, qa, H, D, L, Rr, rt.status)
        fast = rt.attention_kernels
        if D > 0 and (fast is None or not fast.head_linear(q, q.stride(0), D + Rr, self.w_uk_t, qa, H * Dk, Dk, R)):
            ops.head_linear(q, q.stride(0), D + Rr, self.w_uk_t, qa, H * Dk, Dk, R)
        ol = torch.empty(R, H, L, dtype=dt, device=dev)
        if fast is None or not fast.attention_latent(qa, cache, table, step, self.scale, self.window, ol, L, rt, self.sinks):
            ops.attention_latent(qa, cache.k, table, cache.page_size, step.req_of_row, step.positions, self.scale, self.window,
                                 ol, L, rt.status, self.sinks)
        o = torch.empty(R, H * self.vdim, dtype=dt, device=dev)
        if fast is None or not fast.head_linear(ol, H * L, L, self.w_uv, o, H * self.vdim, self.vdim, R, gate):
            ops.head_linear(ol, H * L, L, self.w_uv, o, H * self.vdim, self.vdim, R, gate)
        return linear(rt, o, self.w_out, out_dtype=torch.float32, defer=True)
