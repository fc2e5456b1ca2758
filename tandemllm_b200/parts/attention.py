"""The attention mixer: grouped-query attention over the paged cache with optional per-head q/k RMS norms,
a position encoding, and an optional sliding window.

  q = norm_D(q_proj n), k = norm_D(k_proj n), v = v_proj n; position encoding on q, k; k, v written to the
  cache at the row's position; s = q k^T * scale over the visible keys; softmax in 32-bit; o = a v;
  query head h reads KV head h // (Hq / Hk); out = out_proj(o)      (engine/models/lfm2_moe/ref.py:153-178)

Options, each a parameter of the spec so that another design can name its own combination:
  `values`: "projected" (a v matrix of its own) or "keys" (no v matrix: a key as projected, before its norm, is its value);
  `qk_norm`: a norm kind for q and k per head (`rmsnorm` with weights, `unit_rms` without), or None;
  `head_mix`: the name of a tensor M [Hq, Hq]: after the softmax the heads' weights are mixed, p'_h = sum_g M[h, g] p_g,
              and head h applies p'_h to the values of its own KV head;
  `gate`: the name of a matrix [Hq, hidden]: head h's output is multiplied by sigmoid(gate n)_h before the out projection;
  `weight_suffix`: what follows a matrix's name in the folder (".weight" by default);
  `value_dim`: the size of a value a head where it is not the keys';
  `softcap` c: score <- c tanh(score / c) before the mask and the softmax;
  `keep_first` n (with a window): a row also sees the keys at positions below n, at their true positions;
  `value_rotation` base: the value at position j is turned by j over all its entries (halves layout, pair m by
              j base^(-2m / value_dim)) and cached so; a head's output at position i is turned back by -i before any gate;
  `entry_gate`: the name of a matrix [Hq * value_dim, hidden]: the concatenated heads times sigmoid(gate n) entry by entry;
  `borrows_keys`: the layer has no k and v matrices: its site reads the cache of the site its run order names;
  `cache_window`, `cache_keep_first`: what the pages must keep readable when other sites read them through wider masks;
  `bias`: q, k, v and the out projection have biases (`<matrix's name without the weight suffix><bias_suffix>`, ".b" by
              default), added in the products;
  `value_carry` {key, blend}: values carried from layer to layer within a step. The first layer of a step that names `key`
              leaves its values as projected (`blend` None there); a later layer with the same `key` caches and attends over
              (1 - l) v + l v_first, l the one number stored as `<prefix><blend>`, v_first the first layer's values of the same
              row. Both must have the same number of KV heads and value size.
A position encoding whose sines and cosines carry a factor (`magnitude`) passes it to the q/k kernel.
Any of these takes the mixer to the kernels of csrc/attention_flex.cu, which have all of them as arguments.

Every size (heads, KV heads, head size), the scale, the window and the names of its tensors are
parameters. The q, k and v matrices are fused into one product at bind time, as the reference's loader
does (engine/models/lfm2_moe/load.py:125-135). A site that reads another site's cache computes its own
q and attends over the keys and values the other site wrote.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import PagedNeed, Part, make_part, register_part
from .linear import linear

@register_part("mixer", "attention")
class AttentionMixer(Part):
    @property
    def graph_safe(self) -> bool:
        return self.position.graph_safe

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} query heads are not a multiple of {self.num_kv_heads} KV heads")
        if spec.get("head_mix") or spec.get("gate"):
            if not 1 <= self.head_dim <= 256:       # the head-mixing kernels take any head size the q/k kernel does
                raise ValueError(f"head size {self.head_dim}: 1 to 256 are implemented")
        elif any(spec.get(k) for k in ("softcap", "keep_first", "value_rotation", "entry_gate", "borrows_keys", "bias",
                                       "value_carry")) or \
                int(spec.get("value_dim") or self.head_dim) != self.head_dim:
            if not (1 <= self.head_dim <= 256 and 1 <= int(spec.get("value_dim") or self.head_dim) <= 256):
                raise ValueError(f"head sizes {self.head_dim} and {spec.get('value_dim')}: 1 to 256 are implemented")
        elif self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"head size {self.head_dim}: multiples of 16 from 16 to 256 are implemented")
        self.scale = float(spec.get("scale") or self.head_dim ** -0.5)
        self.window = spec.get("window")
        names = spec["names"]
        self.n = {k: prefix + v for k, v in names.items()}
        qk = spec.get("qk_norm")
        self.q_norm = make_part("norm", qk, prefix=self.n.get("q_norm", "") + ".", size=self.head_dim) if qk else None
        self.k_norm = make_part("norm", qk, prefix=self.n.get("k_norm", "") + ".", size=self.head_dim) if qk else None
        self.position = make_part("position_encoding", spec["position"], head_dim=self.head_dim)
        self.bias = bool(spec.get("bias", False))
        self.values = str(spec.get("values", "projected"))
        if self.values not in ("projected", "keys"):
            raise ValueError(f"values {self.values!r}: projected or keys")
        self.suffix = str(spec.get("weight_suffix", ".weight"))
        self.head_mix_name = prefix + spec["head_mix"] if spec.get("head_mix") else None
        self.gate_name = prefix + spec["gate"] if spec.get("gate") else None
        self.qk_flags = (ops.QK_UNIT_NORM if qk and qk.kind == "unit_rms" else 0) | \
                        (ops.QK_VALUES_ARE_KEYS if self.values == "keys" else 0)
        self.head_mix = None
        self.value_dim = int(spec.get("value_dim") or self.head_dim)
        self.softcap = spec.get("softcap")
        self.keep_first = int(spec.get("keep_first") or 0)
        self.value_rotation = spec.get("value_rotation")
        self.entry_gate_name = prefix + spec["entry_gate"] if spec.get("entry_gate") else None
        self.borrows_keys = bool(spec.get("borrows_keys", False))
        self.cache_window = spec.get("cache_window", self.window)
        self.cache_keep_first = int(spec.get("cache_keep_first", self.keep_first) or 0)
        carry = spec.get("value_carry")
        self.carry_key = str(carry["key"]) if carry else None
        self.carry_blend_name = prefix + carry["blend"] if carry and carry.get("blend") else None
        self.bias_suffix = str(spec.get("bias_suffix", ".b"))
        self.flex = bool(self.value_dim != self.head_dim or self.softcap or self.keep_first or self.value_rotation
                         or self.entry_gate_name or self.borrows_keys or self.bias or carry
                         or getattr(self.position, "magnitude", 1.0) != 1.0)
        if self.flex:
            if self.head_mix_name or self.gate_name or self.q_norm or self.values != "projected":
                raise ValueError("capped scores, kept first tokens, turned values, an entry-wise gate and borrowed keys do "
                                 "not combine with mixed heads, a gate a head, q/k norms or values that are the keys")
            if self.value_rotation and self.value_dim % 2:
                raise ValueError(f"values of odd size {self.value_dim} cannot be turned in pairs")
            if carry and (self.value_rotation or self.borrows_keys):
                raise ValueError("carried values are neither turned nor borrowed")
        self.inv_freq_v = self.b_qkv = self.b_out = self.carry_blend = None

    @property
    def out_dim(self) -> int:
        return self.num_heads * self.value_dim

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    def weight_specs(self, present=None):
        H, sfx = self.hidden_size, self.suffix
        if self.flex:
            out = [TensorSpec(self.n["q"] + sfx, (self.q_dim, H))]
            if not self.borrows_keys:
                out += [TensorSpec(self.n["k"] + sfx, (self.kv_dim, H)),
                        TensorSpec(self.n["v"] + sfx, (self.num_kv_heads * self.value_dim, H))]
            if self.entry_gate_name:
                out.append(TensorSpec(self.entry_gate_name + sfx, (self.out_dim, H)))
            out.append(TensorSpec(self.n["out"] + sfx, (H, self.out_dim)))
            if self.bias:
                sizes = {"q": self.q_dim, "k": self.kv_dim, "v": self.num_kv_heads * self.value_dim, "out": H}
                out += [TensorSpec(self.n[x] + self.bias_suffix, (sizes[x],), "vector", "bias")
                        for x in (("q", "out") if self.borrows_keys else ("q", "k", "v", "out"))]
            if self.carry_blend_name:
                out.append(TensorSpec(self.carry_blend_name, (), "vector", "bias"))
            return out
        out = [TensorSpec(self.n["q"] + sfx, (self.q_dim, H)), TensorSpec(self.n["k"] + sfx, (self.kv_dim, H))]
        if self.values == "projected":
            out.append(TensorSpec(self.n["v"] + sfx, (self.kv_dim, H)))
        out.append(TensorSpec(self.n["out"] + sfx, (H, self.q_dim)))
        if self.head_mix_name:
            out.append(TensorSpec(self.head_mix_name, (self.num_heads, self.num_heads), role="vector", init="mix"))
        if self.gate_name:
            out.append(TensorSpec(self.gate_name, (self.num_heads, H)))
        if self.q_norm:
            out += self.q_norm.weight_specs() + self.k_norm.weight_specs()
        return out

    def bind(self, read, runtime):
        self.runtime = runtime
        sfx = self.suffix
        if self.flex:
            # one product for everything that reads the normed row: q, then k and v (unless borrowed), then the gate; every
            # part begins at a multiple of 8 columns
            parts = ["q"] + ([] if self.borrows_keys else ["k", "v"])
            mats = [(x, runtime.matrix(read(self.n[x] + sfx))) for x in parts]
            if self.entry_gate_name:
                mats.append(("gate", runtime.matrix(read(self.entry_gate_name + sfx))))
            rows, self.col, at = [], {}, 0
            for name, m in mats:
                self.col[name] = at
                pad = -m.shape[0] % 8
                rows += [m, torch.zeros(pad, m.shape[1], dtype=m.dtype, device=m.device)] if pad else [m]
                at += m.shape[0] + pad
            self.w_qkv = torch.cat(rows).contiguous()
            self.w_out = runtime.matrix(read(self.n["out"] + sfx))
            if self.bias:       # the fused product's bias: every part's own at the part's columns, zero at the gate's and the fill
                self.b_qkv = torch.zeros(self.w_qkv.shape[0], dtype=torch.float32, device=runtime.device)
                for x in parts:
                    b = runtime.vector(read(self.n[x] + self.bias_suffix))
                    self.b_qkv[self.col[x]:self.col[x] + b.shape[0]] = b
                self.b_out = runtime.vector(read(self.n["out"] + self.bias_suffix))
            if self.carry_blend_name:
                self.carry_blend = runtime.vector(read(self.carry_blend_name)).reshape(1)
            self.position.bind(read, runtime)
            if self.value_rotation:
                vd = self.value_dim
                f = float(self.value_rotation) ** (-torch.arange(0, vd, 2, dtype=torch.float64) / vd)
                self.inv_freq_v = f.to(torch.float32).to(runtime.device)
            return
        rows = [runtime.matrix(read(self.n[x] + sfx)) for x in (("q", "k", "v") if self.values == "projected" else ("q", "k"))]
        self.gate_at = sum(r.shape[0] for r in rows)        # the column of the fused product where the gates' logits begin
        if self.gate_name:
            # the gate's rows ride at the end of the fused product, filled up with zero rows to a multiple of 8 so that a
            # row of the product keeps the 16-byte alignment the vector loads and stores want
            g = runtime.matrix(read(self.gate_name))
            pad = -(self.gate_at + g.shape[0]) % 8
            rows += [g, torch.zeros(pad, g.shape[1], dtype=g.dtype, device=g.device)] if pad else [g]
        self.w_qkv = torch.cat(rows).contiguous()
        self.w_out = runtime.matrix(read(self.n["out"] + sfx))
        if self.head_mix_name:
            self.head_mix = runtime.vector(read(self.head_mix_name))
        if self.q_norm:
            self.q_norm.bind(read, runtime)
            self.k_norm.bind(read, runtime)
        self.position.bind(read, runtime)

    def cache_need(self):
        if self.flex:
            return PagedNeed(self.num_kv_heads, self.head_dim, self.cache_window,
                             value_dim=self.value_dim if self.value_dim != self.head_dim else None,
                             keep_first=self.cache_keep_first if self.cache_window else 0)
        return PagedNeed(self.num_kv_heads, self.head_dim, self.window)

    def forward_inner(self, x, step, cache, writes_cache: bool, out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
        """The concatenated heads (gated, times `out_scale`) into `out` [rows, heads * value_dim], which may be a column
        slice of a wider tensor: what the out projection `w_out` is applied to."""
        if not self.flex:
            raise NotImplementedError("the concatenated heads of this combination of options are not handed out")
        R, dt, dev = x.shape[0], x.dtype, x.device
        Hq, Hk, D, VD = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        status = self.runtime.status
        qkv = linear(self.runtime, x, self.w_qkv, self.b_qkv)
        q = torch.empty(R, Hq, D, dtype=dt, device=dev)
        table = step.block_tables[cache.group]
        inv_freq, rot = self.position.fused_rotary()
        own = writes_cache and not self.borrows_keys
        v_other = None
        if self.carry_key is not None:
            # the step's first layer with this key leaves its values for the later ones, which blend theirs with them
            mine = qkv[:, self.col["v"]:self.col["v"] + Hk * VD]
            v_other = step.carried.get(self.carry_key) if self.carry_blend is not None else None
            if self.carry_blend is None:
                step.carried[self.carry_key] = mine
            elif v_other is None:
                raise RuntimeError(f"{self.prefix}: values to blend with under {self.carry_key!r}, and no earlier layer left any")
        ops.qkv_rotate_store(qkv, self.col["q"], self.col["k"] if own else -1, self.col["v"] if own else -1, inv_freq, rot,
                             self.inv_freq_v, step.positions, step.req_of_row, table, cache.page_size, q,
                             cache.k if own else None, cache.v if own else None, Hq, Hk, D, VD, status,
                             float(getattr(self.position, "magnitude", 1.0)), v_other, self.carry_blend)
        gate = qkv[:, self.col["gate"]:] if self.entry_gate_name else None
        fast = self.runtime.attention_kernels
        if fast is not None and hasattr(fast, "attention_flex") and fast.attention_flex(self, q, cache, table, step, gate,
                                                                                       qkv.stride(0), out_scale, out):
            return out
        return ops.attention_flex(q, cache.k, cache.v, table, cache.page_size, step.req_of_row, step.positions, self.scale,
                                  self.softcap, self.window, self.keep_first, self.inv_freq_v, gate, qkv.stride(0), out_scale,
                                  out, status)

    def forward(self, x, step, cache, writes_cache: bool = True):
        if self.flex:
            o = torch.empty(x.shape[0], self.out_dim, dtype=x.dtype, device=x.device)
            self.forward_inner(x, step, cache, writes_cache, o)
            return linear(self.runtime, o, self.w_out, self.b_out, out_dtype=torch.float32, defer=True)
        R, dt, dev = x.shape[0], x.dtype, x.device
        Hq, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        status = self.runtime.status
        qkv = linear(self.runtime, x, self.w_qkv)
        q = torch.empty(R, Hq, D, dtype=dt, device=dev)
        table = step.block_tables[cache.group]
        qw = self.q_norm.weight if self.q_norm else None
        kw = self.k_norm.weight if self.k_norm else None
        eps = self.q_norm.eps if self.q_norm else 0.0
        fused = self.position.fused_rotary()
        if fused is not None and writes_cache:
            inv_freq, rot = fused
            ops.qk_prepare(qkv, qw, kw, eps, inv_freq, rot, step.positions, step.req_of_row, table, cache.page_size,
                           q, cache.k, cache.v, None, None, Hq, Hk, D, status, self.qk_flags)
        else:
            k = torch.empty(R, Hk, D, dtype=dt, device=dev)
            v = torch.empty(R, Hk, D, dtype=dt, device=dev)
            inv_freq, rot = fused if fused is not None else (None, 0)
            ops.qk_prepare(qkv, qw, kw, eps, inv_freq, rot, step.positions, step.req_of_row, None, 0,
                           q, None, None, k, v, Hq, Hk, D, status, self.qk_flags)
            if fused is None:
                self.position.apply(q, k, step.positions)
            if writes_cache:
                ops.kv_store(k, v, step.positions, step.req_of_row, table, cache.page_size, cache.k, cache.v, status)
        o = torch.empty(R, Hq, D, dtype=dt, device=dev)
        fast = self.runtime.attention_kernels
        if self.head_mix is not None or self.gate_name:
            # the heads' weights are mixed after the softmax (and the output gated a head): kernels of their own
            gate = qkv[:, self.gate_at:] if self.gate_name else None
            if fast is None or not fast.attention_headmix(q, cache, table, step, self.scale, self.window, self.head_mix, gate,
                                                          qkv.stride(0), o, self.runtime):
                ops.attention_headmix(q, cache.k, cache.v, table, cache.page_size, step.req_of_row, step.positions,
                                      self.scale, self.window, self.head_mix, gate, qkv.stride(0), o, step.max_context,
                                      self.runtime, status)
        elif fast is None or not fast.attention(q, cache, table, step, self.scale, self.window, o, self.runtime):
            spans = ops.attention_spans(step.max_context)
            scratch = self.runtime.scratch("attention", ops.attention_scratch_floats(R, Hq, D, spans))
            ops.paged_attention_split(q, cache.k, cache.v, table, cache.page_size, step.req_of_row, step.positions,
                                      self.scale, self.window, o, scratch, spans, status)
        return linear(self.runtime, o.view(R, Hq * D), self.w_out, out_dtype=torch.float32, defer=True)
