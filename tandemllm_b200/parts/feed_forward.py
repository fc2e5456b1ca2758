"""Feed-forward parts: the dense gated feed-forward (SwiGLU) and the routed top-k gated experts.

  dense    out = down( act(gate n) * (up n) ), act = silu             engine/models/lfm2_moe/ref.py:180-183
  experts  logits = router(n) in 32-bit; s = sigmoid(logits); the choice is the top-k of s + expert_bias
           (the bias for the choice only); w = s[chosen], divided by (sum w + norm_floor) when normalised,
           times scale; out = sum over the chosen experts in ascending expert id of w * expert(n)
                                                                         ref.py:185-214

The gate's activation (`activation`: silu, gelu, relu2, identity) and the router's scoring function (`scoring`:
sigmoid, or softmax over all experts) are parameters of the parts' specs, passed to the kernels as codes; LFM2 uses
silu and sigmoid, and another architecture's gated or routed feed-forward reuses the same fused kernels by naming its own.

Gate and up are fused into one matrix at bind time ([2I, H], gate first), per expert for the experts
([E, 2I, H] and [E, H, I], engine/models/lfm2_moe/load.py:136-161). Experts may be stored one by one
(`<experts>.<e>.<gate|up|down>.weight`) or stacked (`<experts>.gate_up_proj [E, 2I, H]`,
`<experts>.down_proj [E, H, I]`); what the folder holds decides. Routing never leaves the device: the
plan of (row, slot) pairs sorted by expert and its tile map are built by kernels, and the expert
products skip experts nobody chose.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import FEED_FORWARDS, Part, register_part
from .linear import linear

def gate_constants_of(spec):
    """The constants of a gate form that has some, from a part's spec: `clamped_swish` reads `gate_limit` and `gate_slope`
    (g' = min(g, limit), u' = clamp(u, -limit, limit), out = g' sigmoid(slope g') (u' + 1)); None for the others."""
    if spec.get("activation", "silu") != "clamped_swish":
        return None
    return float(spec["gate_limit"]), float(spec.get("gate_slope", 1.702))


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.inter = int(spec["intermediate_size"])
        self.act = ops.activation_code(spec.get("activation", "silu"))
        self.gate_constants = gate_constants_of(spec)
        self.suffix = str(spec.get("weight_suffix", ".weight"))
        self.n = {k: prefix + v for k, v in spec["names"].items()}

    def weight_specs(self, present=None):
        H, I, sfx = self.hidden_size, self.inter, self.suffix
        return [TensorSpec(self.n["gate"] + sfx, (I, H)), TensorSpec(self.n["up"] + sfx, (I, H)),
                TensorSpec(self.n["down"] + sfx, (H, I))]

    def bind(self, read, runtime):
        self.runtime = runtime
        sfx = self.suffix
        self.w_gate_up = torch.cat([runtime.matrix(read(self.n["gate"] + sfx)),
                                    runtime.matrix(read(self.n["up"] + sfx))]).contiguous()
        self.w_down = runtime.matrix(read(self.n["down"] + sfx))

    def forward(self, x, step):
        act = torch.empty(x.shape[0], self.inter, dtype=x.dtype, device=x.device)
        tc = self.runtime.tensorcore
        if self.gate_constants is not None:
            ops.gate_constants(*self.gate_constants)
        if tc is None or not tc.gated(x, self.w_gate_up, act, self.act):      # prompts: gate, up and act(gate) * up in one kernel
            gu = linear(self.runtime, x, self.w_gate_up)
            ops.gated_mul(gu, act, self.act)
        return linear(self.runtime, act, self.w_down, out_dtype=torch.float32, defer=True)


@register_part("feed_forward", "dense_act")
class DenseActivation(Part):
    """The ungated dense feed-forward: out = down( act(up n) ). `activation` names the function (a name of
    `ops.ACTIVATIONS`); `xielu` reads its two numbers (p, q) from the tensor `act_params` names and uses
    softplus(p) z^2 + z / 2 for z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise. The two factors are
    formed once at bind time, in 32-bit, and travel to the kernels as plain numbers."""
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.inter = int(spec["intermediate_size"])
        self.activation = str(spec.get("activation", "gelu"))
        self.act = ops.activation_code(self.activation)
        self.n = {k: prefix + v for k, v in spec["names"].items()}
        self.a0 = self.a1 = 0.0

    def weight_specs(self, present=None):
        H, I = self.hidden_size, self.inter
        out = [TensorSpec(self.n["up"], (I, H)), TensorSpec(self.n["down"], (H, I))]
        if self.activation == "xielu":
            out.append(TensorSpec(self.n["act_params"], (2,), role="vector", init="bias"))
        return out

    def bind(self, read, runtime):
        self.runtime = runtime
        self.w_up = runtime.matrix(read(self.n["up"]))
        self.w_down = runtime.matrix(read(self.n["down"]))
        if self.activation == "xielu":
            pq = read(self.n["act_params"]).to(torch.float32).cpu()
            sp = torch.nn.functional.softplus(pq)
            self.a0, self.a1 = float(sp[0]), float(0.5 + sp[1])

    def forward(self, x, step):
        tc = self.runtime.tensorcore
        if tc is not None and x.dtype == torch.bfloat16:
            act = tc.linear_act(x, self.w_up, self.act, self.a0, self.a1)
            if act is not None:
                return linear(self.runtime, act, self.w_down, out_dtype=torch.float32, defer=True)
        act = linear(self.runtime, x, self.w_up)
        ops.activation(act, act, self.act, self.a0, self.a1)
        return linear(self.runtime, act, self.w_down, out_dtype=torch.float32, defer=True)


@register_part("feed_forward", "none")
class NoFeedForward(Part):
    """A layer without a feed-forward: the mixer's output goes on, unadded, to the next layer's first norm."""
    graph_safe = True
    absent = True

    def forward(self, x, step):
        return None

    def forward_from(self, norm, residual, delta, step):
        return delta


@register_part("feed_forward", "sigmoid_topk_experts")
class SigmoidTopKExperts(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.num_experts = int(spec["num_experts"])
        self.top_k = int(spec["top_k"])
        self.inter = int(spec["intermediate_size"])
        self.use_bias = bool(spec.get("expert_bias", True))
        self.normalize = bool(spec.get("normalize", True))
        self.scale = float(spec.get("scale", 1.0))
        self.norm_floor = float(spec.get("norm_floor", 1e-6))
        self.scoring = str(spec.get("scoring", "sigmoid"))
        self.groups = tuple(int(v) for v in spec["groups"]) if spec.get("groups") else None     # (count, how many are kept)
        if self.groups is not None and self.num_experts % self.groups[0]:
            raise ValueError(f"{self.num_experts} experts do not fall into {self.groups[0]} equal groups")
        ops.route_flags(self.normalize, self.scoring, self.groups)      # an unknown scoring function is refused here
        self.act = ops.activation_code(spec.get("activation", "silu"))
        self.gate_constants = gate_constants_of(spec)
        self.suffix = str(spec.get("weight_suffix", ".weight"))
        self.sep = str(spec.get("expert_separator", "."))       # between the experts' common name and an expert's number
        if not 0 < self.top_k <= self.num_experts:
            raise ValueError(f"top-{self.top_k} of {self.num_experts} experts")
        if self.num_experts > 1024 or self.top_k > 32:
            raise ValueError(f"{self.num_experts} experts top-{self.top_k}: up to 1024 experts and top-32 are implemented")
        self.n = dict(spec["names"])
        self.base = prefix + self.n["experts"]
        self._plans: dict[int, ops.MoePlan] = {}
        self._outgrown: list[ops.MoePlan] = []
        self.stacked = False
        self.load = None            # see `count_into`

    def _stacked(self, present) -> bool:
        return present is not None and (self.base + ".gate_up_proj") in present

    def weight_specs(self, present=None):
        H, I, E = self.hidden_size, self.inter, self.num_experts
        out = [TensorSpec(self.prefix + self.n["router"] + self.suffix, (E, H))]
        if self.use_bias:
            out.append(TensorSpec(self.prefix + self.n["bias"], (E,), "vector", "bias"))
        self.stacked = self._stacked(present)
        if self.stacked:
            out += [TensorSpec(self.base + ".gate_up_proj", (E, 2 * I, H)), TensorSpec(self.base + ".down_proj", (E, H, I))]
        else:
            for e in range(E):
                out += [TensorSpec(self._expert(e, "gate"), (I, H)), TensorSpec(self._expert(e, "up"), (I, H)),
                        TensorSpec(self._expert(e, "down"), (H, I))]
        return out

    def _expert(self, e: int, which: str) -> str:
        return f"{self.base}{self.sep}{e}.{self.n[which]}{self.suffix}"

    def bind(self, read, runtime):
        self.runtime = runtime
        H, I, E = self.hidden_size, self.inter, self.num_experts
        # the router's product is 32-bit in both precisions: its weights are kept in 32-bit (E x H is small)
        self.w_router = runtime.vector(read(self.prefix + self.n["router"] + self.suffix))
        self.expert_bias = runtime.vector(read(self.prefix + self.n["bias"])) if self.use_bias else None
        if self.stacked:
            self.w_gate_up = runtime.matrix(read(self.base + ".gate_up_proj"))
            self.w_down = runtime.matrix(read(self.base + ".down_proj"))
        else:
            self.w_gate_up = torch.empty(E, 2 * I, H, dtype=runtime.dtype, device=runtime.device)
            self.w_down = torch.empty(E, H, I, dtype=runtime.dtype, device=runtime.device)
            for e in range(E):
                self.w_gate_up[e, :I].copy_(read(self._expert(e, "gate")))
                self.w_gate_up[e, I:].copy_(read(self._expert(e, "up")))
                self.w_down[e].copy_(read(self._expert(e, "down")))

    def expected_experts_read(self, rows: int) -> float:
        """Distinct experts that `rows` rows choose when every expert is as likely as any other."""
        E, k = self.num_experts, self.top_k
        return E * (1.0 - (1.0 - k / E) ** rows)

    def step_bytes(self, elem: int, experts_read: float | None = None, rows: int = 1, **_) -> int:
        """The router (32-bit) and the expert bias, and `experts_read` experts' matrices (default: the expected number
        of distinct experts `rows` rows choose)."""
        H, I, E = self.hidden_size, self.inter, self.num_experts
        n = self.expected_experts_read(rows) if experts_read is None else experts_read
        return int(E * H * 4 + (E * 4 if self.use_bias else 0) + n * 3 * H * I * elem)

    def count_into(self, counts: torch.Tensor | None) -> None:
        """From now on every pass adds the pairs it routed to each expert to `counts` (an integer tensor [experts] on
        the device; None stops it). The adding is a kernel of the pass, so it also happens in steps replayed from CUDA
        graphs that were captured while it was on; the engine drops its graphs when it switches this."""
        self.load = counts

    def forward_from(self, norm, residual, delta, step):
        """The norm in front and this layer in one go. The router's logits are 32-bit end to end: for few rows the norm
        kernel runs the router itself on its unrounded output as it goes; for many, it also hands the unrounded rows."""
        route = self.router_args(residual.shape[-2], residual.device)
        if route is not None:
            x = norm.add_norm(residual, delta, route=route)
            return self.forward(x, step, routing=(route["ids"], route["wts"]))
        x, x32 = norm.add_norm(residual, delta, want32=True)
        return self.forward(x, step, x32=x32)

    def router_args(self, rows: int, device):
        """What the norm kernel in front of the layer needs to run this layer's router on its `rows` output rows
        (for many rows the kernel norms several rows per block, so the router's weights are read once per block)."""
        return {"weight": self.w_router, "bias": self.expert_bias, "k": self.top_k, "normalize": self.normalize,
                "scoring": self.scoring, "groups": self.groups, "floor": self.norm_floor, "scale": self.scale,
                "ids": torch.empty(rows, self.top_k, dtype=torch.int32, device=device),
                "wts": torch.empty(rows, self.top_k, dtype=torch.float32, device=device)}

    def route(self, x32):
        """(ids int32 [R, k], weights float32 [R, k]) of the 32-bit rows x32."""
        R = x32.shape[0]
        logits = ops.gemm_simt(x32, self.w_router, None, torch.empty(R, self.num_experts, dtype=torch.float32,
                                                                      device=x32.device))
        ids = torch.empty(R, self.top_k, dtype=torch.int32, device=x32.device)
        wts = torch.empty(R, self.top_k, dtype=torch.float32, device=x32.device)
        ops.router_topk(logits, self.expert_bias, self.top_k, self.normalize, self.norm_floor, self.scale, ids, wts,
                        self.scoring, self.groups)
        return ids, wts

    def plan_for(self, pairs: int, device, tile_rows: int | None = None) -> ops.MoePlan:
        """The routing-plan buffers for up to `pairs` pairs and token tiles of `tile_rows` rows (kept and reused)."""
        tile_rows = tile_rows or ops.simt_tile_rows()
        plan = self._plans.get(tile_rows)
        if plan is None or plan.max_pairs < pairs:
            cap = max(pairs, 64) if plan is None else max(pairs, 2 * plan.max_pairs)
            if plan is not None:
                self._outgrown.append(plan)         # a captured decode graph may still use the smaller plan's buffers
            plan = self._plans[tile_rows] = ops.MoePlan(cap, self.num_experts, tile_rows, device)
        return plan

    def forward(self, x, step, x32=None, routing=None):
        """The layer's output as `ops.ExpertRows`: one 32-bit row per (row, slot) pair, which the consuming norm
        kernel weighs and adds in ascending expert id. `routing` = (ids, wts) when the norm in front already ran
        the router; else it runs here, on `x32` (the unrounded normed rows) where given."""
        R, H = x.shape[0], self.hidden_size
        ids, wts = routing if routing is not None else self.route(x32 if x32 is not None else x.float())
        if step is not None and step.trace is not None:
            step.trace.setdefault("routes", []).append((self.prefix, ids))
        tc = self.runtime.tensorcore
        if self.gate_constants is not None:
            ops.gate_constants(*self.gate_constants)
        if tc is not None and x.dtype == torch.bfloat16:
            rows = tc.experts(self, x, ids, wts)
            if rows is not None:
                return rows
        plan = self.plan_for(R * self.top_k, x.device).build(ids)
        if self.load is not None:
            self.load.add_(plan.counts)
        act = torch.empty(R * self.top_k, self.inter, dtype=x.dtype, device=x.device)
        ops.gemm_simt_grouped(x, plan.sorted_pairs, self.top_k, self.w_gate_up, act, plan, swiglu=self.act)
        y = torch.empty(R * self.top_k, H, dtype=torch.float32, device=x.device)
        ops.gemm_simt_grouped(act, None, 1, self.w_down, y, plan, swiglu=False)
        return ops.ExpertRows(y, plan.pos_of_pair, ids, wts)


@register_part("feed_forward", "shared_and_routed")
class SharedAndRouted(Part):
    """A routed feed-forward beside a dense one that every row uses: out = routed(n) + sigmoid(gate n) * shared(n), the gate
    one number a row (`shared_gate`: the name of its [1, hidden] matrix; None: no gate). `routed` and `shared` are specs of
    feed-forward kinds of their own. The sum is not formed here: the three pieces go on as `ops.GatedSum`, which a norm
    behind the branch adds in its own kernel (`ops.materialize` forms it for anything else)."""

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.routed = FEED_FORWARDS[spec["routed"].kind](spec["routed"], prefix=prefix, hidden_size=hidden_size)
        self.shared = FEED_FORWARDS[spec["shared"].kind](spec["shared"], prefix=prefix, hidden_size=hidden_size)
        self.gate_name = prefix + spec["shared_gate"] if spec.get("shared_gate") else None
        self.w_gate = None

    @property
    def graph_safe(self) -> bool:
        return self.routed.graph_safe and self.shared.graph_safe

    def weight_specs(self, present=None):
        out = self.routed.weight_specs(present) + self.shared.weight_specs(present)
        if self.gate_name:
            out.append(TensorSpec(self.gate_name, (1, self.hidden_size)))
        return out

    def bind(self, read, runtime):
        self.runtime = runtime
        self.routed.bind(read, runtime)
        self.shared.bind(read, runtime)
        if self.gate_name:
            self.w_gate = runtime.matrix(read(self.gate_name))

    # the routed part's accounts and records are this part's
    def expected_experts_read(self, rows: int) -> float:
        return self.routed.expected_experts_read(rows)

    def step_bytes(self, elem: int, experts_read: float | None = None, rows: int = 1, **_) -> int:
        return (self.routed.step_bytes(elem, experts_read=experts_read, rows=rows) + self.shared.step_bytes(elem)
                + (self.hidden_size * elem if self.gate_name else 0))

    def count_into(self, counts) -> None:
        self.routed.count_into(counts)

    @property
    def num_experts(self) -> int:
        return self.routed.num_experts

    def router_args(self, rows: int, device):
        return self.routed.router_args(rows, device)

    def forward_from(self, norm, residual, delta, step):
        route = self.routed.router_args(residual.shape[-2], residual.device)
        x = norm.add_norm(residual, delta, route=route)
        return self.forward(x, step, routing=(route["ids"], route["wts"]))

    def forward(self, x, step, routing=None):
        routed = self.routed.forward(x, step, routing=routing)
        shared = self.shared.forward(x, step)
        gate = None
        if self.w_gate is not None:
            gate = ops.row_dot(x, self.w_gate, torch.empty(x.shape[0], 1, dtype=torch.float32, device=x.device))
        return ops.GatedSum(shared, gate, routed)
