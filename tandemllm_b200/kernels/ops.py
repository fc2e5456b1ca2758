"""Python entry points of the CUDA kernels: tensors in, launches on torch's current stream.

Each function checks what the kernel cannot (device, dtype, contiguity), passes raw pointers and the
stream handle through ctypes, and raises `KernelError` with the library's own message when a launcher
refuses its arguments. There is no fallback: a missing library is an error at load time.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load

FP32, BF16 = 0, 1
TL_BAD_ARGUMENT = 100001
# the gate activations of gated products (TL_ACT_* of csrc/common.cuh) and the router's scoring functions (TL_SCORE_*
# of csrc/route.cuh), by the names a part's spec gives them
ACTIVATIONS = {"silu": 1, "gelu": 2, "relu2": 3, "identity": 4, "xielu": 5, "clamped_swish": 6, "softcap": 7, "tanh": 8, "scale": 9}
SCORINGS = {"sigmoid": 0, "softmax": 1}


def activation_code(name: str) -> int:
    if name not in ACTIVATIONS:
        raise KernelError(f"gate activation {name!r}: one of {', '.join(ACTIVATIONS)}")
    return ACTIVATIONS[name]


def route_flags(normalize: bool, scoring: str = "sigmoid", groups: tuple[int, int] | None = None) -> int:
    """The routers' `normalize` argument: bit 0 = divide the chosen weights by their sum, bits 1..3 = the scoring function,
    bits 4..9 = the number of expert groups and bits 10..15 = how many of them are kept (`groups` = (count, keep); None: the
    choice is free)."""
    if scoring not in SCORINGS:
        raise KernelError(f"router scoring function {scoring!r}: one of {', '.join(SCORINGS)}")
    count, keep = groups or (0, 0)
    if groups is not None and not (1 <= keep <= count <= 32):
        raise KernelError(f"router groups: {keep} of {count} kept; 1 <= keep <= count <= 32")
    return int(bool(normalize)) | (SCORINGS[scoring] << 1) | (count << 4) | (keep << 10)


def gate_constants(a0: float, a1: float) -> None:
    """The constants of a gate form that has some (`clamped_swish`: the limit and the slope) for the gated launches this
    thread makes from now on, in every loaded library."""
    core().tl_set_gate_constants(float(a0), float(a1))
    from . import tensorcore
    if tensorcore.loaded():
        tensorcore.lib().tl_tc_set_gate_constants(float(a0), float(a1))


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return FP32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dtype} is not implemented; float32 and bfloat16 are")


_SIGNATURES = {
    "tl_embed_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p],
    "tl_embed_rows_copies": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_int, c_longlong,
                             c_void_p],
    "tl_add_rmsnorm_streams": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p,
                               c_int, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_float, c_float, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p],
    "tl_add_rmsnorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                       c_void_p,
                       c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                       c_float, c_float, c_void_p, c_void_p, c_void_p],
    "tl_gated_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "tl_gemm_simt": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int,
                     c_int, c_int, c_void_p],
    "tl_gemm_simt_grouped": [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p,
                             c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_int, c_void_p],
    "tl_gemm_simt_tile_rows": [],
    "tl_short_conv": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_int, c_int, c_void_p],
    "tl_short_conv_decode": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tl_short_conv_state": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "tl_qk_prepare": [c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                      c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_void_p, c_void_p],
    "tl_add_dyt": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                   c_int, c_void_p],
    "tl_activation": [c_void_p, c_void_p, c_longlong, c_int, c_float, c_float, c_int, c_void_p],
    "tl_headmix_spans": [c_int, c_int, c_int],
    "tl_attention_headmix": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
                             c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_void_p, c_void_p],
    "tl_kv_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_void_p, c_void_p],
    "tl_paged_attention_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "tl_attention_spans": [c_int],
    "tl_paged_attention_split": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "tl_attention_join": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tl_router_topk": [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p,
                       c_void_p],
    "tl_moe_max_tiles": [c_int, c_int, c_int],
    "tl_moe_plan_copies_rows": [c_int, c_int],
    "tl_moe_plan": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p],
    "tl_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "tl_argmax": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p],
    "tl_add_normed": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p,
                      c_int, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "tl_add_vector": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "tl_row_dot": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "tl_causal_conv_act": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_longlong, c_int, c_int, c_int, c_int, c_void_p],
    "tl_conv_state": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "tl_ssm_scan": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "tl_gated_group_norm": [c_void_p, c_void_p, c_longlong, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "tl_latent_prepare": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                          c_void_p],
    "tl_rmsnorm_rows": [c_void_p, c_longlong, c_void_p, c_float, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p],
    "tl_head_linear": [c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_int,
                       c_int, c_int, c_void_p, c_longlong, c_void_p],
    "tl_attention_latent": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "tl_add_layernorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                         c_int, c_void_p],
    "tl_qkv_rotate_store": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_float, c_void_p, c_longlong, c_void_p, c_void_p],
    "tl_attention_flex": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_float,
                          c_int, c_int, c_void_p, c_void_p, c_longlong, c_float, c_void_p, c_longlong, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_void_p, c_void_p],
    "tl_recurrence_scan": [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                           c_float, c_float, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                           c_int, c_int, c_void_p, c_longlong, c_int, c_int, c_float, c_void_p],
    "tl_recurrence_scratch_floats": [c_longlong, c_int, c_int, c_int, c_int],
    "tl_group_norm_gate": [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_float, c_float, c_void_p, c_longlong, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tl_set_gate_constants": [c_float, c_float],
    "tl_graph_capture_begin": [c_void_p],
    "tl_graph_capture_end": [c_void_p, c_void_p, c_void_p],
    "tl_graph_launch": [c_void_p, c_void_p],
    "tl_graph_destroy": [c_void_p],
    "tl_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p],
    "tl_penalize": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "tl_count_tokens": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p],
}

_core = None


def core():
    """The loaded core library with its signatures declared (built at the first call)."""
    global _core
    if _core is None:
        lib = load("core")
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        lib.tl_headmix_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
        lib.tl_headmix_scratch_floats.restype = c_longlong
        lib.tl_recurrence_scratch_floats.restype = c_longlong
        lib.tl_ssm_scan_scratch.argtypes = [c_int, c_int, c_int, c_int, c_int]
        lib.tl_ssm_scan_scratch.restype = c_longlong
        lib.tl_last_error.restype = ctypes.c_char_p
        lib.tl_cuda_error_string.restype = ctypes.c_char_p
        lib.tl_cuda_error_string.argtypes = [c_int]
        _core = lib
    return _core


launches = 0        # kernels of this package launched so far (a launcher that starts two kernels counts both)


def check(code: int, what: str, lib=None, kernels: int = 1) -> None:
    global launches
    if code == 0:
        launches += kernels
        return
    lib = lib or core()
    if code == TL_BAD_ARGUMENT:
        raise KernelError(lib.tl_last_error().decode())
    raise KernelError(f"{what}: CUDA error {code}: {core().tl_cuda_error_string(code).decode()}")


# The current stream's handle is asked for once a launch: through torch's own C entry points where it has them (a
# fraction of a microsecond), else through `torch.cuda.current_stream()`, whose Python checks cost more than the launch.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def stream() -> int:
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA tensors only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} is {t.dtype}, expected {dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


# ------------------------------------------------------------------------------------------ rows
def embed_rows(table: torch.Tensor, tokens: torch.Tensor, residual: torch.Tensor, status: torch.Tensor,
               scale: float = 1.0) -> None:
    """residual[r] = table[tokens[r]] * scale in 32-bit; a residual of several streams [streams, rows, hidden] gets the row in
    every stream."""
    _need(table, None, "embedding table"); _need(tokens, torch.int32, "tokens"); _need(residual, torch.float32, "residual")
    copies = residual.shape[0] if residual.dim() == 3 else 1
    rows, hidden = residual.shape[-2:]
    check(core().tl_embed_rows_copies(ptr(table), ptr(tokens), ptr(residual), rows, hidden, table.shape[0],
                                      dtype_code(table.dtype), ptr(status), float(scale), copies, rows * hidden, stream()),
          "embed_rows")


class PartialSums:
    """A product's output still in `parts` partial sums [parts, rows, hidden] (32-bit), to be added in order and, when
    `dtype` is given, rounded to it (what the product's own reduction would have stored)."""

    def __init__(self, data: torch.Tensor, parts: int, rows: int, hidden: int, dtype: torch.dtype | None = None):
        self.data, self.parts, self.rows, self.hidden, self.dtype = data, parts, rows, hidden, dtype

    def materialize(self) -> torch.Tensor:
        parts = self.data[:self.parts * self.rows * self.hidden].view(self.parts, self.rows, self.hidden)
        total = torch.zeros_like(parts[0])
        for part in parts:
            total += part
        return total if self.dtype is None else total.to(self.dtype)


class ExpertRows:
    """A routed expert layer's output still as one row per (row, slot) pair in expert-sorted order [pairs, hidden]
    (32-bit), with what is needed to weigh and add them per row."""

    def __init__(self, rows: torch.Tensor, pos_of_pair: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, parts: int = 1):
        """`parts` > 1: `rows` is [parts, pairs, hidden], partial sums of a down projection split along k."""
        self.rows, self.pos_of_pair, self.ids, self.wts, self.parts = rows, pos_of_pair, ids, wts, parts

    def materialize(self) -> torch.Tensor:
        rows = self.rows
        if self.parts > 1:
            rows = rows[0].clone()
            for part in self.rows[1:]:
                rows += part
        out = torch.empty(self.ids.shape[0], rows.shape[-1], dtype=torch.float32, device=rows.device)
        check(core().tl_moe_combine(ptr(rows), ptr(self.pos_of_pair), ptr(self.ids), ptr(self.wts), ptr(out),
                                    out.shape[0], out.shape[1], self.ids.shape[1], stream()), "moe_combine")
        return out


class GatedSum:
    """A branch output in three pieces: dense [rows, hidden] (a tensor or `PartialSums`) times sigmoid(gate[r]) (float32
    [rows, 1] logits; None: no gate), plus the weighed rows of `experts` (`ExpertRows` or None)."""

    def __init__(self, dense, gate: torch.Tensor | None, experts: "ExpertRows | None"):
        self.dense, self.gate, self.experts = dense, gate, experts

    def materialize(self) -> torch.Tensor:
        total = materialize(self.dense).float()
        if self.gate is not None:
            total = total * torch.sigmoid(self.gate.view(-1, 1))
        return total if self.experts is None else total + self.experts.materialize()


class StreamUpdate:
    """What a sublayer leaves for a residual of several streams [streams, rows, hidden] (hyper-connections): its output `delta`
    (None, a tensor or a deferred form) with the weights that take it into the streams, all streams at once from the old
    ones, x_t <- sum_s mix[s, t] x_s + out[t] delta (`mix` float32 [streams, streams], `out` float32 [streams]; both None:
    nothing is added yet), and the weights `read` (float32 [streams]; None: all one) with which the next norm sums the
    streams into the row it norms. The norm kernel does all of it."""

    def __init__(self, delta, mix: torch.Tensor | None, out: torch.Tensor | None, read: torch.Tensor | None = None):
        self.delta, self.mix, self.out, self.read = delta, mix, out, read

    def reading(self, read: torch.Tensor | None) -> "StreamUpdate":
        return StreamUpdate(self.delta, self.mix, self.out, read)


def materialize(branch):
    """A branch output as a plain tensor, whatever form a part returned it in."""
    return branch.materialize() if isinstance(branch, (PartialSums, ExpertRows, GatedSum)) else branch


def add_rmsnorm(residual: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor,
                gather: torch.Tensor | None = None, out32: torch.Tensor | None = None, route: dict | None = None
                ) -> torch.Tensor:
    """residual += delta (32-bit); out = weight * rms_normalised(residual). `delta` is None, a float32 tensor, a
    `PartialSums` or an `ExpertRows`. With `gather` (int32 row indices) the output row i is computed from row
    gather[i] and the residual is left unchanged. `out32` also receives the normalised rows unrounded. `route`
    (router weights float32 [E, hidden], bias, k, normalize, scoring, floor, scale, ids, wts) also runs the router on the
    unrounded rows and fills ids int32 [rows, k] and wts float32 [rows, k]. A residual of several streams [streams, rows,
    hidden] takes a `StreamUpdate`: its delta rewrites the streams and their weighed sum is what is normed."""
    _need(residual, torch.float32, "residual"); _need(weight, torch.float32, "norm weight"); _need(out, None, "normed")
    if out32 is not None:
        _need(out32, torch.float32, "normed32")
    streams, hc = 0, None
    if isinstance(delta, StreamUpdate):
        hc, delta = delta, delta.delta
        if residual.dim() != 3 or (hc.mix is not None and tuple(hc.mix.shape) != (residual.shape[0],) * 2):
            raise KernelError(f"a stream update for a residual of shape {tuple(residual.shape)}")
        for t in (hc.mix, hc.out, hc.read):
            if t is not None:
                _need(t, torch.float32, "stream weights")
        streams = residual.shape[0]
    elif residual.dim() != 2:
        raise KernelError(f"a residual of shape {tuple(residual.shape)} without a stream update")
    dense = parts = stride = 0
    rows_ptr = pos = ids = wts = None
    top_k, eparts, estride = 0, 1, 0
    if isinstance(delta, PartialSums):
        dense, parts, stride = delta.data.data_ptr(), delta.parts, delta.rows * delta.hidden
    elif isinstance(delta, ExpertRows):
        rows_ptr, pos, ids, wts, top_k = delta.rows, delta.pos_of_pair, delta.ids, delta.wts, delta.ids.shape[1]
        if delta.parts > 1:
            eparts, estride = delta.parts, delta.rows.shape[1] * delta.rows.shape[2]
    elif delta is not None:
        delta = materialize(delta)
        _need(delta, torch.float32, "delta")
        dense, parts = delta.data_ptr(), 1
    hidden = residual.shape[-1]
    n_out = out.shape[0]
    r = route or {}
    if route:
        _need(r["weight"], torch.float32, "router weight"); _need(r["ids"], torch.int32, "ids"); _need(r["wts"], torch.float32, "wts")
    check(core().tl_add_rmsnorm_streams(
        ptr(residual), dense or None, parts, stride, ptr(rows_ptr), eparts, estride, ptr(pos), ptr(ids), ptr(wts), top_k,
        ptr(weight),
        ptr(out), ptr(out32), ptr(gather), n_out, hidden, float(eps), dtype_code(out.dtype), ptr(r.get("weight")),
        ptr(r.get("bias")), r["weight"].shape[0] if route else 0, int(r.get("k", 0)),
        route_flags(r.get("normalize", 0), r.get("scoring", "sigmoid"), r.get("groups")),
        float(r.get("floor", 0.0)), float(r.get("scale", 1.0)), ptr(r.get("ids")), ptr(r.get("wts")),
        streams, residual.stride(0) if streams else 0, ptr(hc.mix) if hc else None, ptr(hc.out) if hc else None,
        ptr(hc.read) if hc else None, stream()), "add_rmsnorm")
    return out


def gated_mul(gate_up: torch.Tensor, out: torch.Tensor, act: int = 1) -> torch.Tensor:
    """out = act(gate_up[:, :inter]) * gate_up[:, inter:], `act` a code of ACTIVATIONS (1: SiLU)."""
    _need(gate_up, out.dtype, "gate_up"); _need(out, None, "out")
    rows, inter = out.shape
    check(core().tl_gated_mul(ptr(gate_up), ptr(out), rows, inter, int(act), dtype_code(out.dtype), stream()), "gated_mul")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    return gated_mul(gate_up, out, ACTIVATIONS["silu"])


def add_dyt(residual: torch.Tensor, delta, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor, out: torch.Tensor,
            gather: torch.Tensor | None = None) -> torch.Tensor:
    """residual += delta (32-bit); out = tanh(alpha * residual) * weight + bias, element by element. `delta` is None, a
    float32 tensor or a branch output in a deferred form (`PartialSums` is added part by part in order; anything else is
    made a tensor first). `alpha` is a float32 tensor of one element on the device. With `gather` (int32 row indices)
    output row i is made from row gather[i] and the residual is left unchanged."""
    _need(residual, torch.float32, "residual"); _need(weight, torch.float32, "norm weight"); _need(bias, torch.float32, "norm bias")
    _need(alpha, torch.float32, "norm alpha"); _need(out, None, "normed")
    data, parts, stride = None, 0, 0
    if isinstance(delta, PartialSums) and delta.dtype is None:
        data, parts, stride = delta.data, delta.parts, delta.rows * delta.hidden
    elif delta is not None:
        data, parts = materialize(delta), 1
        _need(data, torch.float32, "delta")
    check(core().tl_add_dyt(ptr(residual), ptr(data), parts, stride, ptr(weight), ptr(bias), ptr(alpha), ptr(out), ptr(gather),
                            out.shape[0], residual.shape[-1], dtype_code(out.dtype), stream()), "add_dyt")
    return out


def activation(x: torch.Tensor, out: torch.Tensor, act: int, a0: float = 0.0, a1: float = 0.0) -> torch.Tensor:
    """out = act(x) element by element (may be x itself); `act` a code of ACTIVATIONS, `a0`, `a1` its constants (xielu: the
    factors of its two branches)."""
    _need(x, out.dtype, "x"); _need(out, None, "out")
    check(core().tl_activation(ptr(x), ptr(out), x.numel(), int(act), float(a0), float(a1), dtype_code(out.dtype), stream()),
          "activation")
    return out


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap), in place."""
    return activation(x, x, ACTIVATIONS["softcap"], float(cap))


def add_layernorm(residual: torch.Tensor, delta, weight: torch.Tensor, bias: torch.Tensor, eps: float, out: torch.Tensor,
                  gather: torch.Tensor | None = None) -> torch.Tensor:
    """residual += delta (None, a float32 tensor or `PartialSums`); out = (residual - mean) / sqrt(var + eps) * weight + bias,
    mean and variance over the row in 32-bit. With `gather` output row i is made from row gather[i] and the residual stays."""
    _need(residual, torch.float32, "residual"); _need(out, None, "out")
    parts, stride, data = 0, 0, None
    if isinstance(delta, PartialSums):
        parts, data = delta.parts, delta.data
        stride = delta.rows * delta.hidden
    elif delta is not None:
        delta = materialize(delta)
        _need(delta, torch.float32, "delta")
        parts, data = 1, delta
    check(core().tl_add_layernorm(ptr(residual), ptr(data), parts, stride, ptr(weight), ptr(bias), float(eps), ptr(out),
                                  ptr(gather), out.shape[0], residual.shape[-1], dtype_code(out.dtype), stream()),
          "add_layernorm")
    return out


def add_normed(residual: torch.Tensor, delta, weight: torch.Tensor, eps: float, gate: torch.Tensor | None = None,
               experts: "ExpertRows | None" = None, then: tuple | None = None) -> torch.Tensor | None:
    """The norm behind a branch, fused with the residual add: d = delta (None, a float32 tensor or `PartialSums`), times
    sigmoid(gate[r]) where `gate` (float32 [rows] logits) is given, plus the weighed rows of `experts`;
    residual += weight * d / rms(d). `then` = (next norm's weight, its eps, out, gather or None): the kernel also writes
    the next norm's rows of the new residual into `out` (with `gather`, only of those rows, whose residual then stays as it
    was); returns `out` or None."""
    _need(residual, torch.float32, "residual"); _need(weight, torch.float32, "norm weight")
    dense, parts, stride = None, 0, 0
    if isinstance(delta, PartialSums):
        if delta.dtype is not None:
            delta = delta.materialize().float()
        else:
            dense, parts, stride = delta.data.data_ptr(), delta.parts, delta.rows * delta.hidden
    if isinstance(delta, ExpertRows):
        experts, delta = delta, None
    if isinstance(delta, torch.Tensor):
        _need(delta, torch.float32, "delta")
        dense, parts = delta.data_ptr(), 1
    rows_ptr = pos = ids = wts = None
    top_k, eparts, estride = 0, 1, 0
    if experts is not None:
        rows_ptr, pos, ids, wts, top_k = experts.rows, experts.pos_of_pair, experts.ids, experts.wts, experts.ids.shape[1]
        if experts.parts > 1:
            eparts, estride = experts.parts, experts.rows.shape[1] * experts.rows.shape[2]
    if gate is not None:
        _need(gate, torch.float32, "gate logits")
    hidden = residual.shape[-1]
    pre_w, pre_eps, out, gather = then if then is not None else (None, 0.0, None, None)
    rows = residual.shape[0] if gather is None else out.shape[0]
    check(core().tl_add_normed(ptr(residual), dense, parts, stride, ptr(gate), ptr(rows_ptr), eparts, estride, ptr(pos), ptr(ids),
                               ptr(wts), top_k, ptr(weight), float(eps), ptr(pre_w), float(pre_eps), ptr(out), ptr(gather),
                               rows, hidden, dtype_code(out.dtype) if out is not None else FP32, stream()), "add_normed")
    return out


def row_dot(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = x[r] . w in 32-bit: one number a row (w: a vector or a [1, hidden] matrix of x's type; out float32 [rows] or
    [rows, 1])."""
    _need(w, x.dtype, "w"); _need(out, torch.float32, "out")
    if x.stride(-1) != 1 or w.numel() != x.shape[1] or out.numel() != x.shape[0]:
        raise KernelError(f"row dot: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    check(core().tl_row_dot(ptr(x), x.stride(0), ptr(w), ptr(out), x.shape[0], x.shape[1], dtype_code(x.dtype), stream()), "row_dot")
    return out


def add_vector(residual: torch.Tensor, vec: torch.Tensor) -> None:
    """residual[r, :] += vec for every row."""
    _need(residual, torch.float32, "residual"); _need(vec, torch.float32, "vector")
    if vec.numel() != residual.shape[-1]:
        raise KernelError(f"a vector of {vec.numel()} for rows of {residual.shape[-1]}")
    check(core().tl_add_vector(ptr(residual), ptr(vec), residual.shape[0], residual.shape[1], stream()), "add_vector")


# ------------------------------------------------------------------------------------------ state-space mixer
CONV_ACTIVATIONS = {"none": 0, "silu": 1}


def causal_conv_act(x: torch.Tensor, channels: int, taps, bias, state: torch.Tensor, state_slot, req_of_row, row_start,
                    out: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """out[r, c] = act(bias[c] + sum_k taps[c, k] x[r - (K - 1) + k, c]) over each request's own rows; inputs before the
    step come from the request's slot of `state` (float32 [slots, floats]; the first (K - 1) * channels floats of a slot
    are its last K - 1 inputs, oldest first). `x` is a float32 view whose first `channels` columns are convolved."""
    _need(taps, torch.float32, "taps"); _need(state, torch.float32, "state"); _need(out, torch.float32, "out")
    if x.dtype != torch.float32 or x.stride(-1) != 1:
        raise KernelError("causal conv: float32 rows with unit stride")
    check(core().tl_causal_conv_act(ptr(x), x.stride(0), ptr(taps), ptr(bias), ptr(state), state.stride(0), ptr(state_slot),
                                    ptr(req_of_row), ptr(row_start), ptr(out), out.stride(0), x.shape[0], channels,
                                    taps.shape[1], CONV_ACTIVATIONS[act], stream()), "causal_conv_act")
    return out


def conv_state(x: torch.Tensor, channels: int, taps: int, state: torch.Tensor, state_slot, row_start, requests: int) -> None:
    """After a step: each request's slot holds its last `taps - 1` inputs (rows of `x`, or what the slot held)."""
    check(core().tl_conv_state(ptr(x), x.stride(0), ptr(state), state.stride(0), ptr(state_slot), ptr(row_start), requests,
                               channels, taps, stream()), "conv_state", kernels=1 if taps > 1 else 0)


SCAN_CHUNK = 128            # rows of a chunk when a long portion's recurrence is cut into chunks that run side by side
SCAN_CHUNKED_FROM = 256     # the longest portion of a step from which on it is


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, dt_bias, a_log, d_skip, state: torch.Tensor, state_offset: int, state_slot,
             row_start, requests: int, y: torch.Tensor, heads: int, cols: int, n_state: int, groups: int,
             write_state: bool = True, max_rows_per_request: int = 0, runtime=None) -> torch.Tensor:
    """The selective state-space recurrence of csrc/ssm.cu over each request's rows. `xbc` float32 [rows, H P + 2 G N];
    `dt` a float32 view [rows, H] of the raw step sizes; a slot's recurrent state [H, P, N] begins `state_offset` floats
    into its row of `state`; `y` float32 [rows, H P]. With `max_rows_per_request` (the step's longest portion) of
    SCAN_CHUNKED_FROM rows or more and a `runtime` to keep the scratch, portions are cut into chunks of SCAN_CHUNK rows:
    every chunk's own contribution from a zero state, the states the chunks start from, then every chunk's outputs."""
    _need(xbc, torch.float32, "xbc"); _need(y, torch.float32, "y"); _need(state, torch.float32, "state")
    if dt.dtype != torch.float32 or dt.stride(-1) != 1:
        raise KernelError("ssm scan: float32 step sizes with unit stride")
    chunk = chunks = 0
    scratch = None
    if runtime is not None and max_rows_per_request >= SCAN_CHUNKED_FROM:
        chunk, chunks = SCAN_CHUNK, -(-max_rows_per_request // SCAN_CHUNK)
        if requests * chunks > 65535:
            chunk = chunks = 0
        else:
            scratch = runtime.scratch("ssm_chunks", core().tl_ssm_scan_scratch(requests, chunks, heads, cols, n_state))
    check(core().tl_ssm_scan(ptr(xbc), xbc.stride(0), ptr(dt), dt.stride(0), ptr(dt_bias), ptr(a_log), ptr(d_skip),
                             state.data_ptr() + 4 * state_offset, state.stride(0), ptr(state_slot), ptr(row_start), ptr(y),
                             requests, heads, cols, n_state, groups, int(write_state), chunk, chunks, ptr(scratch), stream()),
          "ssm_scan", kernels=3 if chunks > 1 else 1)
    return y


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight, eps: float, groups: int, out: torch.Tensor) -> torch.Tensor:
    """out = weight * v / rms(v) in `groups` equal parts of a row, v = y * silu(z); `z` a float32 view [rows, inner]."""
    _need(y, torch.float32, "y"); _need(weight, torch.float32, "norm weight"); _need(out, None, "out")
    if z.dtype != torch.float32 or z.stride(-1) != 1:
        raise KernelError("gated group norm: a float32 gate with unit stride")
    check(core().tl_gated_group_norm(ptr(y), ptr(z), z.stride(0), ptr(weight), float(eps), ptr(out), y.shape[0], y.shape[1],
                                     groups, dtype_code(out.dtype), stream()), "gated_group_norm")
    return out


# ------------------------------------------------------------------------------------------ latent attention
def latent_prepare(q, kv, c_weight, eps, inv_freq, rot_dims, positions, req_of_row, table, page_size, cache, q_out,
                   heads: int, dim: int, latent: int, rot_dim: int, status) -> None:
    """Writes the normed latent and the rotated shared key part of every row into its page, and every head's rotated query
    part into `q_out` (float32 [rows, heads, latent + rot_dim]) behind the place of its absorbed part (csrc/attention_latent.cu)."""
    _need(q, cache.dtype, "q"); _need(q_out, torch.float32, "q'")
    if kv.dtype != cache.dtype or kv.stride(-1) != 1:
        raise KernelError("latent prepare: the latent's rows in the cache's type with unit stride")
    check(core().tl_latent_prepare(ptr(q), q.stride(0), ptr(kv), kv.stride(0), ptr(c_weight), float(eps), ptr(inv_freq),
                                   int(rot_dims), ptr(positions), ptr(req_of_row), ptr(table), table.shape[1], int(page_size),
                                   cache.shape[0], ptr(cache), ptr(q_out), q.shape[0], heads, dim, latent, rot_dim,
                                   dtype_code(q.dtype), ptr(status), stream()), "latent_prepare")


def rmsnorm_rows(x: torch.Tensor, n: int, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out[r, :n] = weight * x[r, :n] / rms(x[r, :n]): a plain RMS norm over the first n columns of strided rows, 32-bit
    inside, rows in and out in the compute dtype."""
    _need(weight, torch.float32, "norm weight")
    if x.dtype != out.dtype or x.stride(-1) != 1 or out.stride(-1) != 1:
        raise KernelError("rmsnorm rows: rows in and out of one type with unit stride")
    check(core().tl_rmsnorm_rows(ptr(x), x.stride(0), ptr(weight), float(eps), ptr(out), out.stride(0), x.shape[0], int(n),
                                 dtype_code(x.dtype), stream()), "rmsnorm_rows")
    return out


def head_linear(a: torch.Tensor, ld_a: int, a_head: int, w: torch.Tensor, out: torch.Tensor, ld_out: int, out_head: int,
                rows: int, gate: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, h, n] = sum_k a[r, h, k] w[h, n, k] with w [heads, N, K]; `a` and `out` addressed by a row stride and a head
    stride (elements). With `gate` (logits [rows, heads * N] of the operands' type, unit inner stride) the result is
    multiplied entry by entry by sigmoid(gate)."""
    _need(w, a.dtype, "head weights")
    H, N, K = w.shape
    if gate is not None and (gate.dtype != a.dtype or gate.stride(-1) != 1):
        raise KernelError("head product: a gate of the operands' type with unit stride")
    check(core().tl_head_linear(ptr(a), int(ld_a), int(a_head), ptr(w), ptr(out), int(ld_out), int(out_head), rows, H, N, K,
                                dtype_code(a.dtype), dtype_code(out.dtype), ptr(gate), gate.stride(0) if gate is not None else 0,
                                stream()), "head_linear")
    return out


def attention_latent(q, cache, table, page_size, req_of_row, positions, scale, window, out, latent: int, status,
                     sinks: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, h, :latent] = softmax over the visible keys of scale * q[r, h] . key, applied to the keys' latent parts. With
    `sinks` (float32 [heads]) a head's denominator also holds exp(sink), which has no key and no value."""
    _need(q, torch.float32, "q'"); _need(out, cache.dtype, "out")
    rows, H, Dk = q.shape
    check(core().tl_attention_latent(ptr(q), ptr(cache), ptr(table), table.shape[1], int(page_size), cache.shape[0],
                                     ptr(req_of_row), ptr(positions), float(scale), int(window or 0), ptr(out), rows, H, latent,
                                     Dk, dtype_code(cache.dtype), ptr(status), ptr(sinks), stream()), "attention_latent")
    return out


# ------------------------------------------------------------------------------------------ products
def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias) on the CUDA cores with 32-bit accumulation."""
    _need(x, w.dtype, "x"); _need(w, None, "w"); _need(out, None, "out")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    check(core().tl_gemm_simt(ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(bias), ptr(out), out.stride(0), M, N, K,
                              dtype_code(x.dtype), dtype_code(out.dtype), stream()), "gemm_simt")
    return out


def gemm_simt_grouped(a: torch.Tensor, a_gather: torch.Tensor | None, a_div: int, w: torch.Tensor, out: torch.Tensor,
                      plan: "MoePlan", swiglu: bool | int) -> torch.Tensor:
    """Per sorted row i of the plan: out[i] = A[row(i)] @ w[expert(i)]^T, with w [E, N(*2 when swiglu), K]. `swiglu`:
    False for a plain product, True or a code of ACTIVATIONS for act(gate rows) * (up rows)."""
    _need(a, w.dtype, "a"); _need(w, None, "w"); _need(out, None, "out")
    E, n_rows_w, K = w.shape
    N = n_rows_w // 2 if swiglu else n_rows_w
    check(core().tl_gemm_simt_grouped(ptr(a), a.stride(0), ptr(a_gather), a_div, ptr(w), w.stride(1), w.stride(0),
                                      ptr(out), out.stride(0), plan.pairs, N, K, ptr(plan.tile_group),
                                      ptr(plan.tile_row0), ptr(plan.tile_rows), ptr(plan.n_tiles), plan.max_tiles,
                                      int(swiglu), dtype_code(a.dtype), dtype_code(out.dtype), stream()),
          "gemm_simt_grouped")
    return out


def simt_tile_rows() -> int:
    return core().tl_gemm_simt_tile_rows()


# ------------------------------------------------------------------------------------------ short conv
def short_conv(bcx, taps, bias, state, state_slot, req_of_row, row_start, positions, out) -> torch.Tensor:
    _need(bcx, out.dtype, "bcx"); _need(taps, torch.float32, "taps"); _need(state, torch.float32, "conv state")
    rows, hidden = out.shape
    K = taps.shape[1]
    check(core().tl_short_conv(ptr(bcx), ptr(taps), ptr(bias), ptr(state), ptr(state_slot), ptr(req_of_row),
                               ptr(row_start), ptr(positions), ptr(out), rows, hidden, K, dtype_code(out.dtype),
                               stream()), "short_conv")
    return out


def short_conv_decode(bcx, taps, bias, state, state_slot, req_of_row, positions, out, write_state: bool = True):
    """The convolution and the state's shift for a step of one row a request; `bcx` a tensor or `PartialSums`."""
    _need(taps, torch.float32, "taps"); _need(state, torch.float32, "conv state")
    rows, hidden = out.shape
    partial, parts, stride, data = None, 0, 0, None
    if isinstance(bcx, PartialSums):
        if bcx.dtype not in (None, out.dtype) or bcx.hidden != 3 * hidden or bcx.rows != rows:
            raise KernelError("short_conv_decode: partial sums of another shape or precision")
        partial, parts, stride = bcx.data, bcx.parts, bcx.rows * bcx.hidden
    else:
        _need(bcx, out.dtype, "bcx")
        data = bcx
    check(core().tl_short_conv_decode(ptr(data), ptr(partial), parts, stride, ptr(taps), ptr(bias), ptr(state),
                                      ptr(state_slot), ptr(req_of_row), ptr(positions), ptr(out), rows, hidden,
                                      taps.shape[1], dtype_code(out.dtype), int(write_state), stream()),
          "short_conv_decode")
    return out


def short_conv_state(bcx, state, state_slot, row_start, positions, requests: int, hidden: int, taps: int) -> None:
    _need(bcx, None, "bcx"); _need(state, torch.float32, "conv state")
    check(core().tl_short_conv_state(ptr(bcx), ptr(state), ptr(state_slot), ptr(row_start), ptr(positions), requests,
                                     hidden, taps, dtype_code(bcx.dtype), stream()), "short_conv_state")


# ------------------------------------------------------------------------------------------ attention
QK_UNIT_NORM, QK_VALUES_ARE_KEYS = 1, 2      # `flags` of qk_prepare (TL_QK_* of csrc/attention_simt.cu)


def qk_prepare(qkv, q_weight, k_weight, eps, inv_freq, rotary_dim, positions, req_of_row, block_table, page_size,
               q_out, k_cache, v_cache, k_out, v_out, num_heads, num_kv_heads, head_dim, status, flags: int = 0) -> None:
    """`flags`: QK_UNIT_NORM brings q and k to unit root mean square without norm weights; QK_VALUES_ARE_KEYS: the rows
    hold query and key heads only, and a key as projected (before its norm) is stored as its value."""
    _need(qkv, None, "qkv")
    rows = qkv.shape[0]
    max_pages = block_table.shape[1] if block_table is not None else 0
    check(core().tl_qk_prepare(ptr(qkv), qkv.stride(0), ptr(q_weight), ptr(k_weight), float(eps), ptr(inv_freq),
                               int(rotary_dim), ptr(positions), ptr(req_of_row), ptr(block_table), max_pages,
                               int(page_size), k_cache.shape[0] if k_cache is not None else 0, ptr(q_out), ptr(k_cache),
                               ptr(v_cache), ptr(k_out), ptr(v_out), rows,
                               num_heads, num_kv_heads, head_dim, dtype_code(qkv.dtype), int(flags), ptr(status), stream()),
          "qk_prepare")


def kv_store(k, v, positions, req_of_row, block_table, page_size, k_cache, v_cache, status) -> None:
    _need(k, k_cache.dtype, "k"); _need(v, v_cache.dtype, "v")
    rows, Hk, D = k.shape
    check(core().tl_kv_store(ptr(k), ptr(v), ptr(positions), ptr(req_of_row), ptr(block_table), block_table.shape[1],
                             int(page_size), k_cache.shape[0], ptr(k_cache), ptr(v_cache), rows, Hk, D, dtype_code(k.dtype),
                             ptr(status), stream()), "kv_store")


def paged_attention_simt(q, k_cache, v_cache, block_table, page_size, req_of_row, positions, scale, window, out,
                         status) -> torch.Tensor:
    _need(q, k_cache.dtype, "q"); _need(out, q.dtype, "out")
    rows, Hq, D = q.shape
    Hk = k_cache.shape[1]
    check(core().tl_paged_attention_simt(ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.shape[1],
                                         int(page_size), k_cache.shape[0], ptr(req_of_row), ptr(positions), float(scale),
                                         int(window or 0), ptr(out), rows, Hq, Hk, D, dtype_code(q.dtype), ptr(status),
                                         stream()), "paged_attention")
    return out


def attention_spans(max_context: int) -> int:
    """Key spans the split kernel cuts a context of `max_context` positions into."""
    return core().tl_attention_spans(int(max_context))


def attention_scratch_floats(rows: int, num_heads: int, head_dim: int, n_spans: int) -> int:
    return rows * num_heads * n_spans * (head_dim + 2)


def paged_attention_split(q, k_cache, v_cache, block_table, page_size, req_of_row, positions, scale, window, out,
                          scratch, n_spans: int, status) -> torch.Tensor:
    """Attention of every row over its request's cached keys, split along the keys; `scratch` is float32 with at
    least attention_scratch_floats(rows, Hq, D, n_spans) elements and n_spans covers the longest context."""
    _need(q, k_cache.dtype, "q"); _need(out, q.dtype, "out"); _need(scratch, torch.float32, "scratch")
    rows, Hq, D = q.shape
    Hk = k_cache.shape[1]
    if scratch.numel() < attention_scratch_floats(rows, Hq, D, n_spans):
        raise KernelError(f"attention scratch of {scratch.numel()} floats, "
                          f"{attention_scratch_floats(rows, Hq, D, n_spans)} needed")
    check(core().tl_paged_attention_split(ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.shape[1],
                                          int(page_size), k_cache.shape[0], ptr(req_of_row), ptr(positions), float(scale),
                                          int(window or 0), ptr(out), ptr(scratch), rows, Hq, Hk, D, int(n_spans),
                                          dtype_code(q.dtype), ptr(status), stream()), "paged_attention_split",
          kernels=2 if n_spans > 1 else 1)
    return out


SPAN_KEYS = 256     # key positions per span of `paged_attention_split`


def attention_join(scratch, positions, window, out, n_spans: int, span_keys: int = SPAN_KEYS) -> None:
    """Adds the key spans (of `span_keys` positions each) another kernel left in `scratch` (layout of
    `paged_attention_split`) into `out`."""
    rows, Hq, D = out.shape
    check(core().tl_attention_join(ptr(scratch), ptr(positions), int(window or 0), ptr(out), rows, Hq, D, int(n_spans),
                                   int(span_keys), dtype_code(out.dtype), stream()), "attention_join",
          kernels=1 if n_spans > 1 else 0)


def qkv_rotate_store(qkv, q_col: int, k_col: int, v_col: int, inv_freq, rot: int, inv_freq_v, positions, req_of_row, table,
                     page_size: int, q_out, k_cache, v_cache, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                     status, rot_magnitude: float = 1.0, v_other=None, v_blend=None) -> None:
    """From the rows of one fused product (`q_col`, `k_col`, `v_col`: where each part begins in a row; `k_col` < 0: the rows
    hold queries only): rotary over the first `rot` entries of every q and k head (halves layout; `inv_freq` None: none), its
    sines and cosines times `rot_magnitude`; the values turned over all their entries by `inv_freq_v` (None: as projected), or
    blended with the same rows of `v_other` (a view [rows, kv heads * value_dim] of the compute dtype, unit inner stride):
    (1 - l) v + l v_other with l = `v_blend` (float32, one number on the device); q to `q_out`, k and v into their pages."""
    _need(qkv, None, "qkv"); _need(q_out, qkv.dtype, "q")
    if v_other is not None and (v_other.dtype != qkv.dtype or v_other.stride(1) != 1 or
                                v_other.shape != (qkv.shape[0], num_kv_heads * value_dim)):
        raise KernelError(f"values to blend with of shape {tuple(v_other.shape)}, dtype {v_other.dtype}")
    check(core().tl_qkv_rotate_store(ptr(qkv), qkv.stride(0), int(q_col), int(k_col), int(v_col), ptr(inv_freq), int(rot),
                                     ptr(inv_freq_v), ptr(positions), ptr(req_of_row), ptr(table),
                                     table.shape[1] if table is not None else 0, int(page_size),
                                     k_cache.shape[0] if k_cache is not None else 0, ptr(q_out), ptr(k_cache), ptr(v_cache),
                                     qkv.shape[0], num_heads, num_kv_heads, head_dim, value_dim, dtype_code(qkv.dtype),
                                     ptr(status), float(rot_magnitude), ptr(v_other),
                                     v_other.stride(0) if v_other is not None else 0, ptr(v_blend), stream()),
          "qkv_rotate_store")


def attention_flex(q, k_cache, v_cache, table, page_size: int, req_of_row, positions, scale: float, softcap, window,
                   keep_first: int, inv_freq_out, gate, ld_gate: int, out_scale: float, out, status) -> torch.Tensor:
    """Attention of every row over its request's pages: capped scores (`softcap` None: none), a window that also keeps the
    first `keep_first` tokens (`window` None: all keys), the output turned back by `inv_freq_out` (None: not), times
    sigmoid(`gate`) entry by entry (a tensor of the compute dtype beginning at the first logit, rows `ld_gate` apart), times
    `out_scale`. `out` [rows, heads * value_dim] may be a column slice of a wider tensor."""
    _need(q, k_cache.dtype, "q")
    rows, Hq, D = q.shape
    Hk, VD = k_cache.shape[1], v_cache.shape[3]
    if out.dtype != q.dtype or out.stride(1) != 1 or out.shape != (rows, Hq * VD):
        raise KernelError(f"attention output of shape {tuple(out.shape)}, dtype {out.dtype}")
    check(core().tl_attention_flex(ptr(q), ptr(k_cache), ptr(v_cache), ptr(table), table.shape[1], int(page_size),
                                   k_cache.shape[0], ptr(req_of_row), ptr(positions), float(scale), float(softcap or 0.0),
                                   int(window or 0), int(keep_first or 0), ptr(inv_freq_out), ptr(gate), int(ld_gate),
                                   float(out_scale), ptr(out), out.stride(0), rows, Hq, Hk, D, VD, dtype_code(q.dtype),
                                   ptr(status), stream()), "attention_flex")
    return out


RECURRENCE_STAGED_ROWS = 8      # a request that brings more rows than this takes the step to the two-kernel form


def recurrence_scan(proj, q_col: int, k_col: int, v_col: int, state, state_slot, row_start, requests: int, y, heads: int,
                    key_dim: int, value_dim: int, *, head_decay=None, a_col: int = -1, w=None, w0=None, a_bias=None,
                    rate: float = 0.0, key_eps: float = 0.0, silu_inputs: bool = False, write_state: bool = True,
                    max_rows: int = 1, q_scale: float = 1.0) -> torch.Tensor:
    """The recurrence over a matrix state a head (csrc/recurrence.cu): with `head_decay` (float32 [heads]) the decayed sum of
    outer products, with `w` (float32 [rows, heads * key_dim], the decay's logits) and `a_col` the generalized delta rule,
    with `w` alone the gated outer products (a decay sigmoid(w + w0)^rate a key channel). q is multiplied by `q_scale`. `proj`:
    float32 rows holding q, k, v (and the removal logits at `a_col`) at the given columns; `state` [slots, heads, key_dim,
    value_dim] float32; `y` [rows, heads * value_dim] float32. `max_rows`: the most rows a request brings; above
    RECURRENCE_STAGED_ROWS the tokens' activations, decays and unit keys are formed side by side first and the scan fetches
    them ahead of its loop."""
    _need(proj, torch.float32, "projections"); _need(state, torch.float32, "state"); _need(y, torch.float32, "y")
    if w is not None:
        _need(w, torch.float32, "decay logits")
    rows = proj.shape[0]
    rule = 0 if w is None else (1 if a_col >= 0 else 2)
    scratch = None
    if max_rows > RECURRENCE_STAGED_ROWS:
        scratch = torch.empty(core().tl_recurrence_scratch_floats(rows, heads, key_dim, value_dim, rule),
                              dtype=torch.float32, device=proj.device)
    check(core().tl_recurrence_scan(ptr(proj), proj.stride(0), int(q_col), int(k_col), int(v_col), int(a_col), ptr(w),
                                    w.stride(0) if w is not None else 0, ptr(w0), ptr(a_bias), ptr(head_decay), float(rate),
                                    float(key_eps), int(silu_inputs), ptr(state), state[0].numel(), ptr(state_slot),
                                    ptr(row_start), int(requests), ptr(y), heads, key_dim, value_dim, int(write_state),
                                    ptr(scratch), rows, sm_count(), rule, float(q_scale), stream()), "recurrence_scan",
          kernels=2 if scratch is not None else 1)
    return y


def group_norm_gate(y, gate, ld_gate: int, weight, eps: float, groups: int, scale: float, out, gate_activation: str = "sigmoid"
                    ) -> torch.Tensor:
    """out = y / rms(y) over each of `groups` equal parts of a row, times `weight`, times sigmoid(gate) (or, with
    `gate_activation` "silu", gate sigmoid(gate)), times `scale`. `gate` begins at the first logit, rows `ld_gate` apart
    (32-bit or the compute dtype); `out` may be a column slice. A weight of one part's size is shared by all parts."""
    _need(y, torch.float32, "y")
    rows, width = y.shape
    if out.stride(1) != 1 or out.shape != (rows, width):
        raise KernelError(f"group_norm_gate output of shape {tuple(out.shape)}")
    check(core().tl_group_norm_gate(ptr(y), ptr(gate), int(ld_gate), dtype_code(gate.dtype), ptr(weight), float(eps),
                                    float(scale), ptr(out), out.stride(0), rows, width, int(groups), dtype_code(out.dtype),
                                    int(gate_activation == "silu"), int(weight.numel() * groups == width and groups > 1),
                                    stream()), "group_norm_gate")
    return out


HEADMIX_SPAN = 32       # the fewest keys a span of `attention_headmix` holds: one tile (measured: 40 us a layer at 8 rows and a window of 1024 against 49 with 64 and 82 with 128)


_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def attention_headmix(q, k_cache, v_cache, block_table, page_size, req_of_row, positions, scale, window, mix, gate, ld_gate,
                      out, max_context: int, runtime, status) -> torch.Tensor:
    """Attention with the heads' weights mixed after the softmax by `mix` (float32 [Hq, Hq] or None) and the output of
    head h times sigmoid(gate[r * ld_gate + h]) (`gate`: a tensor of the compute dtype whose data begins at the first
    logit, or None). Few rows and many keys are cut into spans of keys; `runtime.scratch` holds what joins them."""
    _need(q, k_cache.dtype, "q"); _need(out, q.dtype, "out")
    rows, Hq, D = q.shape
    Hk = k_cache.shape[1]
    if mix is not None:
        _need(mix, torch.float32, "head mix")
        if tuple(mix.shape) != (Hq, Hq):
            raise KernelError(f"head mix of shape {tuple(mix.shape)} for {Hq} heads")
    reach = min(max_context, window + 31) if window else max_context
    # few rows and many keys: spans of keys, enough of them for two blocks an SM, none shorter than HEADMIX_SPAN
    wanted = max(1, (2 * sm_count()) // max(rows, 1))
    span = max(HEADMIX_SPAN, -(-reach // wanted))
    span = -(-span // 32) * 32
    spans = core().tl_headmix_spans(int(max_context), int(window or 0), span)
    scratch = None
    if spans > 1:
        scratch = runtime.scratch("attention", core().tl_headmix_scratch_floats(rows, Hq, D, spans))
    check(core().tl_attention_headmix(ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.shape[1],
                                      int(page_size), k_cache.shape[0], ptr(req_of_row), ptr(positions), float(scale),
                                      int(window or 0), ptr(mix), ptr(gate), int(ld_gate), ptr(out), ptr(scratch), rows, Hq,
                                      Hk, D, spans, span, dtype_code(q.dtype), ptr(status), stream()), "attention_headmix",
          kernels=1 if spans == 1 else 3)
    return out


# ------------------------------------------------------------------------------------------ experts
def router_topk(logits, bias, k: int, normalize: bool, floor: float, scale: float, ids, wts, scoring: str = "sigmoid",
                groups: tuple[int, int] | None = None) -> None:
    _need(logits, torch.float32, "router logits"); _need(ids, torch.int32, "ids"); _need(wts, torch.float32, "weights")
    rows, E = logits.shape
    check(core().tl_router_topk(ptr(logits), logits.stride(0), ptr(bias), rows, E, k, route_flags(normalize, scoring, groups), float(floor),
                                float(scale), ptr(ids), ptr(wts), stream()), "router_topk")


class MoePlan:
    """Device buffers of one routing plan: pairs sorted by expert and the map of row tiles."""

    def __init__(self, max_pairs: int, num_experts: int, tile_rows: int, device):
        self.num_experts, self.tile_m, self.max_pairs = num_experts, tile_rows, max_pairs
        self.max_tiles_cap = core().tl_moe_max_tiles(max_pairs, num_experts, tile_rows)
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.zeros(num_experts, **i32)
        self.offsets = torch.zeros(num_experts + 1, **i32)
        self.sorted_pairs = torch.zeros(max(max_pairs, 1), **i32)
        self.pos_of_pair = torch.zeros(max(max_pairs, 1), **i32)
        self.tile_group = torch.zeros(self.max_tiles_cap, **i32)
        self.tile_row0 = torch.zeros(self.max_tiles_cap, **i32)
        self.tile_rows = torch.zeros(self.max_tiles_cap, **i32)
        self.n_tiles = torch.zeros(1, **i32)
        self.block_hist = torch.zeros(-(-max(max_pairs, 1) // 256) * num_experts, **i32)    # per-chunk counts
        self.pairs = 0
        self.max_tiles = 1

    def build(self, ids: torch.Tensor, x: torch.Tensor | None = None, x_sorted: torch.Tensor | None = None) -> "MoePlan":
        """Build the plan for `ids` [rows, k]. With `x` [rows, width] (bfloat16) and `x_sorted` [pairs, width], the
        token rows are copied into expert-sorted order as well when the one-kernel form applies; `self.copied`
        says whether they were."""
        pairs = ids.numel()
        if pairs > self.max_pairs:
            raise KernelError(f"routing plan sized for {self.max_pairs} pairs, got {pairs}")
        self.pairs = pairs
        self.max_tiles = core().tl_moe_max_tiles(pairs, self.num_experts, self.tile_m)
        launched = ctypes.c_int(0)
        check(core().tl_moe_plan(ptr(ids), pairs, self.num_experts, self.tile_m, ids.shape[-1], ptr(self.counts),
                                 ptr(self.offsets), ptr(self.sorted_pairs), ptr(self.pos_of_pair), ptr(self.tile_group),
                                 ptr(self.tile_row0), ptr(self.tile_rows), ptr(self.n_tiles), ptr(self.block_hist), ptr(x),
                                 x.stride(0) if x is not None else 0, ptr(x_sorted), x.shape[1] if x is not None else 0,
                                 ctypes.addressof(launched), stream()), "moe_plan", kernels=0)
        global launches
        launches += launched.value
        self.copied = x is not None and bool(core().tl_moe_plan_copies_rows(pairs, self.num_experts))
        return self


def moe_combine(y, plan: MoePlan, ids, wts, out) -> torch.Tensor:
    _need(y, torch.float32, "expert outputs"); _need(out, torch.float32, "out")
    rows, hidden = out.shape
    check(core().tl_moe_combine(ptr(y), ptr(plan.pos_of_pair), ptr(ids), ptr(wts), ptr(out), rows, hidden, ids.shape[1],
                                stream()), "moe_combine")
    return out


# ------------------------------------------------------------------------------------------ CUDA graphs
class DeviceGraph:
    """A captured CUDA graph on the runtime API (csrc/graphs.cu says why not `torch.cuda.CUDAGraph`). Between
    `capture_begin` and `capture_end` the current stream captures and this thread's allocations come from `pool` (a
    `torch.cuda.MemPool` that the caller keeps as long as any graph captured into it may be replayed): what a captured
    kernel writes stays where it is until the tensor that holds it is dropped, and the memory of tensors dropped since is
    used again by later captures into the same pool, whose graphs therefore must not be replayed side by side."""

    def __init__(self):
        self._exec = ctypes.c_void_p(None)
        self._pool_context = None
        self._stream = None
        self.nodes = 0

    def capture_begin(self, pool) -> None:
        self._stream = stream()
        self._pool_context = torch.cuda.use_mem_pool(pool)
        self._pool_context.__enter__()
        try:
            check(core().tl_graph_capture_begin(self._stream), "graph capture", kernels=0)
        except BaseException:
            self._pool_context.__exit__(None, None, None)
            self._pool_context = None
            raise

    def capture_end(self) -> None:
        nodes = ctypes.c_int(0)
        try:
            code = core().tl_graph_capture_end(self._stream, ctypes.byref(self._exec), ctypes.byref(nodes))
        finally:
            self._pool_context.__exit__(None, None, None)
            self._pool_context = None
        check(code, "graph capture", kernels=0)
        self.nodes = nodes.value

    def replay(self) -> None:
        check(core().tl_graph_launch(self._exec, stream()), "graph launch", kernels=0)

    def __del__(self):
        ex, self._exec = self._exec, ctypes.c_void_p(None)
        if ex and _core is not None:
            _core.tl_graph_destroy(ex)


# ------------------------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(logits, torch.float32, "logits"); _need(out, torch.int32, "out")
    rows, V = logits.shape
    check(core().tl_argmax(ptr(logits), logits.stride(0), rows, V, ptr(out), stream()), "argmax")
    return out


def sample(logits, temperature, top_k, top_p, min_p, seed, position, out) -> torch.Tensor:
    _need(logits, torch.float32, "logits"); _need(temperature, torch.float32, "temperature")
    _need(top_k, torch.int32, "top_k"); _need(top_p, torch.float32, "top_p"); _need(min_p, torch.float32, "min_p")
    _need(seed, torch.int64, "seed"); _need(position, torch.int32, "position"); _need(out, torch.int32, "out")
    rows, V = logits.shape
    check(core().tl_sample(ptr(logits), logits.stride(0), rows, V, ptr(temperature), ptr(top_k), ptr(top_p), ptr(min_p),
                           ptr(seed), ptr(position), ptr(out), stream()), "sample")
    return out


def penalize(logits, counts, slot, repetition, presence, frequency, bias=None) -> torch.Tensor:
    """Penalties and added logits, in place on float32 logits [n, V]. `counts` int32 [slots, V] (None when no row
    has penalties); `slot` int32 [n], negative for a row without penalties; `repetition`, `presence`, `frequency`
    float32 [n]; `bias` None or (begin int32 [n + 1], token int32 [m], value float32 [m])."""
    _need(logits, torch.float32, "logits"); _need(slot, torch.int32, "slot")
    _need(repetition, torch.float32, "repetition"); _need(presence, torch.float32, "presence")
    _need(frequency, torch.float32, "frequency")
    rows, V = logits.shape
    slots, counts_ld, counts_ptr = 0, 0, None
    if counts is not None:
        _need(counts, torch.int32, "counts")
        slots, counts_ld, counts_ptr = counts.shape[0], counts.stride(0), ptr(counts)
        if counts.shape[1] != V:
            raise ValueError(f"counts over {counts.shape[1]} tokens for logits over {V}")
    begin = token = value = None
    if bias is not None:
        _need(bias[0], torch.int32, "bias begin"); _need(bias[1], torch.int32, "bias token")
        _need(bias[2], torch.float32, "bias value")
        if bias[0].numel() != rows + 1 or bias[1].numel() != bias[2].numel():
            raise ValueError("bias: begin needs one entry a row and one more, and a value for every token")
        begin, token, value = ptr(bias[0]), ptr(bias[1]), ptr(bias[2])
    check(core().tl_penalize(ptr(logits), logits.stride(0), rows, V, counts_ptr, counts_ld, slots, ptr(slot),
                             ptr(repetition), ptr(presence), ptr(frequency), begin, token, value, stream()), "penalize")
    return logits


def count_tokens(counts: torch.Tensor, tokens: torch.Tensor, slot) -> None:
    """counts[slot, token] += 1 for int32 tokens [n]; `slot` is an int32 tensor [n] or one row's index."""
    _need(counts, torch.int32, "counts"); _need(tokens, torch.int32, "tokens")
    slots, V = counts.shape
    if isinstance(slot, torch.Tensor):
        _need(slot, torch.int32, "slot")
        if slot.numel() != tokens.numel():
            raise ValueError(f"{slot.numel()} slots for {tokens.numel()} tokens")
        slot_ptr, one = ptr(slot), -1
    else:
        slot_ptr, one = None, int(slot)
    check(core().tl_count_tokens(ptr(counts), counts.stride(0), slots, V, slot_ptr, one, ptr(tokens), tokens.numel(),
                                 stream()), "count_tokens")
