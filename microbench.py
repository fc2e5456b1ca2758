"""Single kernels on small cases, timed with CUDA events: the commands behind the summaries under `profiles/`.

    python microbench.py expert_gemm --tokens 8
    python microbench.py dense_gemm --rows 8 --n 6144 --k 2048
    python microbench.py dense_gemm --rows 2048 --n 6144 --k 2048
    python microbench.py attention --batch 8 --context 8192
    python microbench.py attention --batch 1 --rows 2048 --context 2048
    python microbench.py norm --rows 8
    python microbench.py headmix --batch 8 --window 1024
    python microbench.py headmix --batch 1 --rows 2048 --window 1024
    python microbench.py scan --rows 2048
    python microbench.py latent --rows 2048 --context 2048 --window 1024

Sizes default to the LFM2-8B-A1B layer (hidden 2048, 32 experts of width 1792 top-4, 32/8 heads of 64). Inputs are
larger than the 126 MB L2 or a 256 MB buffer is written between timed launches, so DRAM figures mean something; a
case holds a few GB at most and a run ends in seconds, which is what a profiler capture needs. Each run prints one
JSON line: milliseconds (median), the bytes or flops the kernel has to move or do, and the rate.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

DEV = "cuda:0"


def timed(fn, iters: int, flush: bool = True) -> float:
    junk = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=DEV) if flush else None
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        if flush:
            junk.fill_(1.0)            # 256 MB written: nothing of the last launch is left in L2
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def runtime(prompt_product: str | None = None):
    from tandemllm_b200.parts import Runtime
    from tandemllm_b200.kernels import tensorcore
    rt = Runtime(torch.device(DEV), torch.bfloat16)
    tensorcore.enable(rt)
    if prompt_product:
        tensorcore.PROMPT_PRODUCT = prompt_product
    return rt


def expert_gemm(a) -> dict:
    """The routed experts of one layer: plan + gate/up with SwiGLU + down, for `tokens` rows."""
    from tandemllm_b200.config import PartSpec
    from tandemllm_b200.parts import make_part
    rt = runtime(a.product)
    E, H, I, k, R = a.experts, a.hidden, a.inter, a.top_k, a.tokens
    spec = PartSpec("sigmoid_topk_experts", {"num_experts": E, "top_k": k, "intermediate_size": I, "expert_bias": False,
                                             "normalize": True, "scale": 1.0,
                                             "names": {"router": "gate", "bias": "b", "experts": "experts", "gate": "w1",
                                                       "up": "w3", "down": "w2"}})
    part = make_part("feed_forward", spec, prefix="m.", hidden_size=H)
    part.runtime = rt
    part.w_router = torch.randn(E, H, device=DEV) * 0.5
    part.expert_bias = None
    part.w_gate_up = (torch.randn(E, 2 * I, H, device=DEV) * 0.02).to(torch.bfloat16)
    part.w_down = (torch.randn(E, H, I, device=DEV) * 0.02).to(torch.bfloat16)
    x = torch.randn(R, H, device=DEV).to(torch.bfloat16)
    ids, wts = part.route(x.float())
    touched = int(torch.unique(ids).numel())
    ms = timed(lambda: rt.tensorcore.experts(part, x, ids, wts), a.iters)
    nbytes = touched * 3 * I * H * 2
    flops = 2.0 * R * k * 3 * I * H
    return {"kernel": "experts (plan, gate/up + SwiGLU, down)", "tokens": R, "experts_touched": touched, "ms": ms,
            "bytes": nbytes, "GBps": nbytes / ms / 1e6, "TFLOPs": flops / ms / 1e9}


def dense_gemm(a) -> dict:
    rt = runtime(a.product)
    x = torch.randn(a.rows, a.k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device=DEV) * 0.02).to(torch.bfloat16)
    out = torch.empty(a.rows, a.n, dtype=torch.bfloat16 if a.out == "bf16" else torch.float32, device=DEV)
    ms = timed(lambda: rt.tensorcore.linear(x, w, None, out), a.iters)
    nbytes = (a.n * a.k + a.rows * a.k) * 2 + out.numel() * out.element_size()
    flops = 2.0 * a.rows * a.n * a.k
    return {"kernel": "dense product", "rows": a.rows, "n": a.n, "k": a.k, "ms": ms, "bytes": nbytes,
            "GBps": nbytes / ms / 1e6, "TFLOPs": flops / ms / 1e9}


def attention(a) -> dict:
    """`rows` query rows per request at the end of a context of `context` positions, `batch` requests."""
    from tandemllm_b200.kernels import ops
    rt = runtime()
    Hq, Hk, D, page = a.heads, a.kv_heads, a.head_dim, 16
    B, n, L = a.batch, a.rows, a.context
    pages_per = -(-L // page)
    kc = (torch.randn(B * pages_per, Hk, page, D, device=DEV) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(B * pages_per, Hk, page, D, device=DEV) * 0.5).to(torch.bfloat16)
    table = torch.arange(B * pages_per, dtype=torch.int32, device=DEV).view(B, pages_per)
    R = B * n
    q = torch.randn(R, Hq, D, device=DEV).to(torch.bfloat16)
    positions = torch.cat([torch.arange(L - n, L, dtype=torch.int32) for _ in range(B)]).to(DEV)
    starts = [b * n for b in range(B + 1)]
    step = types.SimpleNamespace(n_requests=B, max_rows_per_request=n, max_context=L, positions=positions,
                                 req_of_row=torch.arange(B, dtype=torch.int32, device=DEV).repeat_interleave(n),
                                 host={"row_start": starts})
    cache = types.SimpleNamespace(k=kc, v=vc, page_size=page)
    out = torch.empty(R, Hq, D, dtype=torch.bfloat16, device=DEV)
    if a.kernel in ("mma", "tc"):
        from tandemllm_b200.kernels import tensorcore
        tensorcore.PROMPT_ATTENTION = "tcgen05" if a.kernel == "tc" else "mma"
        tensorcore.lib().tl_attention_mma_use_tma(int(a.copies == "tma"))
        tensorcore.lib().tl_attention_tc_p_in_tensor_memory(int(a.p == "tmem"))
        fn = lambda: rt.tensorcore.attention(q, cache, table, step, D ** -0.5, None, out, rt)
    else:
        spans = ops.attention_spans(L)
        scratch = torch.empty(ops.attention_scratch_floats(R, Hq, D, spans), device=DEV)
        fn = lambda: ops.paged_attention_split(q, kc, vc, table, page, step.req_of_row, positions, D ** -0.5, None, out,
                                               scratch, spans, rt.status)
    ms = timed(fn, a.iters, flush=kc.numel() * 4 < 512 * 1024 * 1024)
    nbytes = B * L * Hk * D * 2 * 2
    flops = 4.0 * B * Hq * D * (n * (L - n) + n * (n + 1) / 2)
    return {"kernel": f"paged attention ({a.kernel})", "batch": B, "rows": n, "context": L, "ms": ms, "bytes": nbytes,
            "GBps": nbytes / ms / 1e6, "TFLOPs": flops / ms / 1e9}


def norm(a) -> dict:
    from tandemllm_b200.kernels import ops
    ops.core()
    R, H, S = a.rows, a.hidden, a.streams
    delta = torch.randn(R, H, device=DEV)
    w = torch.ones(H, device=DEV)
    out = torch.empty(R, H, dtype=torch.bfloat16, device=DEV)
    if S:       # several residual streams: rewritten from the old ones and the sublayer's output, their weighed sum normed
        res = torch.randn(S, R, H, device=DEV)
        mix = (torch.eye(S) * 0.9 + 0.1 / S).to(DEV)
        upd = ops.StreamUpdate(delta, mix, torch.ones(S, device=DEV), torch.full((S,), 1.0 / S, device=DEV))
        ms = timed(lambda: ops.add_rmsnorm(res, upd, w, 1e-5, out), a.iters)
        nbytes = R * H * (4 * (2 * S + 1) + 2)
        return {"kernel": "streams rewritten + RMS norm", "rows": R, "hidden": H, "streams": S, "ms": ms, "bytes": nbytes,
                "GBps": nbytes / ms / 1e6}
    res = torch.randn(R, H, device=DEV)
    ms = timed(lambda: ops.add_rmsnorm(res, delta, w, 1e-5, out), a.iters)
    nbytes = R * H * (4 + 4 + 4 + 2)
    return {"kernel": "residual add + RMS norm", "rows": R, "hidden": H, "ms": ms, "bytes": nbytes, "GBps": nbytes / ms / 1e6}


def headmix(a) -> dict:
    """Attention with the heads' weights mixed after the softmax: `--rows` 1 is a decode step of `--batch` requests whose
    windows are full (the CUDA-core kernels, keys cut into spans), more rows a prompt portion (the tensor-core kernel)."""
    from tandemllm_b200.kernels import ops, tensorcore
    rt = runtime()
    H, G, D, win, B, R = a.heads, a.kv_heads, a.head_dim, a.window, a.batch, a.rows
    ctx = win + R
    pages_per = -(-ctx // 16) + 1
    pool = B * pages_per
    kc = torch.randn(pool, G, 16, D, device=DEV).to(torch.bfloat16)
    vc = torch.randn(pool, G, 16, D, device=DEV).to(torch.bfloat16)
    table = torch.arange(pool, dtype=torch.int32, device=DEV).view(B, pages_per).contiguous()
    mix = (torch.eye(H) + 0.1 * torch.randn(H, H)).to(DEV)
    q = torch.randn(B * R, H, D, device=DEV).to(torch.bfloat16)
    gate = torch.randn(B * R, H, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    pos = (torch.arange(R, dtype=torch.int32) + win).repeat(B).to(DEV)
    req = torch.arange(B, dtype=torch.int32).repeat_interleave(R).to(DEV)
    pairs = B * sum(min(win + i + 1, win) for i in range(R))
    if R == 1:
        fn = lambda: ops.attention_headmix(q, kc, vc, table, 16, req, pos, D ** -0.5, win, mix, gate, H, out, ctx, rt, rt.status)
        kernel = "head-mixed attention, CUDA cores (statistics, apply, join)"
    else:
        lib = tensorcore.lib()
        if not lib.tl_attention_headmix_mma_supported(H, G, D):
            raise SystemExit(f"the tensor-core kernel does not take {H} heads over {G} of size {D}")
        tiles = torch.tensor([(b, b * R + r0, min(16, R - r0)) for b in range(B) for r0 in range(0, R, 16)],
                             dtype=torch.int32, device=DEV)
        fn = lambda: lib.tl_attention_headmix_mma(
            q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.shape[1], 16, pool, tiles.data_ptr(),
            tiles.shape[0], pos.data_ptr(), D ** -0.5, win, mix.data_ptr(), gate.data_ptr(), H, out.data_ptr(), H, G, D,
            rt.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        kernel = "head-mixed attention, mma.sync (prompt portions)"
    ms = timed(fn, a.iters)
    assert int(rt.status.item()) == 0
    flops = 4.0 * pairs * H * D + 2.0 * pairs * H * H
    nbytes = 2.0 * 2 * B * min(ctx, win + R - 1) * G * D
    return {"kernel": kernel, "batch": B, "rows": R, "window": win, "heads": H, "kv_heads": G, "head_dim": D, "ms": ms,
            "flops": flops, "TFLOPs": flops / ms / 1e9, "kv_bytes": nbytes, "GBps": nbytes / ms / 1e6}


def scan(a) -> dict:
    """The state-space recurrence of one layer over one request's portion (chunked from 256 rows on) or a decode step."""
    from tandemllm_b200.kernels import ops
    from tandemllm_b200.parts import Runtime
    ops.core()
    rt = Runtime(torch.device(DEV), torch.float32)
    H, Pc, N, G, B, R = a.heads, a.cols, a.state, a.groups, a.batch, a.rows
    inner = H * Pc
    xbc = torch.randn(B * R, inner + 2 * G * N, device=DEV)
    dt = torch.randn(B * R, H, device=DEV)
    vecs = [torch.randn(H, device=DEV) * 0.3 for _ in range(3)]
    state = torch.zeros(B, H * Pc * N, device=DEV)
    y = torch.empty(B * R, inner, device=DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    start = torch.arange(0, (B + 1) * R, R, dtype=torch.int32, device=DEV)
    ms = timed(lambda: ops.ssm_scan(xbc, dt, vecs[0], vecs[1] - 1.0, vecs[2], state, 0, slot, start, B, y, H, Pc, N, G,
                                    max_rows_per_request=R, runtime=rt), a.iters)
    flops = 4.0 * B * R * H * Pc * N
    nbytes = 4.0 * (xbc.numel() + dt.numel() + y.numel() + 2 * state.numel())
    return {"kernel": "state-space recurrence", "batch": B, "rows": R, "heads": H, "cols": Pc, "state": N, "ms": ms,
            "flops": flops, "TFLOPs_fp32": flops / ms / 1e9, "bytes": nbytes, "GBps": nbytes / ms / 1e6}


def latent(a) -> dict:
    """Latent attention of one layer on the tensor cores: `batch` requests of `rows` rows at a context of `context`."""
    from tandemllm_b200.parts import PagedSiteCache, StepContext
    rt = runtime()
    H, L, Rr, B, R, ctx, win, page = a.heads, a.kv_rank, a.rot_dim, a.batch, a.rows, a.context, a.window, 16
    Dk = L + Rr
    pages_each = -(-ctx // page)
    cache_t = (torch.randn(B * pages_each, 1, page, Dk, device=DEV) * 0.5).to(torch.bfloat16)
    cache = PagedSiteCache(0, page, cache_t, cache_t)
    table = torch.arange(B * pages_each, dtype=torch.int32, device=DEV).view(B, pages_each)
    q = torch.randn(B * R, H, Dk, device=DEV)
    out = torch.empty(B * R, H, L, dtype=torch.bfloat16, device=DEV)
    pos = torch.cat([torch.arange(ctx - R, ctx, dtype=torch.int32) for _ in range(B)]).to(DEV)
    req = torch.arange(B, dtype=torch.int32).repeat_interleave(R).to(DEV)
    start = torch.arange(0, (B + 1) * R, R, dtype=torch.int32, device=DEV)
    step = StepContext(n_rows=B * R, n_requests=B, token_ids=None, positions=pos, req_of_row=req, row_start=start, state_slot=None,
                       block_tables=[table], out_rows=None, n_out=0, max_rows_per_request=R, max_context=ctx)
    ms = timed(lambda: rt.tensorcore.attention_latent(q, cache, table, step, Dk ** -0.5, win, out, L, rt), a.iters)
    pairs = B * sum(min(p + 1, win) if win else p + 1 for p in range(ctx - R, ctx))
    flops = pairs * H * (2.0 * Dk + 2.0 * L)
    nbytes = 2.0 * B * min(ctx, (win + R) if win else ctx) * Dk + q.numel() * 4 + out.numel() * 2
    return {"kernel": "latent attention (mma.sync)", "batch": B, "rows": R, "context": ctx, "window": win, "heads": H, "kv_rank": L,
            "rot_dim": Rr, "ms": ms, "flops": flops, "TFLOPs": flops / ms / 1e9, "bytes": nbytes, "GBps": nbytes / ms / 1e6}


def recurrence(a) -> dict:
    """The recurrence over a matrix state a head of one layer (`--rule delta`, `decay` or `gated`): `batch` requests of `rows` rows."""
    from tandemllm_b200.kernels import ops
    ops.core()
    H, D, VD, B, R = a.heads, a.dim, a.vdim, a.batch, a.rows
    delta = a.rule == "delta"
    if delta:
        VD = D
    I = H * D
    cols = {"q": 0, "k": I, "v": 2 * I, "a": 2 * I + H * VD}
    proj = torch.randn(B * R, cols["a"] + I, device=DEV) * 0.5
    state = torch.zeros(B, H, D, VD, device=DEV)
    y = torch.empty(B * R, H * VD, device=DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    start = torch.arange(0, (B + 1) * R, R, dtype=torch.int32, device=DEV)
    kw = dict(a_col=cols["a"], w=torch.randn(B * R, I, device=DEV), w0=torch.zeros(I, device=DEV), a_bias=torch.zeros(I, device=DEV),
              rate=0.6, key_eps=1e-6) if delta else dict(head_decay=torch.full((H,), 0.97, device=DEV), silu_inputs=True)
    if a.rule == "gated":       # a decay a key channel and token, sigmoid(w + w0)^rate
        kw = dict(w=torch.randn(B * R, I, device=DEV), w0=torch.full((I,), 3.0, device=DEV), rate=1.0 / 16, q_scale=D ** -0.5)
    ms = timed(lambda: ops.recurrence_scan(proj, cols["q"], cols["k"], cols["v"], state, slot, start, B, y, H, D, VD,
                                           max_rows=R, **kw), a.iters)
    flops = (10.0 if delta else 6.0) * B * R * H * D * VD
    nbytes = 4.0 * (proj.numel() + y.numel() + 2 * state.numel())
    return {"kernel": f"matrix-state recurrence ({a.rule})", "batch": B, "rows": R, "heads": H, "dim": D, "vdim": VD, "ms": ms,
            "flops": flops, "TFLOPs_fp32": flops / ms / 1e9, "bytes": nbytes, "GBps": nbytes / ms / 1e6,
            "ns_per_token_of_a_request": ms * 1e6 / R}


def flex(a) -> dict:
    """Attention with capped scores, a window that keeps first tokens, a turned output and optionally a gate, on the tensor
    cores: `batch` requests of `rows` rows at a context of `context`."""
    from tandemllm_b200.parts import PagedSiteCache, StepContext
    rt = runtime()
    Hq, Hk, D, VD, B, R, ctx, win, page = a.heads, a.kv_heads, a.dim, a.vdim, a.batch, a.rows, a.context, a.window, 16
    pages_each = -(-ctx // page)
    k = (torch.randn(B * pages_each, Hk, page, D, device=DEV) * 0.5).to(torch.bfloat16)
    v = (torch.randn(B * pages_each, Hk, page, VD, device=DEV) * 0.5).to(torch.bfloat16)
    cache = PagedSiteCache(0, page, k, v)
    table = torch.arange(B * pages_each, dtype=torch.int32, device=DEV).view(B, pages_each)
    q = (torch.randn(B * R, Hq, D, device=DEV)).to(torch.bfloat16)
    out = torch.empty(B * R, Hq * VD, dtype=torch.bfloat16, device=DEV)
    pos = torch.cat([torch.arange(ctx - R, ctx, dtype=torch.int32) for _ in range(B)]).to(DEV)
    req = torch.arange(B, dtype=torch.int32).repeat_interleave(R).to(DEV)
    starts = list(range(0, (B + 1) * R, R))
    step = StepContext(n_rows=B * R, n_requests=B, token_ids=None, positions=pos, req_of_row=req,
                       row_start=torch.tensor(starts, dtype=torch.int32, device=DEV), state_slot=None, block_tables=[table],
                       out_rows=None, n_out=0, max_rows_per_request=R, max_context=ctx, host={"row_start": starts})
    inv = (10000.0 ** (-torch.arange(0, VD, 2, dtype=torch.float64) / VD)).float().to(DEV) if a.turned else None
    part = types.SimpleNamespace(scale=D ** -0.5, softcap=a.softcap or None, window=win or None, keep_first=a.keep_first,
                                 inv_freq_v=inv)
    assert rt.tensorcore.attention_flex(part, q, cache, table, step, None, 0, 1.0, out), "sizes the kernel does not take"
    ms = timed(lambda: rt.tensorcore.attention_flex(part, q, cache, table, step, None, 0, 1.0, out), a.iters)
    seen = lambda p: (min(p + 1, win) + min(a.keep_first, max(0, p + 1 - win))) if win else p + 1
    pairs = B * sum(seen(p) for p in range(ctx - R, ctx))
    flops = pairs * Hq * 2.0 * (D + VD)
    nbytes = 2.0 * B * Hk * min(ctx, (win + a.keep_first + R) if win else ctx) * (D + VD) + q.numel() * 2 + out.numel() * 2
    return {"kernel": "attention, capped scores and kept first tokens (mma.sync)", "batch": B, "rows": R, "context": ctx,
            "window": win, "keep_first": a.keep_first, "heads": Hq, "kv_heads": Hk, "dim": D, "vdim": VD, "ms": ms, "flops": flops,
            "TFLOPs": flops / ms / 1e9, "bytes": nbytes, "GBps": nbytes / ms / 1e6}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    e = sub.add_parser("expert_gemm")
    e.add_argument("--tokens", type=int, default=8)
    e.add_argument("--experts", type=int, default=32)
    e.add_argument("--hidden", type=int, default=2048)
    e.add_argument("--inter", type=int, default=1792)
    e.add_argument("--top-k", type=int, default=4)
    d = sub.add_parser("dense_gemm")
    d.add_argument("--rows", type=int, default=8)
    d.add_argument("--n", type=int, default=6144)
    d.add_argument("--k", type=int, default=2048)
    d.add_argument("--out", default="bf16", choices=("bf16", "fp32"))
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--rows", type=int, default=1)
    t.add_argument("--context", type=int, default=8192)
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=8)
    t.add_argument("--head-dim", type=int, default=64)
    t.add_argument("--kernel", default="tc", choices=("tc", "mma", "split"),
                   help="tc: the tcgen05 kernel for prompt portions of head size 64 (decode rows go to the mma.sync kernel "
                        "either way); mma: the mma.sync kernel for everything; split: the CUDA-core kernel")
    t.add_argument("--p", default="tmem", choices=("tmem", "smem"),
                   help="the tcgen05 kernel: P as the MMA's operand from tensor memory, or through shared memory")
    t.add_argument("--copies", default="tma", choices=("tma", "cp.async"),
                   help="decoding with the mma kernel: a producer warp's TMA copies, or cp.async from every thread")
    hm = sub.add_parser("headmix")
    hm.add_argument("--batch", type=int, default=8)
    hm.add_argument("--rows", type=int, default=1)
    hm.add_argument("--window", type=int, default=1024)
    hm.add_argument("--heads", type=int, default=32)
    hm.add_argument("--kv-heads", type=int, default=8)
    hm.add_argument("--head-dim", type=int, default=64)
    sc = sub.add_parser("scan")
    sc.add_argument("--batch", type=int, default=1)
    sc.add_argument("--rows", type=int, default=2048)
    sc.add_argument("--heads", type=int, default=32)
    sc.add_argument("--cols", type=int, default=64)
    sc.add_argument("--state", type=int, default=128)
    sc.add_argument("--groups", type=int, default=4)
    la = sub.add_parser("latent")
    la.add_argument("--batch", type=int, default=1)
    la.add_argument("--rows", type=int, default=2048)
    la.add_argument("--context", type=int, default=2048)
    la.add_argument("--window", type=int, default=1024)
    la.add_argument("--heads", type=int, default=16)
    la.add_argument("--kv-rank", type=int, default=256)
    la.add_argument("--rot-dim", type=int, default=32)
    rc = sub.add_parser("recurrence")
    rc.add_argument("--rule", default="delta", choices=("delta", "decay", "gated"))
    rc.add_argument("--batch", type=int, default=1)
    rc.add_argument("--rows", type=int, default=2048)
    rc.add_argument("--heads", type=int, default=16)
    rc.add_argument("--dim", type=int, default=64)
    rc.add_argument("--vdim", type=int, default=64)
    fl = sub.add_parser("flex")
    fl.add_argument("--batch", type=int, default=1)
    fl.add_argument("--rows", type=int, default=2048)
    fl.add_argument("--context", type=int, default=2048)
    fl.add_argument("--window", type=int, default=512)
    fl.add_argument("--keep-first", type=int, default=4)
    fl.add_argument("--softcap", type=float, default=50.0)
    fl.add_argument("--turned", type=int, default=1)
    fl.add_argument("--heads", type=int, default=16)
    fl.add_argument("--kv-heads", type=int, default=4)
    fl.add_argument("--dim", type=int, default=64)
    fl.add_argument("--vdim", type=int, default=64)
    n = sub.add_parser("norm")
    n.add_argument("--rows", type=int, default=8)
    n.add_argument("--hidden", type=int, default=2048)
    n.add_argument("--streams", type=int, default=0, help="several residual streams (hyper-connections); 0: one residual")
    for p in (e, d):
        p.add_argument("--product", default="pair", choices=("pair", "single"),
                       help="prompt-sized products: the kernel on pairs of SMs (cta_group::2), or the one-CTA persistent kernel")
    for p in (e, d, t, n, hm, sc, la, rc, fl):
        p.add_argument("--iters", type=int, default=20)
    a = ap.parse_args(argv)
    result = {"expert_gemm": expert_gemm, "dense_gemm": dense_gemm, "attention": attention, "norm": norm, "headmix": headmix,
              "scan": scan, "latent": latent, "recurrence": recurrence, "flex": flex}[a.what](a)
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in result.items()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
