"""Niralix on the GPU against the plain implementation (`tests/plain_niralix.py`): every mechanism alone as a part with a
cache of its own, then whole models through the step function, the scheduler and the replay program.

The tiny models (`tests/niralix_configs.py`) differ from one another in every size and constant. Where random weights would
hide a fault (a far key among hundreds, a first token whose trace must last), one input row's query and one row's key are made
large along an entry the rotation leaves alone, so that one score stands out, or a decay is set so close to one that the first
token still shows at the end.

Tolerances as for the engine's other models: 32-bit within 1e-4 of a row's largest magnitude, bfloat16 within 3e-2.
"""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import niralix_configs as C
from tests import plain_niralix as P
from tests.test_gpu_parts import plain, reader, runtime, stepper

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda:0"


def rel(a, b):
    a = torch.as_tensor(np.asarray(a), dtype=torch.float64) if not isinstance(a, torch.Tensor) else a.double().cpu()
    b = torch.as_tensor(np.asarray(b), dtype=torch.float64) if not isinstance(b, torch.Tensor) else b.double().cpu()
    return float(((a - b).abs() / b.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)).max())


def rt_of(dtype):
    """The runtime a served model has: in bfloat16 with the tensor-core kernels switched on."""
    rt = runtime(DT[dtype])
    if dtype == "bfloat16":
        from tandemllm_b200.kernels import tensorcore
        tensorcore.enable(rt)
    return rt


def one_model(layers, width, eps=1e-5, rank=8, seed=0, streams=None):
    from tandemllm_b200.config import NiralixConfig
    cfg = {"architecture": "Niralix", "vocab": 11, "width": width, "norm": {"eps": eps}, "logit_scale": 1.0, "layers": list(layers)}
    if streams:
        cfg["streams"] = streams
    W = C.random_weights(cfg, rank, seed)
    return NiralixConfig.from_dict(cfg).to_spec(), W


def bound(spec, i, W, rt, width):
    from tandemllm_b200.parts import make_part
    part = make_part("mixer", spec.layers[i].mixer, prefix=spec.layers[i].prefix, hidden_size=width)
    if hasattr(part, "shapes_from"):
        part.shapes_from(lambda n: tuple(W[n].shape) if n in W else None)
    part.bind(reader(W), rt)
    return part


def cuts(n, sizes):
    out, i = [], 0
    while n:
        c = min(n, sizes[i % len(sizes)])
        out.append(c)
        n -= c
        i += 1
    return out


def in_portions(part, x, cache, step, portions, rid="r", site=0, before=None):
    outs, at = [], 0
    for n in portions:
        ctx = step([(rid, n)])
        rows = x[at:at + n].to(DEV)
        if before is not None:
            before(rows, ctx)
        outs.append(plain(part.forward(rows, ctx, cache.site_cache[site])))
        at += n
    assert at == x.shape[0]
    return torch.cat(outs)


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams,width", [(1, 44), (2, 328), (3, 1000), (8, 64), (4, 2052)])
def test_the_norm_kernel_rewrites_the_streams_and_norms_what_the_sublayer_reads(dtype, streams, width):
    from tandemllm_b200.kernels import ops
    g = torch.Generator().manual_seed(width + streams)
    R, S = 9, streams
    x = torch.randn(S, R, width, generator=g) * 2
    y = torch.randn(R, width, generator=g)
    mix = torch.eye(S) + 0.3 * torch.randn(S, S, generator=g)
    w_out, w_in = torch.randn(S, generator=g), torch.randn(S, generator=g)
    w = 0.2 * torch.randn(width, generator=g)
    res = x.to(DEV)
    out = torch.empty(R, width, dtype=DT[dtype], device=DEV)
    ops.add_rmsnorm(res, ops.StreamUpdate(y.to(DEV), mix.to(DEV), w_out.to(DEV), w_in.to(DEV)), (1 + w).to(DEV), 1e-5, out)
    new = P.hyper_write(x.double().numpy(), y.double().numpy(), mix.double().numpy(), w_out.double().numpy())
    want = P.offset_norm(P.hyper_read(new, w_in.double().numpy()), w.double().numpy(), 1e-5)
    assert rel(res.reshape(S * R, width), new.reshape(S * R, width)) < 1e-6
    assert rel(out.float(), want) < (2e-5 if dtype == "float32" else 1e-2)
    # nothing to add: the streams stay, their weighed sum is normed
    res2 = x.to(DEV)
    ops.add_rmsnorm(res2, ops.StreamUpdate(None, None, None, w_in.to(DEV)), (1 + w).to(DEV), 1e-5, out)
    assert torch.equal(res2.cpu(), x)
    assert rel(out.float(), P.offset_norm(P.hyper_read(x.double().numpy(), w_in.double().numpy()), w.double().numpy(), 1e-5)) < \
        (2e-5 if dtype == "float32" else 1e-2)
    # the last norm of a model: a few rows, the plain sum of the rewritten streams, the streams left as they were; the
    # sublayer's output may come as partial sums
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, width, dtype=DT[dtype], device=DEV)
    halves = torch.stack([0.25 * y, 0.75 * y]).to(DEV).contiguous()
    ops.add_rmsnorm(res2, ops.StreamUpdate(ops.PartialSums(halves, 2, R, width), mix.to(DEV), w_out.to(DEV), None),
                    (1 + w).to(DEV), 1e-5, out2, rows)
    assert torch.equal(res2.cpu(), x)
    assert rel(out2.float(), P.offset_norm(new.sum(0), w.double().numpy(), 1e-5)[[7, 2]]) < (2e-5 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,tau,rank", [(3, 8, 6, 4.0, 5), (2, 64, 64, 16.0, 16), (3, 40, 72, 8.0, 12), (1, 16, 16, 1.0, 8),
                                                     (2, 128, 128, 16.0, 8), (5, 1, 3, 2.0, 2), (5, 32, 96, 32.0, 24)])
def test_gated_linear_attention_in_portions_in_slots_used_again_and_a_first_token_that_lasts(dtype, heads, dim, vdim, tau, rank):
    """Two requests side by side, one whole and one in portions down to single tokens; a third request takes a slot that was
    given back and must find it zero; with decays near one the first token still shows hundreds of tokens later."""
    width, T = 40, 300
    layer = C._gla(heads, dim, vdim, tau)
    spec, W = one_model([layer], width, eps=3e-5, rank=rank, seed=dim + vdim)
    W["l0.mix.a2.b"] = (W["l0.mix.a2.b"] + 3.0).to(torch.bfloat16).float()        # decays of 0.9 to 0.999
    m, pre = layer["mixer"], "l0.mix."
    w64 = {k: v.double().numpy() for k, v in W.items()}
    g = torch.Generator().manual_seed(3)
    xa = (torch.randn(T, width, generator=g) * 0.7).to(DT[dtype]).float()
    xb = torch.randn(33, width, generator=g).to(DT[dtype]).float()
    want_a = P.mixer_gla(xa.double().numpy(), m, w64, pre, 3e-5)
    want_b, S_b = P.mixer_gla(xb.double().numpy(), m, w64, pre, 3e-5, return_state=True)
    x2 = xa.clone()
    x2[0] = -xa[0] * 3
    assert rel(P.mixer_gla(x2.double().numpy(), m, w64, pre, 3e-5)[-1:], want_a[-1:]) > 1e-3, \
        "the first token must still show at the end for this test to say anything"
    rt = rt_of(dtype)
    part = bound(spec, 0, W, rt, width)
    tol = TOL[dtype] * (3 if dtype == "bfloat16" else 1)
    cache, step = stepper([part.cache_need()], rt, requests=2)
    got_a, at = [], 0
    for i, n in enumerate(cuts(T, [1, 2, 9, 1, 17, 3, 64, 2])):
        batch = [("a", n)] + ([("b", 33)] if i == 2 else [])
        ctx = step(batch)
        rows = torch.cat([xa[at:at + n]] + ([xb] if i == 2 else [])).to(DT[dtype]).to(DEV)
        out = plain(part.forward(rows, ctx, cache.site_cache[0]))
        got_a.append(out[:n])
        if i == 2:
            assert rel(out[n:], want_b) < tol
            slot = cache._slot_of["b"]
            assert rel(cache.site_cache[0].state[slot].reshape(heads, -1), S_b.reshape(heads, -1)) < (1e-4 if dtype == "float32" else 2e-2)
            cache.free("b")
        at += n
    assert rel(torch.cat(got_a), want_a) < tol
    # a newcomer in b's old slot starts from zero
    ctx = step([("c", 33)])
    assert rel(plain(part.forward(xb.to(DT[dtype]).to(DEV), ctx, cache.site_cache[0])), want_b) < tol
    # the whole text at once, and token by token from the start
    cache, step = stepper([part.cache_need()], rt, requests=2)
    assert rel(in_portions(part, xa.to(DT[dtype]), cache, step, [T]), want_a) < tol
    cache, step = stepper([part.cache_need()], rt, requests=2)
    assert rel(in_portions(part, xa[:40].to(DT[dtype]), cache, step, [1] * 40), want_a[:40]) < tol


def spiked(x, W, pre, m, row, key, strength):
    """x and W changed so that `row`'s score with `key` stands out in every head: two input columns are set aside, one drives the
    last (unturned) entry of every query head from `row`, the other the same entry of every key head from `key`."""
    x, W = x.clone(), {k: v.clone() for k, v in W.items()}
    D = m["dim"]
    a, b = 0, 1
    x[:, a] = 0
    x[:, b] = 0
    x[row, a] = strength
    x[key, b] = strength
    for name, col, heads in ((pre + "q", a, m["heads"]), (pre + "k", b, m["kv_heads"])):
        W[name][:, [a, b]] = 0
        for h in range(heads):
            W[name][h * D + D - 1, col] = 1.0
    return x, W


ATTN_CASES = {
    # heads, kv, dim, vdim, scale, rot dims, scaling
    "narrow values, half a head turned, a stretch": (4, 2, 16, 8, 0.3, 8, (4.0, 64, 8.0, 2.0)),
    "tensor-core sizes": (8, 2, 64, 64, 0.125, 32, (8.0, 256, 16.0, 1.0)),
    "one kv head, keys of 128 over values of 48": (6, 1, 128, 48, 0.09, 64, (3.0, 1024, 16.0, 0.5)),
    "as many kv heads as heads, no stretch": (2, 2, 32, 16, 0.15, 16, None),
    "no rotation": (3, 1, 24, 40, 0.2, 0, None),
    "keys of 128, values of 64": (4, 2, 128, 64, 0.09, 64, None),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(ATTN_CASES))
def test_attention_with_biases_a_stretch_and_carried_values_reaches_a_far_key(case, dtype):
    """Two value-mixing layers on the same rows: the first leaves its values, the second blends its own with them. Row 290's
    score with key 3 stands out, so its output is (nearly) that key's blended value: a lost far key, a lost blend or a lost
    bias shows. In portions across pages' edges and token by token."""
    H, G, D, VD, scale, dims, scaling = ATTN_CASES[case]
    width, T = 48, 300
    rot = C._rot(10000.0, dims, scaling) if dims else None
    layers = [C._attn(H, G, D, VD, scale, rot, v_mix=True), C._attn(H, G, D, VD, scale, rot, v_mix=True)]
    spec, W = one_model(layers, width, seed=D + VD)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, width, generator=g).to(DT[dtype]).float()
    x, W = spiked(x, W, "l1.mix.", layers[1]["mixer"], 290, 3, 6.0 / (scale ** 0.5))
    w64 = {k: v.double().numpy() for k, v in W.items()}
    n64 = x.double().numpy()
    first = P.attention_values(n64, layers[0]["mixer"], w64, "l0.mix.")
    want0 = P.mixer_attention(n64, layers[0]["mixer"], w64, "l0.mix.")
    want1 = P.mixer_attention(n64, layers[1]["mixer"], w64, "l1.mix.", first)
    # the far key carries row 290: without it the row would be another
    lost = P.mixer_attention(n64[4:], layers[1]["mixer"], w64, "l1.mix.", first[4:])
    assert rel(lost[290 - 4:291 - 4], want1[290:291]) > 0.05
    rt = rt_of(dtype)
    p0, p1 = bound(spec, 0, W, rt, width), bound(spec, 1, W, rt, width)
    assert p1.carry_blend is not None and p0.carry_blend is None
    tol = TOL[dtype] * (2 if dtype == "bfloat16" else 1)
    for sizes in ([T], [7, 2, 33, 3, 16, 5], [250] + [1] * 50):
        cache, step = stepper([p0.cache_need(), p1.cache_need()], rt, requests=2)
        outs0, outs1, at = [], [], 0
        for n in cuts(T, sizes):
            ctx = step([("r", n)])
            rows = x[at:at + n].to(DT[dtype]).to(DEV)
            outs0.append(plain(p0.forward(rows, ctx, cache.site_cache[0])))
            outs1.append(plain(p1.forward(rows, ctx, cache.site_cache[1])))
            at += n
        assert rel(torch.cat(outs0), want0) < tol, sizes
        assert rel(torch.cat(outs1), want1) < tol, sizes


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,R,VD,L,Q", [(3, 12, 4, 10, 20, 14), (4, 64, 32, 64, 64, 48), (1, 8, 16, 24, 16, 8), (6, 48, 16, 64, 128, 72),
                                          (2, 32, 8, 128, 320, 40)])
def test_latent_attention_with_a_sink_and_an_output_gate(dtype, H, D, R, VD, L, Q):
    """Hundreds of keys, portions across pages' edges, token by token; sinks from far below every score (no effect) to above
    them (most of the weight)."""
    width, T = 56, 280
    layer = C._latent(H, D, R, VD, L, Q, 0.6 / (D + R) ** 0.5, 1000.0)
    spec, W = one_model([layer], width, seed=L + Q)
    W["l0.mix.sink"] = torch.linspace(-30.0, 4.0, H) if H > 1 else torch.tensor([1.0])
    m = layer["mixer"]
    w64 = {k: v.double().numpy() for k, v in W.items()}
    g = torch.Generator().manual_seed(6)
    x = torch.randn(T, width, generator=g).to(DT[dtype]).float()
    want = P.mixer_latent_attention(x.double().numpy(), m, w64, "l0.mix.", 1e-5)
    no_sink = dict(w64)
    no_sink["l0.mix.sink"] = np.full(H, -1e9)
    assert rel(P.mixer_latent_attention(x.double().numpy(), m, no_sink, "l0.mix.", 1e-5), want) > 0.05
    rt = rt_of(dtype)
    part = bound(spec, 0, W, rt, width)
    tol = TOL[dtype] * (2 if dtype == "bfloat16" else 1)
    for sizes in ([T], [7, 2, 33, 3, 16, 5], [240] + [1] * 40):
        cache, step = stepper([part.cache_need()], rt, requests=2)
        assert rel(in_portions(part, x.to(DT[dtype]), cache, step, cuts(T, sizes)), want) < tol, sizes


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,k,ff,rows", [(5, 2, 24, 37), (8, 3, 64, 300), (2, 1, 40, 5), (4, 4, 16, 1), (24, 5, 48, 20)])
def test_experts_chosen_by_softmax_scores_keep_their_scores(dtype, E, k, ff, rows):
    from tandemllm_b200.parts import make_part
    width = 72
    spec, W = one_model([C._gla(1, 8, 8, 2.0, ff=(E, k, ff))], width, seed=E + k, streams=2)
    rt = rt_of(dtype)
    ffp = make_part("feed_forward", spec.layers[0].feed_forward, prefix="l0.", hidden_size=width)
    ffp.bind(reader(W), rt)
    norm = make_part("norm", spec.layers[0].feed_forward_norm, prefix="l0.", size=width)
    norm.bind(reader(W), rt)
    g = torch.Generator().manual_seed(8)
    x = torch.randn(rows, width, generator=g)
    w64 = {k_: v.double().numpy() for k_, v in W.items()}
    # through the norm's kernel, as a layer runs it: the router sees the unrounded normed rows
    from tandemllm_b200.kernels import ops
    res = torch.stack([x, 2 * x]).to(DEV).contiguous()
    read = torch.tensor([0.5, 0.25], device=DEV)
    from tandemllm_b200.parts.block import _Reading
    out = plain(ffp.forward_from(_Reading(norm, read), res, ops.StreamUpdate(None, None, None), None))
    n = P.offset_norm(x.double().numpy(), w64["l0.norm2"], 1e-5)
    # the router reads the unrounded normed rows in both precisions; the experts read them in the compute dtype
    scores = P.softmax(n @ w64["l0.mlp.router"].T)
    fed = torch.from_numpy(n).to(DT[dtype]).double().numpy()
    want = np.zeros((rows, width))
    for t in range(rows):
        for e in np.argsort(-scores[t], kind="stable")[:k]:
            want[t] += scores[t, e] * P.dense_gated(fed[t:t + 1], w64, f"l0.mlp.e{e}.")[0]
    assert np.allclose(P.routed_experts(n, spec_mlp(E, k, ff), w64, "l0.mlp.")[0], P.routed_experts(n[:1], spec_mlp(E, k, ff), w64, "l0.mlp.")[0])
    # a row whose k-th and (k+1)-th scores nearly tie may choose otherwise: such rows are left out
    srt = np.sort(scores, axis=-1)[:, ::-1]
    clear = (srt[:, k - 1] - srt[:, k] > 1e-5 * srt[:, 0]) if k < E else np.ones(rows, bool)
    assert clear.sum() >= max(1, int(0.9 * rows))
    assert rel(out[torch.from_numpy(clear)], want[clear]) < TOL[dtype] * (3 if dtype == "bfloat16" else 1)


def spec_mlp(E, k, ff):
    return {"kind": "moe", "router": {"experts": E, "top": k}, "expert": {"ff": ff}}


# ------------------------------------------------------------------------------------------ whole models
def engine_of(name, dtype, pages=64, parallel=4, cfg=None, W=None, **kw):
    from tandemllm_b200.config import NiralixConfig
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.weights.loader import DictWeights
    cfg = cfg or C.CONFIGS[name]
    W = W or C.weights(name, bf16_exact=True)
    spec = NiralixConfig.from_dict(cfg).to_spec()
    args = EngineArgs(dtype=dtype, max_len=4096, parallel=parallel, block_size=16, kv_blocks=pages, graph=False, **kw)
    return Engine._build(None, spec, DictWeights({k: v.clone() for k, v in W.items()}), args), cfg, W


def run_schedule(engine, requests, schedule):
    """`schedule`: steps of [(request, count), ...]; every position's logits are wanted. Returns request -> logits."""
    from tandemllm_b200.engine import StepEntry
    at = {r: 0 for r in requests}
    got = {r: [] for r in requests}
    for step in schedule:
        entries = []
        for r, n in step:
            if not engine.cache.has(r):
                engine.admit(r)
            entries.append(StepEntry(r, requests[r][at[r]:at[r] + n], list(range(n))))
        logits = engine.step(entries).float().cpu()
        o = 0
        for r, n in step:
            got[r].append(logits[o:o + n])
            o += n
            at[r] += n
            if at[r] == len(requests[r]):
                engine.release(r)
    engine.cache.check()
    return {r: torch.cat(v) for r, v in got.items()}


def held_to_the_plain_model(engine, cfg, W, requests, schedule, dtype, what="", slack=1.0):
    """32-bit: every row within the tolerance. bfloat16: these tiny models norm rows and heads of a dozen numbers, and where
    such a part happens to be small its norm multiplies the rounding of what went in (and a routed row may take another
    expert where two scores nearly tie); so nine rows in ten (of all requests together) are held to the tolerance and every
    row to four times that. A fault moves a row by its own size."""
    got = run_schedule(engine, requests, schedule)
    rows = []
    for r, toks in requests.items():
        want = torch.from_numpy(P.forward(cfg, W, toks))
        g = got[r].double()
        rows.append(((g - want).abs() / want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)).amax(dim=-1))
        if dtype == "float32":
            assert float(rows[-1].max()) < slack * TOL[dtype], (what, r, float(rows[-1].max()))
    if dtype == "bfloat16":
        rows = torch.cat(rows)
        assert float(rows.quantile(0.9)) < slack * TOL[dtype] and float(rows.max()) < 4 * slack * TOL[dtype], \
            (what, float(rows.quantile(0.9)), float(rows.max()))
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["n1", "n2", "n3", "n4"])
def test_whole_prompts_decoding_and_portions_agree_with_the_plain_model(name, dtype):
    engine, cfg, W = engine_of(name, dtype)
    toks = C.tokens(name, 150, seed=3)
    reqs = {"a": toks}
    whole = held_to_the_plain_model(engine, cfg, W, reqs, [[("a", len(toks))]], dtype, "whole")["a"]
    # the first tokens of a sequence alone
    held_to_the_plain_model(engine, cfg, W, {"a": toks[:3]}, [[("a", 1)], [("a", 1)], [("a", 1)]], dtype, "first tokens")
    # most of it at once, then token by token across pages' edges
    held_to_the_plain_model(engine, cfg, W, reqs, [[("a", 60)]] + [[("a", 1)]] * 90, dtype, "decode")
    # token by token from the very first
    held_to_the_plain_model(engine, cfg, W, {"a": toks[:70]}, [[("a", 1)]] * 70, dtype, "every token alone")
    # portions of changing size, down to two tokens
    for sizes in ([2], [7, 2, 33, 3, 16, 5], [64, 2, 31]):
        got = held_to_the_plain_model(engine, cfg, W, reqs, [[("a", c)] for c in cuts(len(toks), sizes)], dtype,
                                      f"portions {sizes}")["a"]
        if dtype == "float32":          # how the prompt was cut changes nothing beyond rounding
            assert rel(got, whole) < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["n1", "n4"])
def test_layer_by_layer(name, dtype):
    """The models cut off behind their first, second, ... layer (the last norm and the head read the streams there): a fault
    shows at the first layer that has it."""
    full, W = C.CONFIGS[name], C.weights(name)
    toks = C.tokens(name, 40, seed=9)
    for n in range(1, len(full["layers"]) + 1):
        cfg = dict(full, layers=full["layers"][:n])
        keep = {k: v for k, v in W.items() if not k.startswith("l") or int(k[1:k.index(".")]) < n}
        engine, _, _ = engine_of(None, dtype, cfg=cfg, W=keep)
        held_to_the_plain_model(engine, cfg, keep, {"a": toks}, [[("a", 33)], [("a", 2)]] + [[("a", 1)]] * 5, dtype, f"{n} layers")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["n1", "n2", "n4"])
def test_unequal_requests_in_one_batch_on_pages_and_slots_that_are_used_again(name, dtype):
    """Seven requests of unequal length through four slots and a pool too small for all of them: portions beside single
    tokens, requests that pause, pages and state slots that come back and are taken again (a slot's state must start at
    zero for its next owner)."""
    lengths = [90, 5, 47, 130, 1, 33, 64]
    reqs = {f"q{i}": C.tokens(name, n, seed=10 + i) for i, n in enumerate(lengths)}
    engine, cfg, W = engine_of(name, dtype, pages=24, parallel=4)
    rng = np.random.default_rng(0)
    at = {r: 0 for r in reqs}
    waiting, live, schedule = list(reqs), [], []
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        step = []
        for r in list(live):
            left = len(reqs[r]) - at[r]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step
            n = min(left, int(rng.choice([1, 1, 2, 3, 16, 29])))
            step.append((r, n))
            at[r] += n
            if at[r] == len(reqs[r]):
                live.remove(r)
        if step:
            schedule.append(step)
    got = held_to_the_plain_model(engine, cfg, W, reqs, schedule, dtype, "mixed")
    if dtype == "float32":
        # each request alone, whole: what else was in the batch changes nothing beyond rounding
        for r, toks in reqs.items():
            alone = run_schedule(engine, {r: toks}, [[(r, len(toks))]])[r]
            assert rel(got[r], alone) < 2e-5, r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    engine, cfg, W = engine_of("n2", dtype, pages=28)
    toks = C.tokens("n2", 330, seed=8)
    held_to_the_plain_model(engine, cfg, W, {"a": toks}, [[("a", 9)]] + [[("a", 1)]] * 321, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype, tmp_path):
    """A folder on disk (config.json chooses the architecture), `Engine.generate`, several requests at once, decode steps
    from CUDA graphs where the engine takes them."""
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    name = "n2"
    folder = C.write_folder(str(tmp_path / "m"), name)
    engine = Engine.from_folder(folder, EngineArgs(dtype=dtype, max_len=256, parallel=3, chunk_size=32, max_batched_tokens=64))
    assert engine.model.spec.architecture == "Niralix" and engine.model.graph_safe
    prompts = [C.tokens(name, n, seed=40 + n) for n in (70, 3, 21, 45)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    cfg, W = C.CONFIGS[name], C.weights(name, bf16_exact=True)
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        # rounding may take another token where two logits are close: every token must be among the plain model's best
        # given the text so far
        text = list(prompt)
        for t in out:
            row = P.forward(cfg, W, text)[-1]
            assert float(row.max() - row[t]) <= (2e-3 if dtype == "float32" else 0.12) * float(np.abs(row).max())
            text.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_on_a_folder(dtype, tmp_path):
    name = "n3"
    folder = C.write_folder(str(tmp_path / "m"), name)
    toks = {"x": C.tokens(name, 40, seed=1), "y": C.tokens(name, 19, seed=2)}
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks["x"][:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks["x"][25:], "want": [14]},
                                     {"id": "y", "tokens": toks["y"], "want": [18]}], "end": ["x", "y"]},
             {"step": 2, "entries": [{"id": "z", "tokens": toks["y"][:2], "want": []}], "end": ["z"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
                        str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    V = C.CONFIGS[name]["vocab"]
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    b = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V)
    cfg, W = C.CONFIGS[name], C.weights(name)
    wx, wy = P.forward(cfg, W, toks["x"]), P.forward(cfg, W, toks["y"])
    assert rel(a, wx[[0, 24]]) < TOL[dtype]
    assert rel(b, np.stack([wx[39], wy[18]])) < TOL[dtype]
    assert not (out / "2.f32").exists()


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_drawn_at_random(seed, dtype):
    cfg, rank = C.random_config(seed)
    W = C.random_weights(cfg, rank, 100 + seed)
    engine, cfg, W = engine_of(None, dtype, cfg=cfg, W=W, pages=32)
    g = torch.Generator().manual_seed(seed)
    toks = {r: torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for r, n in (("a", 97), ("b", 30), ("c", 2))}
    schedule = [[("a", 40), ("b", 1)], [("a", 2), ("b", 17), ("c", 2)], [("a", 1), ("b", 1)], [("a", 31), ("b", 11)],
                [("a", 23)]]
    held_to_the_plain_model(engine, cfg, W, toks, schedule, dtype, f"random {seed}", slack=2.0 if dtype == "bfloat16" else 1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_command_line_writes_a_random_model_and_generates_from_it(dtype, tmp_path):
    """`random-weights` from a config.json of this design (the names the architecture stores, the blend weight that is never
    read left out), then `generate` on the folder: greedy tokens that the plain model agrees with."""
    from tandemllm_b200.weights.safetensors_io import index_file, read_tensor
    cfg_path, folder, out = tmp_path / "config.json", tmp_path / "m", tmp_path / "out.json"
    cfg_path.write_text(json.dumps(C.N1))
    base = [sys.executable, "-m", "tandemllm_b200"]
    r = subprocess.run(base + ["random-weights", "--config", str(cfg_path), "--seed", "5", "--out", str(folder)], cwd=ROOT,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    prompt = C.tokens("n1", 19, seed=6)
    r = subprocess.run(base + ["generate", "--model", str(folder), "--dtype", dtype, "--prompt-ids", ",".join(map(str, prompt)),
                               "--tokens", "8", "--json", str(out)], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = json.loads(out.read_text())["outputs"][0]
    assert len(got) == 8
    W = {k: read_tensor(v).double().numpy() for k, v in index_file(str(folder / "model.safetensors")).items()}
    W.setdefault("l1.mix.vmix", np.array(0.0))
    text = list(prompt)
    for t in got:
        row = P.forward(C.N1, W, text)[-1]
        assert float(row.max() - row[t]) <= (2e-3 if dtype == "float32" else 0.12) * float(np.abs(row).max())
        text.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_of_real_layer_widths(dtype):
    """Layer sizes of a model that would be served (width 1024, heads of 64 and 128, a latent of 256, 16 experts, 4 streams),
    few layers and a small vocabulary: the products, attentions and scans run the forms they take at such sizes (prompt-sized
    tensor-core products, tiles of 64 rows, staged scans). A prompt in two portions, then decoding beside a second request."""
    cfg = {"architecture": "Niralix", "vocab": 1000, "width": 1024, "norm": {"eps": 1e-6}, "logit_scale": 0.5, "streams": 4,
           "layers": [C._gla(16, 64, 64, 16.0, ff=(16, 4, 256)),
                      C._attn(16, 4, 64, 64, 0.125, C._rot(500000.0, 64, (8.0, 8192, 32.0, 1.0)), v_mix=True, ff=1024),
                      C._latent(16, 64, 32, 64, 256, 384, 96 ** -0.5, 10000.0, ff=(16, 4, 256)),
                      C._attn(8, 4, 128, 64, 0.09, C._rot(500000.0, 32, (8.0, 8192, 32.0, 1.0)), v_mix=True, ff=1024)]}
    W = C.random_weights(cfg, 16, 77)
    engine, cfg, W = engine_of(None, dtype, cfg=cfg, W=W, pages=32)
    g = torch.Generator().manual_seed(9)
    toks = {r: torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for r, n in (("a", 200), ("b", 70))}
    schedule = [[("a", 150)], [("a", 40), ("b", 64)]] + [[("a", 1), ("b", 1)]] * 6 + [[("a", 4)]]
    held_to_the_plain_model(engine, cfg, W, toks, schedule, dtype, "real widths")
