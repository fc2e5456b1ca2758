"""Sebilorn on the GPU against the plain implementation (`tests/plain_sebilorn.py`): every mechanism alone as a part
with a cache of its own, then whole models through the step function, the scheduler and the replay program.

The tiny models (`tests/sebilorn_configs.py`) differ from one another in every size and constant. Where random weights
would hide a fault (a far key among hundreds, a kept first token, a window's edge), one input row's query and one row's
key are made large along an entry the rotation leaves alone, so that one score stands out: the row's output is then that
key's value if and only if the key is visible.

Tolerances as for the engine's other models: 32-bit within 1e-4 of a row's largest magnitude, bfloat16 within 3e-2.
"""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import plain_sebilorn as P
from tests import sebilorn_configs as C
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


def one_layer(layer: dict, width: int, eps: float = 1e-5, rank: int = 8, seed: int = 0, layers_before=()):
    """(mixer part spec, weights by name as 64-bit arrays and as tensors, the prefix) of a model that has this one layer
    (after `layers_before`, which a borrowing layer needs)."""
    from tandemllm_b200.config import SebilornConfig
    cfg = {"architecture": "Sebilorn", "vocab": 11, "width": width, "norm": {"eps": eps}, "embedding": {"scale": 1.0},
           "layers": list(layers_before) + [layer]}
    W = C.random_weights(cfg, rank, seed)
    spec = SebilornConfig.from_dict(cfg).to_spec()
    return spec, W, f"l{len(layers_before)}."


def bound(spec, i, W, rt, width):
    from tandemllm_b200.parts import make_part
    part = make_part("mixer", spec.layers[i].mixer, prefix=spec.layers[i].prefix, hidden_size=width)
    if hasattr(part, "shapes_from"):
        part.shapes_from(lambda n: tuple(W[n].shape) if n in W else None)
    part.bind(reader(W), rt)
    return part


def in_portions(part, x, cache, step, cuts, rid="r", site=0):
    outs, at = [], 0
    for n in cuts:
        ctx = step([(rid, n)])
        outs.append(plain(part.forward(x[at:at + n].to(DEV), ctx, cache.site_cache[site])))
        at += n
    assert at == x.shape[0]
    return torch.cat(outs)


def cuts(n, sizes):
    out, i = [], 0
    while n:
        c = min(n, sizes[i % len(sizes)])
        out.append(c)
        n -= c
        i += 1
    return out


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [44, 328, 1000])
def test_layer_norm_with_weight_and_bias(dtype, width):
    from tandemllm_b200.kernels import ops
    g = torch.Generator().manual_seed(width)
    res = torch.randn(9, width, generator=g) * 3 + 1.5          # a mean far from zero: the variance is of the deviations
    delta = torch.randn(9, width, generator=g)
    w, b = 1 + 0.2 * torch.randn(width, generator=g), 0.3 * torch.randn(width, generator=g)
    r = res.to(DEV)
    out = torch.empty(9, width, dtype=DT[dtype], device=DEV)
    ops.add_layernorm(r, delta.to(DEV), w.to(DEV), b.to(DEV), 1e-4, out)
    summed = (res + delta).double().numpy()
    assert rel(r, summed) < 1e-6
    assert rel(out.float(), P.layer_norm(summed, w.double().numpy(), b.double().numpy(), 1e-4)) < (1e-5 if dtype == "float32" else 1e-2)
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, width, dtype=DT[dtype], device=DEV)
    ops.add_layernorm(r, None, w.to(DEV), b.to(DEV), 1e-4, out2, rows)
    assert torch.equal(out2, out[[7, 2]])


ATTN_CASES = {
    # heads, kv, dim, vdim, scale, rot dims, scaling, (window, kept) or None, cap
    "narrow values, half a head turned": (4, 2, 16, 8, 0.3, 8, (4.0, 1.0, 3.0, 64), (5, 2), 7.0),
    "tensor-core sizes": (8, 2, 64, 64, 0.125, 32, (8.0, 1.0, 4.0, 256), (70, 4), 40.0),
    "one kv head, a window of pages": (8, 1, 64, 64, 0.125, 48, None, (64, 6), 50.0),
    "no mask, no cap": (2, 2, 32, 16, 0.15, 16, None, None, None),
    "a window of one": (6, 1, 8, 6, 0.5, 4, None, (1, 0), 30.0),
    "wide values": (2, 1, 128, 256, 0.07, 96, (2.0, 1.0, 2.0, 128), (33, 5), 15.0),
    "kept tokens past a page": (4, 4, 32, 32, 0.2, 16, None, (20, 19), None),
    "keys of 128, values of 64": (4, 2, 128, 64, 0.09, 64, None, (40, 3), 20.0),
    "three heads a kv head, more kept tokens than a key tile": (6, 2, 64, 128, 0.12, 64, (8.0, 1.0, 4.0, 64), (30, 70), 35.0),
}


def spiked(x, W, pre, m, row, key, strength):
    """x and W changed so that `row`'s score with `key` stands out in every head: two input columns are set aside, one
    drives the last (unturned) entry of every query head from `row`, the other the same entry of every key head from `key`."""
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(ATTN_CASES))
def test_attention_sees_its_window_and_its_kept_first_tokens_and_nothing_else(case, dtype):
    """Keys far away, at page borders, just inside and just outside the window, the last kept token and the first that is
    not, for a row inside a prompt's portion and for a row decoded alone."""
    H, G, D, VD, scale, dims, scaling, mask, cap = ATTN_CASES[case]
    width, T = 48, 150
    layer = C._attn(H, G, D, VD, scale, C._rot(9000.0, dims, scaling), mask, cap)
    spec, W, pre = one_layer(layer, width, seed=len(case))
    m = layer["mixer"]
    g = torch.Generator().manual_seed(1)
    x0 = (torch.randn(T, width, generator=g) * 0.5).to(DT[dtype]).float()
    size, keep = mask if mask else (None, 0)
    row_sets = {"prompt": 140, "decoded": 148}
    for where, row in row_sets.items():
        keys = {0, row, row - 1, 16, 15, 1}
        if size:
            keys |= {row - size + 1, row - size, keep - 1, keep}
        for key in sorted(k for k in keys if 0 <= k <= row):
            top = 0.8 * cap / scale if cap else 12.0 / scale
            x, Wk = spiked(x0, W, pre + "mix.", m, row, key, top ** 0.5)
            w64 = {k: v.double().numpy() for k, v in Wk.items()}
            want = P.mixer_attention(x.double().numpy(), m, w64, pre + "mix.", None)
            seen = P.visible(T, size, keep)[row, key]
            unspiked = x.clone()
            unspiked[key, 1] = 0.0          # the same rows without the key's spike
            base = P.mixer_attention(unspiked.double().numpy(), m, w64, pre + "mix.", None)
            moved = np.abs(want[row] - base[row]).max() / np.abs(base[row]).max()
            assert (moved > 1e-3) == bool(seen) or key == row, (case, where, key, moved)
            rt = rt_of(dtype)
            part = bound(spec, 0, Wk, rt, width)
            cache, step = stepper([part.cache_need()], rt, pages=12)        # fewer pages than the sequence has: the window's go back
            got = in_portions(part, x.to(DT[dtype]), cache, step, [31, 2, 111] + [1] * 6)
            assert rel(got, want) < TOL[dtype], (case, where, key)
            assert int(rt.status.item()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,VD,dims", [(3, 3, 12, 20, 4), (8, 2, 64, 64, 64), (4, 2, 64, 128, 32), (2, 1, 32, 32, 16), (4, 1, 128, 128, 64)])
def test_gated_attention_reaches_a_far_key_among_hundreds(dtype, H, G, D, VD, dims):
    """The attention of a side-by-side mixer on its own: causal over all keys, an entry-wise sigmoid gate, no turned values.
    One key hundreds of tokens back stands out; prompts, portions and decoding."""
    width, T = 40, 420
    left = (H, G, D, VD, 0.2, C._rot(500.0, dims))
    layer = C._parallel(left, (1, 8), 1.0, 1.0)
    spec, W, pre = one_layer(layer, width, seed=D)
    m = layer["mixer"]["left"]
    g = torch.Generator().manual_seed(2)
    x0 = (torch.randn(T, width, generator=g) * 0.5).to(DT[dtype]).float()
    rt = rt_of(dtype)
    for row, key in ((300, 3), (419, 17)):
        if dims == D:           # every entry is turned: no spike, random weights only
            x, Wk = x0, W
        else:
            x, Wk = spiked(x0, W, pre + "mix.left.", m, row, key, (10.0 / 0.2) ** 0.5)
        w64 = {k: v.double().numpy() for k, v in Wk.items()}
        want = P.mixer_gated_attention(x.double().numpy(), m, w64, pre + "mix.left.")
        from tandemllm_b200.parts import make_part
        part = make_part("mixer", spec.layers[0].mixer["mixers"][0], prefix=pre, hidden_size=width)     # the left half alone
        part.bind(reader(Wk), rt)
        cache, step = stepper([part.cache_need()], rt, pages=32)
        got = in_portions(part, x.to(DT[dtype]), cache, step, [290, 2, 7, 100, 16] + [1] * 5)
        assert rel(got, want) < TOL[dtype], (row, key)


@pytest.mark.parametrize("mask,cap", [(None, None), ((600, 3), 30.0), ((130, 70), None)])
@pytest.mark.parametrize("H,G,D,VD", [(4, 2, 64, 64), (8, 1, 128, 64), (2, 2, 64, 128)])
def test_decoding_behind_many_key_tiles(H, G, D, VD, mask, cap):
    """Rows decoded alone behind 800 keys (bfloat16): few requests and many key tiles, so several CTAs share a request's
    keys and their shares are merged. A key far back stands out, then the key at the window's edge."""
    width, T = 40, 800
    layer = C._attn(H, G, D, VD, 0.15, C._rot(3000.0, D // 2), mask, cap)
    spec, W, pre = one_layer(layer, width, seed=H + D)
    m = layer["mixer"]
    g = torch.Generator().manual_seed(3)
    x0 = (torch.randn(T, width, generator=g) * 0.5).to(torch.bfloat16).float()
    rt = rt_of("bfloat16")
    row = T - 1
    for key in (1, row - mask[0] + 1 if mask else 400):
        x, Wk = spiked(x0, W, pre + "mix.", m, row, key, ((0.8 * cap if cap else 10.0) / 0.15) ** 0.5)
        w64 = {k: v.double().numpy() for k, v in Wk.items()}
        want = P.mixer_attention(x.double().numpy(), m, w64, pre + "mix.", None)
        part = bound(spec, 0, Wk, rt, width)
        cache, step = stepper([part.cache_need()], rt, pages=64)
        got = in_portions(part, x.to(torch.bfloat16), cache, step, [T - 12] + [1] * 12)
        assert rel(got[T - 12:], want[T - 12:]) < TOL["bfloat16"], (key,)
        assert int(rt.status.item()) == 0


def _half(spec, which, pre, width, W, rt):
    from tandemllm_b200.parts import make_part
    part = make_part("mixer", spec.layers[0].mixer["mixers"][which], prefix=pre, hidden_size=width)
    if hasattr(part, "shapes_from"):
        part.shapes_from(lambda n: tuple(W[n].shape) if n in W else None)
    part.bind(reader(W), rt)
    return part


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rank", [(2, 24, 5), (4, 64, 16), (1, 160, 12), (3, 4, 3), (2, 16, 8), (1, 1, 2)])
def test_the_delta_rule_token_by_token_in_portions_and_in_slots_used_again(dtype, heads, dim, rank):
    """Two requests side by side, one whole and one in portions down to single tokens; then a third request takes a slot that
    was given back and must find it zero."""
    width, T = 40, 70
    layer = C._parallel((2, 1, 8, 8, 0.3, C._rot(100.0, 4)), (heads, dim), 1.0, 1.0)
    spec, W, pre = one_layer(layer, width, eps=3e-5, rank=rank, seed=dim)
    m = layer["mixer"]["right"]
    w64 = {k: v.double().numpy() for k, v in W.items()}
    g = torch.Generator().manual_seed(3)
    xa = torch.randn(T, width, generator=g).to(DT[dtype]).float()
    xb = torch.randn(33, width, generator=g).to(DT[dtype]).float()
    want_a = P.mixer_delta_rule(xa.double().numpy(), m, w64, pre + "mix.right.", 3e-5)
    want_b, S_b = P.mixer_delta_rule(xb.double().numpy(), m, w64, pre + "mix.right.", 3e-5, return_state=True)
    rt = rt_of(dtype)
    part = _half(spec, 1, pre, width, W, rt)
    cache, step = stepper([part.cache_need()], rt, requests=2)
    tol = TOL[dtype] * (3 if dtype == "bfloat16" else 1)
    got_a, at = [], 0
    for i, n in enumerate(cuts(T, [1, 2, 9, 1, 17, 3])):
        batch = [("a", n)] + ([("b", 33)] if i == 2 else [])
        ctx = step(batch)
        rows = torch.cat([xa[at:at + n]] + ([xb] if i == 2 else [])).to(DT[dtype]).to(DEV)
        out = plain(part.forward(rows, ctx, cache.site_cache[0]))
        got_a.append(out[:n])
        if i == 2:
            assert rel(out[n:], want_b) < tol
            slot = cache._slot_of["b"]
            # (bfloat16 rounds the decay's inner product of `rank` numbers; everything behind it is 32-bit in both modes)
            assert rel(cache.site_cache[0].state[slot].reshape(heads, -1), S_b.reshape(heads, -1)) < (1e-4 if dtype == "float32" else 3e-3)
            cache.free("b")
        at += n
    assert rel(torch.cat(got_a), want_a) < tol
    # a newcomer in b's old slot starts from zero
    ctx = step([("c", 33)])
    assert rel(plain(part.forward(xb.to(DT[dtype]).to(DEV), ctx, cache.site_cache[0])), want_b) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim", [(3, 8, 24), (4, 64, 32), (2, 40, 72), (1, 16, 16), (2, 128, 128), (5, 1, 3)])
def test_lightning_attention_in_portions_and_a_first_token_that_still_shows_hundreds_later(dtype, heads, dim, vdim):
    width, T = 56, 400
    decay = [0.999] + [float(np.exp(-0.5 / (h + 1))) for h in range(heads - 1)]
    layer = C._lightning(heads, dim, vdim, decay)
    spec, W, pre = one_layer(layer, width, eps=1e-6, seed=dim + vdim)
    m = layer["mixer"]
    w64 = {k: v.double().numpy() for k, v in W.items()}
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(T, width, generator=g) * 0.7).to(DT[dtype]).float()
    want = P.mixer_lightning(x.double().numpy(), m, w64, pre + "mix.", 1e-6)
    x2 = x.clone()
    x2[0] = -x[0] * 3
    assert rel(P.mixer_lightning(x2.double().numpy(), m, w64, pre + "mix.", 1e-6)[-1:], want[-1:]) > 1e-3, \
        "the first token must still show at the end for this test to say anything"
    rt = rt_of(dtype)
    part = bound(spec, 0, W, rt, width)
    tol = TOL[dtype] * (3 if dtype == "bfloat16" else 1)
    for sizes in ([T], [300] + [1] * 100, [2], [7, 1, 64, 3]):
        cache, step = stepper([part.cache_need()], rt, requests=2)
        got = in_portions(part, x.to(DT[dtype]), cache, step, cuts(T, sizes))
        assert rel(got, want) < tol, sizes


# ------------------------------------------------------------------------------------------ whole models
def engine_of(name, dtype, pages=64, parallel=4, cfg=None, W=None, **kw):
    from tandemllm_b200.config import SebilornConfig
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.weights.loader import DictWeights
    cfg = cfg or C.CONFIGS[name]
    W = W or C.weights(name, bf16_exact=True)
    spec = SebilornConfig.from_dict(cfg).to_spec()
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
    such a part happens to be small its norm multiplies the rounding of what went in; so nine rows in ten (of all requests
    together) are held to the tolerance and every row to three times that. A fault moves a row by its own size."""
    got = run_schedule(engine, requests, schedule)
    rows = []
    for r, toks in requests.items():
        want = torch.from_numpy(P.forward(cfg, W, toks))
        g = got[r].double()
        rows.append(((g - want).abs() / want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)).amax(dim=-1))
        if dtype == "float32":
            assert float(rows[-1].max()) < slack * TOL[dtype], (what, r)
    if dtype == "bfloat16":
        rows = torch.cat(rows)
        assert float(rows.quantile(0.9)) < slack * TOL[dtype] and float(rows.max()) < 3 * slack * TOL[dtype], what
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["b1", "b2", "b3", "b4"])
def test_whole_prompts_decoding_and_portions_agree_with_the_plain_model(name, dtype):
    engine, cfg, W = engine_of(name, dtype)
    toks = C.tokens(name, 150, seed=3)
    reqs = {"a": toks}
    whole = held_to_the_plain_model(engine, cfg, W, reqs, [[("a", len(toks))]], dtype, "whole")["a"]
    # the first tokens of a sequence alone
    held_to_the_plain_model(engine, cfg, W, {"a": toks[:3]}, [[("a", 1)], [("a", 1)], [("a", 1)]], dtype, "first tokens")
    # most of it at once, then token by token across windows' and pages' edges
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
@pytest.mark.parametrize("name", ["b1", "b4"])
def test_layer_by_layer(name, dtype):
    """The models cut off behind their first, second, ... layer (the final norm and the head read the stream there): a
    fault shows at the first layer that has it."""
    full, W = C.CONFIGS[name], C.weights(name)
    toks = C.tokens(name, 40, seed=9)
    for n in range(1, len(full["layers"]) + 1):
        cfg = dict(full, layers=full["layers"][:n])
        keep = {k: v for k, v in W.items() if not k.startswith("l") or int(k[1:k.index(".")]) < n}
        engine, _, _ = engine_of(None, dtype, cfg=cfg, W=keep)
        held_to_the_plain_model(engine, cfg, keep, {"a": toks}, [[("a", 33)], [("a", 2)]] + [[("a", 1)]] * 5, dtype, f"{n} layers")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["b1", "b2", "b4"])
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
@pytest.mark.parametrize("name", ["b1", "b2"])
def test_long_decoding_past_every_window(name, dtype):
    engine, cfg, W = engine_of(name, dtype, pages=28)
    toks = C.tokens(name, 400, seed=8)
    held_to_the_plain_model(engine, cfg, W, {"a": toks}, [[("a", 9)]] + [[("a", 1)]] * 391, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype, tmp_path):
    """A folder on disk (config.json chooses the architecture), `Engine.generate`, several requests at once, decode steps
    from CUDA graphs where the engine takes them."""
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    name = "b2"
    folder = C.write_folder(str(tmp_path / "m"), name)
    engine = Engine.from_folder(folder, EngineArgs(dtype=dtype, max_len=256, parallel=3, chunk_size=32, max_batched_tokens=64))
    assert engine.model.spec.architecture == "Sebilorn"
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
    name = "b3"
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
