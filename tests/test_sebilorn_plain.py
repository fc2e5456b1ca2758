"""Sebilorn without a GPU: the configuration reader, the sites and caches it makes, the tensors the parts ask for, and the
plain implementation's own consistency (a prefix does not change when the sequence goes on; a key outside a window changes
nothing and a kept first token does; the recurrences equal their unrolled sums)."""

import copy
import math

import numpy as np
import pytest

from tests import plain_sebilorn as P
from tests import sebilorn_configs as C


def w64(name):
    return {k: v.double().numpy() for k, v in C.weights(name).items()}


def test_the_reader_names_every_tensor_of_the_design():
    from tandemllm_b200.config import SebilornConfig, architecture_of
    from tandemllm_b200.parts.model import DecoderModel
    for name, cfg in C.CONFIGS.items():
        assert architecture_of(cfg).name == "sebilorn"
        spec = SebilornConfig.from_dict(cfg).to_spec()
        model = DecoderModel(spec)
        rank = C.RANKS[name]
        shapes = C.tensor_shapes(cfg, rank)
        for layer in model.layers:
            for part in layer.parts:
                if hasattr(part, "shapes_from"):
                    part.shapes_from(lambda n: shapes.get(n))
        got = {s.name: tuple(s.shape) for s in model.weight_specs(None)}
        assert got == shapes, name


def test_a_borrowing_layer_reads_its_owners_site_and_the_owner_keeps_the_widest_mask():
    from tandemllm_b200.config import SebilornConfig
    from tandemllm_b200.parts.base import PagedNeed, SlotNeed
    from tandemllm_b200.parts.model import DecoderModel
    spec = SebilornConfig.from_dict(C.B1).to_spec()
    assert [s.cache_of for s in spec.schedule] == [None, 0, None, None, None]
    needs = DecoderModel(spec).cache_needs()
    # layer 0 has a window of 5 keeping 2; its borrower a window of 9 keeping 3: the pages keep 9 and 3
    assert needs[0] == PagedNeed(2, 16, 9, value_dim=8, keep_first=3)
    assert needs[1] is None
    left, right = needs[2]
    assert left == PagedNeed(3, 12, None, value_dim=20) and isinstance(right, SlotNeed) and right.shape == (2, 24, 24)
    assert isinstance(needs[3], SlotNeed) and needs[3].shape == (3, 8, 24)
    assert needs[4] == PagedNeed(1, 8, 1, value_dim=6)
    # a borrower without a mask leaves its owner without a window
    cfg = copy.deepcopy(C.B2)
    del cfg["layers"][3]["mixer"]["mask"]
    assert DecoderModel(SebilornConfig.from_dict(cfg).to_spec()).cache_needs()[1].window is None


def test_unknown_keys_and_bad_sizes_are_refused_by_name():
    from tandemllm_b200.config import SebilornConfig
    bad = copy.deepcopy(C.B2)
    bad["layers"][1]["mixer"]["heads_kv"] = 2
    with pytest.raises(ValueError, match="heads_kv"):
        SebilornConfig.from_dict(bad)
    bad = copy.deepcopy(C.B2)
    bad["layers"][1]["mixer"]["rot"]["scaling"]["mid"] = 2.0
    with pytest.raises(ValueError, match="mid"):
        SebilornConfig.from_dict(bad)
    bad = copy.deepcopy(C.B2)
    bad["layers"][3]["mixer"]["kv_from"] = 2            # a parallel layer owns no borrowable keys
    with pytest.raises(ValueError, match="kv_from"):
        SebilornConfig.from_dict(bad)
    bad = copy.deepcopy(C.B1)
    bad["layers"][3]["mixer"]["decay"] = [0.5, 0.9]
    with pytest.raises(ValueError, match="decays"):
        SebilornConfig.from_dict(bad)
    bad = copy.deepcopy(C.B1)
    bad["layers"][0]["type"] = "retention"
    with pytest.raises(ValueError, match="retention"):
        SebilornConfig.from_dict(bad)
    bad = copy.deepcopy(C.B1)
    bad["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError, match="moe"):
        SebilornConfig.from_dict(bad)
    assert SebilornConfig.from_dict(C.B4).to_dict() == C.B4


def test_the_engines_frequencies_are_the_plain_ones():
    from tandemllm_b200.parts.position import RotaryNeox
    for base, dims, scaling in [(10000.0, 8, None), (500000.0, 64, (8.0, 1.0, 4.0, 1024)), (100.0, 16, (2.0, 1.0, 2.0, 32)),
                                (50000.0, 96, (4.0, 0.5, 3.0, 200))]:
        s = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
        part = RotaryNeox({"theta": base, "rotary_dim": dims, "scaling": s, "precise": True}, head_dim=dims)
        want = P.rotary_frequencies(base, dims, s)
        assert np.allclose(part.frequencies().double().numpy(), want, rtol=1e-6, atol=0)
    # all three branches of the scaling occur in one table
    f = P.rotary_frequencies(100.0, 16, {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 32})
    raw = P.rotary_frequencies(100.0, 16)
    kinds = {"kept" if a == b else ("slowed" if math.isclose(a, b / 2.0) else "blend") for a, b in zip(f, raw)}
    assert kinds == {"kept", "slowed", "blend"}


def test_the_plain_model_is_causal_and_its_windows_end_where_they_should():
    cfg, W = C.B1, w64("b1")
    toks = C.tokens("b1", 30, seed=1)
    whole = P.forward(cfg, W, toks)
    assert np.allclose(P.forward(cfg, W, toks[:13]), whole[:13], atol=1e-10)
    m = cfg["layers"][0]["mixer"]
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    rng = np.random.default_rng(3)
    h = rng.standard_normal((14, cfg["width"]))
    base = P.mixer_attention(h, m, W, "l0.mix.", None)
    for at, seen in [(13 - size, False), (13 - size + 1, True), (keep - 1, True), (keep, False)]:
        h2 = h.copy()
        h2[at] += 3.0
        same = np.allclose(P.mixer_attention(h2, m, W, "l0.mix.", None)[13], base[13], atol=1e-12)
        assert same != seen, (at, seen)


def test_turning_the_values_and_turning_the_output_back_leaves_relative_angles():
    """sum_j p_j R(j) v_j turned by -i equals sum_j p_j R(j - i) v_j."""
    rng = np.random.default_rng(0)
    T, VD = 7, 12
    v = rng.standard_normal((T, 1, VD))
    f = P.rotary_frequencies(300.0, VD)
    p = rng.random((T, T)) * P.visible(T, None, 0)
    p /= p.sum(-1, keepdims=True)
    turned = P.rotate_halves(v, np.arange(T), f)
    got = P.rotate_halves((p @ turned[:, 0])[:, None], np.arange(T), f, sign=-1.0)[:, 0]
    for i in range(T):
        want = sum(p[i, j] * P.rotate_halves(v[j:j + 1], np.array([j - i]), f)[0, 0] for j in range(i + 1))
        assert np.allclose(got[i], want, atol=1e-12)


def test_the_lightning_recurrence_equals_its_unrolled_sum():
    cfg, W = C.B1, w64("b1")
    m = cfg["layers"][3]["mixer"]
    rng = np.random.default_rng(5)
    T = 9
    n = rng.standard_normal((T, cfg["width"]))
    H, D, VD = m["heads"], m["dim"], m["vdim"]
    p = "l3.mix."
    q = P.silu(n @ W[p + "q"].T).reshape(T, H, D)
    k = P.silu(n @ W[p + "k"].T).reshape(T, H, D)
    v = P.silu(n @ W[p + "v"].T).reshape(T, H, VD)
    o = np.zeros((T, H, VD))
    for h in range(H):
        for t in range(T):
            for s in range(t + 1):
                o[t, h] += m["decay"][h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h]
    o = P.unit_rms(o.reshape(T, H * VD), 1e-4) * W[p + "norm"] * P.sigmoid(n @ W[p + "g"].T)
    assert np.allclose(P.mixer_lightning(n, m, W, p, 1e-4), o @ W[p + "o"].T, atol=1e-10)
    # in two portions through the state
    a, S = P.mixer_lightning(n[:4], m, W, p, 1e-4, return_state=True)
    b = P.mixer_lightning(n[4:], m, W, p, 1e-4, state=S)
    assert np.allclose(np.concatenate([a, b]), o @ W[p + "o"].T, atol=1e-10)


def test_the_delta_rule_reads_the_old_state_in_both_terms():
    """One head, two keys: after a first token the second step is written out by hand."""
    w = {"x.r": np.eye(2), "x.k": np.eye(2), "x.v": np.eye(2), "x.a": np.zeros((2, 2)), "x.a.b": np.array([0.3, -0.2]),
         "x.w1": np.zeros((1, 2)), "x.w2": np.zeros((2, 1)), "x.w0": np.array([0.5, -1.0]), "x.g": np.zeros((2, 2)),
         "x.norm": np.ones(2), "x.o": np.eye(2)}
    m = {"heads": 1, "dim": 2}
    n = np.array([[1.0, 2.0], [0.5, -1.5]])
    _, S = P.mixer_delta_rule(n, m, w, "x.", 1e-5, return_state=True)
    d = np.exp(-math.exp(-0.5) * P.sigmoid(w["x.w0"]))
    a = P.sigmoid(w["x.a.b"])
    S1 = np.outer(n[0], n[0])
    u = n[1] / math.sqrt(n[1] @ n[1] + 1e-6)
    S2 = d[:, None] * S1 - np.outer(a * u, u @ S1) + np.outer(n[1], n[1])
    assert np.allclose(S[0], S2, atol=1e-12)
    # and a portion that starts from a state goes on as the whole sequence does
    cfg, W = C.B1, w64("b1")
    rng = np.random.default_rng(2)
    h = rng.standard_normal((8, cfg["width"]))
    mm = cfg["layers"][2]["mixer"]["right"]
    whole = P.mixer_delta_rule(h, mm, W, "l2.mix.right.", 1e-4)
    a_, S = P.mixer_delta_rule(h[:3], mm, W, "l2.mix.right.", 1e-4, return_state=True)
    b_ = P.mixer_delta_rule(h[3:], mm, W, "l2.mix.right.", 1e-4, state=S)
    assert np.allclose(np.concatenate([a_, b_]), whole, atol=1e-10)


def test_models_drawn_at_random_are_read():
    from tandemllm_b200.config import SebilornConfig
    from tandemllm_b200.parts.model import DecoderModel
    for seed in range(20):
        cfg, rank = C.random_config(seed)
        spec = SebilornConfig.from_dict(cfg).to_spec()
        model = DecoderModel(spec)
        shapes = C.tensor_shapes(cfg, rank)
        for layer in model.layers:
            for part in layer.parts:
                if hasattr(part, "shapes_from"):
                    part.shapes_from(lambda n: shapes.get(n))
        assert {s.name: tuple(s.shape) for s in model.weight_specs(None)} == shapes, seed
