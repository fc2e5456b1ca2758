"""Niralix without a GPU: the configuration reader, the caches it asks for, the tensors the parts ask for, the engine's
stretched frequencies, and the plain implementation's own consistency (a prefix does not change when the sequence goes on;
the gated recurrence equals its unrolled sum; streams with an identity mixing are one residual; a sink only takes weight
away; mixed values are the first mixing layer's)."""

import copy
import math

import numpy as np
import pytest

from tests import niralix_configs as C
from tests import plain_niralix as P


def w64(name):
    return {k: v.double().numpy() for k, v in C.weights(name).items()}


def test_the_reader_names_every_tensor_of_the_design():
    from tandemllm_b200.config import NiralixConfig, architecture_of
    from tandemllm_b200.parts.model import DecoderModel
    for name, cfg in C.CONFIGS.items():
        assert architecture_of(cfg).name == "niralix"
        spec = NiralixConfig.from_dict(cfg).to_spec()
        model = DecoderModel(spec)
        shapes = C.tensor_shapes(cfg, C.RANKS[name])
        for layer in model.layers:
            for part in layer.parts:
                if hasattr(part, "shapes_from"):
                    part.shapes_from(lambda n: shapes.get(n))
        got = {s.name: tuple(s.shape) for s in model.weight_specs(None)}
        # the first value-mixing layer's own blend weight is stored and never read (the other ignored names are what a folder
        # may hold for a sublayer or a blend that is not there)
        assert set(shapes) - set(got) <= set(spec.ignored_names) and not set(got) & set(spec.ignored_names), name
        assert got == {k: v for k, v in shapes.items() if k not in spec.ignored_names}, name
        assert NiralixConfig.from_dict(NiralixConfig.from_dict(cfg).to_dict()).to_spec() == spec


def test_caches_states_and_streams_follow_the_configuration():
    from tandemllm_b200.config import NiralixConfig
    from tandemllm_b200.parts.base import PagedNeed, SlotNeed
    from tandemllm_b200.parts.model import DecoderModel
    spec = NiralixConfig.from_dict(C.N1).to_spec()
    assert spec.streams == 3 and spec.logit_scale == 0.7 and spec.head_name is None
    assert all(l.arrangement == "hyper_connections" for l in spec.layers)
    needs = DecoderModel(spec).cache_needs()
    assert isinstance(needs[0], SlotNeed) and needs[0].shape == (3, 8, 6)
    assert needs[1] == PagedNeed(2, 16, None, value_dim=8)
    assert needs[2] == PagedNeed(1, 24, None, values=False)            # the latent and the shared rotated key part
    assert needs[3] == PagedNeed(2, 8, None)
    # the first mixing layer leaves its values, the later ones blend with them
    carries = [l.mixer.get("value_carry") for l in spec.layers]
    assert carries[1]["blend"] is None and carries[3]["blend"] == "mix.vmix" and carries[1]["key"] == carries[3]["key"]
    assert "l1.mix.vmix" in spec.ignored_names and "l3.mix.vmix" not in spec.ignored_names
    plain = NiralixConfig.from_dict(C.N3).to_spec()
    assert plain.streams == 0 and all(l.arrangement == "prenorm_residual" for l in plain.layers)
    assert all(l.mixer.get("value_carry") is None for l in plain.layers if l.mixer.kind == "attention")


def test_unknown_keys_and_bad_sizes_are_refused_by_name():
    from tandemllm_b200.config import NiralixConfig
    bad = copy.deepcopy(C.N2)
    bad["layers"][0]["mixer"]["window"] = 4
    with pytest.raises(ValueError, match="window"):
        NiralixConfig.from_dict(bad)
    bad = copy.deepcopy(C.N2)
    bad["layers"][2]["mixer"]["rot"]["scaling"] = {"factor": 2.0}
    with pytest.raises(ValueError, match="scaling"):
        NiralixConfig.from_dict(bad)
    bad = copy.deepcopy(C.N2)
    bad["layers"][3]["mixer"]["vdim"] = 32          # mixes with layer 0's values of 64
    with pytest.raises(ValueError, match="sizes differ"):
        NiralixConfig.from_dict(bad)
    bad = copy.deepcopy(C.N1)
    bad["layers"][1]["mlp"]["router"]["top"] = 6
    with pytest.raises(ValueError, match="top 6 of 5"):
        NiralixConfig.from_dict(bad)
    bad = copy.deepcopy(C.N1)
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError, match="conv"):
        NiralixConfig.from_dict(bad)
    bad = copy.deepcopy(C.N1)
    bad["streams"] = 9
    with pytest.raises(ValueError, match="streams 9"):
        NiralixConfig.from_dict(bad)


def test_the_engines_frequencies_are_the_plain_ones():
    from tandemllm_b200.parts.position import RotaryNeox
    cases = [(10000.0, 8, None), (300000.0, 48, (3.0, 1024, 16.0, 0.5)), (100.0, 16, (8.0, 64, 8.0, 2.0)),
             (50000.0, 128, (2.0, 128, 1e9, 1e-9)), (300.0, 2, (4.0, 16, 3.0, 1.0))]
    for base, dims, scaling in cases:
        s = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
        part = RotaryNeox({"theta": base, "rotary_dim": dims, "scaling": s, "precise": True}, head_dim=dims)
        want, magnitude = P.stretched_frequencies(base, dims, s)
        assert np.allclose(part.frequencies().double().numpy(), want, rtol=1e-6, atol=0)
        assert math.isclose(part.magnitude, magnitude, rel_tol=1e-12)
    # kept, slowed and blended pairs occur in one table, and the magnitude follows the factor
    f, mag = P.stretched_frequencies(100.0, 16, {"factor": 8.0, "original": 64, "fast": 8.0, "slow": 2.0})
    raw, one = P.stretched_frequencies(100.0, 16, None)
    kinds = {"kept" if a == b else ("slowed" if math.isclose(a, b / 8.0) else "blend") for a, b in zip(f, raw)}
    assert kinds == {"kept", "slowed", "blend"} and one == 1.0 and math.isclose(mag, 1.0 + 0.1 * math.log(8.0))


def test_a_prefix_does_not_change_when_the_sequence_goes_on():
    for name in ("n1", "n3"):
        toks = C.tokens(name, 40, seed=2)
        whole = P.forward(C.CONFIGS[name], w64(name), toks)
        assert np.allclose(P.forward(C.CONFIGS[name], w64(name), toks[:17]), whole[:17], rtol=1e-9, atol=1e-9)


def test_the_gated_recurrence_equals_its_unrolled_sum_and_carries_its_state():
    m = {"heads": 2, "dim": 5, "vdim": 3, "tau": 4.0}
    g = np.random.default_rng(0)
    width, T, rank = 12, 9, 4
    w = {"q": g.normal(size=(10, width)), "k": g.normal(size=(10, width)), "v": g.normal(size=(6, width)),
         "g": g.normal(size=(6, width)), "o": g.normal(size=(width, 6)), "norm": 1 + 0.1 * g.normal(size=3),
         "a1": g.normal(size=(rank, width)), "a2": g.normal(size=(10, rank)), "a2.b": g.normal(size=10)}
    n = g.normal(size=(T, width))
    out, S = P.mixer_gla(n, m, w, "", 1e-5, return_state=True)
    # the state by its closed form: S_T = sum_t (prod over s > t of alpha_s) * k_t v_t^T
    alpha = P.gla_decay(n, m, w, "")
    k = (n @ w["k"].T).reshape(T, 2, 5)
    v = (n @ w["v"].T).reshape(T, 2, 3)
    for h in range(2):
        want = sum(np.prod(alpha[t + 1:, h], axis=0)[:, None] * np.outer(k[t, h], v[t, h]) for t in range(T))
        assert np.allclose(S[h], want, rtol=1e-10, atol=1e-12)
    # two portions from a carried state are the whole
    a, Sa = P.mixer_gla(n[:4], m, w, "", 1e-5, return_state=True)
    b = P.mixer_gla(n[4:], m, w, "", 1e-5, state=Sa)
    assert np.allclose(np.concatenate([a, b]), out, rtol=1e-10, atol=1e-12)
    # a decay is sigmoid(z) to the power 1 / tau
    z = (n @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    assert np.allclose(alpha.reshape(T, -1) ** 4.0, 1 / (1 + np.exp(-z)), rtol=1e-10)


def test_streams_with_an_identity_mixing_are_one_residual():
    cfg = copy.deepcopy(C.N1)
    W = w64("n1")
    S = cfg["streams"]
    for key in list(W):
        if ".hc" in key:
            last = key.rsplit(".", 1)[-1]
            W[key] = np.eye(S) if last == "mix" else (np.full(S, 1.0 / S) if last == "in" else np.ones(S))
    toks = C.tokens("n1", 21, seed=5)
    many = P.forward(cfg, W, toks, return_layers=True)[1]
    del cfg["streams"]
    one = P.forward(cfg, {k: v for k, v in W.items() if ".hc" not in k}, toks, return_layers=True)[1]
    # every stream is then the plain residual, and their sum is S times it
    assert np.allclose(many, S * one, rtol=1e-9, atol=1e-9)


def test_streams_are_rewritten_all_at_once_from_the_old_ones():
    x = np.arange(12, dtype=np.float64).reshape(2, 3, 2)
    y = np.ones((3, 2))
    mix = np.array([[0.0, 1.0], [1.0, 0.0]])          # [from, to]: the streams change places
    new = P.hyper_write(x, y, mix, np.array([10.0, 0.0]))
    assert np.array_equal(new[0], x[1] + 10.0) and np.array_equal(new[1], x[0])
    assert np.array_equal(P.hyper_read(x, np.array([1.0, -1.0])), x[0] - x[1])


def test_a_sink_only_takes_weight_away_and_values_are_mixed_with_the_first_layers():
    cfg, W = C.N1, w64("n1")
    m = cfg["layers"][2]["mixer"]
    n = np.random.default_rng(1).normal(size=(7, cfg["width"]))
    W2 = dict(W)
    W2["l2.mix.sink"] = np.full(3, -1e9)
    with_sink = P.mixer_latent_attention(n, m, W, "l2.mix.", 1e-4)
    without = P.mixer_latent_attention(n, m, W2, "l2.mix.", 1e-4)
    assert not np.allclose(with_sink, without, rtol=1e-3)
    # at the first position the only key has weight 1 / (1 + exp(sink - score)) instead of 1
    W3 = dict(W)
    W3["l2.mix.sink"] = np.full(3, 1e9)
    assert np.allclose(P.mixer_latent_attention(n, m, W3, "l2.mix.", 1e-4) , 0.0, atol=1e-12)
    # a blend weight of one makes a later layer attend over the first layer's values alone
    a = cfg["layers"][3]["mixer"]
    W4 = dict(W)
    W4["l3.mix.vmix"] = np.array(1.0)
    first = np.random.default_rng(2).normal(size=(7, a["kv_heads"], a["vdim"]))
    got = P.mixer_attention(n, a, W4, "l3.mix.", first)
    W5 = dict(W4)
    W5["l3.mix.v"] = np.zeros_like(W["l3.mix.v"])
    W5["l3.mix.v.b"] = np.zeros_like(W["l3.mix.v.b"])
    assert np.allclose(got, P.mixer_attention(n, a, W5, "l3.mix.", first), rtol=1e-12, atol=1e-12)


def test_the_chosen_experts_keep_their_scores_as_weights():
    cfg, W = C.N1, w64("n1")
    mlp = cfg["layers"][1]["mlp"]
    n = np.random.default_rng(3).normal(size=(6, cfg["width"]))
    out, choice = P.routed_experts(n, mlp, W, "l1.mlp.", return_choice=True)
    s = P.softmax(n @ W["l1.mlp.router"].T)
    for t in range(6):
        assert set(choice[t]) == set(np.argsort(-s[t])[:2])
        want = sum(s[t, e] * P.dense_gated(n[t:t + 1], W, f"l1.mlp.e{e}.")[0] for e in choice[t])
        assert np.allclose(out[t], want, rtol=1e-12) and s[t, choice[t]].sum() < 1.0


def test_models_drawn_at_random_are_read():
    from tandemllm_b200.config import NiralixConfig
    from tandemllm_b200.parts.model import DecoderModel
    for seed in range(12):
        cfg, rank = C.random_config(seed)
        spec = NiralixConfig.from_dict(cfg).to_spec()
        model = DecoderModel(spec)
        shapes = C.tensor_shapes(cfg, rank)
        for layer in model.layers:
            for part in layer.parts:
                if hasattr(part, "shapes_from"):
                    part.shapes_from(lambda n: shapes.get(n))
        got = {s.name: tuple(s.shape) for s in model.weight_specs(None)}
        assert got == {k: v for k, v in shapes.items() if k not in spec.ignored_names}, seed
        W = {k: v.double().numpy() for k, v in C.random_weights(cfg, rank, seed).items()}
        assert np.isfinite(P.forward(cfg, W, list(range(9)))).all()
