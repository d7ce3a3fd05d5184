"""Tenusun without a GPU: the configuration reader and its plan, what the cache keeps for the windows of latent layers,
and the plain implementation's mechanisms on cases worked out by hand."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_tenusun as plain
from tenusun_models import CONFIGS, make_weights, tensor_shapes


def test_configuration_round_trip_and_plan():
    from pico_engine.config import (ConfigError, GatedAttentionSpec, GatedMLPSpec, LatentAttentionSpec, LayerNormSpec, MixtureSpec,
                                    RotaryHalvesSpec, config_from_dict)
    for name, d in CONFIGS.items():
        cfg = config_from_dict(copy.deepcopy(d))
        assert cfg.to_dict() == d, name
        plan = cfg.plan()
        assert plan.embedding_scale == d["embedding"]["scale"] and plan.head is None and type(plan.final_norm) is LayerNormSpec
        assert len(plan.layers) == len(plan.schedule) == len(d["layers"])
        blending = [i for i, l in enumerate(d["layers"]) if l["mixer"].get("v_mix")]
        for i, (l, spec) in enumerate(zip(d["layers"], plan.layers)):
            m = l["mixer"]
            assert spec.arrangement == "sandwich" and type(spec.mixer_norm) is type(spec.mixer_out_norm) is LayerNormSpec
            assert (spec.mixer_norm.weight, spec.mixer_out_norm.weight, spec.mixer_out_norm.bias) == (f"l{i}.norm1", f"l{i}.norm1b", f"l{i}.norm1b.b")
            assert (spec.feed_forward is None) == (l["mlp"] is None) == (spec.feed_forward_out_norm is None)
            assert type(spec.mixer.position) is RotaryHalvesSpec and spec.mixer.position.dims == m["rot"]["dims"]
            if l["type"] == "latent_attention":
                assert type(spec.mixer) is LatentAttentionSpec and spec.mixer.gate is None and spec.mixer.q_rank == m["q_rank"]
                assert spec.mixer.window == (m.get("mask") or {}).get("size") and spec.mixer.position.stretch is None
            else:
                assert type(spec.mixer) is GatedAttentionSpec and spec.mixer.fixed_sink == 0.0 and spec.mixer.window is None
                sc = m["rot"].get("scaling")
                assert spec.mixer.position.stretch == (None if sc is None else (sc["factor"], sc["original"], sc["fast"], sc["slow"]))
                role = None if i not in blending else ("source" if i == blending[0] else "reader")
                assert spec.mixer.value_blend_role == role and (spec.mixer.value_blend == "vmix") == (role == "reader")
            if l["mlp"] is not None and l["mlp"]["kind"] == "dense":
                assert type(spec.feed_forward) is GatedMLPSpec and spec.feed_forward.limit == l["mlp"]["limit"] and spec.feed_forward.alpha == 1.702
            elif l["mlp"] is not None:
                f, r = spec.feed_forward, l["mlp"]["router"]
                assert type(f) is MixtureSpec and f.scores == "sigmoid" and f.correction_name == "correction" and f.group_best == 2
                assert (f.n_groups, f.keep_groups) == ((r["groups"]["count"], r["groups"]["keep"]) if "groups" in r else (1, 1))

    def broken(name, change, match):
        bad = copy.deepcopy(CONFIGS[name])
        change(bad)
        with pytest.raises(ConfigError, match=match):
            config_from_dict(bad)
    broken("T1", lambda c: c["layers"][1].update(type="mamba"), "type")
    broken("T1", lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank")
    broken("T1", lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "rot.dims")
    broken("T1", lambda c: c["layers"][1]["mixer"]["rot"].update(scaling={"factor": 2.0, "original": 8, "fast": 1.0, "slow": 1.0}), "not stretched")
    broken("T1", lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "does not divide")
    broken("T1", lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=1), "do not fit")
    broken("T1", lambda c: c["layers"][2]["mixer"].update(vdim=24), "mix values")
    broken("T1", lambda c: c["layers"][2]["mlp"].pop("limit"), "limit")
    broken("T2", lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "evenly")
    broken("T2", lambda c: c["layers"][2]["mixer"].update(v_mix="yes"), "v_mix")


def test_the_model_names_the_tensors_of_the_design():
    from pico_engine.config import config_from_dict
    from pico_engine.config.registry import architecture
    from pico_engine.weights.loader import check
    for name, d in CONFIGS.items():
        model = architecture("Tenusun").build_model(config_from_dict(d), torch.bfloat16, "meta")
        stored = tensor_shapes(d)
        expected = {k: tuple(v.shape) for k, v in model.expected_tensors().items()}
        unread = set(stored) - set(expected)
        first = next((i for i, l in enumerate(d["layers"]) if l["mixer"].get("v_mix")), None)
        assert unread == ({f"l{first}.mix.vmix"} if first is not None else set()), name      # the first blending layer's number is stored and unused
        assert expected == {k: v for k, v in stored.items() if k not in unread}, name
        check(model.expected_tensors(), stored, model.plan.ignorable_tensors)                    # and loads without a warning
        needs = model.cache_needs()
        assert len(needs) == len(d["layers"])
        for l, need in zip(d["layers"], needs):
            m = l["mixer"]
            if l["type"] == "latent_attention":
                assert (need.kv.n_kv_heads, need.kv.head_dim, need.kv.value_shape[0]) == (1, m["kv_rank"] + m["rot_dim"], 0)
                assert need.kv.window == (m.get("mask") or {}).get("size")
            else:
                assert (need.kv.n_kv_heads, need.kv.head_dim, need.kv.value_shape, need.kv.window) == (m["kv_heads"], m["dim"], (m["kv_heads"], m["vdim"]), None)


def test_latent_pages_leave_with_the_window_and_the_others_stay():
    from pico_engine.cache import Cache
    from pico_engine.config import config_from_dict
    from pico_engine.config.registry import architecture
    model = architecture("Tenusun").build_model(config_from_dict(CONFIGS["T4"]), torch.float32, "meta")
    cache = Cache(model.cache_needs(), 64 * 12, 2, torch.float32, "cpu", allocate=False)
    windows = {g.need.window: g for g in cache.groups}
    assert set(windows) == {130, 45, None}
    s = cache.open()
    cache.reserve(s, 500); cache.advance(s, 500)
    # the next query stands at 500: a window of 130 begins at 371 (page 5), one of 45 at 456 (page 7)
    assert [p >= 0 for p in windows[130].table[s]] == [False] * 5 + [True] * 3
    assert [p >= 0 for p in windows[45].table[s]] == [False] * 7 + [True]
    assert all(p >= 0 for p in windows[None].table[s])
    cache.check()
    cache.close(s)
    assert all(g.pages.free_count == g.pages.n for g in cache.groups)


# ------------------------------------------------------------------ the plain implementation on cases worked out by hand

def test_plain_norms_masks_and_the_extra_place():
    x = torch.tensor([[1.0, 3.0]], dtype=torch.float64)
    got = plain.layer_norm(x, torch.tensor([2.0, 2.0]).double(), torch.tensor([0.5, -0.5]).double(), 0.0)
    assert torch.allclose(got, torch.tensor([[-1.5, 1.5]], dtype=torch.float64))
    assert plain.causal_mask(4, 2).tolist() == [[True, False, False, False], [True, True, False, False],
                                                 [False, True, True, False], [False, False, True, True]]
    assert plain.causal_mask(3).tolist() == torch.tril(torch.ones(3, 3)).bool().tolist()
    s = torch.tensor([[math.log(3.0), math.log(4.0)]], dtype=torch.float64)
    seen = torch.tensor([[True, True]])
    assert torch.allclose(plain.softmax_rows(s, seen, extra_one=True), torch.tensor([[3 / 8, 4 / 8]], dtype=torch.float64))
    assert torch.allclose(plain.softmax_rows(s, seen), torch.tensor([[3 / 7, 4 / 7]], dtype=torch.float64))
    low = torch.tensor([[-1000.0, -1001.0]], dtype=torch.float64)                      # very low scores: the extra place takes everything
    assert float(plain.softmax_rows(low, seen, extra_one=True).sum()) < 1e-300


def test_plain_rotation_by_hand():
    u = torch.tensor([[1.0, 5.0, 0.0, 6.0, 7.0]] * 2, dtype=torch.float64)                # four rotated entries: pairs (0, 2) and (1, 3)
    f = plain.plain_frequencies(4, 100.0)
    assert f == [1.0, 0.1]
    r = plain.rotate_half(u, 4, f, magnitude=2.0)
    assert torch.allclose(r[0], torch.tensor([2.0, 10.0, 0.0, 12.0, 7.0], dtype=torch.float64))
    c1, s1, c2, s2 = math.cos(1.0), math.sin(1.0), math.cos(0.1), math.sin(0.1)
    want = [2 * c1, 2 * (5 * c2 - 6 * s2), 2 * s1, 2 * (6 * c2 + 5 * s2), 7.0]
    assert torch.allclose(r[1], torch.tensor(want, dtype=torch.float64))
    # a ramp from entry 1 to entry 3 of four: entry 0 keeps its frequency, entry 3 has it divided by the factor
    dims, base = 8, 10.0
    original = 2 * math.pi * 10.0 ** (2 * 1 / dims)                                        # where(1.0) = 1 and where(t) falls as t grows
    sc = {"factor": 4.0, "original": original, "fast": 0.99, "slow": 1.01 * 10.0 ** (-2 * 2 / dims)}      # where: 1.02 and 2.98
    freqs, mag = plain.stretched_frequencies(dims, base, sc)
    plainf = plain.plain_frequencies(dims, base)
    assert freqs[0] == plainf[0] and abs(freqs[3] - plainf[3] / 4.0) < 1e-15 and plainf[2] / 4.0 < freqs[2] < plainf[2]
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-15


def test_plain_routing_by_hand():
    """Four experts in two groups, one group stays.  Scores (0.5, 0.5, 0.9, 0.1) with corrections (0, 0, -2, -2): the choice scores
    of the second group are negative, the first group wins (1.0 against -2.9); the weights are the scores without correction."""
    big = 50.0
    w = {"p.router": torch.tensor([[0.0], [0.0], [math.log(9.0)], [-math.log(9.0)]], dtype=torch.float64),
         "p.correction": torch.tensor([0.0, 0.0, -2.0, -2.0], dtype=torch.float64)}
    mlp = {"router": {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}}
    got = plain.route(torch.ones(1, 1, dtype=torch.float64), mlp, w, "p.")[0]
    assert [e for e, _ in got] == [0, 1] and all(abs(float(s) - 0.5) < 1e-12 for _, s in got)
    # corrections that lift the second group: it wins, and its weights are still the plain scores 0.9 and 0.1
    w["p.correction"] = torch.tensor([-1.0, -1.0, 0.0, 0.0], dtype=torch.float64)
    got = plain.route(torch.ones(1, 1, dtype=torch.float64), mlp, w, "p.")[0]
    assert [e for e, _ in got] == [2, 3] and abs(float(got[0][1]) - 0.9) < 1e-12 and abs(float(got[1][1]) - 0.1) < 1e-12
    # every choice score negative: the experts outside the group that stays must not come back as zeros
    w["p.correction"] = torch.tensor([-3.0, -3.0, -5.0, -5.0], dtype=torch.float64)
    assert [e for e, _ in plain.route(torch.ones(1, 1, dtype=torch.float64), mlp, w, "p.")[0]] == [0, 1]
    # without groups the two largest choice scores of all
    w["p.correction"] = torch.tensor([0.0, -1.0, 0.0, big], dtype=torch.float64)
    got = plain.route(torch.ones(1, 1, dtype=torch.float64), {"router": {"experts": 4, "top": 2}}, w, "p.")[0]
    assert [e for e, _ in got] == [3, 2]


def test_plain_dense_feed_forward_by_hand():
    w = {"p.gate": torch.tensor([[1.0], [1.0]]).double(), "p.up": torch.tensor([[1.0], [-1.0]]).double(), "p.down": torch.tensor([[1.0, 10.0]]).double()}
    y = plain.dense_ff(torch.tensor([[3.0]], dtype=torch.float64), {"limit": 2.0}, w, "p.")
    g = 2.0 / (1 + math.exp(-1.702 * 2.0))
    assert abs(float(y) - (g * 3.0 + 10 * g * -1.0)) < 1e-12                                # up clamps to 2 and -2, then + 1


def test_plain_values_blend_with_the_first_blending_layer_only():
    cfg = CONFIGS["T2"]
    w = {n: t.double() for n, t in make_weights(cfg, 5).items()}
    toks = [3, 9, 27, 81, 5]
    with torch.no_grad():
        a = plain.logits(cfg, w, toks)
        w2 = dict(w); w2["l2.mix.vmix"] = w["l2.mix.vmix"] + 0.5                              # the first blending layer's number is unused
        b = plain.logits(cfg, w2, toks)
        w3 = dict(w); w3["l3.mix.vmix"] = w["l3.mix.vmix"] + 0.5
        c = plain.logits(cfg, w3, toks)
    assert torch.equal(a, b) and not torch.allclose(a, c)


def test_plain_prefix_does_not_depend_on_what_follows():
    """Causality of the whole plain model: the logits of a prefix equal the first rows of the longer run."""
    cfg = CONFIGS["T1"]
    w = {n: t.double() for n, t in make_weights(cfg, 3).items()}
    toks = torch.randint(0, cfg["vocab"], (60,), generator=torch.Generator().manual_seed(1)).tolist()
    with torch.no_grad():
        a, b = plain.logits(cfg, w, toks), plain.logits(cfg, w, toks[:47])
    assert torch.allclose(a[:47], b, atol=1e-10)
