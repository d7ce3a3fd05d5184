"""Pupidra without a GPU: the configuration reader and its plan, what the cache keeps for a window with kept first tokens,
and the plain implementation's mechanisms on cases worked out by hand."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_pupidra as plain
from pupidra_models import CONFIGS, make_weights, tensor_shapes


def test_configuration_round_trip_and_plan():
    from pico_engine.config import ConfigError, GatedAttentionSpec, LatentAttentionSpec, MixtureSpec, StateSpaceSpec, config_from_dict
    for name, d in CONFIGS.items():
        cfg = config_from_dict(copy.deepcopy(d))
        assert cfg.to_dict() == d, name
        plan = cfg.plan()
        assert len(plan.layers) == len(plan.schedule) == len(d["layers"])
        for i, (l, spec, entry) in enumerate(zip(d["layers"], plan.layers, plan.schedule)):
            kind = {"attention": GatedAttentionSpec, "latent_attention": LatentAttentionSpec, "mamba2": StateSpaceSpec}[l["type"]]
            assert type(spec.mixer) is kind and spec.arrangement == "post_norm"
            assert spec.mixer_scale == f"l{i}.ls1" and (spec.feed_forward is None) == (l["mlp"] is None)
            assert entry.cache_of == l["mixer"].get("kv_from")
            if l["mlp"] is not None:
                assert type(spec.feed_forward) is MixtureSpec and not spec.feed_forward.gated and spec.feed_forward.scores == "softmax_all"
                assert spec.feed_forward.route_scale == l["mlp"]["router"]["scale"]
    bad = copy.deepcopy(CONFIGS["P1"]); bad["layers"][3]["mixer"]["kv_from"] = 3
    with pytest.raises(ConfigError, match="earlier"):
        config_from_dict(bad)
    bad = copy.deepcopy(CONFIGS["P1"]); bad["layers"][3]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError, match="attention layer"):
        config_from_dict(bad)
    bad = copy.deepcopy(CONFIGS["P1"]); bad["layers"][3]["mixer"]["dim"] = 16
    with pytest.raises(ConfigError, match="must be equal"):
        config_from_dict(bad)
    bad = copy.deepcopy(CONFIGS["P1"]); bad["layers"][1]["type"] = "mamba3"
    with pytest.raises(ConfigError, match="type"):
        config_from_dict(bad)
    bad = copy.deepcopy(CONFIGS["P2"]); del bad["layers"][0]["mixer"]["state"]
    with pytest.raises(ConfigError, match="state"):
        config_from_dict(bad)


def test_the_cache_spans_every_reader_of_a_layers_keys():
    """Layer 0 of P1 looks 40 back and keeps 5, its reader looks 70 back and keeps none: the cache keeps 70 and 5.  In P4 the
    readers' windows are narrower than the owner's."""
    from pico_engine.config import config_from_dict
    plan = config_from_dict(CONFIGS["P1"]).plan()
    assert plan.layers[0].mixer.cache_span == (70, 5) and plan.layers[0].mixer.window == 40 and plan.layers[0].mixer.keep_first == 5
    assert plan.layers[3].mixer.window == 70 and plan.layers[3].mixer.keep_first == 0 and not plan.layers[3].mixer.own_kv
    plan = config_from_dict(CONFIGS["P4"]).plan()
    assert plan.layers[1].mixer.cache_span == (130, 70)
    plan = config_from_dict(CONFIGS["P2"]).plan()
    assert plan.layers[1].mixer.cache_span == (None, 0)


def test_the_model_names_the_tensors_of_the_design():
    from pico_engine.config import config_from_dict
    from pico_engine.config.registry import architecture
    for name, d in CONFIGS.items():
        model = architecture("Pupidra").build_model(config_from_dict(d), torch.bfloat16, "meta")
        assert {k: tuple(v.shape) for k, v in model.expected_tensors().items()} == tensor_shapes(d), name
        needs = model.cache_needs()
        assert len(needs) == len(d["layers"]) + (1 if d.get("embedding") else 0)
        for l, need in zip(d["layers"], needs):
            assert (need is None) == (l["mixer"].get("kv_from") is not None)


def test_kept_first_pages_stay_while_the_window_moves_on():
    from pico_engine.cache import Cache, CacheNeeds, KVNeed
    cache = Cache([CacheNeeds(kv=KVNeed(1, 8, window=70, keep_first=65)), CacheNeeds(kv=KVNeed(1, 8, window=70))], 64 * 12, 2,
                  torch.float32, "cpu", allocate=False)
    s = cache.open()
    cache.reserve(s, 500); cache.advance(s, 500)
    kept, plain_window = (cache.groups[i].table[s] for i in (0, 1))
    # the next query stands at 500 and sees keys from 431 on: page 6 (384..447) is the first that is needed
    assert [p >= 0 for p in plain_window] == [False] * 6 + [True] * 2
    assert [p >= 0 for p in kept] == [True] * 2 + [False] * 4 + [True] * 2          # 65 kept tokens lie on two pages
    cache.check()
    cache.close(s)
    assert all(g.pages.free_count == g.pages.n for g in cache.groups)


# ------------------------------------------------------------------ the plain implementation on cases worked out by hand

def test_plain_mask_slopes_and_pairs():
    seen = plain.window_keep_mask(6, 2, 1)
    assert seen.tolist() == [[True, False, False, False, False, False], [True, True, False, False, False, False],
                             [True, True, True, False, False, False], [True, False, True, True, False, False],
                             [True, False, False, True, True, False], [True, False, False, False, True, True]]
    assert plain.window_keep_mask(4, None, 0).tolist() == torch.tril(torch.ones(4, 4)).bool().tolist()
    assert plain.distance_slopes(4) == [0.25, 0.0625, 0.015625, 0.00390625]
    assert plain.distance_slopes(1) == [2.0 ** -8]
    w = {"embed": torch.arange(12.0).view(6, 2), "bigram": 100 * torch.arange(8.0).view(4, 2)}
    got = plain.embed([5, 1, 1], w, {"buckets": 3, "mul_prev": 2, "mul_cur": 5})
    rows = [3, (5 * 2 + 1 * 5) % 3, (1 * 2 + 1 * 5) % 3]
    assert torch.equal(got, torch.stack([w["embed"][t] + w["bigram"][r] for t, r in zip([5, 1, 1], rows)]))


def test_plain_attention_by_hand():
    """Two keys, one head: the weights are the softmax of (q.k * scale - slope * distance)."""
    q = torch.tensor([[[1.0, 0.0]], [[2.0, 0.0]]], dtype=torch.float64)
    k = torch.tensor([[[1.0, 0.0]], [[3.0, 0.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[5.0]]], dtype=torch.float64)
    o = plain.biased_attention(q, k, v, 0.5, None, 0)
    s0, s1 = 2.0 * 1.0 * 0.5 - 2.0 ** -8, 2.0 * 3.0 * 0.5
    p0 = math.exp(s0) / (math.exp(s0) + math.exp(s1))
    assert abs(float(o[0, 0, 0]) - 1.0) < 1e-12 and abs(float(o[1, 0, 0]) - (p0 * 1.0 + (1 - p0) * 5.0)) < 1e-12


def test_plain_rotation_convolution_and_recurrence_by_hand():
    u = torch.tensor([[1.0, 0.0, 7.0], [1.0, 0.0, 7.0]], dtype=torch.float64)
    r = plain.rotate_pairs(u, 2, 10.0)
    assert torch.allclose(r[0], u[0]) and torch.allclose(r[1], torch.tensor([math.cos(1.0), math.sin(1.0), 7.0], dtype=torch.float64))
    y = plain.causal_conv(torch.tensor([[1.0], [2.0], [3.0]]), torch.tensor([[10.0, 1.0]]), torch.tensor([0.5]))
    assert y.view(-1).tolist() == [1.5, 12.5, 23.5]
    # one head, one state row, one column: S_t = exp(A dt) S + dt B x; y = S C + D x
    xs, B, C = (torch.tensor(t, dtype=torch.float64) for t in ([[[2.0]], [[3.0]]], [[[1.0]], [[0.5]]], [[[1.0]], [[4.0]]]))
    dt, A, D = (torch.tensor(t, dtype=torch.float64) for t in ([[0.5], [2.0]], [-1.0], [10.0]))
    y = plain.ssm_recurrence(xs, B, C, dt, A, D).view(-1).tolist()
    S0 = 0.5 * 1.0 * 2.0
    S1 = math.exp(-2.0) * S0 + 2.0 * 0.5 * 3.0
    assert abs(y[0] - (S0 * 1.0 + 20.0)) < 1e-12 and abs(y[1] - (S1 * 4.0 + 30.0)) < 1e-12


def test_plain_mixture_weights_are_not_renormalised():
    g = torch.Generator().manual_seed(0)
    W, F, E = 6, 4, 3
    w = {"p.router": torch.tensor([[1.0] + [0.0] * 5, [0.0, 1.0] + [0.0] * 4, [0.0] * 6], dtype=torch.float64)}
    for e in range(E):
        w[f"p.e{e}.up"], w[f"p.e{e}.down"] = torch.randn(F, W, generator=g).double(), torch.randn(W, F, generator=g).double()
    h = torch.tensor([[2.0, 1.0, 0.3, -0.2, 0.1, 0.5]], dtype=torch.float64)
    got = plain.mixture(h, {"router": {"experts": 3, "top": 2, "scale": 1.5}}, w, "p.")
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=torch.float64), 0)
    want = sum(1.5 * s[e] * (w[f"p.e{e}.down"] @ torch.clamp(w[f"p.e{e}.up"] @ h[0], min=0) ** 2) for e in (0, 1))
    assert torch.allclose(got[0], want)


def test_plain_prefix_does_not_depend_on_what_follows():
    """Causality of the whole plain model: the logits of a prefix equal the first rows of the longer run."""
    cfg = CONFIGS["P1"]
    w = {n: t.double() for n, t in make_weights(cfg, 3).items()}
    toks = torch.randint(0, cfg["vocab"], (60,), generator=torch.Generator().manual_seed(1)).tolist()
    with torch.no_grad():
        a, b = plain.logits(toks, cfg, w), plain.logits(toks[:47], cfg, w)
    assert torch.allclose(a[:47], b, atol=1e-10)
