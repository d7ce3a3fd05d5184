"""Tenusun on the GPU against the plain implementation: each mechanism's kernel alone on inputs that show a fault, and the
whole model through the library's step function, cache, scheduler and entry points, in both dtypes, for every way of
cutting requests into steps."""
from __future__ import annotations

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_tenusun as plain
import replay
from conftest import write_model
from tenusun_models import CONFIGS, make_weights, plain_logits, requests_for

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CASES = [(n, d) for n in sorted(CONFIGS) for d in ("float32", "bfloat16")]
LENGTHS = {"T1": [1, 2, 3, 47, 70, 131, 64, 5], "T2": [65, 1, 150, 9, 33, 2], "T3": [3, 129, 31, 64, 1, 70], "T4": [4, 1, 290, 17, 66, 135]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{(config, dtype): (engine, cfg, weights, folder)}."""
    from pico_engine.engine.engine import Engine
    root = tmp_path_factory.mktemp("tenusun")
    out = {}
    for k, (name, cfg) in enumerate(sorted(CONFIGS.items())):
        for dtype in DTYPES:                              # bfloat16 runs get routers that rounding cannot turn (tenusun_models.make_weights)
            weights = make_weights(cfg, 80 + k, steady_routing=dtype == "bfloat16")
            folder = write_model(root / f"{name}-{dtype}", cfg, weights)
            out[(name, dtype)] = (Engine(folder, dtype=dtype), cfg, weights, folder)
    return out


def compare(got, cfg, w, reqs, dtype, what, only_got=False):
    """Against the plain logits.  float32: every place, by the rule of the engine tests.  bfloat16 (models whose routers make no
    close calls; should the plain run still record one, that place and the two behind it are left out): none may be off by more
    than a tenth of the logits' size, and at most one in a hundred by more than the engine tests' 4e-2 (a sublayer's output is
    normed before it is added, so a small output carries its rounding at full size into the stream)."""
    close = set()
    want = plain_logits(cfg, w, reqs, close)
    if only_got:
        want = {k: v for k, v in want.items() if k in got}
    if dtype != "bfloat16":
        return replay.compare(got, want, dtype, what)
    assert set(got) == set(want), (what, sorted(set(want) - set(got))[:5], sorted(set(got) - set(want))[:5])
    close |= {(r, p + d) for r, p in close for d in (1, 2)}
    assert len(close & set(want)) < 0.1 * len(want)
    over = []
    for key in sorted(set(want) - close, key=lambda k: (str(k[0]), k[1])):
        scale = max(1.0, float(np.abs(want[key]).max()))
        err = float(np.abs(np.asarray(got[key], dtype=np.float64) - want[key]).max()) / scale
        assert err <= 1e-1, f"{what}: request {key[0]!r} position {key[1]}: max error {err:.3e} of the logits' size {scale:.3f}"
        if err > 4e-2:
            over.append((key, round(err, 4)))
    assert len(over) <= max(1, len(set(want) - close) // 100), (what, over[:8])


def check(models, name, dtype, steps, reqs, what):
    eng, cfg, w, _ = models[(name, dtype)]
    compare(replay.run_in_process(eng, steps), cfg, w, reqs, dtype, what)


# ------------------------------------------------------------------ the whole model, every way of cutting

@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_and_first_tokens(models, name, dtype):
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 1)
    check(models, name, dtype, replay.whole(reqs), reqs, "whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(models, name, dtype):
    """Every request again with its last tokens one at a time (the shortest ones entirely), 100 for the long ones: the
    windows pass over decoded tokens, pages behind them are given back, and a decoded token's values blend with the first
    blending layer's values of the same step."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 2)
    check(models, name, dtype, replay.tail(reqs, 100), reqs, "tail")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompts_in_portions(models, name, dtype):
    """Portions of unequal sizes, then portions of two, three and five tokens and single tokens in turn: every portion starts
    inside its sequence from the cache pages the portion before it left."""
    cfg = CONFIGS[name]
    reqs = requests_for(cfg, LENGTHS[name], 3)
    check(models, name, dtype, replay.pieces(reqs), reqs, "pieces")
    small = requests_for(cfg, [23, 11, 70], 4)
    plan = {}
    for i, (r, toks) in enumerate(small.items()):
        cuts, left, k = [], len(toks), i
        while left:
            c = min(left, (2, 3, 1, 2, 5)[k % 5])
            cuts.append(c); left -= c; k += 1
        plan[r] = (i, cuts)
    check(models, name, dtype, replay.scheduled(small, plan), small, "small portions")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("batch_size,fraction", [(3, 0.5), (8, 0.9)])
def test_unequal_batches_reuse_slots_and_pages(models, name, dtype, batch_size, fraction):
    """Batches one after another in a cache sized for one: slots and pages are used again, and a request's logits do not
    depend on its neighbours (compared with the plain run of each alone)."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name] + LENGTHS[name][::-1], 5)
    check(models, name, dtype, replay.batched(reqs, batch_size, fraction), reqs, "batched")


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_steps(models, name, dtype):
    """Steps that carry a fresh prompt, a later portion of another and single tokens side by side."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 6)
    check(models, name, dtype, replay.mixed(reqs), reqs, "mixed")


@pytest.mark.parametrize("name,dtype", [("T1", "float32"), ("T1", "bfloat16"), ("T4", "bfloat16"), ("T3", "float32")])
def test_batches_of_more_rows_than_the_decode_products_fuse(models, name, dtype):
    """Twenty short requests start together and are decoded together: steps of 17 and more rows take the products that prompts take."""
    reqs = requests_for(CONFIGS[name], [3 + (7 * i) % 23 for i in range(20)], 13)
    check(models, name, dtype, replay.batched(reqs, 20, 0.5), reqs, "twenty rows")


@pytest.mark.parametrize("name", ["T1", "T3", "T4"])
def test_long_decoding(models, name):
    """300 tokens one by one from a one-token prompt: windows and pages given back over many steps, keys far back without a window."""
    reqs = requests_for(CONFIGS[name], [301], 12)
    check(models, name, "float32", replay.tail(reqs, 300), reqs, "long decoding")


def test_a_freed_slot_starts_from_nothing(models):
    eng, cfg, w, _ = models[("T1", "float32")]
    reqs = requests_for(cfg, [40, 6], 8)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"], "want": [39]}], "end": ["r0"]},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"], "want": list(range(6))}], "end": ["r1"]}]
    got = replay.run_in_process(eng, steps, max_tokens=64)
    compare(got, cfg, w, reqs, "float32", "slot reuse", only_got=True)


@pytest.mark.parametrize("name", ["T1", "T4"])
@pytest.mark.parametrize("use_graph", [False, True])
def test_greedy_generation_through_the_entry_point(models, name, use_graph):
    """Engine.generate (scheduler, batches, captured decode steps) against the plain greedy loop."""
    eng, cfg, w, _ = models[(name, "float32")]
    w64 = {n: t.double() for n, t in w.items()}
    prompts = list(requests_for(cfg, [5, 1, 19, 66], 9).values())
    news = [12, 20, 7, 9]
    outs = eng.generate(prompts, max_tokens=news, temperature=0.0, use_graph=use_graph, stop_token_ids=[])
    for p, o, n in zip(prompts, outs, news):
        with torch.no_grad():
            assert o == plain.greedy(cfg, w64, p, n), (len(p), o)


def test_bfloat16_generation_with_graphs_matches_eager(models):
    eng, cfg, w, _ = models[("T3", "bfloat16")]
    prompts = list(requests_for(cfg, [7, 30, 2], 11).values())
    a = eng.generate(prompts, max_tokens=10, temperature=0.0, use_graph=False, stop_token_ids=[])
    b = eng.generate(prompts, max_tokens=10, temperature=0.0, use_graph=True, stop_token_ids=[])
    assert a == b


def test_trace_replay_program(models, tmp_path):
    eng, cfg, w, folder = models[("T2", "float32")]
    reqs = requests_for(cfg, [40, 3, 77], 10)
    steps = replay.batched(reqs, 3, 0.6)
    got = replay.run_binary(folder, "float32", steps, str(tmp_path / "out"), cfg["vocab"])
    compare(got, cfg, w, reqs, "float32", "bin/trace_run")


def test_command_line_generates(models):
    import json, subprocess, sys
    eng, cfg, w, folder = models[("T1", "float32")]
    out = subprocess.run([sys.executable, "-m", "pico_engine", folder, "--prompt", "5,17,3", "--max-tokens", "6", "--temperature", "0",
                          "--dtype", "float32"], capture_output=True, text=True, cwd=replay.ROOT, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    with torch.no_grad():
        assert json.loads(line)["output"] == plain.greedy(cfg, {n: t.double() for n, t in w.items()}, [5, 17, 3], 6)


def test_the_blending_number_of_a_later_layer_counts_and_the_first_ones_does_not(models, tmp_path):
    """The same model with the first blending layer's stored number changed gives the same logits; with a later layer's changed, others."""
    from pico_engine.engine.engine import Engine
    _, cfg, w, _ = models[("T2", "float32")]
    toks = requests_for(cfg, [20], 3)["r0"]
    rows = {}
    for tag, name in (("same", None), ("first", "l2.mix.vmix"), ("later", "l3.mix.vmix")):
        w2 = dict(w)
        if name:
            w2[name] = w[name] + 0.25
        eng = Engine(write_model(tmp_path / tag, cfg, w2), dtype="float32")
        rows[tag] = replay.run_in_process(eng, replay.whole({"r0": toks}))[("r0", 19)]
    assert np.array_equal(rows["same"], rows["first"]) and np.abs(rows["same"] - rows["later"]).max() > 1e-3


# ------------------------------------------------------------------ attention with one more place in the denominator, alone

def paged(k, dt, first_page=1):
    """k [n, G, D] as cache pages [pages + first_page, G, 64, D] and the page table of one sequence."""
    n, G, D = k.shape
    pages = (n + 63) // 64
    pool = torch.zeros(pages + first_page, G, 64, D, dtype=dt).cuda()
    for p in range(n):
        pool[first_page + p // 64, :, p % 64] = k[p].to(dt).cuda()
    return pool, torch.arange(first_page, pages + first_page, dtype=torch.int32).view(1, -1).cuda()


def run_attention(q, kp, vp, table, dt, spans, window, scale, Dv, sink=None, values_in_keys=False):
    """``kernels.attention_headmix`` for the query positions of ``spans`` (each a step of one sequence); q [n, H, D]."""
    from pico_engine.ops import kernels
    n, H, D = q.shape
    G = kp.shape[1]
    out = torch.zeros(n, H * Dv)
    sk = None if sink is None else torch.full((H,), float(sink), dtype=torch.float32).cuda()
    for a, b in spans:
        ctx = SimpleNamespace(one_token_each=(b - a == 1), scratch={}, lens=[b - a], starts=[a], max_context=b, dtype=dt)
        pos, row = torch.arange(a, b, dtype=torch.int32).cuda(), torch.zeros(b - a, dtype=torch.int32).cuda()
        qq = q[a:b].reshape(b - a, H * D).to(dt).cuda().contiguous()
        o = kernels.attention_headmix(qq, H * D, H, G, D, Dv, kp, vp, table, table.shape[1], pos, row, window, scale, sk, None, ctx,
                                      values_in_keys=values_in_keys)
        out[a:b] = o.float().cpu()
    return out.view(n, H, Dv)


def plain_attention(q, k, v, scale, window, extra_one):
    n, H, _ = q.shape
    G = k.shape[1]
    seen = plain.causal_mask(n, window)
    return torch.stack([plain.softmax_rows((q[:, h] @ k[:, h // (H // G)].T) * scale, seen, extra_one) @ v[:, h // (H // G)]
                        for h in range(H)], dim=1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv", [(6, 2, 32, 16), (3, 1, 24, 12), (8, 1, 64, 64), (4, 4, 16, 24), (6, 3, 128, 32), (2, 1, 128, 128)])
def test_attention_with_one_added_to_the_denominator(dtype, H, G, D, Dv):
    """Random queries, keys and values against the plain function: as one prompt, in portions, and the last 80 tokens one by one.
    The scores are small, so that the added one is a large share of every denominator."""
    dt = DTYPES[dtype]
    n = 230
    g = torch.Generator().manual_seed(H * 100 + D)
    q, k, v = ((torch.randn(n, h, d, generator=g)).to(dt).float() for h, d in ((H, D), (G, D), (G, Dv)))
    scale = 0.5 * D ** -0.5
    want = plain_attention(q.double(), k.double(), v.double(), scale, None, True)
    without = plain_attention(q.double(), k.double(), v.double(), scale, None, False)
    assert (want - without).abs().max() > 0.1                           # the added one shows
    kp, table = paged(k, dt)
    vp, _ = paged(v, dt)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for spans in ([(0, n)], [(0, 3), (3, 70), (70, 72), (72, 200), (200, n)], [(0, 150)] + [(p, p + 1) for p in range(150, n)]):
        got = run_attention(q, kp, vp, table, dt, spans, None, scale, Dv, sink=0.0)
        assert (got.double() - want).abs().max() < tol * max(1.0, float(want.abs().max())), spans[:2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,Dv", [(32, 16), (64, 64), (128, 128)])
def test_very_low_scores_leave_the_added_one_alone(dtype, D, Dv):
    """Every score far below zero: the weights vanish beside the added one and the output is zero, not a mean of the values;
    the first token of a sequence, which sees only itself, included (at the head sizes of every attention kernel)."""
    dt = DTYPES[dtype]
    n, H, G = 70, 2, 1
    q, k, v = torch.zeros(n, H, D), torch.zeros(n, G, D), torch.ones(n, G, Dv) * 5
    q[:, :, 0], k[:, :, 0] = 8.0, -8.0                                  # every score is -64
    kp, table = paged(k, dt)
    vp, _ = paged(v, dt)
    for spans in ([(0, n)], [(0, 1)] + [(p, p + 1) for p in range(1, n)]):
        got = run_attention(q, kp, vp, table, dt, spans, None, 1.0, Dv, sink=0.0)
        assert got.abs().max() < 1e-20
    q[:, :, 0] = -8.0                                                   # every score is +64: the added one vanishes
    got = run_attention(q, kp, vp, table, dt, [(0, n)], None, 1.0, Dv, sink=0.0)
    assert (got - 5.0).abs().max() < 1e-3


@pytest.mark.parametrize("H,G,D", [(4, 2, 64), (2, 1, 128), (3, 1, 64), (16, 2, 128)])
def test_long_prompts_in_bfloat16_at_head_sizes_of_the_tensor_memory_kernel(H, G, D):
    """Prompts of 900 tokens with the added one at the sizes the tcgen05 prompt kernel and the cluster kernel for single tokens take:
    whole, in portions that begin and end off the borders of pages and of the kernel's runs of tokens, and with the last 330 tokens
    one by one (the ranges of keys that several blocks share are merged before the added one joins)."""
    dt, n = torch.bfloat16, 900
    g = torch.Generator().manual_seed(H * 100 + D)
    q, k, v = ((torch.randn(n, h, D, generator=g)).to(dt).float() for h in (H, G, G))
    scale = 0.3 * D ** -0.5
    want = plain_attention(q.double(), k.double(), v.double(), scale, None, True)
    assert (want - plain_attention(q.double(), k.double(), v.double(), scale, None, False)).abs().max() > 0.05
    kp, table = paged(k, dt)
    vp, _ = paged(v, dt)
    for spans in ([(0, n)], [(0, 130), (130, 133), (133, 517), (517, n)], [(0, 570)] + [(p, p + 1) for p in range(570, n)]):
        got = run_attention(q, kp, vp, table, dt, spans, None, scale, D, sink=0.0)
        assert (got.double() - want).abs().max() < 2e-2 * max(1.0, float(want.abs().max())), spans[:2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 63, 64, 65, 447])
def test_a_key_from_far_back(dtype, far):
    """Without a window one key that matches the last query must come through from any distance, beside the added one, for
    grouped heads with unequal key and value sizes and in the kernel's form for latent rows; in a prompt and as a single token."""
    dt = DTYPES[dtype]
    H, n = 4, 700
    for G, D, Dv, in_keys in ((2, 32, 24, False), (1, 48, 40, True)):
        g = torch.Generator().manual_seed(far)
        q, k, v = 0.01 * torch.randn(n, H, D, generator=g), 0.01 * torch.randn(n, G, D, generator=g), torch.randn(n, G, Dv, generator=g)
        k[far] = 0; k[far, :, D - 1] = 40.0
        q[-1] = 0; q[-1, :, D - 1] = 40.0
        if in_keys:
            v = k[:, :, :Dv].clone()
            v[far] = k[far, :, :Dv] = 8.0
            k[far, :, D - 1] = 40.0
        else:
            v[far] = 8.0
        kp, table = paged(k, dt)
        vp = None if in_keys else paged(v, dt)[0]
        for spans in ([(0, n)], [(n - 1, n)]):
            got = run_attention(q, kp, vp, table, dt, spans, None, 1.0, Dv, None if in_keys else 0.0, in_keys)
            assert (got[-1] - 8.0).abs().max() < 0.1, (far, in_keys, got[-1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,rank,R,window", [(3, 48, 16, 33), (5, 20, 6, 2), (4, 64, 32, 130), (2, 9, 4, 64), (2, 9, 4, 1), (8, 80, 16, 44)])
def test_window_edges_over_latent_rows_in_prompt_and_decoding(dtype, H, rank, R, window):
    """In the kernel's form for latent rows (one key head whose first entries are the value) one key is made to dominate for
    the queries that follow it: it must be seen by the query window - 1 places after it and not by the next one; in a prompt
    step and token by token, with the key on either side of a page border and at a sequence's first places."""
    dt = DTYPES[dtype]
    D = rank + R
    for key_at in (0, 1, 58, 63, 64, 127):
        n = key_at + window + 70
        g = torch.Generator().manual_seed(key_at)
        q, k = 0.01 * torch.randn(n, H, D, generator=g), 0.01 * torch.randn(n, 1, D, generator=g)
        k[key_at] = 0; k[key_at, :, D - 1] = 30.0; k[key_at, :, :rank] = 100.0      # the value is the front of the key row
        q[key_at + 1:] = 0; q[key_at + 1:, :, D - 1] = 30.0
        kp, table = paged(k, dt)
        for spans in ([(0, n)], [(0, key_at + 1)] + [(p, p + 1) for p in range(key_at + 1, n)], [(0, key_at + 1), (key_at + 1, key_at + 3), (key_at + 3, n)]):
            got = run_attention(q, kp, None, table, dt, spans, window, 1.0, rank, None, True)
            for p in range(key_at + 1, n):
                seen = p - key_at < window
                assert ((got[p] - 100.0).abs().max() < 1.0) == seen, (key_at, p, len(spans), got[p].abs().max())


# ------------------------------------------------------------------ rotation of halves, blended values and the cache write, alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,dims,scaling,blend", [(6, 2, 32, 16, 16, (4.0, 64, 8.0, 2.0), True), (3, 1, 24, 12, 10, (8.0, 32, 4.0, 0.5), False),
                                                         (4, 4, 16, 24, 16, None, True), (2, 2, 16, 16, 0, None, True), (4, 2, 128, 32, 48, (6.0, 2048, 24.0, 1.5), True),
                                                         (2, 1, 200, 8, 200, (2.0, 16, 64.0, 32.0), False)])
@pytest.mark.parametrize("shift", [1, 2])
def test_rotation_of_halves_with_blended_values_kernel(dtype, H, G, D, Dv, dims, scaling, blend, shift):
    """Against the plain rotation at positions up to 5000 on rows that carry more columns than q, k and v; the keys and values
    land at the tokens' places of their pages; blended values are rewritten in the rows and cached; the other columns stay.  The
    rows the values are blended with begin ``shift`` entries into wider rows (an odd shift keeps the kernel off its 4-byte path)."""
    from pico_engine.config import RotaryHalvesSpec
    from pico_engine.ops import kernels
    from pico_engine.parts.attention_gated import halves_frequencies
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(D + dims)
    pos = torch.tensor([0, 1, 2, 63, 64, 65, 700, 4999], dtype=torch.int32)
    T, extra = len(pos), 5
    rows = torch.randn(T, (H + G) * D + G * Dv + extra, generator=g).to(dt)
    other = torch.randn(T, G * Dv + 4, generator=g).to(dt)
    lam = torch.tensor(0.375, dtype=dt)
    sc = None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling))
    freqs, mag = plain.stretched_frequencies(dims, 1000.0, sc)
    freq, magnitude = halves_frequencies(RotaryHalvesSpec(D, dims, 1000.0, scaling), "cuda")
    assert abs(magnitude - mag) < 1e-12
    pages = 4999 // 64 + 1
    kp, vp = torch.zeros(pages + 1, G, 64, D, dtype=dt).cuda(), torch.zeros(pages + 1, G, 64, Dv, dtype=dt).cuda()
    table = torch.arange(1, pages + 1, dtype=torch.int32).view(1, -1).cuda()
    dev, odev = rows.cuda().clone(), other.cuda()
    kernels.rotary_half_store(dev, H, G, D, Dv, freq if dims else None, dims, magnitude, False, 1e-6, pos.cuda(), torch.zeros(T, dtype=torch.int32).cuda(),
                              kp, vp, table, pages, odev[:, shift:shift + G * Dv] if blend else None, lam.cuda() if blend else None)
    got = dev.float().cpu()
    r64 = rows.double()
    want_qk = torch.stack([plain.rotate_half(r64[t:t + 1, :(H + G) * D].view(1, H + G, D), dims, freqs, mag, first=int(pos[t]))[0] for t in range(T)])
    want_v = r64[:, (H + G) * D:(H + G) * D + G * Dv]
    if blend:
        want_v = (1 - lam.double()) * want_v + lam.double() * other.double()[:, shift:shift + G * Dv]
    tol = 3e-5 if dtype == "float32" else 2e-2
    turn = pos.double().view(T, 1, 1) * 2.5e-7 * 5          # the angle is a float32 product: its rounding grows with the position
    assert ((got[:, :(H + G) * D].double().view(T, H + G, D) - want_qk).abs() < tol * 5 + turn).all()
    assert (got[:, (H + G) * D:(H + G) * D + G * Dv].double() - want_v).abs().max() < tol * 5
    assert torch.equal(got[:, -extra:], rows[:, -extra:].float())
    for t, p in enumerate(pos.tolist()):
        page, at = 1 + p // 64, p % 64
        assert torch.equal(kp[page, :, at].float().cpu().view(-1), got[t, H * D:(H + G) * D])
        assert torch.equal(vp[page, :, at].float().cpu().view(-1), got[t, (H + G) * D:(H + G) * D + G * Dv])
    assert float(kp[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,R,rank,q_rank", [(3, 24, 16, 48, 40), (5, 12, 6, 20, 14), (2, 10, 4, 9, 30), (4, 32, 32, 64, 96)])
def test_latent_rows_in_the_layout_of_halves(dtype, H, D, R, rank, q_rank):
    """The kernel that norms the latent row, turns the shared key part and the heads' rotated query parts (halves) and builds the
    query rows, with the queries in rows of their own; and the norm of a run of columns in front of it."""
    from pico_engine.ops import kernels
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(D + R)
    pos = torch.tensor([0, 1, 63, 64, 300, 4999], dtype=torch.int32)
    T = len(pos)
    proj = torch.randn(T, q_rank + rank + R + 3, generator=g).to(dt)
    qrows = torch.randn(T, H * (D + R), generator=g).to(dt)
    qa = torch.randn(H, T, rank, generator=g).to(dt)
    nw, qw = (1 + 0.1 * torch.randn(rank, generator=g)).to(dt), (1 + 0.1 * torch.randn(q_rank, generator=g)).to(dt)
    freqs = plain.plain_frequencies(R, 500.0)
    freq = torch.tensor(freqs, dtype=torch.float64).float().cuda()
    pages = 4999 // 64 + 1
    kp = torch.zeros(pages + 1, 1, 64, rank + R, dtype=dt).cuda()
    table = torch.arange(1, pages + 1, dtype=torch.int32).view(1, -1).cuda()
    eps = 1e-5
    q = kernels.latent_prepare(proj.cuda(), H, D, R, rank, q_rank, nw.cuda(), eps, freq, R, qa.cuda(), pos.cuda(), torch.zeros(T, dtype=torch.int32).cuda(),
                               kp, table, pages, halves=True, q_rows=qrows.cuda()).float().cpu().view(T, H, rank + R)
    tol = 3e-5 if dtype == "float32" else 2e-2
    p64 = proj.double()
    for t, p in enumerate(pos.tolist()):
        c = plain.rms_unit(p64[t, q_rank:q_rank + rank], eps) * nw.double()
        kr = plain.rotate_half(p64[t:t + 1, q_rank + rank:q_rank + rank + R], R, freqs, first=p)[0]
        row = kp[1 + p // 64, 0, p % 64].double().cpu()
        turn = p * 2.5e-7 * 5                             # the angle is a float32 product: its rounding grows with the position
        assert (row[:rank] - c).abs().max() < tol * 5 and (row[rank:] - kr).abs().max() < tol * 5 + turn
        qr = plain.rotate_half(qrows.double()[t:t + 1].view(1, H, D + R)[..., D:], R, freqs, first=p)[0]
        assert (q[t, :, rank:].double() - qr).abs().max() < tol * 5 + turn
        assert torch.equal(q[t, :, :rank], qa[:, t].float())
    got = kernels.rmsnorm_cols(proj.cuda(), 0, q_rank, qw.cuda(), eps).double().cpu()
    assert (got - plain.rms_unit(p64[:, :q_rank], eps) * qw.double()).abs().max() < tol * 5


# ------------------------------------------------------------------ norms on a sublayer's output, the clamped activation, the choice of experts

@pytest.mark.parametrize("ydtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W", [50, 272, 1000, 3584, 4100])
def test_normed_output_into_the_stream_and_the_next_norm(ydtype, W):
    from pico_engine.ops import kernels
    g = torch.Generator().manual_seed(W)
    T, eps = 9, 1e-5
    x, y = torch.randn(T, W, generator=g) * 3 + 1, (torch.randn(T, W, generator=g) * 0.5 + 2).to(DTYPES[ydtype])
    w1, b1, w2, b2 = (torch.randn(W, generator=g).to(torch.bfloat16) for _ in range(4))
    want_x = x.double() + plain.layer_norm(y.double(), w1.double(), b1.double(), eps)
    want_h = plain.layer_norm(want_x, w2.double(), b2.double(), 2 * eps)
    dev = x.cuda().clone()
    assert kernels.layernorm_add(dev, y.cuda(), w1.cuda(), b1.cuda(), eps) is None
    tol = 1e-4                                           # (the plain norm reads the same rounded y)
    assert (dev.double().cpu() - want_x).abs().max() < tol
    for out_dtype in (torch.float32, torch.bfloat16):
        dev = x.cuda().clone()
        h = kernels.layernorm_add(dev, y.cuda(), w1.cuda(), b1.cuda(), eps, (w2.cuda(), b2.cuda(), 2 * eps), out_dtype)
        assert h.dtype == out_dtype and (dev.double().cpu() - want_x).abs().max() < tol
        assert (h.double().cpu() - want_h).abs().max() < (tol if out_dtype == torch.float32 else 5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("ff", [36, 344])
def test_clamped_activation_kernel(dtype, ff):
    from pico_engine.ops import kernels
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(ff)
    gu = (torch.randn(7, 2 * ff, generator=g) * 2).to(dt)
    gu[0, :4] = torch.tensor([1.25, 1.2499, 9.0, -9.0]).to(dt)
    gu[0, ff:ff + 4] = torch.tensor([-1.25, 1.25, -9.0, 9.0]).to(dt)
    lim = 1.25
    gg, uu = torch.clamp(gu[:, :ff].double(), max=lim), torch.clamp(gu[:, ff:].double(), min=-lim, max=lim)
    want = gg * plain.sigmoid(1.702 * gg) * (uu + 1)
    got = kernels.gated_act(gu.cuda(), "clamped_sigmoid", limit=lim, alpha=1.702).double().cpu()
    assert (got - want).abs().max() < (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("E,top,groups", [(8, 3, (4, 2)), (12, 3, (3, 1)), (6, 2, (6, 3)), (6, 1, (3, 1)), (4, 3, (1, 1)), (2, 2, None), (64, 6, (8, 3)), (256, 8, (8, 4)), (40, 40, (5, 5))])
def test_choice_of_experts_among_groups(E, top, groups):
    """The routing kernel against the plain choice on random logits and corrections of either sign (many choice scores are negative:
    experts outside the groups that stay must not return as zeros); weights are the plain scores."""
    from pico_engine.ops import kernels
    g = torch.Generator().manual_seed(E + top)
    T = 50
    logits = torch.randn(T, E, generator=g) * 2
    corr = torch.randn(E, generator=g) * 0.5 - 0.8
    r = {"experts": E, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    w = {"p.router": torch.eye(E, dtype=torch.float64), "p.correction": corr.double()}
    chosen = plain.route(logits.double(), {"router": r}, w, "p.")
    ids = torch.zeros(T, top, dtype=torch.int32).cuda()
    got = kernels.moe_route_grouped(logits.cuda(), E, top, corr.cuda(), groups[0] if groups else 1, groups[1] if groups else 1, 2, 1.0, ids).cpu()
    for t in range(T):
        want = torch.zeros(E, dtype=torch.float64)
        for e, s in chosen[t]:
            want[e] = s
        assert (got[t].double() - want).abs().max() < 1e-6, (t, got[t], want)
        assert ids[t].tolist() == [e for e, _ in chosen[t]]
    assert (got > 0).sum(1).tolist() == [top] * T


@pytest.mark.parametrize("K,E,top,groups", [(50, 6, 2, (6, 3)), (80, 8, 3, (4, 2)), (192, 10, 2, (2, 1)), (1000, 64, 6, (8, 3)), (128, 2, 2, (1, 1))])
def test_router_on_the_stream_through_its_layer_norm(K, E, top, groups):
    """Layer norm, router product and the choice among groups in one kernel on float32 rows, against the plain functions."""
    from pico_engine.ops import kernels
    g = torch.Generator().manual_seed(K + E)
    T, eps = 40, 1e-5
    x = torch.randn(T, K, generator=g) * 3 + 0.5
    nw, nb = (1 + 0.2 * torch.randn(K, generator=g)).to(torch.bfloat16), (0.2 * torch.randn(K, generator=g)).to(torch.bfloat16)
    router, corr = torch.randn(E, K, generator=g) * 1.5 * K ** -0.5, torch.randn(E, generator=g) - 0.3
    h = plain.layer_norm(x.double(), nw.double(), nb.double(), eps)
    w = {"p.router": router.double(), "p.correction": corr.double()}
    plain.ROUTER_GAPS = []
    chosen = plain.route(h, {"router": {"experts": E, "top": top, "groups": {"count": groups[0], "keep": groups[1]}}}, w, "p.")
    gaps, plain.ROUTER_GAPS = plain.ROUTER_GAPS[0], None
    ids = torch.zeros(T, top, dtype=torch.int32).cuda()
    got = kernels.moe_route_stream_grouped(x.cuda(), nw.cuda(), nb.cuda(), eps, router.cuda(), E, top, corr.cuda(), groups[0], groups[1], 2, 1.0, ids).cpu()
    compared = 0
    for t in range(T):
        if gaps[t] < 1e-4:                                   # (a choice that float32 rounding can turn)
            continue
        compared += 1
        want = torch.zeros(E, dtype=torch.float64)
        for e, sc in chosen[t]:
            want[e] = sc
        assert (got[t].double() - want).abs().max() < 1e-5, (t, got[t], want)
        assert ids[t].tolist() == [e for e, _ in chosen[t]]
    assert compared > T // 2


@pytest.mark.parametrize("ff,experts", [(24, 8), (32, 8), (20, 6), (64, 4)])
def test_gated_activation_times_expert_weights_leaves_unused_experts_at_zero(ff, experts):
    """silu(gate) * up * weight(token, expert) with the hidden units of all experts side by side; experts a token does not use give
    exact zeros, also where they hold infinities (their columns are not read where the kernel can tell)."""
    from pico_engine.ops import kernels
    g = torch.Generator().manual_seed(ff)
    T, I = 9, ff * experts
    for dt in (torch.float32, torch.bfloat16):
        gu = torch.randn(T, 2 * I, generator=g).to(dt)
        wts = torch.rand(T, experts, generator=g)
        wts[torch.rand(T, experts, generator=g) < 0.6] = 0.0
        col = wts.repeat_interleave(ff, dim=1).double()
        want = gu[:, :I].double() * plain.sigmoid(gu[:, :I].double()) * gu[:, I:].double() * col
        got = kernels.gated_act(gu.cuda(), "silu", wts.cuda(), ff).double().cpu()
        assert (got - want).abs().max() < (1e-5 if dt == torch.float32 else 2e-2)
        assert bool((got[col == 0] == 0).all())
