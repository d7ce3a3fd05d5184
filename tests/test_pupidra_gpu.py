"""Pupidra on the GPU against the plain implementation: each mechanism's kernel alone on inputs that show a fault, and the
whole model through the library's step function, cache, scheduler and entry points, in both dtypes, for every way of
cutting requests into steps."""
from __future__ import annotations

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_pupidra as plain
import replay
from conftest import write_model
from pupidra_models import CONFIGS, make_weights, plain_logits, requests_for

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CASES = [(n, d) for n in sorted(CONFIGS) for d in ("float32", "bfloat16")]
LENGTHS = {"P1": [1, 2, 3, 47, 70, 131, 64, 5], "P2": [65, 1, 150, 9, 33, 2], "P3": [3, 129, 31, 64, 1, 70], "P4": [4, 1, 290, 17, 66, 135]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{(config, dtype): (engine, cfg, weights, folder)}."""
    from pico_engine.engine.engine import Engine
    root = tmp_path_factory.mktemp("pupidra")
    out = {}
    for k, (name, cfg) in enumerate(sorted(CONFIGS.items())):
        weights = make_weights(cfg, 60 + k)
        folder = write_model(root / name, cfg, weights)
        for dtype in DTYPES:
            out[(name, dtype)] = (Engine(folder, dtype=dtype), cfg, weights, folder)
    return out


def compare(got, cfg, w, reqs, dtype, what, only_got=False):
    """Against the plain logits.  float32: every place, by the rule of the engine tests.  bfloat16: without the places where
    the plain router's choice was a close call and the two places behind each (which weigh that place's keys, values and
    convolution inputs most, and inherit another choice of experts there); of the others none may be off by more than a tenth of the logits' size, and
    at most one in a hundred by more than the engine tests' 4e-2 (a sublayer's output is normed before it is added, so a
    small output carries its rounding at full size into the stream: a few places lie just above the rule of the pre-norm designs)."""
    close = set()
    want = plain_logits(cfg, w, reqs, close)
    if only_got:
        want = {k: v for k, v in want.items() if k in got}
    if dtype != "bfloat16":
        return replay.compare(got, want, dtype, what)
    assert set(got) == set(want), (what, sorted(set(want) - set(got))[:5], sorted(set(got) - set(want))[:5])
    close |= {(r, p + d) for r, p in close for d in (1, 2)}
    assert len(close & set(want)) < 0.6 * len(want)
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
    windows pass over decoded tokens, pages behind them are given back while kept ones stay, and the states and the
    token before are carried from step to step."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 2)
    check(models, name, dtype, replay.tail(reqs, 100), reqs, "tail")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompts_in_portions(models, name, dtype):
    """Portions of unequal sizes, then portions of two, three and five tokens and single tokens in turn: every portion starts
    inside its sequence from the state and the cache pages the portion before it left."""
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
    """Batches one after another in a cache sized for one: slots, pages and state rows are used again, and a request's logits
    do not depend on its neighbours (compared with the plain run of each alone)."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name] + LENGTHS[name][::-1], 5)
    check(models, name, dtype, replay.batched(reqs, batch_size, fraction), reqs, "batched")


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_steps(models, name, dtype):
    """Steps that carry a fresh prompt, a later portion of another and single tokens side by side."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 6)
    check(models, name, dtype, replay.mixed(reqs), reqs, "mixed")


@pytest.mark.parametrize("name,dtype", [("P1", "float32"), ("P1", "bfloat16"), ("P4", "bfloat16"), ("P3", "float32")])
def test_batches_of_more_rows_than_the_decode_products_fuse(models, name, dtype):
    """Twenty short requests start together and are decoded together: steps of 17 and more rows take the products that prompts
    take, and the recurrence walks twenty sequences side by side."""
    reqs = requests_for(CONFIGS[name], [3 + (7 * i) % 23 for i in range(20)], 13)
    check(models, name, dtype, replay.batched(reqs, 20, 0.5), reqs, "twenty rows")


@pytest.mark.parametrize("name", ["P1", "P3", "P4"])
def test_long_decoding(models, name):
    """300 tokens one by one from a one-token prompt: windows, kept first tokens, pages given back, and states over many steps."""
    reqs = requests_for(CONFIGS[name], [301], 12)
    check(models, name, "float32", replay.tail(reqs, 300), reqs, "long decoding")


def test_a_freed_slot_starts_from_nothing(models):
    """A sequence that takes over a slot must not see the matrix states, the convolution's inputs or the last token left there."""
    eng, cfg, w, _ = models[("P1", "float32")]
    reqs = requests_for(cfg, [40, 6], 8)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"], "want": [39]}], "end": ["r0"]},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"], "want": list(range(6))}], "end": ["r1"]}]
    got = replay.run_in_process(eng, steps, max_tokens=64)
    compare(got, cfg, w, reqs, "float32", "slot reuse", only_got=True)


@pytest.mark.parametrize("name", ["P1", "P4"])
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
            assert o == plain.greedy(p, cfg, w64, n), (len(p), o)


def test_bfloat16_generation_with_graphs_matches_eager(models):
    eng, cfg, w, _ = models[("P3", "bfloat16")]
    prompts = list(requests_for(cfg, [7, 30, 2], 11).values())
    a = eng.generate(prompts, max_tokens=10, temperature=0.0, use_graph=False, stop_token_ids=[])
    b = eng.generate(prompts, max_tokens=10, temperature=0.0, use_graph=True, stop_token_ids=[])
    assert a == b


def test_trace_replay_program(models, tmp_path):
    eng, cfg, w, folder = models[("P2", "float32")]
    reqs = requests_for(cfg, [40, 3, 77], 10)
    steps = replay.batched(reqs, 3, 0.6)
    got = replay.run_binary(folder, "float32", steps, str(tmp_path / "out"), cfg["vocab"])
    compare(got, cfg, w, reqs, "float32", "bin/trace_run")


def test_command_line_generates(models):
    import json, subprocess, sys
    eng, cfg, w, folder = models[("P1", "float32")]
    out = subprocess.run([sys.executable, "-m", "pico_engine", folder, "--prompt", "5,17,3", "--max-tokens", "6", "--temperature", "0",
                          "--dtype", "float32"], capture_output=True, text=True, cwd=replay.ROOT, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    with torch.no_grad():
        assert json.loads(line)["output"] == plain.greedy([5, 17, 3], cfg, {n: t.double() for n, t in w.items()}, 6)


# ------------------------------------------------------------------ attention with a distance bias, a window and kept first keys, alone

def paged(k, dt, first_page=1):
    """k [n, G, D] as cache pages [pages + first_page, G, 64, D] and the page table of one sequence."""
    n, G, D = k.shape
    pages = (n + 63) // 64
    pool = torch.zeros(pages + first_page, G, 64, D, dtype=dt).cuda()
    for p in range(n):
        pool[first_page + p // 64, :, p % 64] = k[p].to(dt).cuda()
    return pool, torch.arange(first_page, pages + first_page, dtype=torch.int32).view(1, -1).cuda()


def run_attention(q, kp, vp, table, dt, spans, window, keep, scale, slopes, Dv, values_in_keys=False):
    """``kernels.attention_headmix`` for the query positions of ``spans`` (each a step of one sequence); q [n, H, D]."""
    from pico_engine.ops import kernels
    n, H, D = q.shape
    G = kp.shape[1]
    out = torch.zeros(n, H * Dv)
    sl = None if slopes is None else torch.tensor(slopes, dtype=torch.float32).cuda()
    for a, b in spans:
        ctx = SimpleNamespace(one_token_each=(b - a == 1), scratch={}, lens=[b - a], starts=[a], max_context=b, dtype=dt)
        pos, row = torch.arange(a, b, dtype=torch.int32).cuda(), torch.zeros(b - a, dtype=torch.int32).cuda()
        qq = q[a:b].reshape(b - a, H * D).to(dt).cuda().contiguous()
        o = kernels.attention_headmix(qq, H * D, H, G, D, Dv, kp, vp, table, table.shape[1], pos, row, window, scale, None, None, ctx,
                                      slopes=sl, keep_first=keep, values_in_keys=values_in_keys)
        out[a:b] = o.float().cpu()
    return out.view(n, H, Dv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,window,keep", [(6, 2, 32, 16, 40, 5), (3, 1, 24, 12, 2, 1), (8, 1, 64, 64, 130, 70), (2, 2, 16, 16, 64, 64),
                                                  (4, 4, 16, 24, None, 0), (4, 2, 48, 40, 70, 0), (2, 1, 128, 128, 65, 3)])
def test_biased_attention_kernel(dtype, H, G, D, Dv, window, keep):
    """Random queries, keys and values against the plain function: as one prompt, in portions, and the last 80 tokens one by one."""
    dt = DTYPES[dtype]
    n = 230
    g = torch.Generator().manual_seed(H * 100 + D)
    q, k, v = ((torch.randn(n, h, d, generator=g)).to(dt).float() for h, d in ((H, D), (G, D), (G, Dv)))
    scale = 0.5 * D ** -0.5
    want = plain.biased_attention(q.double(), k.double(), v.double(), scale, window, keep)
    kp, table = paged(k, dt)
    vp, _ = paged(v, dt)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for spans in ([(0, n)], [(0, 3), (3, 70), (70, 72), (72, 200), (200, n)], [(0, 150)] + [(p, p + 1) for p in range(150, n)]):
        got = run_attention(q, kp, vp, table, dt, spans, window, keep, scale, plain.distance_slopes(H), Dv)
        assert (got.double() - want).abs().max() < tol * max(1.0, float(want.abs().max())), spans[:2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,window,keep", [(6, 2, 32, 16, 40, 5), (3, 1, 24, 12, 2, 1), (8, 1, 64, 64, 130, 70), (2, 2, 16, 16, 64, 64),
                                                  (2, 1, 64, 64, 66, 3), (2, 2, 128, 128, 40, 65)])
def test_window_and_kept_edges_in_prompt_and_decoding(dtype, H, G, D, Dv, window, keep):
    """One key is made to dominate for the queries that follow it.  A key behind the kept ones must be seen by the query
    window - 1 places after it and not by the next one; the last kept key must be seen from everywhere and the first key
    that is not kept only inside its window; in a prompt step and token by token, with the key on either side of a page border."""
    dt = DTYPES[dtype]
    for key_at in sorted({keep - 1, keep, keep + 58, keep + 59, 63 + keep, 64 + keep, 127 + keep} - {-1}):
        n = key_at + window + 70
        g = torch.Generator().manual_seed(key_at)
        q, k, v = 0.01 * torch.randn(n, H, D, generator=g), 0.01 * torch.randn(n, G, D, generator=g), torch.randn(n, G, Dv, generator=g)
        k[key_at] = 0; k[key_at, :, 1] = 30.0
        q[key_at + 1:] = 0; q[key_at + 1:, :, 1] = 30.0              # a score of 900 against a distance bias of 0.5 a place at most
        v[key_at] = 100.0
        kp, table = paged(k, dt)
        vp, _ = paged(v, dt)
        for spans in ([(0, n)], [(0, key_at + 1)] + [(p, p + 1) for p in range(key_at + 1, n)]):
            got = run_attention(q, kp, vp, table, dt, spans, window, keep, 1.0, plain.distance_slopes(H), Dv)
            for p in range(key_at + 1, n):
                seen = p - key_at < window or key_at < keep
                assert ((got[p] - 100.0).abs().max() < 1.0) == seen, (key_at, p, len(spans), got[p].abs().max())


@pytest.mark.parametrize("H,G,D,window,keep", [(4, 2, 64, 100, 70), (2, 1, 128, 65, 3), (2, 2, 64, 64, 0), (3, 1, 64, None, 0),
                                               (2, 2, 128, 200, 128), (2, 1, 64, 300, 1)])
def test_long_prompts_in_bfloat16_at_head_sizes_of_the_tensor_memory_kernel(H, G, D, window, keep):
    """Prompts long enough that the pages of the kept first keys and the pages of the window lie apart, whole, in portions
    that begin and end off the borders of pages and of the kernel's runs of tokens, and with the last 330 tokens one by one."""
    dt, n = torch.bfloat16, 900
    g = torch.Generator().manual_seed(H * 100 + D + (window or 0))
    q, k, v = ((torch.randn(n, h, D, generator=g)).to(dt).float() for h in (H, G, G))
    scale = 0.7 * D ** -0.5
    want = plain.biased_attention(q.double(), k.double(), v.double(), scale, window, keep)
    kp, table = paged(k, dt)
    vp, _ = paged(v, dt)
    for spans in ([(0, n)], [(0, 130), (130, 133), (133, 517), (517, n)], [(0, 570)] + [(p, p + 1) for p in range(570, n)]):
        got = run_attention(q, kp, vp, table, dt, spans, window, keep, scale, plain.distance_slopes(H), D)
        assert (got.double() - want).abs().max() < 2e-2 * max(1.0, float(want.abs().max())), spans[:2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 63, 64, 65, 447])
def test_a_key_from_far_back(dtype, far):
    """Without a window, and in the kernel's form for latent rows (one key head whose first entries are the value), one key
    that matches the last query must come through from any distance, although the distance bias counts against it."""
    dt = DTYPES[dtype]
    H, n = 4, 700
    for G, D, Dv, in_keys in ((2, 32, 24, False), (1, 48, 40, True)):
        g = torch.Generator().manual_seed(far)
        q, k, v = 0.01 * torch.randn(n, H, D, generator=g), 0.01 * torch.randn(n, G, D, generator=g), torch.randn(n, G, Dv, generator=g)
        k[far] = 0; k[far, :, D - 1] = 40.0
        q[-1] = 0; q[-1, :, D - 1] = 40.0                            # 1600 against at most 0.5 * 700
        if in_keys:
            v = k[:, :, :Dv].clone()
            v[far] = k[far, :, :Dv] = 8.0
            k[far, :, D - 1] = 40.0
        else:
            v[far] = 8.0
        kp, table = paged(k, dt)
        vp = None if in_keys else paged(v, dt)[0]
        for spans in ([(0, n)], [(n - 1, n)]):
            got = run_attention(q, kp, vp, table, dt, spans, None, 0, 1.0, None if in_keys else plain.distance_slopes(H), Dv, in_keys)
            assert (got[-1] - 8.0).abs().max() < 0.1, (far, in_keys, got[-1])


# ------------------------------------------------------------------ the state-space mixer's kernels, alone

def run_state_space(proj, m, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, eps, dt, lens, cuts, chunked=False):
    """Convolution, recurrence and gated norm on packed sequences of ``lens`` tokens (rows of proj = z | x | B | C | dt), brought
    in steps that cut every sequence at the fractions ``cuts``; returns [T, inner] and the final matrix states."""
    from pico_engine.ops import kernels
    H, P, N, G, taps, groups = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner, conv = H * P, H * P + 2 * G * N
    T, B = proj.shape[0], len(lens)
    elems = kernels.state_space_elems(H, P, N)
    state = torch.full((B + 2, 5 + elems + (taps - 1) * conv), 3.0).cuda()      # the part's state begins at offset 5 of a slot's row
    state[1:B + 1, 5:] = 0
    slots = torch.tensor([b + 1 for b in range(B)], dtype=torch.int32).cuda()
    dev = proj.to(dt).cuda().contiguous()
    cw, cb, nw = conv_w.to(dt).cuda(), conv_b.to(dt).cuda(), norm_w.to(dt).cuda()
    f32 = [t.float().cuda() for t in (dt_bias, a_log, d_skip)]
    first = np.concatenate([[0], np.cumsum(lens)])
    out = torch.zeros(T, inner)
    done = [0] * B
    for c in cuts:
        upto = [n if c == cuts[-1] else max(d, int(n * c)) for n, d in zip(lens, done)]
        rows = [b for b in range(B) if upto[b] > done[b]]
        idx = torch.cat([torch.arange(first[b] + done[b], first[b] + upto[b]) for b in rows])
        step_lens = [upto[b] - done[b] for b in rows]
        rf = torch.tensor(np.concatenate([[0], np.cumsum(step_lens)]), dtype=torch.int32).cuda()
        rl = torch.tensor(step_lens, dtype=torch.int32).cuda()
        tr = torch.tensor(np.repeat(np.arange(len(rows)), step_lens), dtype=torch.int32).cuda()
        sl = slots[torch.tensor(rows).cuda()].contiguous()
        p = dev[idx.cuda()].contiguous()
        xbc = kernels.conv_silu(p, inner, conv, cw, cb, state, 5 + elems, tr, rf, rl, sl)
        y = kernels.state_space_scan(xbc, p, inner + conv, *f32, state, 5, rf, rl, sl, H, P, N, G, chunked=chunked)
        out[idx] = kernels.gate_norm(y, inner // groups, p, 0, nw, eps).float().cpu()
        done = upto
    assert float(state[0].min()) == 3.0 and float(state[B + 1].min()) == 3.0 and float(state[:, :5].min()) == 3.0
    return out


def plain_state_space(proj, m, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, eps, lens):
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    outs, at = [], 0
    for n in lens:
        pr = proj[at:at + n].double()
        z, xbc, dtr = pr[:, :inner], pr[:, inner: 2 * inner + 2 * G * N], pr[:, 2 * inner + 2 * G * N:]
        xbc = plain.silu(plain.causal_conv(xbc, conv_w.double(), conv_b.double()))
        y = plain.ssm_recurrence(xbc[:, :inner].reshape(n, H, P), xbc[:, inner: inner + G * N].reshape(n, G, N),
                                 xbc[:, inner + G * N:].reshape(n, G, N), plain.softplus(dtr + dt_bias.double()),
                                 -torch.exp(a_log.double()), d_skip.double()).reshape(n, inner) * plain.silu(z)
        groups = m["norm_groups"]
        outs.append(plain.rms_unit(y.view(n, groups, inner // groups), eps).reshape(n, inner) * norm_w.double())
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,P,N,G,taps,groups", [(4, 16, 24, 2, 3, 4), (2, 8, 40, 1, 2, 1), (3, 5, 7, 3, 1, 3), (4, 32, 128, 4, 4, 2),
                                                  (2, 64, 16, 2, 4, 1), (1, 40, 200, 1, 5, 8), (6, 24, 64, 3, 4, 2)])
def test_state_space_kernels(dtype, H, P, N, G, taps, groups):
    """Sequences of many lengths as one prompt step, in portions, and with the last tokens one by one; a sequence's walk and the
    three passes over chunks of 64."""
    dt = DTYPES[dtype]
    m = {"heads": H, "vdim": P, "state": N, "groups": G, "conv": taps, "norm_groups": groups}
    g = torch.Generator().manual_seed(H * 1000 + N)
    lens = [1, 2, 9, 70, 3, 131, 64, 200]
    T, inner, conv = sum(lens), H * P, H * P + 2 * G * N
    r = lambda *s: torch.randn(*s, generator=g)
    rounded = lambda t: t.to(dt).float()
    proj = rounded(r(T, 2 * inner + 2 * G * N + H))
    conv_w, conv_b, norm_w = rounded(0.6 * r(conv, taps)), rounded(0.3 * r(conv)), rounded(1 + 0.1 * r(inner))
    dt_bias, a_log, d_skip = r(H) - 1.0, 0.7 * r(H) - 0.5, 1 + 0.3 * r(H)
    args = (m, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, 1e-5)
    want = plain_state_space(proj, *args, lens)
    tol = (3e-5 if dtype == "float32" else 1.5e-2) * max(1.0, float(want.abs().max()))
    for cuts in ((1.0,), (0.4, 0.75, 1.0), (0.97, 0.98, 0.99, 1.0)):
        for chunked in (False, True):
            got = run_state_space(proj, *args, dt, lens, cuts, chunked)
            assert (got.double() - want).abs().max() < tol, (cuts, chunked)


@pytest.mark.parametrize("far", [0, 1, 7, 8, 9, 63, 64, 65, 447, 511, 512])
def test_state_keeps_an_input_from_far_back(far):
    """With a decay of nearly 1 an input whose B matches the last token's C must come through from any distance: the first
    positions, the borders of the kernel's groups of tokens and of its chunks, hundreds of tokens back, also when the last token
    comes alone."""
    m = {"heads": 1, "vdim": 4, "state": 8, "groups": 1, "conv": 1, "norm_groups": 1}
    n, inner, N = 600, 4, 8
    g = torch.Generator().manual_seed(far)
    proj = 0.01 * torch.randn(n, 2 * inner + 2 * N + 1, generator=g)
    proj[:, :inner] = 5.0                                        # gate silu(5) ~ 5
    proj[:, -1] = 3.0                                            # dt ~ 3
    proj[far, inner: 2 * inner] = 9.0                            # x (silu(9) ~ 9)
    proj[far, 2 * inner + 3] = 9.0                               # B, state row 3
    proj[-1, 2 * inner + N + 3] = 9.0                            # C of the last token, state row 3
    ones, zeros = torch.ones(inner + 2 * N, 1), torch.zeros(inner + 2 * N)
    args = (m, ones, zeros, torch.zeros(1), torch.full((1,), -12.0), torch.zeros(1), torch.ones(inner), 1e-5)
    want = plain_state_space(proj, *args, [n])
    assert float(want[-1].abs().min()) > 0.9                      # the norm makes it 1: the far input dominates the last row
    for cuts, chunked in (((1.0,), False), ((1.0,), True), ((0.5, (n - 1) / n, 1.0), False), ((0.3, (n - 1) / n, 1.0), True)):
        got = run_state_space(proj, *args, torch.float32, [n], cuts, chunked)
        assert (got[-1].double() - want[-1]).abs().max() < 1e-3, (far, cuts, chunked)


# ------------------------------------------------------------------ the router, the experts' hidden units, pairs of tokens

@pytest.mark.parametrize("E,top,shared", [(5, 2, True), (3, 1, False), (7, 3, True), (2, 2, True), (64, 6, False)])
def test_routing_over_all_experts(E, top, shared):
    from pico_engine.ops import kernels
    g = torch.Generator().manual_seed(E)
    T, K = 50, 72
    x = torch.randn(T, K, generator=g)
    router = torch.randn(E, K, generator=g) * 0.5
    z = x.double() @ router.double().T
    s = torch.softmax(z, -1)
    want = torch.zeros(T, E + (1 if shared else 0), dtype=torch.float64)
    idx = s.topk(top, -1).indices
    want[:, :E].scatter_(1, idx, s.gather(1, idx) * 1.7)
    if shared:
        want[:, E] = 1.0
    extra = "one" if shared else False
    got = kernels.moe_route_stream(x.cuda(), None, 0.0, router.cuda().contiguous(), E, top, extra, over_all=True, factor=1.7)
    assert (got.cpu().double() - want).abs().max() < 1e-5
    got = kernels.moe_route(z.float().cuda().contiguous(), E, top, extra, over_all=True, factor=1.7)
    assert (got.cpu().double() - want).abs().max() < 1e-5
    # hidden units: relu^2 times the weight of the expert that owns the column; the shared expert's columns come last and may be wider
    # (widths that are multiples of 8 take 16-byte accesses in bfloat16); an infinite hidden unit behind a zero weight gives zero
    for ff, sff in ((12, 20), (16, 40)):
        h = torch.randn(T, E * ff + (sff if shared else 0), generator=g)
        unused = [e for e in range(E) if want[0, e] == 0]
        if unused:
            h[0, unused[0] * ff + 1] = float("inf")
        for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            hh = h.to(dt)
            out = kernels.weighted_act(hh.cuda().contiguous(), "relu2", got, ff).float().cpu()
            col = torch.clamp(torch.arange(h.shape[1]) // ff, max=want.shape[1] - 1)
            w = want[:, col]
            ref = torch.where(w == 0, torch.zeros_like(w), plain.relu2(hh.double()) * w)
            assert (out.double() - ref).abs().max() < tol * float(ref.abs().max())
            assert bool((out[ref == 0] == 0).all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pairs_of_tokens_in_the_embedding(dtype):
    """Whole sequences, then the same cut into steps so that the token before comes from the state; slots are used again."""
    from pico_engine.ops import kernels
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(5)
    V, W, buckets, mp, mc = 50, 24, 13, 29, 3
    table, pairs = torch.randn(V, W, generator=g).to(dt), torch.randn(buckets + 1, W, generator=g).to(dt)
    big = {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (1, 7, 20)]
    w = {"embed": table.double(), "bigram": pairs.double()}
    want = [plain.embed(s, w, big) for s in seqs]
    state = torch.full((5, 1), 77, dtype=torch.int32).cuda()          # rows 0 and 4 belong to nobody
    for cuts in ([1.0], [0.5, 1.0], [0.2, 0.3, 0.9, 1.0]):
        done = [0] * len(seqs)
        got = [torch.zeros(len(s), W) for s in seqs]
        for c in cuts:
            upto = [len(s) if c == cuts[-1] else max(d, int(len(s) * c)) for s, d in zip(seqs, done)]
            rows = [b for b in range(len(seqs)) if upto[b] > done[b]]
            ids = torch.tensor([t for b in rows for t in seqs[b][done[b]:upto[b]]], dtype=torch.int32).cuda()
            lens = [upto[b] - done[b] for b in rows]
            pos = torch.tensor([p for b in rows for p in range(done[b], upto[b])], dtype=torch.int32).cuda()
            tr = torch.tensor(np.repeat(np.arange(len(rows)), lens), dtype=torch.int32).cuda()
            rf = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32).cuda()
            slots = torch.tensor([b + 1 for b in rows], dtype=torch.int32).cuda()
            out = kernels.embed_pairs(table.cuda(), pairs.cuda(), ids, pos, tr, rf, slots, state, buckets, mp, mc).cpu()
            at = 0
            for b, n in zip(rows, lens):
                got[b][done[b]:upto[b]] = out[at:at + n]; at += n
            done = upto
        for a, b in zip(got, want):
            assert (a.double() - b).abs().max() < 1e-6
        assert int(state[0, 0]) == 77 and int(state[4, 0]) == 77
        assert state[1:4, 0].tolist() == [s[-1] for s in seqs]
