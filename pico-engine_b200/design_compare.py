"""Two designs side by side at equal layer widths: the Mebalorn decoder (layer norm + input convolution, attention
with mixed heads or a minGRU recurrence, a dense relu^2 feed-forward, both halves in parallel), the Kevelorn decoder
(linear attention with fixed or learned decay, windowed softmax attention with an output gate beside it, gated dense
feed-forwards and mixtures of experts) or the Pupidra decoder (post-norm layers with layer scale; windowed attention with a
distance bias and kept first keys, also on another layer's keys and values; latent attention; a state-space mixer; ungated
mixtures; a bigram embedding) or the Tenusun decoder (a layer norm before and after each sublayer; latent attention with a query
row behind a sliding window; grouped attention with one added to the softmax denominator, stretched rotation of halves, blended values and an
output gate; a clamped gated feed-forward; mixtures chosen by sigmoid scores among groups of experts; its kernels also beside Pupidra's like
kernels) and the dense Qwen2 decoder, this library's closest other model.  Random weights; prefill and decode throughput of a few layers, and
the kernels of the new design each beside the Qwen2 kernel that does the like job, as fractions of the measured
copy bandwidth or matrix throughput.

    python -m pico_engine.design_compare [--design mebalorn|kevelorn|pupidra|tenusun] [--sizes s,m,l] [--tokens 2048] [--batch 8] [--context 2048] [--output FILE]
"""
from __future__ import annotations

import argparse
import json
from typing import Callable, Dict

import torch

from . import benchmark as B
from .config import config_from_dict
from .ops import kernels

# layer widths that resemble real models: (width, heads, key/value heads, head size, feed-forward width, layers)
SIZES = {"s": (896, 14, 2, 64, 4864, 4), "m": (2048, 16, 4, 128, 8192, 4), "l": (3584, 28, 4, 128, 18944, 2)}
VOCAB = 32768
TAPS = 4


def mebalorn_config(size: str) -> dict:
    from .config.shapes import mebalorn_shape
    W, H, G, D, F, L = SIZES[size]
    return mebalorn_shape(W, H, G, D, F, L, VOCAB, taps=TAPS)


def kevelorn_config(size: str, layers: int | None = None) -> dict:
    from .config.shapes import kevelorn_shape
    W, H, G, D, F, L = SIZES[size]
    return kevelorn_shape(W, H, G, D, F, layers or L, VOCAB)


def pupidra_config(size: str, layers: int | None = None) -> dict:
    from .config.shapes import pupidra_shape
    W, H, G, D, F, L = SIZES[size]
    return pupidra_shape(W, H, G, D, F, layers or max(L, 4), VOCAB)          # four layers: every kind of mixer once


def tenusun_config(size: str, layers: int | None = None) -> dict:
    from .config.shapes import tenusun_shape
    W, H, G, D, F, L = SIZES[size]
    return tenusun_shape(W, H, G, D, F, layers or max(L, 4), VOCAB)          # four layers: both kinds of layer twice (the second attention blends values)


DESIGNS = {"mebalorn": mebalorn_config, "kevelorn": kevelorn_config, "pupidra": pupidra_config, "tenusun": tenusun_config}
FOUR_LAYERS = ("pupidra", "tenusun")


def qwen2_config(size: str, layers: int | None = None) -> dict:
    W, H, G, D, F, L = SIZES[size]
    L = layers or L
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "torch_dtype": "bfloat16",
            "num_hidden_layers": L, "hidden_size": W, "num_attention_heads": H, "num_key_value_heads": G, "head_dim": D,
            "intermediate_size": F, "vocab_size": VOCAB, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
            "max_position_embeddings": 32768, "tie_word_embeddings": False, "use_sliding_window": False}


_flush = {}


def _graph_ms(body: Callable[[], object], replays: int = 5) -> float:
    """Median milliseconds of a replay of the CUDA graph that ``body`` records."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            body()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return B.percentile(times, 50)


def device_us(fn: Callable[[], object], calls: int = 8) -> float:
    """Microseconds of ``fn`` on the device.  ``calls`` times [write a 256 MB buffer (which empties the L2), fn] are
    captured in one CUDA graph, so that no launch waits for the host; the same graph without fn is timed too and
    subtracted.  CUDA events around the replays, the median of five, after a warm-up call and replay."""
    buf = _flush.get("buf")
    if buf is None:
        buf = _flush["buf"] = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn()
    torch.cuda.synchronize()

    def both():
        for _ in range(calls):
            buf.zero_()
            fn()

    def flush_only():
        for _ in range(calls):
            buf.zero_()
    return max(0.0, (_graph_ms(both) - _graph_ms(flush_only)) * 1000.0 / calls)


def _prompt_context(eng, tokens: int):
    slot = eng.cache.open()
    ids = torch.randint(0, eng.model.plan.vocab_size, (tokens,), generator=torch.Generator().manual_seed(0)).tolist()
    eng.stepper.step([slot], [ids], [[]])                     # fills the cache and the states of this slot
    eng.cache.close(slot)
    slot = eng.cache.open()
    lay, host, starts = eng.stepper.describe([slot], [tokens], None, [ids])
    dev = eng.stepper.upload(host)
    return slot, eng.stepper.context(lay, dev, [tokens], starts, [slot])


def _decode_context(eng, batch: int, context: int):
    slots = B.open_sequences(eng, batch, context - 1)
    lay, host, starts = eng.stepper.describe(slots, [1] * batch, None, [[1]] * batch)
    dev = eng.stepper.upload(host)
    return slots, eng.stepper.context(lay, dev, [1] * batch, starts, slots)


def kevelorn_kernel_times(eng, size: str, tokens: int, batch: int, context: int, entry) -> None:
    """The kernels that only the Kevelorn parts have, each at the sizes of this shape's layers."""
    W, H, G, D, F, L = SIZES[size]
    bf = torch.bfloat16
    sched = eng.model.plan.schedule
    kind = lambda e: type(eng.model.layers[sched[e].layer].mixer).__name__
    e_fix = next(e for e in range(len(sched)) if kind(e) == "LinearAttention" and eng.model.layers[sched[e].layer].mixer.head_decay is not None)
    e_gla = next(e for e in range(len(sched)) if kind(e) == "LinearAttention" and eng.model.layers[sched[e].layer].mixer.head_decay is None)
    e_par = next(e for e in range(len(sched)) if kind(e) == "BranchSum")
    fix = eng.model.layers[sched[e_fix].layer].mixer
    left = eng.model.layers[sched[e_par].layer].mixer.branches[0]
    moe = eng.model.layers[sched[e_gla].layer].feed_forward
    state_bytes = H * D * D * 4

    def recurrences(ctx, T, B, chunked, label):
        proj = torch.randn(T, 4 * H * D, device="cuda").to(bf)
        z = torch.randn(T, H * D, device="cuda")
        work = 4.0 * H * D * D * T * (2 if chunked else 1)        # multiply-adds x 2, and the chunked way walks every chunk twice
        moved = T * 4 * H * D * 2 + T * H * D * 4 + 2 * B * state_bytes
        us = device_us(lambda: kernels.linear_attention(proj, 0, H * D, 2 * H * D, H, D, D, ctx.state(e_fix), 0, ctx.row_first, ctx.row_lens,
                                                        ctx.slots, chunked, head_decay=fix.head_decay, qk_activation="silu", v_activation="silu"))
        entry(f"{label} recurrence, fixed decay", us, nbytes=moved)
        out[f"{label} recurrence, fixed decay"]["float32_tflops_per_s"] = work / us / 1e6
        us = device_us(lambda: kernels.linear_attention(proj, 0, H * D, 2 * H * D, H, D, D, ctx.state(e_gla), 0, ctx.row_first, ctx.row_lens,
                                                        ctx.slots, chunked, decay_logits=z, inv_tau=1 / 16.0, q_scale=D ** -0.5))
        entry(f"{label} recurrence, learned decay", us, nbytes=moved + T * H * D * 4)
        out[f"{label} recurrence, learned decay"]["float32_tflops_per_s"] = work / us / 1e6

    out = entry.out
    slot, ctx = _prompt_context(eng, tokens)
    kv = ctx.kv(e_par)
    recurrences(ctx, tokens, 1, True, "prefill")
    qkvg = torch.randn(tokens, left.w_in.shape[0], device="cuda").to(bf)
    entry("prefill pair rotation + unit norm + cache write", device_us(lambda: kernels.rotary_norm_store(
        qkvg, H, G, D, D, left.freq, D, True, 1e-6, ctx.tok_pos, ctx.tok_row, kv.k, kv.v, kv.table, kv.stride)), nbytes=tokens * (H + 2 * G) * D * 2 * 2)
    window = left.spec.window
    seen = sum(min(p + 1, window) for p in range(tokens))
    entry("prefill attention (window)", device_us(lambda: kernels.attention(
        qkvg, qkvg.shape[1], H, G, D, kv.k, kv.v, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, window, D ** -0.5, ctx)), flops=4.0 * H * D * seen)
    o = torch.randn(tokens, H * D, device="cuda")
    entry("prefill norm over heads x gate", device_us(lambda: kernels.gated_norm(o, H * D, fix.norm, 1e-6, qkvg, 0, "sigmoid", bf)),
          nbytes=tokens * H * D * (4 + 2 + 2))
    entry("prefill norm per head x gate", device_us(lambda: kernels.gated_norm(o, D, fix.norm[:D].contiguous(), 1e-6, qkvg, 0, "silu", bf)),
          nbytes=tokens * H * D * (4 + 2 + 2))
    ob = o.to(bf)
    entry("prefill heads x gate", device_us(lambda: kernels.gated_norm(ob, 0, None, 1e-6, qkvg, 0, "sigmoid", bf)), nbytes=tokens * H * D * 2 * 3)
    x = torch.randn(tokens, W, device="cuda")
    ys = [torch.randn(tokens, W, device="cuda") for _ in range(2)]
    ws = eng.model.layers[sched[e_par].layer].mixer.out_norms
    entry("prefill two normed branches into the stream", device_us(lambda: kernels.normed_sum_add(x, ys, ws, 1e-6, 0.25)), nbytes=tokens * W * 4 * 4)
    entry("prefill scaled residual sum", device_us(lambda: kernels.scaled_add(x, ys[0], 0.5)), nbytes=tokens * W * 4 * 3)
    gu = torch.randn(tokens, 2 * F, device="cuda").to(bf)
    entry("prefill gelu(gate) x up", device_us(lambda: kernels.gated_act(gu, "gelu_tanh")), nbytes=tokens * F * 2 * 3)
    I = moe.w_down.shape[1]
    gum = torch.randn(tokens, 2 * I, device="cuda").to(bf)
    logits = torch.randn(tokens, moe.spec.n_experts + 1, device="cuda")
    wts = kernels.moe_route(logits, moe.spec.n_experts, moe.spec.top_k, True)
    norm2 = eng.model.layers[sched[e_gla].layer].feed_forward_norm
    entry("prefill norm + router + choice of experts", device_us(lambda: kernels.moe_route_stream(
        x, norm2.weight, norm2.eps, moe.w_router, moe.spec.n_experts, moe.spec.top_k, True)), nbytes=tokens * (W * 4 + (moe.spec.n_experts + 1) * 4))
    entry("prefill silu(gate) x up x expert weight", device_us(lambda: kernels.gated_act(gum, "silu", wts, moe.spec.intermediate)), nbytes=tokens * I * 2 * 3)
    eng.cache.close(slot)
    slots, ctx = _decode_context(eng, batch, context)
    recurrences(ctx, batch, batch, False, "decode")
    kv = ctx.kv(e_par)
    q1 = torch.randn(batch, left.w_in.shape[0], device="cuda").to(bf)
    entry("decode attention (window)", device_us(lambda: kernels.attention(
        q1, q1.shape[1], H, G, D, kv.k, kv.v, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, window, D ** -0.5, ctx)),
        nbytes=batch * min(context, window) * 2 * G * D * 2)
    B.close_sequences(eng, slots)


def pupidra_kernel_times(eng, size: str, tokens: int, batch: int, context: int, entry) -> None:
    """The kernels that only the Pupidra parts have (or that they use in a new form), each at the sizes of this shape's layers."""
    W, H, G, D, F, L = SIZES[size]
    bf = torch.bfloat16
    out = entry.out
    layers = eng.model.layers
    e_att, e_ssm, e_lat, e_read = 0, 1, 2, 3
    att, ssm, lat = layers[e_att].mixer, layers[e_ssm].mixer, layers[e_lat].mixer
    moe = layers[e_att].feed_forward
    sa, ss, sl = att.spec, ssm.spec, lat.spec
    inner, bc, conv = ssm._sizes()
    rank, R = sl.kv_rank, sl.rot_dim
    q_w, dkv_w, _ = lat._widths()
    state_floats = ssm.matrix_state_elems()

    def attention_calls(ctx, T, label, seen_biased, seen_all, nbytes_biased=None, nbytes_latent=None):
        kv = ctx.kv(e_att)
        qkv = torch.randn(T, att.w_in.shape[0], device="cuda").to(bf)
        how = dict(flops=4.0 * H * D * seen_biased) if nbytes_biased is None else dict(nbytes=nbytes_biased)
        entry(f"{label} attention (distance bias, window, kept first keys)", device_us(lambda: kernels.attention_headmix(
            qkv, qkv.shape[1], H, G, D, D, kv.k, kv.v, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, sa.window, sa.scale, None, None, ctx,
            slopes=att.slopes, keep_first=sa.keep_first)), **how)
        kl = ctx.kv(e_lat)
        ql = torch.randn(T, H * (rank + R), device="cuda").to(bf)
        how = dict(flops=2.0 * H * (2 * rank + R) * seen_all) if nbytes_latent is None else dict(nbytes=nbytes_latent)
        entry(f"{label} attention over latent rows", device_us(lambda: kernels.attention_headmix(
            ql, ql.shape[1], H, 1, rank + R, rank, kl.k, None, kl.table, kl.stride, ctx.tok_pos, ctx.tok_row, None, sl.scale, None, None, ctx,
            values_in_keys=True)), **how)

    def state_space_calls(ctx, T, B, label):
        proj = torch.randn(T, ssm.w_in.shape[0], device="cuda").to(bf)
        state = ctx.state(e_ssm)
        entry(f"{label} convolution + silu", device_us(lambda: kernels.conv_silu(
            proj, inner, conv, ssm.conv_w, ssm.conv_b, state, ssm.state_offset + state_floats, ctx.tok_row, ctx.row_first, ctx.row_lens,
            ctx.slots)), nbytes=T * conv * (2 + 4))
        xbc = torch.randn(T, conv, device="cuda")
        us = device_us(lambda: kernels.state_space_scan(xbc, proj, inner + conv, ssm.dt_bias, ssm.a_log, ssm.d_skip, state, ssm.state_offset,
                                                        ctx.row_first, ctx.row_lens, ctx.slots, ss.n_heads, ss.head_dim, ss.state, ss.n_groups,
                                                        chunked=ssm.chunks_pay(ctx.lens)))
        entry(f"{label} state-space recurrence", us, nbytes=T * (conv + inner) * 4 + 2 * B * state_floats * 4)
        out[f"{label} state-space recurrence"]["float32_tflops_per_s"] = 4.0 * inner * ss.state * T / us / 1e6
        y = torch.randn(T, inner, device="cuda")
        entry(f"{label} gate x output, norm over groups", device_us(lambda: kernels.gate_norm(
            y, inner // ss.norm_groups, proj, 0, ssm.norm, ss.norm_eps)), nbytes=T * inner * (4 + 2 + 2))

    slot, ctx = _prompt_context(eng, tokens)
    window, keep = sa.window, sa.keep_first
    seen_biased = sum(min(p + 1, window + min(keep, max(0, p + 1 - window))) for p in range(tokens))
    attention_calls(ctx, tokens, "prefill", seen_biased, tokens * (tokens + 1) / 2)
    kv = ctx.kv(e_att)
    qkv = torch.randn(tokens, att.w_in.shape[0], device="cuda").to(bf)
    entry("prefill unit norm of q and k + cache write", device_us(lambda: kernels.rotary_norm_store(
        qkv, H, G, D, D, None, 0, True, sa.norm_eps, ctx.tok_pos, ctx.tok_row, kv.k, kv.v, kv.table, kv.stride)), nbytes=tokens * (H + 2 * G) * D * 2 * 2)
    kl = ctx.kv(e_lat)
    proj = torch.randn(tokens, lat.w_in.shape[0], device="cuda").to(bf)
    q_out = torch.randn(tokens, H * (rank + R), device="cuda").to(bf)      # (the batched product has written the carried parts there)
    entry("prefill latent norm + rotation + cache write + rotated query parts", device_us(lambda: kernels.latent_prepare(
        proj, H, sl.head_dim, R, rank, q_w, lat.dkv_norm, sl.norm_eps, lat.freq, sl.position.dims, None, ctx.tok_pos, ctx.tok_row, kl.k,
        kl.table, kl.stride, q_out=q_out)), nbytes=tokens * 2 * 2 * (H * R + rank + R))
    o = torch.randn(H, tokens, sl.v_head_dim, device="cuda").to(bf)
    entry("prefill heads x sigmoid gate (head-major in)", device_us(lambda: kernels.head_gate(o, proj, q_w + dkv_w)), nbytes=tokens * H * sl.v_head_dim * 2 * 2)
    state_space_calls(ctx, tokens, 1, "prefill")
    x = torch.randn(tokens, W, device="cuda")
    y = torch.randn(tokens, W, device="cuda")
    folded = layers[e_att].mixer_scale.times(layers[e_att].mixer_norm.weight)
    entry("prefill norm x layer scale into the stream", device_us(lambda: kernels.normed_sum_add(x, [y], [folded], 1e-5, 1.0)), nbytes=tokens * W * 4 * 3)
    E, top = moe.spec.n_experts, moe.spec.top_k
    entry("prefill router + softmax over all + choice of experts", device_us(lambda: kernels.moe_route_stream(
        x, None, 0.0, moe.w_router, E, top, moe._extra(), over_all=True, factor=moe.spec.route_scale)), nbytes=tokens * (W * 4 + (E + 1) * 4))
    I = moe.w_down.shape[1]
    hid = torch.randn(tokens, I, device="cuda").to(bf)
    wts = kernels.moe_route_stream(x, None, 0.0, moe.w_router, E, top, moe._extra(), over_all=True, factor=moe.spec.route_scale)
    entry("prefill relu^2 x expert weight", device_us(lambda: kernels.weighted_act(hid, "relu2", wts, moe.spec.intermediate)), nbytes=tokens * I * 2 * 2)
    if eng.model.pair_table is not None:
        ids = torch.randint(0, VOCAB, (tokens,), device="cuda", dtype=torch.int32)
        prev = torch.zeros(eng.cache.max_seqs + 2, 1, dtype=torch.int32, device="cuda")
        big = eng.model.plan.embedding_pairs
        entry("prefill token rows + bigram rows", device_us(lambda: kernels.embed_pairs(
            eng.model.embedding, eng.model.pair_table, ids, ctx.tok_pos, ctx.tok_row, ctx.row_first, ctx.slots, prev, big.buckets, big.mul_prev,
            big.mul_cur)), nbytes=tokens * W * (2 + 2 + 4))
    eng.cache.close(slot)
    slots, ctx = _decode_context(eng, batch, context)
    attention_calls(ctx, batch, "decode", 0, 0, nbytes_biased=batch * min(context, window + keep) * 2 * G * D * 2,
                    nbytes_latent=batch * context * (rank + R) * 2)
    state_space_calls(ctx, batch, batch, "decode")
    B.close_sequences(eng, slots)


def tenusun_kernel_times(eng, size: str, tokens: int, batch: int, context: int, entry) -> None:
    """The kernels of the Tenusun parts at the sizes of this shape's layers (layers 0 and 2 latent attention + dense feed-forward,
    layers 1 and 3 attention + mixture; layer 3 blends its values with layer 1's)."""
    W, H, G, D, F, L = SIZES[size]
    bf = torch.bfloat16
    layers = eng.model.layers
    e_lat, e_att, e_mix = 0, 1, 3
    lat, att, att2 = layers[e_lat].mixer, layers[e_att].mixer, layers[e_mix].mixer
    dense, moe = layers[e_lat].feed_forward, layers[e_att].feed_forward
    sa, sl = att.spec, lat.spec
    Dv, rank, R = sa.v_head_dim, sl.kv_rank, sl.rot_dim
    q_w, dkv_w, _ = lat._widths()

    def attention_calls(ctx, T, label, seen_all, seen_window, nbytes_plain=None, nbytes_latent=None):
        kv = ctx.kv(e_att)
        qkv = torch.randn(T, att.w_in.shape[0], device="cuda").to(bf)
        how = dict(flops=2.0 * H * (D + Dv) * seen_all) if nbytes_plain is None else dict(nbytes=nbytes_plain)
        entry(f"{label} attention (one added to the denominator)", device_us(lambda: kernels.attention_headmix(
            qkv, qkv.shape[1], H, G, D, Dv, kv.k, kv.v, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, None, sa.scale, att.sink, None, ctx)), **how)
        kl = ctx.kv(e_lat)
        ql = torch.randn(T, H * (rank + R), device="cuda").to(bf)
        how = dict(flops=2.0 * H * (2 * rank + R) * seen_window) if nbytes_latent is None else dict(nbytes=nbytes_latent)
        entry(f"{label} attention over latent rows (window)", device_us(lambda: kernels.attention_headmix(
            ql, ql.shape[1], H, 1, rank + R, rank, kl.k, None, kl.table, kl.stride, ctx.tok_pos, ctx.tok_row, sl.window, sl.scale, None, None, ctx,
            values_in_keys=True)), **how)

    slot, ctx = _prompt_context(eng, tokens)
    window = sl.window or tokens
    attention_calls(ctx, tokens, "prefill", tokens * (tokens + 1) / 2, sum(min(p + 1, window) for p in range(tokens)))
    kv = ctx.kv(e_mix)
    qkv = torch.randn(tokens, att2.w_in.shape[0], device="cuda").to(bf)
    other = torch.randn(tokens, att.w_in.shape[0], device="cuda").to(bf)[:, (H + G) * D:(H + G) * D + G * Dv]
    entry("prefill rotation of halves + blended values + cache write", device_us(lambda: kernels.rotary_half_store(
        qkv, H, G, D, Dv, att2.freq, sa.position.dims, att2.magnitude, False, sa.norm_eps, ctx.tok_pos, ctx.tok_row, kv.k, kv.v, kv.table, kv.stride,
        other, att2.blend_weight)), nbytes=tokens * ((H + G) * D * 2 * 2 + G * D * 2 + G * Dv * 2 * 4))
    a = torch.randn(tokens, H * Dv, device="cuda").to(bf)
    entry("prefill heads x sigmoid(gate)", device_us(lambda: kernels.gated_norm(a, 0, None, sa.norm_eps, qkv, (H + G) * D + G * Dv, "sigmoid", bf)),
          nbytes=tokens * H * Dv * 2 * 3)
    kl = ctx.kv(e_lat)
    proj = torch.randn(tokens, lat.w_in.shape[0], device="cuda").to(bf)
    entry("prefill norm of the query row", device_us(lambda: kernels.rmsnorm_cols(proj, 0, sl.q_rank, lat.dq_norm, sl.norm_eps)), nbytes=tokens * sl.q_rank * 2 * 2)
    q_rows = torch.randn(tokens, H * (sl.head_dim + R), device="cuda").to(bf)
    q_out = torch.randn(tokens, H * (rank + R), device="cuda").to(bf)      # (the batched product has written the carried parts there)
    entry("prefill latent norm + rotation + cache write + rotated query parts", device_us(lambda: kernels.latent_prepare(
        proj, H, sl.head_dim, R, rank, q_w, lat.dkv_norm, sl.norm_eps, lat.freq, sl.position.dims, None, ctx.tok_pos, ctx.tok_row, kl.k,
        kl.table, kl.stride, halves=True, q_rows=q_rows, q_out=q_out)), nbytes=tokens * 2 * 2 * (H * R + rank + R))
    x = torch.randn(tokens, W, device="cuda")
    y = torch.randn(tokens, W, device="cuda")
    n1, n2 = layers[e_lat].mixer_out_norm, layers[e_lat].feed_forward_norm
    entry("prefill output norm into the stream + next norm", device_us(lambda: kernels.layernorm_add(
        x, y, n1.weight, n1.bias, n1.eps, (n2.weight, n2.bias, n2.eps), bf)), nbytes=tokens * W * (4 * 3 + 2))
    gu = torch.randn(tokens, 2 * F, device="cuda").to(bf)
    entry("prefill clamped gate x (up + 1)", device_us(lambda: kernels.gated_act(gu, "clamped_sigmoid", limit=dense.spec.limit, alpha=dense.spec.alpha)),
          nbytes=tokens * F * 2 * 3)
    E, top = moe.spec.n_experts, moe.spec.top_k
    h = torch.randn(tokens, W, device="cuda").to(bf)
    n3 = layers[e_att].feed_forward_norm
    entry("prefill layer norm + router + sigmoid scores + choice among groups", device_us(lambda: kernels.moe_route_stream_grouped(
        x, n3.weight, n3.bias, n3.eps, moe.w_router, E, top, moe.correction, moe.spec.n_groups, moe.spec.keep_groups, moe.spec.group_best,
        moe.spec.route_scale)), nbytes=tokens * (W * 4 + E * 4))
    I = moe.w_down.shape[1]
    gum = torch.randn(tokens, 2 * I, device="cuda").to(bf)
    wts = moe.routing(h)
    entry("prefill silu(gate) x up x expert weight", device_us(lambda: kernels.gated_act(gum, "silu", wts, moe.spec.intermediate)), nbytes=tokens * I * 2 * 3)
    ids = torch.randint(0, VOCAB, (tokens,), device="cuda", dtype=torch.int32)
    entry("prefill token rows x scale", device_us(lambda: kernels.embed(eng.model.embedding, ids, scale=eng.model.plan.embedding_scale)), nbytes=tokens * W * (2 + 4))
    eng.cache.close(slot)
    slots, ctx = _decode_context(eng, batch, context)
    attention_calls(ctx, batch, "decode", 0, 0, nbytes_plain=batch * context * G * (D + Dv) * 2,
                    nbytes_latent=batch * min(context, window) * (rank + R) * 2)
    B.close_sequences(eng, slots)


def kernel_times(size: str, tokens: int, batch: int, context: int, peaks: dict, design: str = "mebalorn") -> Dict[str, dict]:
    """Every kernel of the new design beside the like kernel of the Qwen2 decoder: microseconds, the bytes or
    multiply-adds it must move or do, and that as a fraction of the measured peak."""
    from .engine.engine import Engine
    W, H, G, D, F, L = SIZES[size]
    out: Dict[str, dict] = {}
    bf = torch.bfloat16

    def entry(name, us, nbytes=None, flops=None):
        rec = {"us": us}
        if nbytes is not None:
            rec.update(gbytes_per_s=nbytes / us / 1e3, frac=nbytes / us / 1e3 / peaks["hbm_gbs"], bound="hbm")
        if flops is not None:
            rec.update(tflops_per_s=flops / us / 1e6, frac=flops / us / 1e6 / peaks["bf16_tflops"], bound="bf16")
        out[name] = rec

    entry.out = out
    # (the kernels of the Kevelorn parts are timed in a model of three layers, which has every kind of part once)
    first = kevelorn_config(size, 3) if design == "kevelorn" else DESIGNS[design](size)
    runs = [(design, first), ("qwen2", qwen2_config(size))]
    if design == "tenusun":                                  # its kernels also beside the like kernels of Pupidra
        runs.insert(1, ("pupidra beside", pupidra_config(size)))
    for design, cfg in runs:
        if design in ("pupidra", "pupidra beside", "tenusun"):
            eng = Engine.from_config(config_from_dict(cfg), seed=1, draw_on="cuda", dtype="bfloat16")
            eng.ensure_cache(max(tokens, batch * context) + 64 * batch, max(tokens, context), max_seqs=batch + 1)
            if design == "tenusun":
                tenusun_kernel_times(eng, size, tokens, batch, context, entry)
            elif design == "pupidra":
                pupidra_kernel_times(eng, size, tokens, batch, context, entry)
            else:
                pupidra_kernel_times(eng, size, tokens, batch, context, _prefixed(entry, out))
            kernels.check_status(eng.device)
            del eng
            torch.cuda.empty_cache()
            continue
        eng = Engine.from_config(config_from_dict(cfg), seed=1, draw_on="cuda", dtype="bfloat16")
        eng.ensure_cache(max(tokens, batch * context) + 64 * batch, max(tokens, context), max_seqs=batch + 1)
        if design == "kevelorn":
            kevelorn_kernel_times(eng, size, tokens, batch, context, entry)
            kernels.check_status(eng.device)
            del eng
            torch.cuda.empty_cache()
            continue
        e_att = next(e for e, s in enumerate(eng.model.plan.schedule) if hasattr(eng.model.layers[s.layer].mixer.spec, "n_heads"))
        att = eng.model.layers[e_att].mixer
        seen = tokens * (tokens + 1) / 2
        # ---- a prompt of `tokens`
        slot, ctx = _prompt_context(eng, tokens)
        kv = ctx.kv(e_att)
        x = torch.randn(tokens, W, device="cuda")
        qkv = torch.randn(tokens, (H + 2 * G) * D, device="cuda").to(bf)
        if design == "mebalorn":
            layer = eng.model.layers[e_att]
            state = ctx.state(e_att)
            halves = [(n.weight, n.bias, f.taps_weight, o) for n, f, o in zip((layer.mixer_norm, layer.feed_forward_norm),
                      (layer.mixer_input, layer.feed_forward_input), layer.state_offsets())]
            entry("prefill norm+conv, both halves", device_us(lambda: kernels.dual_layernorm_conv(
                x, halves, 1e-6, state, ctx.tok_row, ctx.row_first, ctx.row_lens, ctx.slots, bf, False)), nbytes=tokens * W * (4 + 2 * 2))
            entry("prefill attention (mixed heads)", device_us(lambda: kernels.attention_headmix(
                qkv, qkv.shape[1], H, G, D, D, kv.k, kv.v, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, None, D ** -0.5, att.sink,
                att.head_mix, ctx)), flops=4.0 * H * D * seen)
            e_rec = next(e for e, s in enumerate(eng.model.plan.schedule) if not hasattr(eng.model.layers[s.layer].mixer.spec, "n_heads"))
            proj = torch.randn(tokens, 3 * W, device="cuda").to(bf)
            entry("prefill recurrence", device_us(lambda: kernels.mingru(proj, ctx.state(e_rec), 0, ctx.tok_row, ctx.row_first, ctx.row_lens,
                                                                        ctx.slots, chunked=True)), nbytes=tokens * W * 2 * 4)
            up = torch.randn(tokens, F, device="cuda").to(bf)
            entry("prefill relu^2", device_us(lambda: kernels.activation(up, "relu2", out=up)), nbytes=tokens * F * 2 * 2)
            entry("prefill q/k norm + cache write", device_us(lambda: kernels.qknorm_store(
                qkv, H, G, D, D, att.q_norm, att.k_norm, 1e-6, ctx.tok_pos, ctx.tok_row, kv.k, kv.v, kv.table, kv.stride)),
                nbytes=tokens * (H + 2 * G) * D * 2 * 2)
        else:
            norm = eng.model.layers[0].mixer_norm
            entry("qwen2 prefill rmsnorm, twice", device_us(lambda: (kernels.rmsnorm(x, norm.weight, 1e-6, bf), kernels.rmsnorm(x, norm.weight, 1e-6, bf))),
                  nbytes=tokens * W * 2 * (4 + 2))
            entry("qwen2 prefill attention", device_us(lambda: kernels.attention(
                qkv, qkv.shape[1], H, G, D, kv.k, kv.v, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, None, D ** -0.5, ctx)),
                flops=4.0 * H * D * seen)
            gu = torch.randn(tokens, 2 * F, device="cuda").to(bf)
            entry("qwen2 prefill swiglu", device_us(lambda: kernels.swiglu(gu)), nbytes=tokens * F * 2 * 3)
            cos, sin = att._tables(ctx)
            entry("qwen2 prefill rope + cache write", device_us(lambda: kernels.rope_store(
                qkv, H, G, D, cos, sin, ctx.tok_pos, ctx.tok_row, kv.k, kv.v, kv.table, kv.stride)), nbytes=tokens * (H + 2 * G) * D * 2 * 2)
        eng.cache.close(slot)
        # ---- a step of `batch` single tokens at `context`
        slots, ctx = _decode_context(eng, batch, context)
        kv = ctx.kv(e_att)
        q1 = torch.randn(batch, (H + 2 * G) * D, device="cuda").to(bf)
        kv_bytes = batch * context * 2 * G * D * 2
        if design == "mebalorn":
            entry("decode attention (mixed heads)", device_us(lambda: kernels.attention_headmix(
                q1, q1.shape[1], H, G, D, D, kv.k, kv.v, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, None, D ** -0.5, att.sink,
                att.head_mix, ctx)), nbytes=kv_bytes)
        else:
            entry("qwen2 decode attention", device_us(lambda: kernels.attention(
                q1, q1.shape[1], H, G, D, kv.k, kv.v, kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, None, D ** -0.5, ctx)), nbytes=kv_bytes)
        B.close_sequences(eng, slots)
        kernels.check_status(eng.device)
        del eng, ctx, kv
        torch.cuda.empty_cache()
    return out


class _prefixed:
    """``entry`` under names that begin with "pupidra ": the like kernels of another design in the same record."""

    def __init__(self, entry, out):
        self.entry, self.out = entry, _PrefixedDict(out)

    def __call__(self, name, us, nbytes=None, flops=None):
        self.entry("pupidra " + name, us, nbytes, flops)


class _PrefixedDict:
    def __init__(self, out):
        self._out = out

    def __getitem__(self, name):
        return self._out["pupidra " + name]


def throughput(size: str, tokens: int, batch: int, context: int, steps: int = 64, design: str = "mebalorn") -> Dict[str, dict]:
    """Prefill of one prompt and decode of ``batch`` sequences through the engines' own steps, both designs (for Tenusun also Pupidra)."""
    from .engine.engine import Engine
    out = {}
    n_layers = max(SIZES[size][5], 4) if design in FOUR_LAYERS else None    # the same number of layers on both sides
    runs = [(design, DESIGNS[design](size)), ("qwen2", qwen2_config(size, n_layers))]
    if design == "tenusun":
        runs.insert(1, ("pupidra", pupidra_config(size)))
    for design, cfg in runs:
        eng = Engine.from_config(config_from_dict(cfg), seed=1, draw_on="cuda", dtype="bfloat16")
        pre = B.prefill_device(eng, tokens)
        dec = B.decode_device(eng, batch, context, steps, 4)
        out[design] = {"prefill_tokens_per_s": pre["tokens_per_s"], "prefill_ms": pre["ms"], "prefill_tflops_per_s": pre["tflops_per_s"],
                       "decode_tokens_per_s": dec["tokens_per_s"], "decode_ms_per_step": dec["ms_per_step"],
                       "decode_gbytes_per_s": dec["gbytes_per_s"], "decode_launches_per_step": dec["launches_per_step"],
                       "weight_bytes": eng.model.step_weight_bytes()}
        del eng
        torch.cuda.empty_cache()
    return out


def compare(sizes, tokens: int, batch: int, context: int, peaks: dict, design: str = "mebalorn") -> dict:
    record = {"tokens": tokens, "batch": batch, "context": context,
              "layers": {s: max(SIZES[s][5], 4) if design in FOUR_LAYERS else SIZES[s][5] for s in sizes},
              "widths": {s: dict(zip(("width", "heads", "kv_heads", "head_dim", "ff"), SIZES[s][:5])) for s in sizes}, "sizes": {}}
    for s in sizes:
        record["sizes"][s] = {"throughput": throughput(s, tokens, batch, context, design=design),
                              "kernels": kernel_times(s, tokens, batch, context, peaks, design)}
    return record


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--design", default="mebalorn", choices=sorted(DESIGNS))
    p.add_argument("--sizes", default="s,m")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--hbm-gbs", type=float, default=6650.0)
    p.add_argument("--bf16-tflops", type=float, default=1590.0)
    p.add_argument("--output")
    a = p.parse_args(argv)
    rec = compare([s for s in a.sizes.split(",") if s], a.tokens, a.batch, a.context, {"hbm_gbs": a.hbm_gbs, "bf16_tflops": a.bf16_tflops}, a.design)
    for s, r in rec["sizes"].items():
        for d, t in r["throughput"].items():
            print(f"{s} {d}: prefill {t['prefill_tokens_per_s']:.0f} tok/s ({t['prefill_ms']:.2f} ms), decode {t['decode_tokens_per_s']:.0f} tok/s "
                  f"({t['decode_ms_per_step']:.3f} ms a step, {t['decode_launches_per_step']} launches)")
        for k, t in r["kernels"].items():
            print(f"{s} {k}: {t['us']:.1f} us, {t['frac']:.3f} of the {t['bound']} peak")
    if a.output:
        with open(a.output, "w") as f:
            json.dump(rec, f, indent=1)


if __name__ == "__main__":
    main()
