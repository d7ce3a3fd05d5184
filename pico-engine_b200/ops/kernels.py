"""One Python function per CUDA kernel: argument checks, then the launch on torch's current
stream.  Tensors are passed as raw device pointers; outputs are allocated by the caller or
here with torch's allocator.  There is no other implementation behind these functions.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .library import DTYPE_CODE, KernelError, check, core, extras, gated, mixers, stream_ptr

PAGE = 64     # tokens per cache page; PE_PAGE in csrc/common.cuh


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    # the passing case first and cheaply: these checks run a few hundred times a step
    if (t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype)
            and (shape is None or t.shape == shape or tuple(t.shape) == tuple(shape))):
        return
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, not {t.dtype}")
    raise KernelError(f"{name} must have shape {tuple(shape)}, not {tuple(t.shape)}")


def _code(t: torch.Tensor, name: str) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{name} must be float32 or bfloat16, not {t.dtype}") from None


def embed(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """Rows ``ids`` (int32, [T]) of ``table`` [V, H] as float32 [T, H], multiplied by ``scale``."""
    V, H = table.shape
    T = ids.shape[0]
    _need(table, "table"); _need(ids, "ids", torch.int32, (T,))
    if out is None:
        out = torch.empty(T, H, dtype=torch.float32, device=table.device)
    _need(out, "out", torch.float32, (T, H))
    check(core().pe_embed(table.data_ptr(), _code(table, "table"), ids.data_ptr(), out.data_ptr(), T, H, V,
                          float(scale), stream_ptr()), "embed")
    return out


def select_tokens(ids: torch.Tensor, prev: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``ids[j] = prev[src[j]]`` where ``src[j] >= 0`` (all int32, on the device): the ids of rows whose
    token the step before chose and the host has not read yet."""
    n = ids.shape[0]
    _need(ids, "ids", torch.int32, (n,)); _need(prev, "prev", torch.int32); _need(src, "src", torch.int32, (n,))
    check(core().pe_select_tokens(ids.data_ptr(), prev.data_ptr(), src.data_ptr(), n, stream_ptr()), "select_tokens")
    return ids


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows_index: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows [T, H]; with ``rows_index`` (int32 [R]) only of those rows."""
    T, H = x.shape
    _need(x, "x", torch.float32); _need(weight, "weight", None, (H,))
    rows = T if rows_index is None else rows_index.shape[0]
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32)
    if out is None:
        out = torch.empty(rows, H, dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype, (rows, H))
    check(core().pe_rmsnorm(x.data_ptr(), _ptr(rows_index), weight.data_ptr(), _code(weight, "weight"), float(eps),
                            out.data_ptr(), _code(out, "out"), rows, H, stream_ptr()), "rmsnorm")
    return out


def add_rmsnorm(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += y (float32 rows [T, H], in place), then RMSNorm of every row: the residual sum and the
    norm that follows it in one pass over the stream."""
    T, H = x.shape
    _need(x, "x", torch.float32); _need(y, "y", None, (T, H)); _need(weight, "weight", None, (H,))
    if out is None:
        out = torch.empty(T, H, dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype, (T, H))
    check(core().pe_add_rmsnorm(x.data_ptr(), y.data_ptr(), _code(y, "y"), weight.data_ptr(), _code(weight, "weight"),
                                float(eps), out.data_ptr(), _code(out, "out"), T, H, stream_ptr()), "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate) * up of [T, 2I] (gate first) as [T, I]."""
    T, I2 = gate_up.shape
    _need(gate_up, "gate_up")
    if I2 % 2:
        raise KernelError("gate_up needs an even number of columns")
    if out is None:
        out = torch.empty(T, I2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _need(out, "out", gate_up.dtype, (T, I2 // 2))
    check(core().pe_swiglu(gate_up.data_ptr(), out.data_ptr(), _code(gate_up, "gate_up"), T, I2 // 2, stream_ptr()),
          "swiglu")
    return out


def residual_add(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x += y in float32; x is the float32 residual stream."""
    _need(x, "x", torch.float32); _need(y, "y", None, x.shape)
    check(core().pe_residual_add(x.data_ptr(), y.data_ptr(), _code(y, "y"), x.numel(), stream_ptr()), "residual_add")
    return x


def bias_add(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    M, N = y.shape
    _need(y, "y"); _need(bias, "bias", None, (N,))
    check(core().pe_bias_add(y.data_ptr(), _code(y, "y"), bias.data_ptr(), _code(bias, "bias"), M, N, stream_ptr()),
          "bias_add")
    return y


def rope_store(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int, cos: Optional[torch.Tensor],
               sin: Optional[torch.Tensor], tok_pos: torch.Tensor, tok_row: torch.Tensor,
               k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
               table_stride: int) -> None:
    """Rotate the query and key heads of ``qkv`` [T, (n_q + 2 n_kv) * head_dim] in place and
    write keys and values to the cache pages of their sequences (skipped when ``k_pool`` is None)."""
    T = qkv.shape[0]
    _need(qkv, "qkv", None, (T, (n_q + 2 * n_kv) * head_dim))
    _need(tok_pos, "tok_pos", torch.int32); _need(tok_row, "tok_row", torch.int32)
    if cos is not None:
        _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32, cos.shape)
        if cos.shape[1] != head_dim // 2:
            raise KernelError("cos/sin tables need head_dim/2 columns")
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype, k_pool.shape)
        _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim):
            raise KernelError(f"cache pool must be [pages, {n_kv}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    check(core().pe_rope_store(qkv.data_ptr(), _code(qkv, "qkv"), T, n_q, n_kv, head_dim, _ptr(cos), _ptr(sin),
                               tok_pos.data_ptr(), tok_row.data_ptr(), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                               table_stride, 1 if store else 0, stream_ptr()), "rope_store")


_EPILOGUE_STORE = {torch.float32: 0, torch.bfloat16: 1}


def linear_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, accumulate_into: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T (+ bias) with float32 multiply-adds.  Either stored as
    ``out_dtype`` or added into the float32 tensor ``accumulate_into`` [M, N]."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a"); _need(w, "w", None, (N, K))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    if accumulate_into is not None:
        _need(accumulate_into, "accumulate_into", torch.float32, (M, N))
        out, epilogue = accumulate_into, 2
    else:
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        _need(out, "out", None, (M, N))
        epilogue = _EPILOGUE_STORE[out.dtype]
    check(core().pe_linear_simt(a.data_ptr(), _code(a, "a"), w.data_ptr(), _code(w, "w"), _ptr(bias),
                                0 if bias is None else _code(bias, "bias"), out.data_ptr(), epilogue, M, N, K,
                                stream_ptr()), "linear_simt")
    return out


def attention_generic(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                      tok_pos: torch.Tensor, tok_row: torch.Tensor, window: Optional[int], scale: float,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of T tokens over the cache.  ``q`` holds the query heads of token t at
    ``t * q_stride + h * head_dim``; the result is [T, n_heads * head_dim] in q's dtype."""
    T = tok_pos.shape[0]
    _need(q, "q"); _need(k_pool, "k_pool", q.dtype); _need(v_pool, "v_pool", q.dtype, k_pool.shape)
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pool must be [pages, {n_kv_heads}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    _need(block_table, "block_table", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32, (T,)); _need(tok_row, "tok_row", torch.int32, (T,))
    if out is None:
        out = torch.empty(T, n_heads * head_dim, dtype=q.dtype, device=q.device)
    _need(out, "out", q.dtype, (T, n_heads * head_dim))
    check(core().pe_attention_generic(q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                      _code(q, "q"), block_table.data_ptr(), table_stride, tok_pos.data_ptr(),
                                      tok_row.data_ptr(), T, n_heads, n_kv_heads, head_dim, window or 0, float(scale),
                                      stream_ptr()), "attention_generic")
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    B, V = logits.shape
    _need(logits, "logits", torch.float32)
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, (B,))
    from .workspace import scratch
    lib = core()
    ws = scratch("argmax.partial", lib.pe_argmax_scratch_bytes(B, V), logits.device)
    check(lib.pe_argmax(logits.data_ptr(), out.data_ptr(), B, V, ws.data_ptr(), stream_ptr()), "argmax", 2)
    return out


def sample_settings_words(temperature: float, top_k: int, top_p: float, seed: int):
    """The six int32 words of the sampler's settings as the kernels read them from device memory."""
    import struct
    return list(struct.unpack("<6i", struct.pack("<fifiQ", float(temperature), int(top_k), float(top_p), 0,
                                                 int(seed) & ((1 << 64) - 1))))


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, request: torch.Tensor,
           step: torch.Tensor, out: Optional[torch.Tensor] = None, settings: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One draw per row of float32 logits [B, V]; row b uses the uniform of (seed, request[b], step[b]).
    ``settings`` (int32 [6] on the device, ``sample_settings_words``): where given, the kernels read
    temperature, top_k, top_p and the seed from there at run time (a captured launch then follows settings
    that change); the arguments still decide which passes run, i.e. whether there is a cut by rank and by mass."""
    B, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(request, "request", torch.int32, (B,)); _need(step, "step", torch.int32, (B,))
    if not temperature > 0:
        raise KernelError("sample needs a positive temperature; use argmax for greedy choice")
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, (B,))
    from .workspace import scratch
    lib = core()
    ws = scratch("sample.state", lib.pe_sample_scratch_bytes(B, V), logits.device, zeroed=True)
    cut_k, cut_p = 0 < top_k < V, top_p < 1.0
    if settings is not None:
        _need(settings, "settings", torch.int32, (6,))
        if settings.data_ptr() % 8:
            raise KernelError("settings must start on an 8-byte boundary")
    check(lib.pe_sample(logits.data_ptr(), out.data_ptr(), B, V, float(temperature), int(top_k), float(top_p),
                        int(seed) & ((1 << 64) - 1), request.data_ptr(), step.data_ptr(), ws.data_ptr(), _ptr(settings),
                        stream_ptr()),
          "sample", 2 + 3 * cut_k + 3 * cut_p)
    return out


def draw_uniform(seed: int, request: int, step: int) -> float:
    """The uniform the sampling kernel uses for (seed, request, step), computed on the host."""
    m = (1 << 64) - 1
    return float(core().pe_draw_uniform(seed & m, request & m, step & m))


# ---------------------------------------------------------------------------- tensor-core kernels (bfloat16)

def linear_mma_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes these operands (else another one is used)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] <= 64 and a.shape[1] % 8 == 0
            and a.is_contiguous() and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear_mma(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None, accumulate_into: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M <= 64, K] . w [N, K]^T (+ bias), bfloat16 operands, float32 accumulation on the
    tensor cores; stored as ``out_dtype`` or added into float32 ``accumulate_into``."""
    from .workspace import scratch
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16, (N, K))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    if accumulate_into is not None:
        _need(accumulate_into, "accumulate_into", torch.float32, (M, N))
        out, epilogue = accumulate_into, 2
    else:
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        _need(out, "out", None, (M, N))
        epilogue = _EPILOGUE_STORE[out.dtype]
    lib = extras()
    partial = tickets = None
    if lib.pe_linear_mma_splits(N, K) > 1:
        partial = scratch("linear_mma.partial", lib.pe_linear_mma_scratch_bytes(64, N, K), a.device).data_ptr()
        tickets = scratch("linear_mma.tickets", 4 * ((N + 15) // 16), a.device, zeroed=True).data_ptr()
    check(lib.pe_linear_mma(a.data_ptr(), w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"),
                            out.data_ptr(), epilogue, M, N, K, partial, tickets, stream_ptr()), "linear_mma")
    return out


def attention_decode(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int,
                     k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                     tok_pos: torch.Tensor, tok_row: torch.Tensor, window: Optional[int], scale: float,
                     max_context: int, out: Optional[torch.Tensor] = None, early_pages: bool = True, keep_first: int = 0,
                     slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of T single tokens (bfloat16) over the cache; ``max_context`` bounds every
    token's position + 1 and fixes the launch shape.  ``keep_first``: with a window, a sequence's first so many keys stay
    visible.  ``slopes`` float32 [H]: slope_h * (i - j) is taken off the score of query i and key j.  ``sinks`` float32 [H]: one more place of
    score sinks[h] joins every softmax denominator of head h and carries no value.  With ``early_pages`` the kernel copies cache pages
    while the two kernels before it on the stream may still run: they must have written keys and values
    at each token's own position only (the library's own parts do).  A part that rewrites other cache
    rows shortly before attending passes False: the kernel then starts when everything before it has ended."""
    from .library import for_head_dim
    T = tok_pos.shape[0]
    _need(q, "q", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pool must be [pages, {n_kv_heads}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    _need(block_table, "block_table", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32, (T,)); _need(tok_row, "tok_row", torch.int32, (T,))
    if out is None:
        out = torch.empty(T, n_heads * head_dim, dtype=torch.bfloat16, device=q.device)
    _need(out, "out", torch.bfloat16, (T, n_heads * head_dim))
    lib = for_head_dim(head_dim)
    check(lib.pe_attention_decode(q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                  block_table.data_ptr(), table_stride, tok_pos.data_ptr(), tok_row.data_ptr(), T,
                                  n_heads, n_kv_heads, head_dim, window or 0, float(scale), int(max_context),
                                  1 if early_pages else 0, status_ptr(q.device), stream_ptr(), int(keep_first) if window else 0,
                                  _ptr(slopes), _ptr(sinks)), "attention_decode")
    return out


PREFILL_TILE = 64             # AP_QTILE of csrc/attention_prefill.cu
PREFILL_TILE_TCGEN05 = 128    # AT_QTILE of csrc/attention_prefill_tcgen05.cu
TCGEN05_HEAD_DIMS = (64, 128)


def prefill_tile_rows(lens, starts, tile: int = PREFILL_TILE):
    """[(batch row, first packed token, tokens, position of the first token), ...]: the packed tokens of a
    step cut into runs of at most ``tile`` tokens of one sequence, the runs that see the most keys first
    (they take longest, so they are scheduled first)."""
    rows = []
    tok = 0
    for b, (n, st) in enumerate(zip(lens, starts)):
        for off in range(0, n, tile):
            rows.append((b, tok + off, min(tile, n - off), st + off))
        tok += n
    rows.sort(key=lambda r: -(r[3] + r[2]))
    return rows


def prefill_tiles(lens, starts, device, tile: int = PREFILL_TILE) -> torch.Tensor:
    """``prefill_tile_rows`` as int32 [tiles, 4] on ``device``."""
    return torch.tensor(prefill_tile_rows(lens, starts, tile), dtype=torch.int32).to(device, non_blocking=True)


def _prefill_args(q, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, tiles, n_tokens, out):
    _need(q, "q", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pool must be [pages, {n_kv_heads}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    _need(block_table, "block_table", torch.int32); _need(tiles, "tiles", torch.int32)
    if out is None:
        out = torch.empty(n_tokens, n_heads * head_dim, dtype=torch.bfloat16, device=q.device)
    _need(out, "out", torch.bfloat16, (n_tokens, n_heads * head_dim))
    return out


def attention_prefill(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                      tiles: torch.Tensor, n_tokens: int, window: Optional[int], scale: float,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention (bfloat16) of the token runs ``tiles`` (of at most 64 tokens) over the cache:
    the mma.sync kernel, which takes every head size."""
    from .library import for_head_dim
    out = _prefill_args(q, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, tiles, n_tokens, out)
    check(for_head_dim(head_dim).pe_attention_prefill(
        q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
        table_stride, tiles.data_ptr(), None, None, tiles.shape[0], n_heads, n_kv_heads, head_dim, window or 0,
        float(scale), stream_ptr()), "attention_prefill")
    return out


def attention_prefill_tcgen05_takes(head_dim: int, scale: float) -> bool:
    return head_dim in TCGEN05_HEAD_DIMS and scale > 0


def attention_prefill_tcgen05(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int,
                              k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                              tiles: torch.Tensor, n_tokens: int, window: Optional[int], scale: float,
                              out: Optional[torch.Tensor] = None, keep_first: int = 0,
                              slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same on the tcgen05 tensor cores, for head sizes 64 and 128 and runs ``tiles`` of at most
    128 tokens.  ``q`` is a view of ``n_tokens`` rows, ``q_stride`` elements apart.  ``keep_first``: with a window, the first so
    many keys of a sequence stay visible.  ``slopes`` float32 [heads]: slope_h * (i - j) is taken off the score of query i and
    key j.  ``sinks`` float32 [heads]: one more place of score sinks[h] joins every softmax denominator of head h and carries no value."""
    from .library import for_head_dim
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, (n_heads,))
    out = _prefill_args(q, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, tiles, n_tokens, out)
    check(for_head_dim(head_dim).pe_attention_prefill_tcgen05(
        q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0], block_table.data_ptr(),
        table_stride, tiles.data_ptr(), tiles.shape[0], n_tokens, n_heads, n_kv_heads, head_dim, window or 0,
        float(scale), keep_first if window else 0, _ptr(slopes), status_ptr(q.device), stream_ptr(), _ptr(sinks)), "attention_prefill_tcgen05")
    return out


def attention(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int, k_pool: torch.Tensor,
              v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int, tok_pos: torch.Tensor,
              tok_row: torch.Tensor, window: Optional[int], scale: float, ctx, own_rows_only: bool = True) -> torch.Tensor:
    """Attention of the step's tokens over the cache, with the kernel the step calls for:
    bfloat16 uses the tensor-core kernels (single tokens: decode; longer runs: prefill),
    float32 the float32 kernel.  ``own_rows_only``: the kernels launched just before wrote no cache row
    but each token's own (see ``attention_decode``); a caller that cannot promise this passes False."""
    if q.dtype == torch.bfloat16:
        if ctx.one_token_each:
            return attention_decode(q, q_stride, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table,
                                    table_stride, tok_pos, tok_row, window, scale, ctx.max_context,
                                    early_pages=own_rows_only)
        tcgen05 = attention_prefill_tcgen05_takes(head_dim, scale)
        name = "prefill_tiles_128" if tcgen05 else "prefill_tiles"
        tiles = ctx.scratch.get(name)
        if tiles is None:
            tiles = ctx.scratch[name] = prefill_tiles(ctx.lens, ctx.starts, q.device,
                                                      PREFILL_TILE_TCGEN05 if tcgen05 else PREFILL_TILE)
        run = attention_prefill_tcgen05 if tcgen05 else attention_prefill
        return run(q, q_stride, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, table_stride, tiles,
                   tok_pos.shape[0], window, scale)
    return attention_generic(q, q_stride, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, table_stride,
                             tok_pos, tok_row, window, scale)


# ---------------------------------------------------------------------------- fused decode products (bfloat16, up to 16 rows)

FUSED_MAX_ROWS = 16


_status_words = {}


def status_word(device) -> torch.Tensor:
    """The int32 word in which a kernel records that a bounded wait of its own ran out (0: none did)."""
    word = _status_words.get(device)
    if word is None:
        from .workspace import scratch
        word = _status_words[device] = scratch("status", 4, torch.device(device), zeroed=True)[:4].view(torch.int32)
        _status_ptrs[device] = word.data_ptr()
    return word


_status_ptrs = {}


def status_ptr(device) -> int:
    """The address of ``status_word(device)``."""
    ptr = _status_ptrs.get(device)
    if ptr is None:
        ptr = status_word(device).data_ptr()
    return ptr


def check_status(device) -> None:
    """Raise if a kernel gave up waiting for its own copies since the last check.  Synchronises."""
    word = status_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        raise KernelError(f"a kernel gave up a bounded wait (status {code}); its results are incomplete")


# A weight this large streams faster through the library's product even for a few rows: measured on a B200 at
# 8 rows, 37888 x 3584 (271 MB): 46 us (5.9 TB/s) against 61 us; 3584 x 18944 (136 MB): 28 us against 33 us;
# 151936 x 896 (272 MB, into float32): 52 us against 72 us.  The fused kernel's CTAs restart their pipeline
# for every tile; smaller weights are faster there, with what precedes and follows the product fused in.
FUSED_MAX_WEIGHT_BYTES = int(os.environ.get("PICO_ENGINE_FUSED_MAX_MB", "100")) << 20


def fused_takes(rows: int, w: torch.Tensor, *others: torch.Tensor, max_rows: int = FUSED_MAX_ROWS) -> bool:
    """Whether the fused decode kernels take a product with ``rows`` rows and weight ``w``."""
    return (rows <= max_rows and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0 and all(t.is_contiguous() and t.data_ptr() % 16 == 0 for t in others)
            and w.numel() * 2 <= FUSED_MAX_WEIGHT_BYTES)


# The same fused products for 17 to 64 rows are another kernel (csrc/linear_batch.cu: 64 rows of the weight a CTA
# instead of 16, operands through shared memory by TMA); the three functions below take either number of rows.
# It is not what a decode step of that many rows runs unless PICO_ENGINE_BATCH_FUSED=1: measured on a B200 at the
# Qwen2.5-0.5B widths and 64 rows, in captured graphs, norm + q/k/v + rotation take 10.9 us in it against 7.5 us as
# three kernels around the library's product, the output projection 6.5 against 5.3, norm + gate/up + SwiGLU 25.6
# against 9.1, the down projection 9.7 against 10.1; at the 7B widths it streams weights at 1.2 to 2.1 TB/s where
# the library reaches 4 to 5.  Two things bound it: mma.sync runs at about a quarter of the tcgen05 rate (1,000
# cycles for a chunk of 128 columns), and every CTA converts the float32 rows of the residual stream itself, which
# for gate/up (152 CTAs x 229 KB) is all the L2 delivers.
BATCH_MAX_ROWS = 64
BATCH_ENABLED = os.environ.get("PICO_ENGINE_BATCH_FUSED", "0") == "1"


def decode_fused_takes(rows: int, w: torch.Tensor, *others: torch.Tensor) -> bool:
    """Whether a decode step of ``rows`` sequences can run this product fused with its neighbours."""
    return fused_takes(rows, w, *others, max_rows=BATCH_MAX_ROWS if BATCH_ENABLED else FUSED_MAX_ROWS)


def set_batch_fused(on: bool) -> bool:
    """Let decode steps of 17 to 64 rows run the fused products of csrc/linear_batch.cu (or not); returns what was set."""
    global BATCH_ENABLED
    was, BATCH_ENABLED = BATCH_ENABLED, bool(on)
    return was


def linear_fused(a: Optional[torch.Tensor], w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, accumulate_into: Optional[torch.Tensor] = None,
                 norm_of: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                 eps: float = 0.0, scale: float = 1.0) -> torch.Tensor:
    """a [M <= 64, K] . w [N, K]^T (+ bias); with ``norm_of`` (float32 [M, K]) the operand is
    RMSNorm(norm_of) with ``norm_weight`` instead of ``a``.  (More than 16 rows: bfloat16 or accumulated results.)
    ``scale`` (up to 16 rows, with ``accumulate_into``): accumulate_into += scale * product."""
    src = norm_of if norm_of is not None else a
    M, K = src.shape
    N = w.shape[0]
    _need(w, "w", torch.bfloat16, (N, K))
    if norm_of is not None:
        _need(norm_of, "norm_of", torch.float32); _need(norm_weight, "norm_weight", None, (K,))
    else:
        _need(a, "a", torch.bfloat16)
    if bias is not None:
        _need(bias, "bias", None, (N,))
    if accumulate_into is not None:
        _need(accumulate_into, "accumulate_into", torch.float32, (M, N))
        out, epilogue = accumulate_into, 2
    else:
        out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=w.device)
        epilogue = _EPILOGUE_STORE[out.dtype]
    if scale != 1.0:
        if M > FUSED_MAX_ROWS or accumulate_into is None:
            raise KernelError("a scaled sum into the stream is taken for up to 16 rows")
        check(core().pe_linear_fused_scaled(_ptr(a), _ptr(norm_of), _ptr(norm_weight), 0 if norm_weight is None else _code(norm_weight, "norm_weight"),
                                            float(eps), w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"), out.data_ptr(),
                                            epilogue, float(scale), M, N, K, status_ptr(w.device), stream_ptr()), "linear_fused")
        return out
    fn, name = (core().pe_linear_fused, "linear_fused") if M <= FUSED_MAX_ROWS else (extras().pe_linear_batch, "linear_batch")
    check(fn(_ptr(a), _ptr(norm_of), _ptr(norm_weight), 0 if norm_weight is None else _code(norm_weight, "norm_weight"), float(eps),
             w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"), out.data_ptr(),
             epilogue, M, N, K, status_ptr(w.device), stream_ptr()), name)
    return out


def norm_gate_up_swiglu(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(h Wg^T) * (h Wu^T) with h = RMSNorm(x); x float32 [M <= 64, K], w_gate_up [2I, K] (gate rows first)."""
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x, "x", torch.float32); _need(norm_weight, "norm_weight", None, (K,)); _need(w_gate_up, "w_gate_up", torch.bfloat16, (2 * I, K))
    act = torch.empty(M, I, dtype=torch.bfloat16, device=x.device)
    fn = core().pe_norm_gate_up_swiglu if M <= FUSED_MAX_ROWS else extras().pe_batch_norm_gate_up_swiglu
    check(fn(x.data_ptr(), norm_weight.data_ptr(), _code(norm_weight, "norm_weight"), float(eps),
             w_gate_up.data_ptr(), act.data_ptr(), M, I, K, status_ptr(x.device), stream_ptr()), "norm_gate_up_swiglu")
    return act


def norm_qkv_rope_store(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w_qkv: torch.Tensor,
                        b_qkv: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int, cos: Optional[torch.Tensor],
                        sin: Optional[torch.Tensor], tok_pos: torch.Tensor, tok_row: torch.Tensor,
                        k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                        block_table: Optional[torch.Tensor], table_stride: int) -> torch.Tensor:
    """Rotated queries [M, n_q * head_dim] of h = RMSNorm(x); rotated keys and the values go to
    the cache pages (skipped when ``k_pool`` is None)."""
    M, K = x.shape
    N = (n_q + 2 * n_kv) * head_dim
    _need(x, "x", torch.float32); _need(norm_weight, "norm_weight", None, (K,)); _need(w_qkv, "w_qkv", torch.bfloat16, (N, K))
    if b_qkv is not None:
        _need(b_qkv, "b_qkv", None, (N,))
    _need(tok_pos, "tok_pos", torch.int32, (M,)); _need(tok_row, "tok_row", torch.int32, (M,))
    if cos is not None:
        _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32, cos.shape)
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
        _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim):
            raise KernelError(f"cache pool must be [pages, {n_kv}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    q = torch.empty(M, n_q * head_dim, dtype=torch.bfloat16, device=x.device)
    tail = (q.data_ptr(), M, K, n_q, n_kv, head_dim, _ptr(cos), _ptr(sin), tok_pos.data_ptr(), tok_row.data_ptr(), _ptr(k_pool),
            _ptr(v_pool), _ptr(block_table), table_stride, 1 if store else 0, status_ptr(x.device), stream_ptr())
    head = (x.data_ptr(), norm_weight.data_ptr(), _code(norm_weight, "norm_weight"), float(eps), w_qkv.data_ptr(), _ptr(b_qkv),
            0 if b_qkv is None else _code(b_qkv, "b_qkv"))
    if M <= FUSED_MAX_ROWS:
        check(core().pe_norm_qkv_rope_store(None, *head, *tail), "norm_qkv_rope_store")
    else:
        check(extras().pe_batch_norm_qkv_rope_store(*head, *tail), "batch_norm_qkv_rope_store")
    return q


# ---------------------------------------------------------------------------- tcgen05 products for more than 16 rows (bfloat16)

ORIENTATION = {None: 0, "rows": 1, "swapped": 2, "pairs": 3}
# Orientation "splitk" (csrc/gemm_splitk.cu): rows of w on the lanes, K cut into ranges over a thread-block cluster, for up
# to 64 rows of a.  Nothing chooses it by itself: measured on a B200 at the Qwen2.5-0.5B widths and 64 rows, in captured
# graphs, it takes 8.5 / 7.2 / 11.8 / 9.5 us for q/k/v + RoPE, o + residual, gate/up + SwiGLU and down + residual where
# the library's product with the pass that follows it takes 5.9 / 5.3 / 7.7 / 10.1; at the 7B widths it streams
# gate/up at 4.6 to 5.0 TB/s (library 5.2).  One thread issues a stage's three TMA copies and another its four MMAs at
# 150 to 200 cycles an instruction, which is 700 cycles for 24 KB of operands, whatever the accumulators' number.
SPLITK_MAX_ROWS = 64


def gemm_tcgen05_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and w.shape[0] % 8 == 0
            and a.is_contiguous() and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 accumulate_into: Optional[torch.Tensor] = None, swiglu: bool = False,
                 orientation: Optional[str] = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T on the tcgen05 tensor cores with a fused epilogue: bfloat16 result
    (+ bias); or added into the float32 tensor ``accumulate_into``; or, with ``swiglu`` and
    w = [gate rows; up rows], silu(gate) * up as bfloat16 [M, N / 2].  ``orientation``: "rows" puts
    the rows of ``a`` on the accumulator's lanes, "pairs" the same with 256 rows to a pair of CTAs
    (``cta_group::2``), "swapped" the rows of ``w`` (for up to a few hundred rows of ``a``); None
    chooses by M."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16, (N, K))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    if accumulate_into is not None:
        _need(accumulate_into, "accumulate_into", torch.float32, (M, N))
        out, epilogue = accumulate_into, 1
    elif swiglu:
        out, epilogue = torch.empty(M, N // 2, dtype=torch.bfloat16, device=a.device), 2
    else:
        out, epilogue = torch.empty(M, N, dtype=torch.bfloat16, device=a.device), 0
    if orientation == "splitk":                  # rows of w on the lanes, K cut over a cluster (up to 64 rows of a)
        check(extras().pe_gemm_splitk(a.data_ptr(), w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"),
                                    out.data_ptr(), epilogue, M, N, K, status_ptr(a.device), stream_ptr()), "gemm_splitk")
        return out
    check(core().pe_gemm_tcgen05(a.data_ptr(), w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"),
                                 out.data_ptr(), epilogue, M, N, K, ORIENTATION[orientation], status_ptr(a.device),
                                 stream_ptr()), "gemm_tcgen05")
    return out


GEMM_ROPE_HEAD_DIMS = (16, 32, 64, 128)      # a 128-row tile of the weight holds whole heads


def gemm_qkv_rope_store(a: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], n_q: int, n_kv: int,
                        head_dim: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], tok_pos: torch.Tensor,
                        tok_row: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                        block_table: Optional[torch.Tensor], table_stride: int,
                        orientation: Optional[str] = None) -> torch.Tensor:
    """Rotated queries [M, n_q * head_dim] of bfloat16 rows ``a`` [M, K]: the q/k/v product with bias, the
    rotation of q and k and the write of keys and values into their cache pages in one tcgen05 kernel
    (the cache write is skipped when ``k_pool`` is None)."""
    M, K = a.shape
    N = (n_q + 2 * n_kv) * head_dim
    _need(a, "a", torch.bfloat16); _need(w_qkv, "w_qkv", torch.bfloat16, (N, K))
    if head_dim not in GEMM_ROPE_HEAD_DIMS and orientation != "splitk":
        raise KernelError(f"head size {head_dim} is not taken by the fused q/k/v product: {GEMM_ROPE_HEAD_DIMS} are")
    if b_qkv is not None:
        _need(b_qkv, "b_qkv", None, (N,))
    _need(tok_pos, "tok_pos", torch.int32, (M,)); _need(tok_row, "tok_row", torch.int32, (M,))
    if cos is not None:
        _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32, cos.shape)
        if cos.shape[1] != head_dim // 2:
            raise KernelError("cos/sin tables need head_dim/2 columns")
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
        _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim):
            raise KernelError(f"cache pool must be [pages, {n_kv}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    q = torch.empty(M, n_q * head_dim, dtype=torch.bfloat16, device=a.device)
    if orientation == "splitk":
        check(extras().pe_gemm_splitk_rope(a.data_ptr(), w_qkv.data_ptr(), _ptr(b_qkv), 0 if b_qkv is None else _code(b_qkv, "b_qkv"),
                                         q.data_ptr(), M, K, n_q, n_kv, head_dim, _ptr(cos), _ptr(sin), tok_pos.data_ptr(),
                                         tok_row.data_ptr(), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), table_stride,
                                         1 if store else 0, status_ptr(a.device), stream_ptr()), "gemm_splitk_rope")
        return q
    check(core().pe_gemm_tcgen05_rope(a.data_ptr(), w_qkv.data_ptr(), _ptr(b_qkv), 0 if b_qkv is None else _code(b_qkv, "b_qkv"),
                                      q.data_ptr(), M, K, n_q, n_kv, head_dim, _ptr(cos), _ptr(sin), tok_pos.data_ptr(),
                                      tok_row.data_ptr(), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), table_stride,
                                      1 if store else 0, ORIENTATION[orientation], status_ptr(a.device), stream_ptr()),
          "gemm_qkv_rope_store")
    return q


# ---------------------------------------------------------------------------- pointwise kernels of other designs

def add_sinusoid(x: torch.Tensor, tok_pos: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """x[t, 2i] += sin(pos_t * freq_i), x[t, 2i + 1] += cos(pos_t * freq_i) on the float32 stream, in place."""
    T, H = x.shape
    _need(x, "x", torch.float32); _need(tok_pos, "tok_pos", torch.int32, (T,)); _need(freq, "freq", torch.float32, ((H + 1) // 2,))
    check(core().pe_add_sinusoid(x.data_ptr(), tok_pos.data_ptr(), freq.data_ptr(), T, H, stream_ptr()), "add_sinusoid")
    return x


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def activation(h: torch.Tensor, kind: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """relu(h)^2, gelu (tanh formula) or silu of every element, computed in float32, stored in h's dtype."""
    _need(h, "h")
    if out is None:
        out = torch.empty_like(h)
    _need(out, "out", h.dtype, h.shape)
    check(core().pe_activation(h.data_ptr(), out.data_ptr(), _code(h, "h"), ACTIVATIONS[kind], h.numel(), stream_ptr()), "activation")
    return out


def softcap(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """logits <- cap * tanh(logits / cap), float32, in place."""
    _need(logits, "logits", torch.float32)
    check(core().pe_softcap(logits.data_ptr(), float(cap), logits.numel(), stream_ptr()), "softcap")
    return logits


# ---------------------------------------------------------------------------- layer norm and the input convolution

def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float, out_dtype: torch.dtype,
              rows_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Layer norm (weight and bias) of float32 rows [T, H]; with ``rows_index`` (int32 [R]) only of those rows."""
    T, H = x.shape
    _need(x, "x", torch.float32); _need(weight, "weight", None, (H,)); _need(bias, "bias", None, (H,))
    rows = T if rows_index is None else rows_index.shape[0]
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32)
    out = torch.empty(rows, H, dtype=out_dtype, device=x.device)
    check(mixers().pe_layernorm(x.data_ptr(), _ptr(rows_index), weight.data_ptr(), _code(weight, "weight"), bias.data_ptr(),
                                _code(bias, "bias"), float(eps), out.data_ptr(), _code(out, "out"), rows, H, stream_ptr()), "layernorm")
    return out


def _state_args(state: torch.Tensor, offset: int, elems: int):
    """Address of element ``offset`` of slot 0 of a float32 state area [slots, elems of all parts] and its row stride."""
    _need(state, "state", torch.float32)
    if state.dim() != 2 or offset < 0 or offset + elems > state.shape[1]:
        raise KernelError(f"a part's state of {elems} numbers at {offset} does not fit rows of {tuple(state.shape)}")
    return state.data_ptr() + 4 * offset, state.shape[1]


def causal_conv_add(y: torch.Tensor, taps_weight: torch.Tensor, state: torch.Tensor, state_offset: int, tok_row: torch.Tensor,
                    row_first: torch.Tensor, row_lens: torch.Tensor, slots: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """y_t + sum_j c[:, j] y_(t - taps + 1 + j) per channel for float32 rows y [T, H] of packed sequences; the rows before a
    step's first token come from the sequences' state, which is then brought up to date (entry k: the row k + 1 places
    before the next step's first token)."""
    T, H = y.shape
    taps = taps_weight.shape[1]
    _need(y, "y", torch.float32); _need(taps_weight, "taps_weight", None, (H, taps))
    sp, stride = _state_args(state, state_offset, (taps - 1) * H) if taps > 1 else (0, 0)
    B = slots.shape[0]
    out = torch.empty(T, H, dtype=out_dtype, device=y.device)
    lib = mixers()
    check(lib.pe_causal_conv_add(y.data_ptr(), taps_weight.data_ptr(), _code(taps_weight, "taps_weight"), sp, stride,
                                 tok_row.data_ptr(), row_first.data_ptr(), slots.data_ptr(), out.data_ptr(), _code(out, "out"),
                                 T, H, taps, stream_ptr()), "causal_conv_add")
    if taps > 1:
        check(lib.pe_conv_state_update(y.data_ptr(), sp, stride, row_first.data_ptr(), row_lens.data_ptr(), slots.data_ptr(),
                                       B, H, taps, stream_ptr()), "conv_state_update")
    return out


DUAL_NORM_CONV_MAX_TAPS = 8      # LC_MAX_TAPS of csrc/layernorm_conv.cu


def dual_layernorm_conv(x: torch.Tensor, halves, eps: float, state: torch.Tensor, tok_row: torch.Tensor, row_first: torch.Tensor,
                        row_lens: torch.Tensor, slots: torch.Tensor, out_dtype: torch.dtype, one_token_each: bool):
    """Layer norm and input convolution of one or two sublayers that read the same float32 rows x [T, H], in one pass.
    ``halves``: one or two tuples (norm weight, norm bias, taps weight [H, taps], state offset); all share eps and taps.
    Returns one output [T, H] per half.  The sequences' states are brought up to date."""
    T, H = x.shape
    _need(x, "x", torch.float32)
    taps = halves[0][2].shape[1]
    outs, args = [], []
    for w, b, c, off in halves:
        _need(w, "norm weight", None, (H,)); _need(b, "norm bias", None, (H,)); _need(c, "taps weight", None, (H, taps))
        sp, stride = _state_args(state, off, (taps - 1) * H) if taps > 1 else (0, 0)
        o = torch.empty(T, H, dtype=out_dtype, device=x.device)
        outs.append(o)
        args += [w.data_ptr(), _code(w, "w"), b.data_ptr(), _code(b, "b"), c.data_ptr(), _code(c, "c"), sp, o.data_ptr()]
    if len(halves) == 1:
        args += [None, 0, None, 0, None, 0, None, None]
    check(mixers().pe_dual_layernorm_conv(x.data_ptr(), *args, DTYPE_CODE[out_dtype], stride, tok_row.data_ptr(),
                                          row_first.data_ptr(), row_lens.data_ptr(), slots.data_ptr(), float(eps), T,
                                          slots.shape[0], H, taps, 1 if one_token_each else 0, stream_ptr()),
          "dual_layernorm_conv", 1 if one_token_each or taps == 1 else 2)
    return outs


# ---------------------------------------------------------------------------- the gated recurrence

def mingru(proj: torch.Tensor, state: torch.Tensor, state_offset: int, tok_row: torch.Tensor, row_first: torch.Tensor,
           row_lens: torch.Tensor, slots: torch.Tensor, chunked: bool) -> torch.Tensor:
    """S_t = (1 - z) S_(t-1) + z c and y_t = S_t * silu(g) for proj [T, 3W] = z | candidate | gate pre-activations of packed
    sequences; S comes from and returns to the sequences' float32 state.  ``chunked``: as a segmented scan over chunks of the
    packed tokens (three launches) instead of token after token."""
    T, W3 = proj.shape
    W = W3 // 3
    _need(proj, "proj")
    sp, stride = _state_args(state, state_offset, W)
    B = slots.shape[0]
    y = torch.empty(T, W, dtype=proj.dtype, device=proj.device)
    lib = mixers()
    ws = None
    if chunked:
        from .workspace import scratch
        ws = scratch("mingru.carry", 4 * lib.pe_mingru_scratch_floats(T, B, W), proj.device).data_ptr()
    check(lib.pe_mingru(proj.data_ptr(), _code(proj, "proj"), sp, stride, tok_row.data_ptr(), row_first.data_ptr(),
                        row_lens.data_ptr(), slots.data_ptr(), y.data_ptr(), T, B, W, 1 if chunked else 0, ws, stream_ptr()),
          "mingru", 3 if chunked else 1)
    return y


# ---------------------------------------------------------------------------- attention with mixed heads

def qknorm_store(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, v_head_dim: int, q_weight: Optional[torch.Tensor],
                 k_weight: Optional[torch.Tensor], eps: float, tok_pos: torch.Tensor, tok_row: torch.Tensor,
                 k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
                 table_stride: int) -> None:
    """RMS norm of every query and key head of qkv [T, H*D + G*D + G*Dv] in place (a weight vector of D for all query heads,
    one for all key heads; None: that side stays as projected), then keys and values into their cache pages (skipped when
    ``k_pool`` is None)."""
    T = qkv.shape[0]
    _need(qkv, "qkv", None, (T, n_heads * head_dim + n_kv * head_dim + n_kv * v_head_dim))
    for w, name in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, name, None, (head_dim,))
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype); _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim) or tuple(v_pool.shape[1:]) != (n_kv, PAGE, v_head_dim):
            raise KernelError(f"cache pools must be [pages, {n_kv}, {PAGE}, {head_dim}] and [pages, {n_kv}, {PAGE}, {v_head_dim}], "
                              f"not {tuple(k_pool.shape)} and {tuple(v_pool.shape)}")
    check(mixers().pe_qknorm_store(qkv.data_ptr(), _code(qkv, "qkv"), T, n_heads, n_kv, head_dim, v_head_dim, _ptr(q_weight),
                                   0 if q_weight is None else _code(q_weight, "q_weight"), _ptr(k_weight),
                                   0 if k_weight is None else _code(k_weight, "k_weight"), float(eps), tok_pos.data_ptr(),
                                   tok_row.data_ptr(), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), table_stride,
                                   1 if store else 0, stream_ptr()), "qknorm_store")


# Which kernel runs head-mixing attention in bfloat16: "1" the one-pass tensor-core kernel (attention_headmix_flash.cu) where
# it takes the sizes, else the two-pass one (attention_headmix_mma.cu), else float32 FMAs; "two-pass" and "0" skip the first
# or both (the tests run all three).
HEADMIX_TENSOR_CORES = os.environ.get("PICO_ENGINE_HEADMIX_MMA", "1")
_headmix_plans = {}


def headmix_mma_key_block(n_heads: int, n_kv: int, head_dim: int, v_head_dim: int) -> int:
    """Keys a block of the tensor-core kernel visits at a time for these sizes; 0: it does not take them (more than 32
    heads, or a tile that does not fit the shared memory), and the float32-FMA kernel runs."""
    key = (n_heads, n_kv, head_dim, v_head_dim)
    if key not in _headmix_plans:
        import ctypes
        dvs = ctypes.c_int(1)
        _headmix_plans[key] = mixers().pe_attention_headmix_mma_plan(n_heads, n_kv, head_dim, v_head_dim, ctypes.byref(dvs))
    return _headmix_plans[key]


def attention_headmix(q: torch.Tensor, q_stride: int, n_heads: int, n_kv: int, head_dim: int, v_head_dim: int,
                      k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                      tok_pos: torch.Tensor, tok_row: torch.Tensor, window: Optional[int], scale: float,
                      sink: Optional[torch.Tensor], mix: Optional[torch.Tensor], ctx, slopes: Optional[torch.Tensor] = None,
                      keep_first: int = 0, values_in_keys: bool = False) -> torch.Tensor:
    """Attention of the step's tokens over the cache with the softmax weights mixed across heads (``mix`` [H, H]; None: not
    mixed) and a sink logit a head in the denominator (``sink`` [H]; None: none); [T, H * Dv] in q's dtype.  ``slopes``
    float32 [H]: slope_h * (i - j) is taken off the score of query i and key j.  ``keep_first``: with a window, the first so many
    keys of a sequence stay visible.  ``values_in_keys``: a position's value is the first Dv entries of its key row
    (``v_pool`` is not read)."""
    T = tok_pos.shape[0]
    _need(q, "q"); _need(k_pool, "k_pool", q.dtype)
    if values_in_keys:
        if v_head_dim > head_dim:
            raise KernelError("values that are part of the key rows cannot be longer than those")
        v_pool, v_ld = k_pool, head_dim
    else:
        _need(v_pool, "v_pool", q.dtype)
        v_ld = v_head_dim
    if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim) or tuple(v_pool.shape[1:]) != (n_kv, PAGE, v_ld):
        raise KernelError("cache pools do not have the heads and head sizes of this attention")
    if slopes is not None:
        _need(slopes, "slopes", torch.float32, (n_heads,))
    plain_mask = slopes is None and not keep_first and not values_in_keys
    if sink is not None:
        _need(sink, "sink", None, (n_heads,))
    if mix is not None:
        _need(mix, "mix", None, (n_heads, n_heads))
    sink_f32 = sink is None or sink.dtype == torch.float32
    if (q.dtype == torch.bfloat16 and not ctx.one_token_each and sink_f32 and mix is None and not values_in_keys
            and head_dim == v_head_dim and attention_prefill_tcgen05_takes(head_dim, scale) and q_stride % 8 == 0
            and HEADMIX_TENSOR_CORES == "1"):
        # one weight a (query, key) and equal sizes of 64 or 128: the tcgen05 kernel of the plain attention, which takes the
        # distance's share of the score, the kept first keys and a sink logit a head
        tiles = ctx.scratch.get("prefill_tiles_128")
        if tiles is None:
            tiles = ctx.scratch["prefill_tiles_128"] = prefill_tiles(ctx.lens, ctx.starts, q.device, PREFILL_TILE_TCGEN05)
        return attention_prefill_tcgen05(q, q_stride, n_heads, n_kv, head_dim, k_pool, v_pool, block_table, table_stride, tiles, T,
                                         window, scale, keep_first=keep_first, slopes=slopes, sinks=sink)
    if (q.dtype == torch.bfloat16 and ctx.one_token_each and sink_f32 and mix is None and not values_in_keys
            and head_dim == v_head_dim and attention_prefill_tcgen05_takes(head_dim, scale) and q_stride % 8 == 0
            and HEADMIX_TENSOR_CORES == "1"):
        # single tokens at the same sizes: the decode kernel of the plain attention, which knows both as well (the kernels before
        # it in the stream write no cache row but each token's own)
        return attention_decode(q, q_stride, n_heads, n_kv, head_dim, k_pool, v_pool, block_table, table_stride, tok_pos, tok_row,
                                window, scale, ctx.max_context, keep_first=keep_first, slopes=slopes, sinks=sink)
    lib = mixers()
    tiles, n_runs = None, 0
    if not ctx.one_token_each:
        tiles = ctx.scratch.get("prefill_tiles")
        if tiles is None:
            tiles = ctx.scratch["prefill_tiles"] = prefill_tiles(ctx.lens, ctx.starts, q.device, PREFILL_TILE)
        n_runs = tiles.shape[0]
    from .workspace import scratch
    out = torch.empty(T, n_heads * v_head_dim, dtype=q.dtype, device=q.device)
    floats = all(t is None or t.dtype == torch.float32 for t in (sink, mix))
    if q.dtype == torch.bfloat16 and HEADMIX_TENSOR_CORES == "1" and floats:
        cg = lib.pe_attention_flashmix_group(n_heads, n_kv, head_dim, v_head_dim)
        if cg and q_stride % 2 == 0 and v_ld % 8 == 0:
            # one pass over the keys with an output for every (head, value head), then merge + sink + mixing
            blocks = (n_runs * n_heads if tiles is not None else T * n_kv) * ((n_kv + cg - 1) // cg)
            # Few blocks (single tokens with long contexts): the keys are cut into ranges until about one and a half blocks
            # an SM run.  Measured on a B200 (8 tokens at 2,048 keys): 14 heads of 64 on 2 key/value heads 65 / 47 / 29 / 32 /
            # 51 us at 2 / 4 / 8 / 16 / 32 ranges, 16 heads of 128 on 4 key/value heads 82 / 55 / 70 / 97 / 202 us: more ranges
            # mean more partial outputs to write and merge.  A prompt has blocks enough and is not cut (2,048 tokens: 183 us
            # uncut, 209 us in two ranges).
            # (a window leaves a token the pages of its last `window` keys and of the kept first ones: no more ranges than those)
            span = ctx.max_context if not window else min(ctx.max_context, window + PAGE - 1 + (keep_first + PAGE - 1) // PAGE * PAGE)
            splits = max(1, min((224 + blocks - 1) // blocks, (span + 63) // 64, 64))
            ws = scratch("attention_headmix", 4 * lib.pe_attention_flashmix_scratch_floats(T, splits, n_heads, n_kv, v_head_dim, 1 if tiles is None else 0), q.device)
            check(lib.pe_attention_flashmix(q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                            block_table.data_ptr(), table_stride, tok_pos.data_ptr(), tok_row.data_ptr(), _ptr(tiles),
                                            n_runs, T, n_heads, n_kv, head_dim, v_head_dim, window or 0, float(scale), _ptr(sink),
                                            _ptr(mix), splits, ws.data_ptr(), _ptr(slopes), keep_first, v_ld, stream_ptr()),
                  "attention_flashmix", 2)
            return out
    if q.dtype == torch.bfloat16 and HEADMIX_TENSOR_CORES in ("1", "two-pass") and floats and plain_mask:
        kb = headmix_mma_key_block(n_heads, n_kv, head_dim, v_head_dim)
        if kb:
            # bfloat16: the tensor-core kernel; tiles of 16 tokens, ranges of at least two key blocks
            n_tiles = T if tiles is None else n_runs * (PREFILL_TILE // 16)
            splits = 1 if n_tiles >= 148 else max(1, min(296 // n_tiles, (ctx.max_context + 2 * kb - 1) // (2 * kb), 64))
            ws = scratch("attention_headmix", 4 * lib.pe_attention_headmix_mma_scratch_floats(n_tiles, splits, n_heads, v_head_dim), q.device)
            check(lib.pe_attention_headmix_mma(q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                               block_table.data_ptr(), table_stride, tok_pos.data_ptr(), tok_row.data_ptr(),
                                               _ptr(tiles), n_runs, PREFILL_TILE, T, n_heads, n_kv, head_dim, v_head_dim,
                                               window or 0, float(scale), _ptr(sink), _ptr(mix), splits, ws.data_ptr(), stream_ptr()),
                  "attention_headmix_mma", 1 if splits == 1 else 3)
            return out
    qt = lib.pe_attention_headmix_tile(n_heads, n_kv, head_dim, v_head_dim, 0 if mix is None else 1, 1 if tiles is None else 16)
    if qt <= 0:
        raise KernelError(f"attention with {n_heads} heads of size {head_dim}/{v_head_dim} is not taken: heads x value size "
                          f"may be 16384 at most")
    n_tiles = T if tiles is None else n_runs * (PREFILL_TILE // qt)
    # few tiles with many keys (single tokens with long contexts): the keys are cut into ranges so that the GPU is filled
    splits = 1
    if n_tiles < 296:
        splits = max(1, min(296 // max(n_tiles, 1), (ctx.max_context + 255) // 256, 64))
    ws = scratch("attention_headmix", 4 * lib.pe_attention_headmix_scratch_floats(n_tiles, splits, qt, n_heads, v_head_dim), q.device)
    check(lib.pe_attention_headmix(q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), _code(q, "q"),
                                   block_table.data_ptr(), table_stride, tok_pos.data_ptr(), tok_row.data_ptr(), _ptr(tiles),
                                   n_runs, PREFILL_TILE, T, n_heads, n_kv, head_dim, v_head_dim, window or 0, float(scale),
                                   _ptr(sink), 0 if sink is None else _code(sink, "sink"), _ptr(mix),
                                   0 if mix is None else _code(mix, "mix"), qt, splits, ws.data_ptr(), _ptr(slopes), keep_first, v_ld,
                                   stream_ptr()),
          "attention_headmix", 2 + (splits > 1))
    return out


# ---------------------------------------------------------------------------- gated mixers and routed feed-forwards

LA_ACTIVATIONS = {"none": 0, "silu": 1}
GATE_ACTIVATIONS = {"none": 0, "sigmoid": 1, "silu": 2, "gelu_tanh": 3, "relu2": 4, "clamped_sigmoid": 5}


def linear_attention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, n_heads: int, head_dim: int, v_head_dim: int,
                     state: torch.Tensor, state_offset: int, row_first: torch.Tensor, row_lens: torch.Tensor, slots: torch.Tensor,
                     chunked: bool, head_decay: Optional[torch.Tensor] = None, decay_logits: Optional[torch.Tensor] = None,
                     inv_tau: float = 1.0, q_scale: float = 1.0, qk_activation: str = "none",
                     v_activation: str = "none") -> torch.Tensor:
    """o [T, H * Dv] float32 of S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, for q, k, v at columns
    ``q_off``, ``k_off``, ``v_off`` of proj [T, ld] (packed sequences).  The decay is ``head_decay`` [H] float32 (one constant
    a head) or sigmoid(``decay_logits`` float32 [T, H * D])^``inv_tau`` (a number per key channel and token).  S [H, D, Dv] comes from
    and returns to the sequences' float32 state at ``state_offset``.  ``chunked``: prompts, three launches over chunks of
    the sequences; else token after token in one launch."""
    T, ld = proj.shape
    H, D, Dv = n_heads, head_dim, v_head_dim
    _need(proj, "proj")
    if max(q_off + H * D, k_off + H * D, v_off + H * Dv) > ld:
        raise KernelError("q, k and v do not fit the rows of proj")
    if (head_decay is None) == (decay_logits is None):
        raise KernelError("linear attention takes either a decay per head or decay logits per channel")
    if head_decay is not None:
        _need(head_decay, "head_decay", torch.float32, (H,))
    else:
        _need(decay_logits, "decay_logits", torch.float32, (T, H * D))
    sp, stride = _state_args(state, state_offset, H * D * Dv)
    B = slots.shape[0]
    out = torch.empty(T, H * Dv, dtype=torch.float32, device=proj.device)
    lib = gated()
    ws = None
    if chunked:
        from .workspace import scratch
        ws = scratch("linear_attention", 4 * lib.pe_linear_attention_scratch_floats(T, B, H, D, Dv), proj.device).data_ptr()
    check(lib.pe_linear_attention(proj.data_ptr(), _code(proj, "proj"), ld, q_off, k_off, v_off, _ptr(decay_logits),
                                  0 if decay_logits is None else _code(decay_logits, "decay_logits"), H * D, _ptr(head_decay),
                                  float(inv_tau), float(q_scale), LA_ACTIVATIONS[qk_activation], LA_ACTIVATIONS[v_activation],
                                  sp, stride, row_first.data_ptr(), row_lens.data_ptr(), slots.data_ptr(), out.data_ptr(),
                                  T, B, H, D, Dv, 1 if chunked else 0, ws, stream_ptr()), "linear_attention", 3 if chunked else 1)
    return out


def rotary_norm_store(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, v_head_dim: int, freq: Optional[torch.Tensor],
                      rot_dims: int, unit_norm: bool, eps: float, tok_pos: torch.Tensor, tok_row: torch.Tensor,
                      k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
                      table_stride: int) -> None:
    """In every query and key head of qkv [T, ld] (a row begins with H*D query, G*D key and G*Dv value entries), in place: entries (2i, 2i+1) below ``rot_dims`` are turned by
    pos * freq[i] (``freq`` float32 [rot_dims / 2]; rot_dims 0: no rotation), then (``unit_norm``) the head is divided by its
    root mean square; keys and values then go to their cache pages (skipped when ``k_pool`` is None)."""
    T, ld = qkv.shape
    _need(qkv, "qkv")
    if ld < n_heads * head_dim + n_kv * head_dim + n_kv * v_head_dim:
        raise KernelError("queries, keys and values do not fit the rows of qkv")
    if rot_dims:
        _need(freq, "freq", torch.float32, (rot_dims // 2,))
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype); _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim) or tuple(v_pool.shape[1:]) != (n_kv, PAGE, v_head_dim):
            raise KernelError(f"cache pools must be [pages, {n_kv}, {PAGE}, {head_dim}] and [pages, {n_kv}, {PAGE}, {v_head_dim}], "
                              f"not {tuple(k_pool.shape)} and {tuple(v_pool.shape)}")
    check(gated().pe_rotary_norm_store(qkv.data_ptr(), _code(qkv, "qkv"), ld, T, n_heads, n_kv, head_dim, v_head_dim, _ptr(freq),
                                       rot_dims, 1 if unit_norm else 0, float(eps), tok_pos.data_ptr(), tok_row.data_ptr(),
                                       _ptr(k_pool), _ptr(v_pool), _ptr(block_table), table_stride, 1 if store else 0,
                                       stream_ptr()), "rotary_norm_store")


def gated_norm(o: torch.Tensor, group: int, weight: Optional[torch.Tensor], eps: float, gate: Optional[torch.Tensor], gate_offset: int,
               gate_activation: str, out_dtype: torch.dtype) -> torch.Tensor:
    """Rows o [T, C] (float32 or ``out_dtype``): every run of ``group`` channels divided by its root mean square and multiplied
    by ``weight`` [group] (group 0: no norm), then by act(gate[t, gate_offset + c]) of gate [T, ld] (None: no gate)."""
    T, C = o.shape
    _need(o, "o")
    if weight is not None:
        _need(weight, "weight", None, (group,))
    if gate is not None:
        _need(gate, "gate", out_dtype)
        if gate_offset + C > gate.shape[1]:
            raise KernelError("the gate's columns do not fit its rows")
    out = torch.empty(T, C, dtype=out_dtype, device=o.device)
    check(gated().pe_gated_norm(o.data_ptr(), _code(o, "o"), T, C, group, _ptr(weight), 0 if weight is None else _code(weight, "weight"),
                                float(eps), _ptr(gate), 0 if gate is None else gate.shape[1], gate_offset,
                                GATE_ACTIVATIONS[gate_activation], out.data_ptr(), _code(out, "out"), stream_ptr()), "gated_norm")
    return out


def normed_sum_add(x: torch.Tensor, branches, weights, eps: float, scale: float) -> torch.Tensor:
    """x += scale * sum_i rmsnorm(branches[i]) * weights[i] on the float32 stream [T, W]; up to four branches of one dtype."""
    T, W = x.shape
    _need(x, "x", torch.float32)
    n = len(branches)
    for y, w in zip(branches, weights):
        _need(y, "branch", branches[0].dtype, (T, W)); _need(w, "weight", weights[0].dtype, (W,))
    ys = [y.data_ptr() for y in branches] + [None] * (4 - n)
    ws = [w.data_ptr() for w in weights] + [None] * (4 - n)
    check(gated().pe_normed_sum_add(x.data_ptr(), *ys, _code(branches[0], "branch"), *ws, _code(weights[0], "weight"), n, T, W,
                                    float(eps), float(scale), stream_ptr()), "normed_sum_add")
    return x


def scaled_add(x: torch.Tensor, y: torch.Tensor, scale: float) -> torch.Tensor:
    """x += scale * y on the float32 stream; y in either dtype."""
    _need(x, "x", torch.float32); _need(y, "y", None, x.shape)
    check(gated().pe_scaled_add(x.data_ptr(), y.data_ptr(), _code(y, "y"), float(scale), x.numel(), stream_ptr()), "scaled_add")
    return x


def add_rows(x: torch.Tensor, rows: Optional[torch.Tensor], vec: Optional[torch.Tensor]) -> torch.Tensor:
    """x[t] += rows[t] + vec on the float32 stream [T, W]; ``rows`` float32 [T, W] or None, ``vec`` [W] in either dtype or None."""
    T, W = x.shape
    _need(x, "x", torch.float32)
    if rows is not None:
        _need(rows, "rows", torch.float32, (T, W))
    if vec is not None:
        _need(vec, "vec", None, (W,))
    check(gated().pe_add_rows(x.data_ptr(), _ptr(rows), _ptr(vec), 0 if vec is None else _code(vec, "vec"), T, W, stream_ptr()), "add_rows")
    return x


def gated_act(gate_up: torch.Tensor, activation: str, col_weights: Optional[torch.Tensor] = None, group: int = 0,
              limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """act(gate) * up [T, I] for gate_up [T, 2I] = gate | up.  ``col_weights`` float32 [T, n]: column c is also multiplied by
    col_weights[t, min(c // group, n - 1)] (a zero weight gives an exact zero).  ``activation`` "clamped_sigmoid": with
    g = min(gate, limit) and u = clamp(up, -limit, limit) the result is g * sigmoid(alpha * g) * (u + 1)."""
    T, I2 = gate_up.shape
    _need(gate_up, "gate_up")
    n = 0
    if col_weights is not None:
        n = col_weights.shape[1]
        _need(col_weights, "col_weights", torch.float32, (T, n))
    out = torch.empty(T, I2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    check(gated().pe_gated_act(gate_up.data_ptr(), out.data_ptr(), _code(gate_up, "gate_up"), T, I2 // 2, GATE_ACTIVATIONS[activation],
                               _ptr(col_weights), group, n, float(limit), float(alpha), stream_ptr()), "gated_act")
    return out


EXTRA_COLUMN = {False: 0, None: 0, True: 1, "sigmoid": 1, "one": 2}


def moe_route(logits: torch.Tensor, n_experts: int, top_k: int, extra, ids: Optional[torch.Tensor] = None,
              over_all: bool = False, factor: float = 1.0) -> torch.Tensor:
    """Dense routing weights float32 [T, E (+ 1)] from router logits float32 [T, E (+ 1)]: the softmax over each token's ``top_k``
    largest logits at their places, zero elsewhere (``over_all``: their entries of the softmax over all experts instead), times
    ``factor``; with ``extra`` True the last column is sigmoid(its logit), with "one" it is 1 and has no logit.  ``ids`` int32
    [T, top_k] receives the chosen experts."""
    T = logits.shape[0]
    extra = EXTRA_COLUMN[extra]
    cols = n_experts + (1 if extra else 0)
    _need(logits, "logits", torch.float32, (T, n_experts + (1 if extra == 1 else 0)))
    if ids is not None:
        _need(ids, "ids", torch.int32, (T, top_k))
    out = torch.empty(T, cols, dtype=torch.float32, device=logits.device)
    check(gated().pe_moe_route(logits.data_ptr(), logits.shape[1], n_experts, top_k, extra, out.data_ptr(), _ptr(ids), T,
                               1 if over_all else 0, float(factor), stream_ptr()), "moe_route")
    return out


MOE_ROUTE_STREAM_MAX_EXPERTS = 256      # MR_MAX_E of csrc/gated_ops.cu


def moe_route_stream(x: torch.Tensor, norm_weight: Optional[torch.Tensor], eps: float, router: torch.Tensor, n_experts: int, top_k: int,
                     extra, ids: Optional[torch.Tensor] = None, over_all: bool = False, factor: float = 1.0) -> torch.Tensor:
    """``moe_route`` of the logits router . RMSNorm(x): x float32 [T, K] is the residual stream, ``norm_weight`` [K] the norm's
    weight (None: the router reads the stream as it is), ``router`` float32 [E (+ 1), K]; norm, logits and choice are one kernel,
    all in float32 (up to 256 experts)."""
    T, K = x.shape
    extra = EXTRA_COLUMN[extra]
    cols = n_experts + (1 if extra else 0)
    _need(x, "x", torch.float32); _need(router, "router", torch.float32, (n_experts + (1 if extra == 1 else 0), K))
    if norm_weight is not None:
        _need(norm_weight, "norm_weight", None, (K,))
    if ids is not None:
        _need(ids, "ids", torch.int32, (T, top_k))
    out = torch.empty(T, cols, dtype=torch.float32, device=x.device)
    check(gated().pe_moe_route_stream(x.data_ptr(), _ptr(norm_weight), 0 if norm_weight is None else _code(norm_weight, "norm_weight"),
                                      float(eps), router.data_ptr(), K, n_experts, top_k, extra, out.data_ptr(), _ptr(ids), T,
                                      1 if over_all else 0, float(factor), stream_ptr()), "moe_route_stream")
    return out


def weighted_act(h: torch.Tensor, activation: str, col_weights: torch.Tensor, group: int) -> torch.Tensor:
    """act(h) [T, I] with column c multiplied by col_weights[t, min(c // group, n - 1)] (float32 [T, n]; a zero weight gives an
    exact zero): the hidden units of experts without a gate matrix."""
    T, I = h.shape
    _need(h, "h")
    n = col_weights.shape[1]
    _need(col_weights, "col_weights", torch.float32, (T, n))
    out = torch.empty_like(h)
    check(gated().pe_weighted_act(h.data_ptr(), out.data_ptr(), _code(h, "h"), T, I, GATE_ACTIVATIONS[activation], col_weights.data_ptr(),
                                  group, n, stream_ptr()), "weighted_act")
    return out


# ---------------------------------------------------------------------------- pairs of tokens in the embedding

def embed_pairs(table: torch.Tensor, pairs: torch.Tensor, ids: torch.Tensor, tok_pos: torch.Tensor, tok_row: torch.Tensor,
                row_first: torch.Tensor, slots: torch.Tensor, prev: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """table[ids] + pairs[(previous * mul_prev + token * mul_cur) mod buckets] as float32 [T, H]; a sequence's first token takes row
    ``buckets`` of ``pairs``.  ``prev`` int32 [slots, 1] holds every sequence's last token and is brought up to date."""
    V, H = table.shape
    T = ids.shape[0]
    _need(table, "table"); _need(pairs, "pairs", table.dtype, (buckets + 1, H)); _need(ids, "ids", torch.int32, (T,))
    _need(prev, "prev", torch.int32)
    out = torch.empty(T, H, dtype=torch.float32, device=table.device)
    check(core().pe_embed_pairs(table.data_ptr(), pairs.data_ptr(), _code(table, "table"), ids.data_ptr(), tok_pos.data_ptr(),
                                tok_row.data_ptr(), row_first.data_ptr(), slots.data_ptr(), prev.data_ptr(), prev.stride(0), out.data_ptr(),
                                T, H, V, buckets, mul_prev, mul_cur, stream_ptr()), "embed_pairs")
    return out


# ---------------------------------------------------------------------------- the state-space mixer

def state_space_elems(n_heads: int, head_dim: int, state: int) -> int:
    """float32 numbers a sequence's recurrent state takes (the kernel's own order, with its padding rows): the rows of a state
    column are dealt to the smallest power of two of threads that leaves a thread at most 16 (pe_state_space_elems of
    csrc/state_space.cu gives the same number)."""
    ns = 1
    while (state + ns - 1) // ns > 16 and ns < 32:
        ns *= 2
    return n_heads * ((state + ns - 1) // ns) * ns * head_dim


def state_space_split(state: int) -> int:
    """Threads that share a column of the state (pe_state_space_split of csrc/state_space.cu gives the same number)."""
    ns = 1
    while (state + ns - 1) // ns > 16 and ns < 32:
        ns *= 2
    return ns


def conv_silu(proj: torch.Tensor, col_offset: int, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
              state_offset: int, tok_row: torch.Tensor, row_first: torch.Tensor, row_lens: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """silu(bias + sum_j w[:, j] u_(t - taps + 1 + j)) as float32 [T, channels] for the inputs u at columns ``col_offset`` .. of
    proj [T, ld] (packed sequences); inputs before a step's first token come from the sequences' state (float32, (taps - 1) *
    channels numbers at ``state_offset``), which is then brought up to date."""
    from .library import state_space
    T, ld = proj.shape
    taps = weight.shape[1]
    _need(proj, "proj"); _need(weight, "weight", None, (channels, taps))
    if bias is not None:
        _need(bias, "bias", None, (channels,))
    sp, stride = _state_args(state, state_offset, (taps - 1) * channels) if taps > 1 else (0, 0)
    out = torch.empty(T, channels, dtype=torch.float32, device=proj.device)
    check(state_space().pe_conv_silu(proj.data_ptr(), _code(proj, "proj"), ld, col_offset, channels, taps, weight.data_ptr(),
                                     _code(weight, "weight"), _ptr(bias), 0 if bias is None else _code(bias, "bias"), sp, stride,
                                     tok_row.data_ptr(), row_first.data_ptr(), row_lens.data_ptr(), slots.data_ptr(), out.data_ptr(),
                                     T, slots.shape[0], stream_ptr()), "conv_silu", 2 if taps > 1 else 1)
    return out


def state_space_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_offset: int, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
                     state: torch.Tensor, state_offset: int, row_first: torch.Tensor, row_lens: torch.Tensor, slots: torch.Tensor,
                     n_heads: int, head_dim: int, n_state: int, n_groups: int, chunked: bool = False) -> torch.Tensor:
    """y float32 [T, H * P] of S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D x_t with dt = softplus(raw + bias):
    x | B | C are the columns of ``xbc`` float32 [T, H*P + 2 G N], the raw step sizes columns ``dt_offset`` .. of proj.  The states
    come from and return to the sequences' float32 state at ``state_offset``.  ``chunked``: prompts, three launches over chunks of 64
    tokens (every chunk from zero, a carry pass, every chunk from its incoming state) instead of one walk a sequence; both give the
    same numbers up to float32 rounding."""
    from .library import state_space
    T = xbc.shape[0]
    H, P, N, G = n_heads, head_dim, n_state, n_groups
    _need(xbc, "xbc", torch.float32, (T, H * P + 2 * G * N)); _need(proj, "proj")
    for t, name in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        _need(t, name, None, (H,))
    sp, stride = _state_args(state, state_offset, state_space_elems(H, P, N))
    y = torch.empty(T, H * P, dtype=torch.float32, device=xbc.device)
    ws = 0
    if chunked:
        from .workspace import scratch
        ws = scratch("state_space_scan", 4 * state_space().pe_state_space_scratch_floats(T, slots.shape[0], H, P, N), xbc.device).data_ptr()
    check(state_space().pe_state_space_scan(xbc.data_ptr(), xbc.shape[1], proj.data_ptr(), _code(proj, "proj"), proj.shape[1], dt_offset,
                                            dt_bias.data_ptr(), _code(dt_bias, "dt_bias"), a_log.data_ptr(), _code(a_log, "a_log"),
                                            d_skip.data_ptr(), _code(d_skip, "d_skip"), sp, stride, row_first.data_ptr(),
                                            row_lens.data_ptr(), slots.data_ptr(), y.data_ptr(), T, slots.shape[0], H, P, N, G,
                                            1 if chunked else 0, ws, stream_ptr()), "state_space_scan", 3 if chunked else 1)
    return y


def gate_norm(y: torch.Tensor, group: int, proj: torch.Tensor, gate_offset: int, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """u = y * silu(gate) with the gate at columns ``gate_offset`` .. of proj; every run of ``group`` channels of u divided by its root
    mean square and multiplied by ``weight`` [C]; [T, C] in proj's dtype.  y float32 [T, C]."""
    from .library import state_space
    T, C = y.shape
    _need(y, "y", torch.float32); _need(proj, "proj"); _need(weight, "weight", None, (C,))
    out = torch.empty(T, C, dtype=proj.dtype, device=y.device)
    check(state_space().pe_gate_norm(y.data_ptr(), T, C, group, proj.data_ptr(), _code(proj, "proj"), proj.shape[1], gate_offset,
                                     weight.data_ptr(), _code(weight, "weight"), float(eps), out.data_ptr(), stream_ptr()), "gate_norm")
    return out


# ---------------------------------------------------------------------------- attention over low-rank rows

def latent_prepare(proj: torch.Tensor, n_heads: int, head_dim: int, rot_dim: int, rank: int, dkv_offset: int, norm_weight: torch.Tensor,
                   eps: float, freq: Optional[torch.Tensor], rot_dims: int, q_absorbed: Optional[torch.Tensor], tok_pos: torch.Tensor,
                   tok_row: torch.Tensor, k_pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor], table_stride: int,
                   halves: bool = False, q_rows: Optional[torch.Tensor] = None, q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Queries [T, H * (rank + rot_dim)] = [absorbed plain part | turned rotated part] a head, from ``q_absorbed`` [H, T, rank] and the
    rotated parts of the queries in proj [T, ld] (a head = head_dim plain | rot_dim rotated entries); the row [rmsnorm(first rank
    entries at ``dkv_offset``) * norm_weight | turned last rot_dim entries] goes to the token's place in ``k_pool`` [pages, 1, PAGE,
    rank + rot_dim] (skipped when None).  ``halves``: the rotation pairs entry i with entry i + rot_dims / 2 instead of neighbours.
    ``q_rows`` [T, H * (head_dim + rot_dim)]: the queries lie there and not at the front of proj's rows.  ``q_absorbed`` None with ``q_out``
    [T, H * (rank + rot_dim)] given: the absorbed parts stand in ``q_out`` already (a batched product wrote them there) and only the
    rotated parts are filled in."""
    from .library import state_space
    T, ld = proj.shape
    H, W = n_heads, rank + rot_dim
    _need(proj, "proj"); _need(norm_weight, "norm_weight", None, (rank,))
    if q_absorbed is not None:
        _need(q_absorbed, "q_absorbed", proj.dtype, (H, T, rank))
    elif q_out is None:
        raise KernelError("without q_absorbed the queries' rows q_out must be given")
    if q_out is not None:
        _need(q_out, "q_out", proj.dtype, (T, H * W))
    if rot_dims:
        _need(freq, "freq", torch.float32, (rot_dims // 2,))
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", proj.dtype); _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (1, PAGE, W):
            raise KernelError(f"the cache pool must be [pages, 1, {PAGE}, {W}], not {tuple(k_pool.shape)}")
    if q_rows is not None:
        _need(q_rows, "q_rows", proj.dtype, (T, H * (head_dim + rot_dim)))
    q = q_out if q_out is not None else torch.empty(T, H * W, dtype=proj.dtype, device=proj.device)
    check(state_space().pe_latent_prepare(proj.data_ptr(), _code(proj, "proj"), ld, T, H, head_dim, rot_dim, rank, dkv_offset,
                                          norm_weight.data_ptr(), _code(norm_weight, "norm_weight"), float(eps), _ptr(freq), rot_dims,
                                          _ptr(q_absorbed), q.data_ptr(), tok_pos.data_ptr(), tok_row.data_ptr(), _ptr(k_pool),
                                          _ptr(block_table), table_stride, 1 if store else 0, 1 if halves else 0, _ptr(q_rows),
                                          0 if q_rows is None else q_rows.shape[1], stream_ptr()), "latent_prepare")
    return q


def head_gate(o: torch.Tensor, proj: Optional[torch.Tensor], gate_offset: int) -> torch.Tensor:
    """[T, H * Dv] from o [H, T, Dv] (head-major, as a batched product leaves it), head h of token t multiplied by
    sigmoid(proj[t, gate_offset + h]) (proj None: no gate)."""
    from .library import state_space
    H, T, Dv = o.shape
    _need(o, "o")
    if proj is not None:
        _need(proj, "proj", o.dtype)
    out = torch.empty(T, H * Dv, dtype=o.dtype, device=o.device)
    check(state_space().pe_head_gate(o.data_ptr(), _code(o, "o"), _ptr(proj), 0 if proj is None else proj.shape[1], gate_offset, T, H, Dv,
                                     out.data_ptr(), stream_ptr()), "head_gate")
    return out


def rmsnorm_cols(rows: torch.Tensor, offset: int, cols: int, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """[T, cols] in rows' dtype: the RMS norm (float32) of columns ``offset`` .. ``offset + cols`` of rows [T, ld], times ``weight`` [cols]."""
    from .library import state_space
    T, ld = rows.shape
    _need(rows, "rows"); _need(weight, "weight", None, (cols,))
    out = torch.empty(T, cols, dtype=rows.dtype, device=rows.device)
    check(state_space().pe_rmsnorm_cols(rows.data_ptr(), _code(rows, "rows"), ld, offset, cols, weight.data_ptr(), _code(weight, "weight"),
                                        float(eps), out.data_ptr(), T, stream_ptr()), "rmsnorm_cols")
    return out


# ---------------------------------------------------------------------------- rotation of halves with blended values; norms on outputs

def rotary_half_store(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, v_head_dim: int, freq: Optional[torch.Tensor],
                      rot_dims: int, magnitude: float, unit_norm: bool, eps: float, tok_pos: torch.Tensor, tok_row: torch.Tensor,
                      k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
                      table_stride: int, blend: Optional[torch.Tensor] = None, blend_weight: Optional[torch.Tensor] = None) -> None:
    """In every query and key head of qkv [T, ld] (a row begins with H*D query, G*D key and G*Dv value entries), in place: entry
    i < rot_dims / 2 and entry i + rot_dims / 2 are turned by pos * freq[i] with cos and sin multiplied by ``magnitude``; then
    (``unit_norm``) the head is divided by its root mean square.  ``blend`` (a view [T, G*Dv] of rows in qkv's dtype whose row stride
    may be wider; ``blend_weight`` one stored number l): values become (1 - l) v + l blend.  Keys and values then go to their cache
    pages (skipped when ``k_pool`` is None)."""
    T, ld = qkv.shape
    _need(qkv, "qkv")
    if ld < n_heads * head_dim + n_kv * head_dim + n_kv * v_head_dim:
        raise KernelError("queries, keys and values do not fit the rows of qkv")
    if rot_dims:
        _need(freq, "freq", torch.float32, (rot_dims // 2,))
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype); _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim) or tuple(v_pool.shape[1:]) != (n_kv, PAGE, v_head_dim):
            raise KernelError(f"cache pools must be [pages, {n_kv}, {PAGE}, {head_dim}] and [pages, {n_kv}, {PAGE}, {v_head_dim}], "
                              f"not {tuple(k_pool.shape)} and {tuple(v_pool.shape)}")
    blend_ld = 0
    if blend is not None:
        if (blend.dtype != qkv.dtype or blend.device != qkv.device or tuple(blend.shape) != (T, n_kv * v_head_dim) or blend.stride(1) != 1
                or blend_weight is None or blend_weight.numel() != 1):
            raise KernelError("blend must be [T, G * Dv] rows of qkv's dtype with unit column stride, and blend_weight one number")
        blend_ld = blend.stride(0)
    check(gated().pe_rotary_half_store(qkv.data_ptr(), _code(qkv, "qkv"), ld, T, n_heads, n_kv, head_dim, v_head_dim, _ptr(freq), rot_dims,
                                       float(magnitude), 1 if unit_norm else 0, float(eps), tok_pos.data_ptr(), tok_row.data_ptr(),
                                       _ptr(k_pool), _ptr(v_pool), _ptr(block_table), table_stride, 1 if store else 0, _ptr(blend), blend_ld,
                                       _ptr(blend_weight), 0 if blend_weight is None else _code(blend_weight, "blend_weight"), stream_ptr()),
          "rotary_half_store")


def layernorm_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                  then: Optional[tuple] = None, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """x += layernorm(y) * weight + bias on the float32 stream [T, W] (y float32 or bfloat16).  ``then`` = (weight2, bias2, eps2):
    also returns layernorm(x) * weight2 + bias2 of the rows as they then stand, in ``out_dtype``; one kernel either way."""
    T, W = x.shape
    _need(x, "x", torch.float32); _need(y, "y", None, (T, W)); _need(weight, "weight", None, (W,)); _need(bias, "bias", None, (W,))
    out = None
    w2 = b2 = None
    eps2 = 0.0
    if then is not None:
        w2, b2, eps2 = then
        _need(w2, "weight2", None, (W,)); _need(b2, "bias2", None, (W,))
        out = torch.empty(T, W, dtype=out_dtype, device=x.device)
    check(mixers().pe_layernorm_add(x.data_ptr(), y.data_ptr(), _code(y, "y"), weight.data_ptr(), _code(weight, "weight"), bias.data_ptr(),
                                    _code(bias, "bias"), float(eps), T, W, _ptr(w2), 0 if w2 is None else _code(w2, "weight2"), _ptr(b2),
                                    0 if b2 is None else _code(b2, "bias2"), float(eps2), _ptr(out), 0 if out is None else _code(out, "out"),
                                    stream_ptr()), "layernorm_add")
    return out


def moe_route_grouped(logits: torch.Tensor, n_experts: int, top_k: int, correction: Optional[torch.Tensor], n_groups: int, keep: int,
                      group_best: int = 2, factor: float = 1.0, ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense routing weights float32 [T, E] from router logits float32 [T, E] with sigmoid scores.  The choice reads score +
    ``correction`` [E]: experts form ``n_groups`` equal runs of neighbours, a run counts the sum of its ``group_best`` largest, the
    ``keep`` best runs stay, and of their experts the ``top_k`` largest are chosen.  The weights are ``factor`` times the chosen
    experts' plain scores (not renormalised), zero elsewhere.  ``ids`` int32 [T, top_k] receives the chosen experts."""
    T = logits.shape[0]
    _need(logits, "logits", torch.float32, (T, n_experts))
    if correction is not None:
        _need(correction, "correction", None, (n_experts,))
    if ids is not None:
        _need(ids, "ids", torch.int32, (T, top_k))
    out = torch.empty(T, n_experts, dtype=torch.float32, device=logits.device)
    check(gated().pe_moe_route_grouped(logits.data_ptr(), logits.shape[1], n_experts, top_k, _ptr(correction),
                                       0 if correction is None else _code(correction, "correction"), n_groups, keep, group_best,
                                       float(factor), out.data_ptr(), _ptr(ids), T, stream_ptr()), "moe_route_grouped")
    return out


def moe_route_stream_grouped(x: torch.Tensor, norm_weight: torch.Tensor, norm_bias: torch.Tensor, eps: float, router: torch.Tensor,
                             n_experts: int, top_k: int, correction: Optional[torch.Tensor], n_groups: int, keep: int, group_best: int = 2,
                             factor: float = 1.0, ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``moe_route_grouped`` of the logits router . layernorm(x): x float32 [T, K] is the residual stream, ``norm_weight`` and
    ``norm_bias`` [K] the layer norm in front of the router, ``router`` float32 [E, K]; norm, logits and choice are one kernel, all
    in float32 (up to 256 experts)."""
    T, K = x.shape
    _need(x, "x", torch.float32); _need(router, "router", torch.float32, (n_experts, K))
    _need(norm_weight, "norm_weight", None, (K,)); _need(norm_bias, "norm_bias", None, (K,))
    if correction is not None:
        _need(correction, "correction", None, (n_experts,))
    if ids is not None:
        _need(ids, "ids", torch.int32, (T, top_k))
    out = torch.empty(T, n_experts, dtype=torch.float32, device=x.device)
    check(gated().pe_moe_route_stream_grouped(x.data_ptr(), norm_weight.data_ptr(), _code(norm_weight, "norm_weight"), norm_bias.data_ptr(),
                                              _code(norm_bias, "norm_bias"), float(eps), router.data_ptr(), K, n_experts, top_k,
                                              _ptr(correction), 0 if correction is None else _code(correction, "correction"), n_groups, keep,
                                              group_best, float(factor), out.data_ptr(), _ptr(ids), T, stream_ptr()), "moe_route_stream_grouped")
    return out
