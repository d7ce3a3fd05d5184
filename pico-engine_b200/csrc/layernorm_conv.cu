// Layer norm (weight and bias) of the float32 residual stream, the short causal convolution that is added to
// a sublayer's input, and both of them fused for a block whose two halves read the same stream.
//
//   norm:   y = (x - mean) / sqrt(var + eps) * w + b          var = mean of squared deviations, all in float32
//   conv:   o_t = y_t + sum_j c[:, j] * y_(t - taps + 1 + j)   per channel, zeros before the sequence's start
//
// The convolution reaches back taps - 1 tokens.  Inside a step those are earlier rows of the packed tokens of
// the same sequence; before the step's first token they come from the sequence's state: `state` points at
// entry 0 of [taps - 1][H] float32 values of the sequence's slot (slots are `state_stride` floats apart), entry
// k holding the normed row of the token k + 1 places before the step's first token.  A new sequence's state
// is zero, which is the zero padding.  The state is brought up to date by a kernel of its own (one block per
// sequence), after the kernel that reads it: a block that reads a slot's old entries and another that writes
// new ones would otherwise race.  Steps in which every sequence brings one token update the state in the
// kernel that reads it (each thread rewrites the entries of its own channels after it has read them).
#include "common.cuh"

#define LN_THREADS 256

extern "C" void pe_set_pdl(int on) { pe_pdl_enabled() = on ? 1 : 0; }     // (this library's own copy of the switch)

// mean and 1/sqrt(var + eps) of one float32 row, two passes (the deviations are squared, not x).
__device__ __forceinline__ void row_stats(const float* row, int H, float eps, float* scratch, float& mean, float& rstd) {
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) s += row[i];
    mean = block_sum(s, scratch) / (float)H;
    float v = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float d = row[i] - mean; v = fmaf(d, d, v); }
    rstd = 1.0f / sqrtf(block_sum(v, scratch) / (float)H + eps);
}

// ---------------------------------------------------------------- layer norm alone
template <typename TO>
__global__ void __launch_bounds__(LN_THREADS) layernorm_kernel(const float* x, const int* rows_index, const void* w, int w_dtype,
                                                               const void* b, int b_dtype, float eps, TO* out, int H) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const float* row = x + (size_t)(rows_index ? rows_index[r] : r) * H;
    float mean, rstd;
    row_stats(row, H, eps, scratch, mean, rstd);
    TO* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_f<TO>((row[i] - mean) * rstd * load_as_f(w, w_dtype, i) + load_as_f(b, b_dtype, i));
}

extern "C" int pe_layernorm(const float* x, const int* rows_index, const void* w, int w_dtype, const void* b, int b_dtype,
                            float eps, void* out, int out_dtype, int rows, int H, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == PE_F32) PE_TRY(pe_launch(layernorm_kernel<float>, rows, LN_THREADS, 0, s, x, rows_index, w, w_dtype, b, b_dtype, eps, (float*)out, H));
    else if (out_dtype == PE_BF16) PE_TRY(pe_launch(layernorm_kernel<bf16>, rows, LN_THREADS, 0, s, x, rows_index, w, w_dtype, b, b_dtype, eps, (bf16*)out, H));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- the convolution alone (on float32 normed rows)
// y [T, H] float32.  Thread per (token, channel).
template <typename TO>
__global__ void causal_conv_add_kernel(const float* y, const void* c, int c_dtype, const float* state, long long state_stride,
                                       const int* tok_row, const int* row_first, const int* slots, TO* out, int T, int H, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * H) return;
    const int t = (int)(e / H), ch = (int)(e % H);
    const int b = tok_row[t], i = t - row_first[b];
    const float* st = state + (size_t)slots[b] * state_stride;
    float acc = y[e];
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                       // 0: the token itself
        const float v = back <= i ? y[(size_t)(t - back) * H + ch] : st[(size_t)(back - i - 1) * H + ch];
        acc = fmaf(load_as_f(c, c_dtype, (size_t)ch * taps + j), v, acc);
    }
    out[e] = from_f<TO>(acc);
}

extern "C" int pe_causal_conv_add(const float* y, const void* c, int c_dtype, const float* state, long long state_stride,
                                  const int* tok_row, const int* row_first, const int* slots, void* out, int out_dtype,
                                  int T, int H, int taps, void* stream) {
    if (T <= 0) return 0;
    if (taps < 1) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * H;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == PE_F32) PE_TRY(pe_launch(causal_conv_add_kernel<float>, blocks, 256, 0, s, y, c, c_dtype, state, state_stride, tok_row, row_first, slots, (float*)out, T, H, taps));
    else if (out_dtype == PE_BF16) PE_TRY(pe_launch(causal_conv_add_kernel<bf16>, blocks, 256, 0, s, y, c, c_dtype, state, state_stride, tok_row, row_first, slots, (bf16*)out, T, H, taps));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// New state of every sequence of the step from the normed rows y: entry k <- the row of the step's token
// n - 1 - k, or, where the step brought fewer tokens, the old entry k - n.  Entries are rewritten from the oldest
// to the newest, so an old entry is read before it is overwritten.  Block per sequence, thread per channel.
__global__ void conv_state_update_kernel(const float* y, float* state, long long state_stride, const int* row_first,
                                         const int* row_lens, const int* slots, int H, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int n = row_lens[b], first = row_first[b];
    float* st = state + (size_t)slots[b] * state_stride;
    for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < H; ch += gridDim.y * blockDim.x)
        for (int k = taps - 2; k >= 0; --k)
            st[(size_t)k * H + ch] = k < n ? y[(size_t)(first + n - 1 - k) * H + ch] : st[(size_t)(k - n) * H + ch];
}

extern "C" int pe_conv_state_update(const float* y, float* state, long long state_stride, const int* row_first,
                                    const int* row_lens, const int* slots, int B, int H, int taps, void* stream) {
    if (B <= 0 || taps <= 1) return 0;
    PE_TRY(pe_launch(conv_state_update_kernel, dim3(B, (H + 255) / 256), 256, 0, (cudaStream_t)stream, y, state, state_stride,
                     row_first, row_lens, slots, H, taps));
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- both norms and both convolutions of a parallel block
// The two norms of a parallel block read the same rows, so a row's mean and variance are computed once for both;
// the rows of the taps - 1 tokens before a token are normed again where they are needed (they come from L1 or L2)
// rather than written out in float32 and read back.  Half 2 is skipped when out2 is null.
#define LC_MAX_TAPS 8

struct NormConvHalf {
    const void* w; const void* b; const void* c;     // norm weight, norm bias, convolution taps [H, taps]
    int w_dtype, b_dtype, c_dtype;
    float* state;                                     // entry 0 of this half's state in slot 0
    void* out;
};

#define LC_TOKENS 8

// mean and 1/sqrt(var + eps) of a row by one warp (two passes over the row, which stays in L1)
__device__ __forceinline__ void warp_row_stats(const float* row, int H, float eps, float& mean, float& rstd) {
    const int lane = threadIdx.x & 31;
    float s = 0.f;
    if ((H & 3) == 0) {
        for (int i = lane * 4; i < H; i += 128) { const float4 v = *reinterpret_cast<const float4*>(row + i); s += (v.x + v.y) + (v.z + v.w); }
    } else {
        for (int i = lane; i < H; i += 32) s += row[i];
    }
    mean = warp_sum(s) / (float)H;
    float q = 0.f;
    if ((H & 3) == 0) {
        for (int i = lane * 4; i < H; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
            q += (a * a + b * b) + (c * c + d * d);
        }
    } else {
        for (int i = lane; i < H; i += 32) { const float d = row[i] - mean; q = fmaf(d, d, q); }
    }
    rstd = 1.0f / sqrtf(warp_sum(q) / (float)H + eps);
}

// A block takes `tpb` (up to LC_TOKENS) consecutive packed tokens.  First a warp per row computes the statistics of the
// block's rows and of the taps - 1 rows before them; then a thread keeps the norm weights and taps of its channels in
// registers and walks the block's tokens, the normed values of the taps - 1 tokens before in a sliding window of
// registers (a token whose sequence starts later than the window reaches takes those values from the state instead).
// NC channels a thread at a time: 4 (16-byte loads of x) where H is a multiple of 4, else 1.
template <typename TO, int NC, int MT>        // MT: the most taps this instance takes (registers of the window and the taps)
__global__ void __launch_bounds__(LN_THREADS) dual_layernorm_conv_kernel(
    const float* x, NormConvHalf h1, NormConvHalf h2, long long state_stride, const int* tok_row, const int* row_first,
    const int* slots, float eps, int T, int H, int taps, int tpb, int update_state) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float mean_s[LC_TOKENS + LC_MAX_TAPS], rstd_s[LC_TOKENS + LC_MAX_TAPS];
    __shared__ int idx_s[LC_TOKENS];                       // index of each token within its sequence's tokens of this step
    __shared__ long long slot_s[LC_TOKENS];
    const int t0 = blockIdx.x * tpb, n_tok = min(tpb, T - t0);
    const int warp = threadIdx.x >> 5, halo = taps - 1;
    for (int r = warp; r < n_tok + halo; r += LN_THREADS / 32) {      // row r stands for token t0 - halo + r
        const int t = t0 - halo + r;
        if (t >= 0) {
            float mean, rstd;
            warp_row_stats(x + (size_t)t * H, H, eps, mean, rstd);
            if ((threadIdx.x & 31) == 0) { mean_s[r] = mean; rstd_s[r] = rstd; }
        }
    }
    if (threadIdx.x < n_tok) {
        const int b = tok_row[t0 + threadIdx.x];
        idx_s[threadIdx.x] = t0 + threadIdx.x - row_first[b];
        slot_s[threadIdx.x] = (long long)slots[b] * state_stride;
    }
    __syncthreads();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const NormConvHalf& hh = half ? h2 : h1;
        if (hh.out == nullptr) continue;
        for (int ch = threadIdx.x * NC; ch < H; ch += LN_THREADS * NC) {
            float w[NC], bb[NC], c[MT][NC], win[MT][NC];      // win[d]: the normed value d + 1 tokens back
#pragma unroll
            for (int u = 0; u < NC; ++u) {
                w[u] = load_as_f(hh.w, hh.w_dtype, ch + u); bb[u] = load_as_f(hh.b, hh.b_dtype, ch + u);
#pragma unroll
                for (int d = 0; d < MT; ++d)        // c[d]: the tap that meets the token d places back
                    c[d][u] = d < taps ? load_as_f(hh.c, hh.c_dtype, (size_t)(ch + u) * taps + (taps - 1 - d)) : 0.f;
            }
#pragma unroll
            for (int d = 0; d < MT; ++d) {
                const int t = t0 - 1 - d;
                float xv[NC];
#pragma unroll
                for (int u = 0; u < NC; ++u) xv[u] = 0.f;
                if (d < halo && t >= 0) {
                    if (NC == 4) { const float4 v = *reinterpret_cast<const float4*>(x + (size_t)t * H + ch); xv[0] = v.x; xv[1 % NC] = v.y; xv[2 % NC] = v.z; xv[3 % NC] = v.w; }
                    else xv[0] = x[(size_t)t * H + ch];
                }
#pragma unroll
                for (int u = 0; u < NC; ++u)
                    win[d][u] = (d < halo && t >= 0) ? (xv[u] - mean_s[halo - 1 - d]) * rstd_s[halo - 1 - d] * w[u] + bb[u] : 0.f;
            }
            for (int k = 0; k < n_tok; ++k) {
                const int t = t0 + k, i = idx_s[k];
                float* st = hh.state + slot_s[k];
                float xv[NC], own[NC], acc[NC];
                if (NC == 4) { const float4 v = *reinterpret_cast<const float4*>(x + (size_t)t * H + ch); xv[0] = v.x; xv[1 % NC] = v.y; xv[2 % NC] = v.z; xv[3 % NC] = v.w; }
                else xv[0] = x[(size_t)t * H + ch];
#pragma unroll
                for (int u = 0; u < NC; ++u) { own[u] = (xv[u] - mean_s[k + halo]) * rstd_s[k + halo] * w[u] + bb[u]; acc[u] = own[u]; }
#pragma unroll
                for (int u = 0; u < NC; ++u) acc[u] = fmaf(c[0][u], own[u], acc[u]);
#pragma unroll
                for (int back = 1; back < MT; ++back) {
                    if (back < taps) {
#pragma unroll
                        for (int u = 0; u < NC; ++u) {
                            const float v = back <= i ? win[back - 1][u] : st[(size_t)(back - i - 1) * H + ch + u];
                            acc[u] = fmaf(c[back][u], v, acc[u]);
                        }
                    }
                }
                TO* o = (TO*)hh.out + (size_t)t * H + ch;
                if (NC == 4 && sizeof(TO) == 2) {            // four bfloat16 as one 8-byte store
                    const __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc[0], acc[1 % NC]), hi2 = __floats2bfloat162_rn(acc[2 % NC], acc[3 % NC]);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&lo2); pk.y = *reinterpret_cast<const uint32_t*>(&hi2);
                    *reinterpret_cast<uint2*>(o) = pk;
                } else if (NC == 4) {
                    *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1 % NC], acc[2 % NC], acc[3 % NC]);
                } else {
                    o[0] = from_f<TO>(acc[0]);
                }
                if (update_state) {                          // the sequence brings this one token: shift its entries, newest first
#pragma unroll
                    for (int u = 0; u < NC; ++u) {
                        for (int e = taps - 2; e > 0; --e) st[(size_t)e * H + ch + u] = st[(size_t)(e - 1) * H + ch + u];
                        if (taps > 1) st[ch + u] = own[u];
                    }
                }
#pragma unroll
                for (int d = MT - 1; d > 0; --d) {
#pragma unroll
                    for (int u = 0; u < NC; ++u) win[d][u] = win[d - 1][u];
                }
#pragma unroll
                for (int u = 0; u < NC; ++u) win[0][u] = own[u];
            }
        }
    }
}

// The state after a step that brought several tokens to some sequence: block per sequence.
__global__ void __launch_bounds__(LN_THREADS) dual_layernorm_state_kernel(
    const float* x, NormConvHalf h1, NormConvHalf h2, long long state_stride, const int* row_first, const int* row_lens,
    const int* slots, float eps, int H, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int b = blockIdx.x;
    const int n = row_lens[b], first = row_first[b];
    const size_t slot_off = (size_t)slots[b] * state_stride;
    for (int k = taps - 2; k >= 0; --k) {
        float mean = 0.f, rstd = 0.f;
        const float* row = x + (size_t)(first + n - 1 - k) * H;
        if (k < n) row_stats(row, H, eps, scratch, mean, rstd);
        for (int half = 0; half < 2; ++half) {
            const NormConvHalf& hh = half ? h2 : h1;
            if (hh.out == nullptr) continue;
            float* st = hh.state + slot_off;
            for (int ch = threadIdx.x; ch < H; ch += blockDim.x)
                st[(size_t)k * H + ch] = k < n ? (row[ch] - mean) * rstd * load_as_f(hh.w, hh.w_dtype, ch) + load_as_f(hh.b, hh.b_dtype, ch)
                                               : st[(size_t)(k - n) * H + ch];
        }
    }
}

extern "C" int pe_dual_layernorm_conv(const float* x, const void* w1, int w1_dtype, const void* b1, int b1_dtype, const void* c1,
                                      int c1_dtype, float* state1, void* out1, const void* w2, int w2_dtype, const void* b2,
                                      int b2_dtype, const void* c2, int c2_dtype, float* state2, void* out2, int out_dtype,
                                      long long state_stride, const int* tok_row, const int* row_first, const int* row_lens,
                                      const int* slots, float eps, int T, int B, int H, int taps, int one_token_each, void* stream) {
    if (T <= 0) return 0;
    if (taps < 1 || taps > LC_MAX_TAPS || out1 == nullptr) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    NormConvHalf h1 = {w1, b1, c1, w1_dtype, b1_dtype, c1_dtype, state1, out1};
    NormConvHalf h2 = {w2, b2, c2, w2_dtype, b2_dtype, c2_dtype, state2, out2};
    const int inline_update = one_token_each ? 1 : 0;
    // tokens a block: as many as leave a few blocks for every SM
    int tpb = LC_TOKENS;
    while (tpb > 1 && (T + tpb - 1) / tpb < 148) tpb >>= 1;
    const int blocks = (T + tpb - 1) / tpb;
    const bool vec = (H & 3) == 0 && !(((uintptr_t)x | (uintptr_t)out1 | (uintptr_t)out2) & 15);
#define LC_LAUNCH(TO, NC, MT) PE_TRY(pe_launch(dual_layernorm_conv_kernel<TO, NC, MT>, blocks, LN_THREADS, 0, s, x, h1, h2, state_stride, \
                                               tok_row, row_first, slots, eps, T, H, taps, tpb, inline_update))
    if (out_dtype == PE_F32) {
        if (vec) { if (taps <= 4) LC_LAUNCH(float, 4, 4); else LC_LAUNCH(float, 4, LC_MAX_TAPS); }
        else { if (taps <= 4) LC_LAUNCH(float, 1, 4); else LC_LAUNCH(float, 1, LC_MAX_TAPS); }
    } else if (out_dtype == PE_BF16) {
        if (vec) { if (taps <= 4) LC_LAUNCH(bf16, 4, 4); else LC_LAUNCH(bf16, 4, LC_MAX_TAPS); }
        else { if (taps <= 4) LC_LAUNCH(bf16, 1, 4); else LC_LAUNCH(bf16, 1, LC_MAX_TAPS); }
    }
#undef LC_LAUNCH
    PE_LAUNCH_CHECK();
    if (!inline_update && taps > 1) {
        PE_TRY(pe_launch(dual_layernorm_state_kernel, B, LN_THREADS, 0, s, x, h1, h2, state_stride, row_first, row_lens, slots, eps, H, taps));
        PE_LAUNCH_CHECK();
    }
    return 0;
}

// ---------------------------------------------------------------- a sublayer's output, layer-normed, into the stream
// x[t] += layernorm(y[t]) * w + b on the float32 stream (y float32 or bfloat16); with `out` also out[t] = layernorm(x[t]) * w2 + b2
// of the row as it then stands (the norm in front of the sublayer that reads the stream next), stored in out's dtype.  Both norms
// in float32, two passes each (mean, then squared deviations).  A block a token; a thread rereads only entries it wrote itself.
template <typename TY, typename TO>
__global__ void __launch_bounds__(LN_THREADS) layernorm_add_kernel(float* x, const TY* y, const void* w, int w_dtype, const void* b, int b_dtype,
                                                                   float eps, int H, const void* w2, int w2_dtype, const void* b2, int b2_dtype,
                                                                   float eps2, TO* out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const TY* yr = y + (size_t)blockIdx.x * H;
    float* xr = x + (size_t)blockIdx.x * H;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) s += to_f(yr[i]);
    const float mean = block_sum(s, scratch) / (float)H;
    float v = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float d = to_f(yr[i]) - mean; v = fmaf(d, d, v); }
    const float rstd = 1.0f / sqrtf(block_sum(v, scratch) / (float)H + eps);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float n = xr[i] + ((to_f(yr[i]) - mean) * rstd * load_as_f(w, w_dtype, i) + load_as_f(b, b_dtype, i));
        xr[i] = n;
        s2 += n;
    }
    if (!out) return;
    const float mean2 = block_sum(s2, scratch) / (float)H;
    float v2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float d = xr[i] - mean2; v2 = fmaf(d, d, v2); }
    const float rstd2 = 1.0f / sqrtf(block_sum(v2, scratch) / (float)H + eps2);
    TO* o = out + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_f<TO>((xr[i] - mean2) * rstd2 * load_as_f(w2, w2_dtype, i) + load_as_f(b2, b2_dtype, i));
}

// Rows of up to 4096 entries, a multiple of 4, 16-byte aligned: a thread keeps its entries of y and x in registers (NV runs of four),
// so that every row is read once and written once.
__device__ __forceinline__ float4 ln_load4(const float* p, size_t i4) { return reinterpret_cast<const float4*>(p)[i4]; }
__device__ __forceinline__ float4 ln_load4(const bf16* p, size_t i4) {
    const uint2 r = reinterpret_cast<const uint2*>(p)[i4];
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 ln_load4_as_f(const void* p, int dtype, size_t i4) {
    return dtype == PE_F32 ? ln_load4((const float*)p, i4) : ln_load4((const bf16*)p, i4);
}
__device__ __forceinline__ void ln_store4(float* p, size_t i4, float4 v) { reinterpret_cast<float4*>(p)[i4] = v; }
__device__ __forceinline__ void ln_store4(bf16* p, size_t i4, float4 v) {
    uint2 r;
    *reinterpret_cast<__nv_bfloat162*>(&r.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&r.y) = __floats2bfloat162_rn(v.z, v.w);
    reinterpret_cast<uint2*>(p)[i4] = r;
}

template <typename TY, typename TO, int NV>
__global__ void __launch_bounds__(LN_THREADS) layernorm_add_vec_kernel(float* x, const TY* y, const void* w, int w_dtype, const void* b, int b_dtype,
                                                                       float eps, int H, const void* w2, int w2_dtype, const void* b2, int b2_dtype,
                                                                       float eps2, TO* out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int n4 = H / 4;
    const size_t row4 = (size_t)blockIdx.x * n4;
    float4 yv[NV], xv[NV];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = threadIdx.x + LN_THREADS * v;
        if (i < n4) {
            yv[v] = ln_load4(y, row4 + i);
            xv[v] = ln_load4(x, row4 + i);
            s += (yv[v].x + yv[v].y) + (yv[v].z + yv[v].w);
        }
    }
    const float mean = block_sum(s, scratch) / (float)H;
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v)
        if (threadIdx.x + LN_THREADS * v < n4) {
            const float a = yv[v].x - mean, c = yv[v].y - mean, d = yv[v].z - mean, e = yv[v].w - mean;
            q += (a * a + c * c) + (d * d + e * e);
        }
    const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)H + eps);
    float s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = threadIdx.x + LN_THREADS * v;
        if (i < n4) {
            const float4 wv = ln_load4_as_f(w, w_dtype, i), bv = ln_load4_as_f(b, b_dtype, i);
            xv[v].x += fmaf((yv[v].x - mean) * rstd, wv.x, bv.x); xv[v].y += fmaf((yv[v].y - mean) * rstd, wv.y, bv.y);
            xv[v].z += fmaf((yv[v].z - mean) * rstd, wv.z, bv.z); xv[v].w += fmaf((yv[v].w - mean) * rstd, wv.w, bv.w);
            ln_store4(x, row4 + i, xv[v]);
            s2 += (xv[v].x + xv[v].y) + (xv[v].z + xv[v].w);
        }
    }
    if (!out) return;
    const float mean2 = block_sum(s2, scratch) / (float)H;
    float q2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v)
        if (threadIdx.x + LN_THREADS * v < n4) {
            const float a = xv[v].x - mean2, c = xv[v].y - mean2, d = xv[v].z - mean2, e = xv[v].w - mean2;
            q2 += (a * a + c * c) + (d * d + e * e);
        }
    const float rstd2 = 1.0f / sqrtf(block_sum(q2, scratch) / (float)H + eps2);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = threadIdx.x + LN_THREADS * v;
        if (i < n4) {
            const float4 wv = ln_load4_as_f(w2, w2_dtype, i), bv = ln_load4_as_f(b2, b2_dtype, i);
            ln_store4(out, row4 + i, make_float4(fmaf((xv[v].x - mean2) * rstd2, wv.x, bv.x), fmaf((xv[v].y - mean2) * rstd2, wv.y, bv.y),
                                                 fmaf((xv[v].z - mean2) * rstd2, wv.z, bv.z), fmaf((xv[v].w - mean2) * rstd2, wv.w, bv.w)));
        }
    }
}

extern "C" int pe_layernorm_add(float* x, const void* y, int y_dtype, const void* w, int w_dtype, const void* b, int b_dtype, float eps,
                                int T, int H, const void* w2, int w2_dtype, const void* b2, int b2_dtype, float eps2, void* out,
                                int out_dtype, void* stream) {
    if (T <= 0) return 0;
    if (out && (!w2 || !b2)) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define LNA(TY, TO) PE_TRY(pe_launch(layernorm_add_kernel<TY, TO>, T, LN_THREADS, 0, s, x, (const TY*)y, w, w_dtype, b, b_dtype, eps, H, w2, \
                                     w2_dtype, b2, b2_dtype, eps2, (TO*)out))
    const bool obf = out && out_dtype == PE_BF16;
    if (out && out_dtype != PE_BF16 && out_dtype != PE_F32) return PE_ERR_UNSUPPORTED;
    const uintptr_t all = (uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)b | (uintptr_t)w2 | (uintptr_t)b2 | (uintptr_t)out;
    if (H % 4 == 0 && H <= 4 * 4 * LN_THREADS && !(all & 15) && (y_dtype == PE_F32 || y_dtype == PE_BF16)) {
        const int nv = (H / 4 + LN_THREADS - 1) / LN_THREADS;
#define LNV(TY, TO, NV) PE_TRY(pe_launch(layernorm_add_vec_kernel<TY, TO, NV>, T, LN_THREADS, 0, s, x, (const TY*)y, w, w_dtype, b, b_dtype, eps, H, \
                                         w2, w2_dtype, b2, b2_dtype, eps2, (TO*)out))
#define LNV_N(TY, TO) do { if (nv <= 1) LNV(TY, TO, 1); else if (nv == 2) LNV(TY, TO, 2); else LNV(TY, TO, 4); } while (0)
        if (y_dtype == PE_F32) { if (obf) LNV_N(float, bf16); else LNV_N(float, float); }
        else { if (obf) LNV_N(bf16, bf16); else LNV_N(bf16, float); }
#undef LNV_N
#undef LNV
        PE_LAUNCH_CHECK();
        return 0;
    }
    if (y_dtype == PE_F32) { if (obf) LNA(float, bf16); else LNA(float, float); }
    else if (y_dtype == PE_BF16) { if (obf) LNA(bf16, bf16); else LNA(bf16, float); }
    else return PE_ERR_UNSUPPORTED;
#undef LNA
    PE_LAUNCH_CHECK();
    return 0;
}
