// Small kernels around gated mixers and routed feed-forwards: rotation of neighbouring pairs with a unit norm of
// every head and the cache write; a norm over groups of channels times a gate; the sum of several normed
// branches into the residual stream; a scaled residual sum; vectors added to the stream; a gated activation
// with a weight per group of columns; the choice of experts.
#include "common.cuh"

extern "C" void pe_set_pdl(int on) { pe_pdl_enabled() = on ? 1 : 0; }     // (this library's own copy of the switch)

__device__ __forceinline__ float go_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float go_gelu_tanh(float v) {
    return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}
// activations: 0 none, 1 sigmoid, 2 silu, 3 gelu (tanh form), 4 the square of relu
__device__ __forceinline__ float go_act(float v, int act) {
    return act == 1 ? go_sigmoid(v) : act == 2 ? v * go_sigmoid(v) : act == 3 ? go_gelu_tanh(v) : act == 4 ? (v > 0.f ? v * v : 0.f) : v;
}

// ---------------------------------------------------------------- rotation of pairs, unit norm, cache write
// qkv [T, ld] in the step's dtype, a row = H*D query | G*D key | G*Dv value entries (| whatever else the product made).  In every query and key head the entries (2i, 2i+1), 2i+1 < rot_dims,
// are turned by the angle pos * freq[i]: (u, v) -> (u cos - v sin, v cos + u sin); then (norm != 0) the head is divided
// by sqrt(mean(head^2) + eps).  The heads are rewritten in place; keys and values also go to their cache pages.
// A warp a head; a lane keeps its entries of the head in registers (D <= 256).
template <typename T, int NE>
__global__ void __launch_bounds__(256) rotary_norm_store_kernel(T* qkv, int ld, int H, int G, int D, int Dv, const float* freq, int rot_dims,
                                                                int norm, float eps, const int* tok_pos, const int* tok_row,
                                                                T* k_pool, T* v_pool, const int* table, int table_stride, int store) {
    pdl_launch_dependents();
    __shared__ float s_cos[128], s_sin[128];                               // the token's angles, the same for all its heads
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    T* row = qkv + (size_t)t * ld;
    const int pos = tok_pos[t];
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) sincosf((float)pos * freq[i], &s_sin[i], &s_cos[i]);
    long long page = -1;
    if (store) page = table[(size_t)tok_row[t] * table_stride + pos / PE_PAGE];
    __syncthreads();
    for (int u = warp; u < H + 2 * G; u += (int)(blockDim.x >> 5)) {
        if (u < H + G) {
            T* v = row + (size_t)u * D;
            float val[NE];
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < NE; ++e) {
                const int d = lane + 32 * e;
                float f = 0.f;
                if (d < D) {
                    f = to_f(v[d]);
                    if ((d | 1) < rot_dims) {
                        const float sn = s_sin[d >> 1], cs = s_cos[d >> 1];
                        const float other = to_f(v[d ^ 1]);
                        f = (d & 1) ? fmaf(f, cs, other * sn) : fmaf(f, cs, -other * sn);
                    }
                }
                val[e] = f;
                ss = fmaf(f, f, ss);
            }
            const float rstd = norm ? 1.0f / sqrtf(warp_sum(ss) / (float)D + eps) : 1.0f;
            __syncwarp();                                                  // every lane has read its partners
            T* dst = (u >= H && store && page >= 0) ? k_pool + (((size_t)page * G + (u - H)) * PE_PAGE + pos % PE_PAGE) * D : nullptr;
#pragma unroll
            for (int e = 0; e < NE; ++e) {
                const int d = lane + 32 * e;
                if (d < D) {
                    const T o = from_f<T>(val[e] * rstd);
                    v[d] = o;
                    if (dst) dst[d] = o;
                }
            }
        } else if (store && page >= 0) {
            const int c = u - H - G;
            const T* v = row + (size_t)(H + G) * D + (size_t)c * Dv;
            T* dst = v_pool + (((size_t)page * G + c) * PE_PAGE + pos % PE_PAGE) * Dv;
            for (int d = lane; d < Dv; d += 32) dst[d] = v[d];
        }
    }
}

// bfloat16 with even D, Dv and ld: a lane takes whole pairs (4-byte accesses), so a pair is rotated inside one lane.
template <int NP>
__global__ void __launch_bounds__(256) rotary_norm_store_pairs_kernel(bf16* qkv, int ld, int H, int G, int D, int Dv, const float* freq,
                                                                      int rot_dims, int norm, float eps, const int* tok_pos,
                                                                      const int* tok_row, bf16* k_pool, bf16* v_pool, const int* table,
                                                                      int table_stride, int store) {
    pdl_launch_dependents();
    __shared__ float s_cos[128], s_sin[128];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    bf16* row = qkv + (size_t)t * ld;
    const int pos = tok_pos[t];
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) sincosf((float)pos * freq[i], &s_sin[i], &s_cos[i]);
    long long page = -1;
    if (store) page = table[(size_t)tok_row[t] * table_stride + pos / PE_PAGE];
    __syncthreads();
    const int pairs = D / 2;
    for (int u = warp; u < H + 2 * G; u += (int)(blockDim.x >> 5)) {
        if (u < H + G) {
            __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(row + (size_t)u * D);
            float2 val[NP];
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < NP; ++e) {
                const int i = lane + 32 * e;
                float2 f = make_float2(0.f, 0.f);
                if (i < pairs) {
                    f = __bfloat1622float2(v[i]);
                    if (2 * i + 1 < rot_dims) {
                        const float sn = s_sin[i], cs = s_cos[i];
                        f = make_float2(fmaf(f.x, cs, -f.y * sn), fmaf(f.y, cs, f.x * sn));
                    }
                }
                val[e] = f;
                ss += f.x * f.x + f.y * f.y;
            }
            const float rstd = norm ? 1.0f / sqrtf(warp_sum(ss) / (float)D + eps) : 1.0f;
            __nv_bfloat162* dst = (u >= H && store && page >= 0)
                ? reinterpret_cast<__nv_bfloat162*>(k_pool + (((size_t)page * G + (u - H)) * PE_PAGE + pos % PE_PAGE) * D) : nullptr;
#pragma unroll
            for (int e = 0; e < NP; ++e) {
                const int i = lane + 32 * e;
                if (i < pairs) {
                    const __nv_bfloat162 o = __floats2bfloat162_rn(val[e].x * rstd, val[e].y * rstd);
                    v[i] = o;
                    if (dst) dst[i] = o;
                }
            }
        } else if (store && page >= 0) {
            const int c = u - H - G;
            const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(row + (size_t)(H + G) * D + (size_t)c * Dv);
            __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(v_pool + (((size_t)page * G + c) * PE_PAGE + pos % PE_PAGE) * Dv);
            for (int d = lane; d < Dv / 2; d += 32) dst[d] = v[d];
        }
    }
}

extern "C" int pe_rotary_norm_store(void* qkv, int dtype, int ld, int T, int H, int G, int D, int Dv, const float* freq, int rot_dims,
                                    int norm, float eps, const int* tok_pos, const int* tok_row, void* k_pool, void* v_pool,
                                    const int* table, int table_stride, int store, void* stream) {
    if (T <= 0) return 0;
    if (D > 256 || rot_dims > D || (rot_dims & 1) || (rot_dims > 0 && !freq) || ld < (H + G) * D + G * Dv) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H + 2 * G > 16 ? 256 : 128;                        // a warp walks at most about four heads
    if (dtype == PE_BF16 && D % 2 == 0 && Dv % 2 == 0 && ld % 2 == 0 && !(((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) & 3)) {
#define ROT_PAIRS(NP) PE_TRY(pe_launch(rotary_norm_store_pairs_kernel<NP>, T, threads, 0, s, (bf16*)qkv, ld, H, G, D, Dv, freq, rot_dims, norm, eps, \
                                       tok_pos, tok_row, (bf16*)k_pool, (bf16*)v_pool, table, table_stride, store))
        if (D <= 64) ROT_PAIRS(1); else if (D <= 128) ROT_PAIRS(2); else ROT_PAIRS(4);
#undef ROT_PAIRS
        PE_LAUNCH_CHECK();
        return 0;
    }
#define ROT_LAUNCH(TT, NE) PE_TRY(pe_launch(rotary_norm_store_kernel<TT, NE>, T, threads, 0, s, (TT*)qkv, ld, H, G, D, Dv, freq, rot_dims, norm, eps, \
                                            tok_pos, tok_row, (TT*)k_pool, (TT*)v_pool, table, table_stride, store))
    if (dtype == PE_F32) {
        if (D <= 64) ROT_LAUNCH(float, 2); else if (D <= 128) ROT_LAUNCH(float, 4); else ROT_LAUNCH(float, 8);
    } else if (dtype == PE_BF16) {
        if (D <= 64) ROT_LAUNCH(bf16, 2); else if (D <= 128) ROT_LAUNCH(bf16, 4); else ROT_LAUNCH(bf16, 8);
    } else return PE_ERR_UNSUPPORTED;
#undef ROT_LAUNCH
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- rotation of halves, blended values, cache write
// The same rows, with the other layout of a rotation: entry i < rot_dims / 2 of a query or key head pairs with entry i + rot_dims / 2;
// the pair (u, v) becomes (u c - v s, v c + u s) with c = magnitude * cos(pos * freq[i]), s = magnitude * sin(pos * freq[i]); entries
// from rot_dims on stay.  Then (norm != 0) the head is divided by sqrt(mean(head^2) + eps).  Values: with `blend` (rows [T, blend_ld]
// of G * Dv entries in the step's dtype, the values another layer made of the same tokens) every value becomes
// (1 - lambda) v + lambda blend[t], lambda one stored number; formed in float32 and rounded once.  Heads and values are rewritten in
// place; keys and values also go to their cache pages.  A warp a head; a lane keeps its entries of the head in registers (D <= 256).
template <typename T, int NE>
__global__ void __launch_bounds__(256) rotary_half_store_kernel(T* qkv, int ld, int H, int G, int D, int Dv, const float* freq, int rot_dims,
                                                                float magnitude, int norm, float eps, const int* tok_pos, const int* tok_row,
                                                                T* k_pool, T* v_pool, const int* table, int table_stride, int store,
                                                                const T* blend, int blend_ld, const void* lambda, int lambda_dtype) {
    pdl_launch_dependents();
    __shared__ float s_cos[128], s_sin[128];                               // the token's angles, the same for all its heads
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    T* row = qkv + (size_t)t * ld;
    const int pos = tok_pos[t];
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * freq[i], &sn, &cs);
        s_sin[i] = sn * magnitude; s_cos[i] = cs * magnitude;
    }
    long long page = -1;
    if (store) page = table[(size_t)tok_row[t] * table_stride + pos / PE_PAGE];
    const float lam = blend ? load_as_f(lambda, lambda_dtype, 0) : 0.f;
    __syncthreads();
    for (int u = warp; u < H + 2 * G; u += (int)(blockDim.x >> 5)) {
        if (u < H + G) {
            T* v = row + (size_t)u * D;
            float val[NE];
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < NE; ++e) {
                const int d = lane + 32 * e;
                float f = 0.f;
                if (d < D) {
                    f = to_f(v[d]);
                    if (d < rot_dims) {
                        const bool low = d < half;
                        const int i = low ? d : d - half;
                        const float other = to_f(v[low ? d + half : d - half]);
                        f = low ? fmaf(f, s_cos[i], -other * s_sin[i]) : fmaf(f, s_cos[i], other * s_sin[i]);
                    }
                }
                val[e] = f;
                ss = fmaf(f, f, ss);
            }
            const float rstd = norm ? 1.0f / sqrtf(warp_sum(ss) / (float)D + eps) : 1.0f;
            __syncwarp();                                                  // every lane has read its partners
            T* dst = (u >= H && store && page >= 0) ? k_pool + (((size_t)page * G + (u - H)) * PE_PAGE + pos % PE_PAGE) * D : nullptr;
#pragma unroll
            for (int e = 0; e < NE; ++e) {
                const int d = lane + 32 * e;
                if (d < D) {
                    const T o = from_f<T>(val[e] * rstd);
                    v[d] = o;
                    if (dst) dst[d] = o;
                }
            }
        } else {
            const int c = u - H - G;
            T* v = row + (size_t)(H + G) * D + (size_t)c * Dv;
            T* dst = (store && page >= 0) ? v_pool + (((size_t)page * G + c) * PE_PAGE + pos % PE_PAGE) * Dv : nullptr;
            const T* other = blend ? blend + (size_t)t * blend_ld + (size_t)c * Dv : nullptr;
            if (!other && !dst) continue;
            for (int d = lane; d < Dv; d += 32) {
                T o = v[d];
                if (other) { o = from_f<T>(fmaf(lam, to_f(other[d]), (1.0f - lam) * to_f(o))); v[d] = o; }
                if (dst) dst[d] = o;
            }
        }
    }
}

// bfloat16 with even D, Dv, ld and rot_dims / 2: a lane takes whole pairs of neighbours (4-byte accesses); the partners of a lane's
// two entries are the two neighbours half the rotated entries away.
template <int NP>
__global__ void __launch_bounds__(256) rotary_half_store_pairs_kernel(bf16* qkv, int ld, int H, int G, int D, int Dv, const float* freq, int rot_dims,
                                                                      float magnitude, int norm, float eps, const int* tok_pos, const int* tok_row,
                                                                      bf16* k_pool, bf16* v_pool, const int* table, int table_stride, int store,
                                                                      const bf16* blend, int blend_ld, const void* lambda, int lambda_dtype) {
    pdl_launch_dependents();
    __shared__ float s_cos[128], s_sin[128];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    bf16* row = qkv + (size_t)t * ld;
    const int pos = tok_pos[t];
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * freq[i], &sn, &cs);
        s_sin[i] = sn * magnitude; s_cos[i] = cs * magnitude;
    }
    long long page = -1;
    if (store) page = table[(size_t)tok_row[t] * table_stride + pos / PE_PAGE];
    const float lam = blend ? load_as_f(lambda, lambda_dtype, 0) : 0.f;
    __syncthreads();
    const int pairs = D / 2;
    for (int u = warp; u < H + 2 * G; u += (int)(blockDim.x >> 5)) {
        if (u < H + G) {
            __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(row + (size_t)u * D);
            float2 val[NP];
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < NP; ++e) {
                const int i = lane + 32 * e, d = 2 * i;
                float2 f = make_float2(0.f, 0.f);
                if (i < pairs) {
                    f = __bfloat1622float2(v[i]);
                    if (d < rot_dims) {
                        const bool low = d < half;
                        const int a = low ? d : d - half;                  // the angle's index of the first of the two entries
                        const float2 o = __bfloat1622float2(v[low ? i + half / 2 : i - half / 2]);
                        f = low ? make_float2(fmaf(f.x, s_cos[a], -o.x * s_sin[a]), fmaf(f.y, s_cos[a + 1], -o.y * s_sin[a + 1]))
                                : make_float2(fmaf(f.x, s_cos[a], o.x * s_sin[a]), fmaf(f.y, s_cos[a + 1], o.y * s_sin[a + 1]));
                    }
                }
                val[e] = f;
                ss += f.x * f.x + f.y * f.y;
            }
            const float rstd = norm ? 1.0f / sqrtf(warp_sum(ss) / (float)D + eps) : 1.0f;
            __syncwarp();                                                  // every lane has read its partners
            __nv_bfloat162* dst = (u >= H && store && page >= 0)
                ? reinterpret_cast<__nv_bfloat162*>(k_pool + (((size_t)page * G + (u - H)) * PE_PAGE + pos % PE_PAGE) * D) : nullptr;
#pragma unroll
            for (int e = 0; e < NP; ++e) {
                const int i = lane + 32 * e;
                if (i < pairs) {
                    const __nv_bfloat162 o = __floats2bfloat162_rn(val[e].x * rstd, val[e].y * rstd);
                    v[i] = o;
                    if (dst) dst[i] = o;
                }
            }
        } else {
            const int c = u - H - G;
            __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(row + (size_t)(H + G) * D + (size_t)c * Dv);
            __nv_bfloat162* dst = (store && page >= 0)
                ? reinterpret_cast<__nv_bfloat162*>(v_pool + (((size_t)page * G + c) * PE_PAGE + pos % PE_PAGE) * Dv) : nullptr;
            const __nv_bfloat162* other = blend ? reinterpret_cast<const __nv_bfloat162*>(blend + (size_t)t * blend_ld + (size_t)c * Dv) : nullptr;
            if (!other && !dst) continue;
            for (int d = lane; d < Dv / 2; d += 32) {
                __nv_bfloat162 o = v[d];
                if (other) {
                    const float2 a = __bfloat1622float2(o), b = __bfloat1622float2(other[d]);
                    o = __floats2bfloat162_rn(fmaf(lam, b.x, (1.0f - lam) * a.x), fmaf(lam, b.y, (1.0f - lam) * a.y));
                    v[d] = o;
                }
                if (dst) dst[d] = o;
            }
        }
    }
}

extern "C" int pe_rotary_half_store(void* qkv, int dtype, int ld, int T, int H, int G, int D, int Dv, const float* freq, int rot_dims,
                                    float magnitude, int norm, float eps, const int* tok_pos, const int* tok_row, void* k_pool, void* v_pool,
                                    const int* table, int table_stride, int store, const void* blend, int blend_ld, const void* lambda,
                                    int lambda_dtype, void* stream) {
    if (T <= 0) return 0;
    if (D > 256 || rot_dims > D || (rot_dims & 1) || (rot_dims > 0 && !freq) || ld < (H + G) * D + G * Dv || (blend && (!lambda || blend_ld < G * Dv)))
        return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H + 2 * G > 16 ? 256 : 128;
    if (dtype == PE_BF16 && D % 2 == 0 && Dv % 2 == 0 && ld % 2 == 0 && (rot_dims / 2) % 2 == 0 && blend_ld % 2 == 0 &&
        !(((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)blend) & 3)) {
#define ROTH_PAIRS(NP) PE_TRY(pe_launch(rotary_half_store_pairs_kernel<NP>, T, threads, 0, s, (bf16*)qkv, ld, H, G, D, Dv, freq, rot_dims, magnitude, norm, \
                                        eps, tok_pos, tok_row, (bf16*)k_pool, (bf16*)v_pool, table, table_stride, store, (const bf16*)blend, blend_ld,  \
                                        lambda, lambda_dtype))
        if (D <= 64) ROTH_PAIRS(1); else if (D <= 128) ROTH_PAIRS(2); else ROTH_PAIRS(4);
#undef ROTH_PAIRS
        PE_LAUNCH_CHECK();
        return 0;
    }
#define ROTH_LAUNCH(TT, NE) PE_TRY(pe_launch(rotary_half_store_kernel<TT, NE>, T, threads, 0, s, (TT*)qkv, ld, H, G, D, Dv, freq, rot_dims, magnitude, \
                                             norm, eps, tok_pos, tok_row, (TT*)k_pool, (TT*)v_pool, table, table_stride, store, (const TT*)blend,      \
                                             blend_ld, lambda, lambda_dtype))
    if (dtype == PE_F32) {
        if (D <= 64) ROTH_LAUNCH(float, 2); else if (D <= 128) ROTH_LAUNCH(float, 4); else ROTH_LAUNCH(float, 8);
    } else if (dtype == PE_BF16) {
        if (D <= 64) ROTH_LAUNCH(bf16, 2); else if (D <= 128) ROTH_LAUNCH(bf16, 4); else ROTH_LAUNCH(bf16, 8);
    } else return PE_ERR_UNSUPPORTED;
#undef ROTH_LAUNCH
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- norm over groups of channels, times a gate
// in [T, C] (float32 or the step's dtype); group > 0: every run of `group` channels is divided by
// sqrt(mean(run^2) + eps) and multiplied by weight[channel % group]; then (gate != null) by act(gate[t, g_off + c]) of
// gate [T, g_ld].  out [T, C] in the step's dtype.  A block a (token, group).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gated_norm_kernel(const TI* in, int C, int group, const void* weight, int w_dtype, float eps,
                                                         const TO* gate, int g_ld, int g_off, int gate_act, TO* out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x, n = group > 0 ? group : C, c0 = blockIdx.y * n;
    const TI* src = in + (size_t)t * C + c0;
    float rstd = 1.f;
    if (group > 0) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) { const float f = to_f(src[i]); ss = fmaf(f, f, ss); }
        rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float f = to_f(src[i]) * rstd;
        if (group > 0 && weight) f *= load_as_f(weight, w_dtype, i);
        if (gate) f *= go_act(to_f(gate[(size_t)t * g_ld + g_off + c0 + i]), gate_act);
        out[(size_t)t * C + c0 + i] = from_f<TO>(f);
    }
}

// The same for groups of up to 512 channels: a warp a (token, group), eight of them a block, the run kept in registers.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gated_norm_warp_kernel(const TI* in, int C, int group, const void* weight, int w_dtype, float eps,
                                                              const TO* gate, int g_ld, int g_off, int gate_act, TO* out, long long runs) {
    pdl_launch_dependents();
    pdl_wait();
    const long long run = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (run >= runs) return;
    const int per_row = C / group;
    const size_t t = (size_t)(run / per_row);
    const int c0 = (int)(run % per_row) * group;
    const TI* src = in + t * C + c0;
    float val[16];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int i = lane + 32 * e;
        val[e] = i < group ? to_f(src[i]) : 0.f;
        ss = fmaf(val[e], val[e], ss);
    }
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)group + eps);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int i = lane + 32 * e;
        if (i < group) {
            float f = val[e] * rstd;
            if (weight) f *= load_as_f(weight, w_dtype, i);
            if (gate) f *= go_act(to_f(gate[t * g_ld + g_off + c0 + i]), gate_act);
            out[t * C + c0 + i] = from_f<TO>(f);
        }
    }
}

// float32 rows in, bfloat16 out and gate, group a multiple of 4 and all rows aligned: four channels a lane with 16-byte reads of the
// row and 8-byte reads and writes of gate and result; the run stays in registers between the sum of squares and the result.
// WARP: a warp a run of up to 512 channels, eight runs a block; else a block a run of up to 4096 channels.
__device__ __forceinline__ void gn_store4(bf16* out, const bf16* gate, float4 f, int gate_act) {
    if (gate) {
        const uint2 g = *reinterpret_cast<const uint2*>(gate);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        const float2 a = __bfloat1622float2(g2[0]), b = __bfloat1622float2(g2[1]);
        f.x *= go_act(a.x, gate_act); f.y *= go_act(a.y, gate_act); f.z *= go_act(b.x, gate_act); f.w *= go_act(b.y, gate_act);
    }
    uint2 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
    o2[0] = __floats2bfloat162_rn(f.x, f.y); o2[1] = __floats2bfloat162_rn(f.z, f.w);
    *reinterpret_cast<uint2*>(out) = o;
}

template <bool WARP>
__global__ void __launch_bounds__(256) gated_norm_x4_kernel(const float* in, int C, int group, const void* weight, int w_dtype, float eps,
                                                            const bf16* gate, int g_ld, int g_off, int gate_act, bf16* out, long long runs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const long long run = WARP ? (long long)blockIdx.x * 8 + (threadIdx.x >> 5) : (long long)blockIdx.x;
    if (WARP && run >= runs) return;
    const int lane = WARP ? (threadIdx.x & 31) : threadIdx.x, step = WARP ? 32 : 256;
    const int per_row = C / group, nv = group / 4;
    const size_t t = (size_t)(run / per_row);
    const int c0 = (int)(run % per_row) * group;
    const float4* src = reinterpret_cast<const float4*>(in + t * C + c0);
    float4 val[4];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int i = lane + step * e;
        val[e] = i < nv ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += val[e].x * val[e].x + val[e].y * val[e].y + val[e].z * val[e].z + val[e].w * val[e].w;
    }
    const float total = WARP ? warp_sum(ss) : block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(total / (float)group + eps);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int i = lane + step * e;
        if (i < nv) {
            float4 f = make_float4(val[e].x * rstd, val[e].y * rstd, val[e].z * rstd, val[e].w * rstd);
            if (weight) {
                f.x *= load_as_f(weight, w_dtype, 4 * i); f.y *= load_as_f(weight, w_dtype, 4 * i + 1);
                f.z *= load_as_f(weight, w_dtype, 4 * i + 2); f.w *= load_as_f(weight, w_dtype, 4 * i + 3);
            }
            gn_store4(out + t * C + c0 + 4 * i, gate ? gate + t * g_ld + g_off + c0 + 4 * i : nullptr, f, gate_act);
        }
    }
}

template <typename TI, typename TO>
static int gated_norm_launch(const void* in, int T, int C, int group, const void* weight, int w_dtype, float eps, const void* gate, int g_ld,
                             int g_off, int gate_act, void* out, cudaStream_t s) {
    if (group > 0 && group <= 512) {
        const long long runs = (long long)T * (C / group);
        PE_TRY(pe_launch(gated_norm_warp_kernel<TI, TO>, (unsigned)((runs + 7) / 8), 256, 0, s, (const TI*)in, C, group, weight, w_dtype, eps,
                         (const TO*)gate, g_ld, g_off, gate_act, (TO*)out, runs));
    } else {
        const int n = group > 0 ? group : C;
        const int threads = n >= 256 ? 256 : ((n + 31) / 32) * 32;
        PE_TRY(pe_launch(gated_norm_kernel<TI, TO>, dim3(T, C / n), threads, 0, s, (const TI*)in, C, group, weight, w_dtype, eps,
                         (const TO*)gate, g_ld, g_off, gate_act, (TO*)out));
    }
    PE_LAUNCH_CHECK();
    return 0;
}

// bfloat16 rows times act(gate) without a norm: out[t, c] = in[t, c] * act(gate[t, g_off + c]); eight columns a thread.
__global__ void gate_mul_bf16x8_kernel(const bf16* in, int C8, const bf16* gate, int g_ld, int g_off, int act, bf16* out, size_t units) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < units; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / C8, c = (idx % C8) * 8;
        const uint4 a = *reinterpret_cast<const uint4*>(in + idx * 8), g = *reinterpret_cast<const uint4*>(gate + t * g_ld + g_off + c);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 af = __bfloat1622float2(a2[e]), gf = __bfloat1622float2(g2[e]);
            o2[e] = __floats2bfloat162_rn(af.x * go_act(gf.x, act), af.y * go_act(gf.y, act));
        }
        *reinterpret_cast<uint4*>(out + idx * 8) = o;
    }
}

extern "C" int pe_gated_norm(const void* in, int in_dtype, int T, int C, int group, const void* weight, int w_dtype, float eps,
                             const void* gate, int g_ld, int g_off, int gate_act, void* out, int out_dtype, void* stream) {
    if (T <= 0 || C <= 0) return 0;
    if (group < 0 || (group > 0 && C % group)) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == PE_F32 && out_dtype == PE_F32)
        return gated_norm_launch<float, float>(in, T, C, group, weight, w_dtype, eps, gate, g_ld, g_off, gate_act, out, s);
    if (in_dtype == PE_F32 && out_dtype == PE_BF16 && group > 0 && group % 4 == 0 && group <= 4096 && g_ld % 4 == 0 && g_off % 4 == 0 &&
        !((uintptr_t)in & 15) && !((uintptr_t)out & 7) && !((uintptr_t)gate & 7)) {
        const long long runs = (long long)T * (C / group);
        if (group <= 512)
            PE_TRY(pe_launch(gated_norm_x4_kernel<true>, (unsigned)((runs + 7) / 8), 256, 0, s, (const float*)in, C, group, weight, w_dtype, eps,
                             (const bf16*)gate, g_ld, g_off, gate_act, (bf16*)out, runs));
        else
            PE_TRY(pe_launch(gated_norm_x4_kernel<false>, (unsigned)runs, 256, 0, s, (const float*)in, C, group, weight, w_dtype, eps,
                             (const bf16*)gate, g_ld, g_off, gate_act, (bf16*)out, runs));
        PE_LAUNCH_CHECK();
        return 0;
    }
    if (in_dtype == PE_F32 && out_dtype == PE_BF16)
        return gated_norm_launch<float, bf16>(in, T, C, group, weight, w_dtype, eps, gate, g_ld, g_off, gate_act, out, s);
    if (in_dtype == PE_BF16 && out_dtype == PE_BF16 && group == 0 && gate && C % 8 == 0 && g_ld % 8 == 0 && g_off % 8 == 0 &&
        !(((uintptr_t)in | (uintptr_t)out | (uintptr_t)gate) & 15)) {
        // no norm, only the gate: eight columns a thread with 16-byte accesses
        const size_t units = (size_t)T * (C / 8);
        const int blocks = (int)((units + 255) / 256 < 148 * 16 ? (units + 255) / 256 : 148 * 16);
        PE_TRY(pe_launch(gate_mul_bf16x8_kernel, blocks, 256, 0, s, (const bf16*)in, C / 8, (const bf16*)gate, g_ld, g_off, gate_act, (bf16*)out, units));
        PE_LAUNCH_CHECK();
        return 0;
    }
    if (in_dtype == PE_BF16 && out_dtype == PE_BF16)
        return gated_norm_launch<bf16, bf16>(in, T, C, group, weight, w_dtype, eps, gate, g_ld, g_off, gate_act, out, s);
    return PE_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- x += scale * sum_i rmsnorm(y_i) * w_i
// x [T, W] float32; up to 4 branches y_i [T, W] (all of one dtype) with plain weights w_i [W] (all of one dtype).
struct NormedSumArgs { const void* y[4]; const void* w[4]; int n; };

template <typename T>
__global__ void __launch_bounds__(256) normed_sum_add_kernel(float* x, NormedSumArgs a, int w_dtype, int W, float eps, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t t = blockIdx.x;
    float rstd[4];
    for (int b = 0; b < a.n; ++b) {
        const T* y = (const T*)a.y[b] + t * W;
        float ss = 0.f;
        for (int i = threadIdx.x; i < W; i += blockDim.x) { const float f = to_f(y[i]); ss = fmaf(f, f, ss); }
        rstd[b] = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
    }
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float sum = 0.f;
        for (int b = 0; b < a.n; ++b) sum += to_f(((const T*)a.y[b])[t * W + i]) * rstd[b] * load_as_f(a.w[b], w_dtype, i);
        x[t * W + i] = fmaf(scale, sum, x[t * W + i]);
    }
}

// float32 branches, W a multiple of 4 and at most 4096: a thread keeps its up to four float4 of every branch in registers
// between the sums of squares and the result, so every row is read once.
template <int NB>
__global__ void __launch_bounds__(256) normed_sum_add_f32x4_kernel(float* x, NormedSumArgs a, int w_dtype, int W, float eps, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t t = blockIdx.x;
    const int nv = W / 4;
    float4 val[NB][4];
    float rstd[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const float4* y = reinterpret_cast<const float4*>((const float*)a.y[b] + t * W);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = threadIdx.x + 256 * e;
            val[b][e] = i < nv ? y[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += val[b][e].x * val[b][e].x + val[b][e].y * val[b][e].y + val[b][e].z * val[b][e].z + val[b][e].w * val[b][e].w;
        }
        rstd[b] = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
    }
    float4* xr = reinterpret_cast<float4*>(x + t * W);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int i = threadIdx.x + 256 * e;
        if (i < nv) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                sum.x += val[b][e].x * rstd[b] * load_as_f(a.w[b], w_dtype, 4 * i + 0);
                sum.y += val[b][e].y * rstd[b] * load_as_f(a.w[b], w_dtype, 4 * i + 1);
                sum.z += val[b][e].z * rstd[b] * load_as_f(a.w[b], w_dtype, 4 * i + 2);
                sum.w += val[b][e].w * rstd[b] * load_as_f(a.w[b], w_dtype, 4 * i + 3);
            }
            float4 xv = xr[i];
            xv.x = fmaf(scale, sum.x, xv.x); xv.y = fmaf(scale, sum.y, xv.y); xv.z = fmaf(scale, sum.z, xv.z); xv.w = fmaf(scale, sum.w, xv.w);
            xr[i] = xv;
        }
    }
}

extern "C" int pe_normed_sum_add(float* x, const void* y0, const void* y1, const void* y2, const void* y3, int y_dtype,
                                 const void* w0, const void* w1, const void* w2, const void* w3, int w_dtype, int n, int T, int W,
                                 float eps, float scale, void* stream) {
    if (T <= 0) return 0;
    if (n < 1 || n > 4) return PE_ERR_UNSUPPORTED;
    NormedSumArgs a = {{y0, y1, y2, y3}, {w0, w1, w2, w3}, n};
    cudaStream_t s = (cudaStream_t)stream;
    bool aligned = !((uintptr_t)x & 15);
    for (int b = 0; b < n; ++b) aligned = aligned && !((uintptr_t)a.y[b] & 15);
    if (y_dtype == PE_F32 && W % 4 == 0 && W <= 4096 && aligned && n <= 2) {
        if (n == 1) PE_TRY(pe_launch(normed_sum_add_f32x4_kernel<1>, T, 256, 0, s, x, a, w_dtype, W, eps, scale));
        else PE_TRY(pe_launch(normed_sum_add_f32x4_kernel<2>, T, 256, 0, s, x, a, w_dtype, W, eps, scale));
    } else if (y_dtype == PE_F32) PE_TRY(pe_launch(normed_sum_add_kernel<float>, T, 256, 0, s, x, a, w_dtype, W, eps, scale));
    else if (y_dtype == PE_BF16) PE_TRY(pe_launch(normed_sum_add_kernel<bf16>, T, 256, 0, s, x, a, w_dtype, W, eps, scale));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- x += scale * y
template <typename T>
__global__ void scaled_add_kernel(float* x, const T* y, float scale, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = fmaf(scale, to_f(y[i]), x[i]);
}

extern "C" int pe_scaled_add(float* x, const void* y, int dtype, float scale, long long total, void* stream) {
    if (total <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == PE_F32) PE_TRY(pe_launch(scaled_add_kernel<float>, blocks, 256, 0, s, x, (const float*)y, scale, (size_t)total));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(scaled_add_kernel<bf16>, blocks, 256, 0, s, x, (const bf16*)y, scale, (size_t)total));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- x[t, :] += rows[t, :] + vec[:]
// rows [T, W] float32 or null, vec [W] in either dtype or null.
__global__ void add_rows_kernel(float* x, const float* rows, const void* vec, int v_dtype, int W, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float f = x[i];
        if (rows) f += rows[i];
        if (vec) f += load_as_f(vec, v_dtype, i % W);
        x[i] = f;
    }
}

extern "C" int pe_add_rows(float* x, const float* rows, const void* vec, int v_dtype, int T, int W, void* stream) {
    if (T <= 0) return 0;
    const size_t total = (size_t)T * W;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    PE_TRY(pe_launch(add_rows_kernel, blocks, 256, 0, (cudaStream_t)stream, x, rows, vec, v_dtype, W, total));
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- gated activation, a weight per group of columns
// gu [T, 2I] = gate | up; out[t, c] = act(gate[t, c]) * up[t, c] * colw[t, g(c)], with g(c) = min(c / group, n_groups - 1)
// (colw [T, n_groups] float32 or null: no weights).  The product is formed in float32.
// act 5, the clamped form: g = min(gate, limit), u = clamp(up, -limit, limit), out = g sigmoid(alpha g) (u + 1).
template <typename T>
__global__ void gated_act_kernel(const T* gu, T* out, int I, int act, const float* colw, int group, int n_groups, size_t total,
                                 float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, c = idx % I;
        float f;
        if (act == 5) {
            const float g = fminf(to_f(gu[t * 2 * I + c]), limit), u = fminf(fmaxf(to_f(gu[t * 2 * I + I + c]), -limit), limit);
            f = g * go_sigmoid(alpha * g) * (u + 1.0f);
        } else f = go_act(to_f(gu[t * 2 * I + c]), act) * to_f(gu[t * 2 * I + I + c]);
        if (colw) {
            const int g = min((int)(c / group), n_groups - 1);
            const float w = colw[t * n_groups + g];
            f = w == 0.f ? 0.f : f * w;
        }
        out[idx] = from_f<T>(f);
    }
}

// bfloat16, I a multiple of 8, aligned rows: eight columns a thread with 16-byte accesses.  Sigmoid and tanh come from the
// special-function unit's 2^x and reciprocal (relative error about 2^-22, far below the bfloat16 rounding of the result).
__device__ __forceinline__ float go_sigmoid_fast(float v) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * v));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}
__device__ __forceinline__ float go_act_fast(float v, int act) {
    if (act == 2) return v * go_sigmoid_fast(v);
    if (act == 3) return v * go_sigmoid_fast(1.5957691216057308f * (v + 0.044715f * v * v * v));   // 0.5 v (1 + tanh(u)) = v sigmoid(2u)
    if (act == 1) return go_sigmoid_fast(v);
    return v;
}
__global__ void gated_act_bf16x8_kernel(const bf16* gu, bf16* out, int I, int act, const float* colw, int group, int n_groups, size_t units,
                                        float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = I / 8;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < units; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / per_row, c = (idx % per_row) * 8;
        if (colw && (group & 7) == 0 && colw[t * n_groups + min((int)(c / group), n_groups - 1)] == 0.f) {
            // eight columns of an expert the token does not use: exact zeros, and its hidden units are not read
            *reinterpret_cast<uint4*>(out + t * I + c) = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * I + c), u = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 gf = __bfloat1622float2(g2[e]), uf = __bfloat1622float2(u2[e]);
            float a, b;
            if (act == 5) {
                const float ga = fminf(gf.x, limit), gb = fminf(gf.y, limit);
                a = ga * go_sigmoid_fast(alpha * ga) * (fminf(fmaxf(uf.x, -limit), limit) + 1.0f);
                b = gb * go_sigmoid_fast(alpha * gb) * (fminf(fmaxf(uf.y, -limit), limit) + 1.0f);
            } else { a = go_act_fast(gf.x, act) * uf.x; b = go_act_fast(gf.y, act) * uf.y; }
            if (colw) {
                const float wa = colw[t * n_groups + min((int)((c + 2 * e) / group), n_groups - 1)];
                const float wb = colw[t * n_groups + min((int)((c + 2 * e + 1) / group), n_groups - 1)];
                a = wa == 0.f ? 0.f : a * wa;
                b = wb == 0.f ? 0.f : b * wb;
            }
            o2[e] = __floats2bfloat162_rn(a, b);
        }
        *reinterpret_cast<uint4*>(out + t * I + c) = o;
    }
}

extern "C" int pe_gated_act(const void* gu, void* out, int dtype, int T, int I, int act, const float* colw, int group, int n_groups,
                            float limit, float alpha, void* stream) {
    if (T <= 0 || I <= 0) return 0;
    if (colw && (group <= 0 || n_groups <= 0)) return PE_ERR_UNSUPPORTED;
    const size_t total = (size_t)T * I;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_BF16 && I % 8 == 0 && !(((uintptr_t)gu | (uintptr_t)out) & 15)) {
        const size_t units = total / 8;
        const int b8 = (int)((units + 255) / 256 < 148 * 16 ? (units + 255) / 256 : 148 * 16);
        PE_TRY(pe_launch(gated_act_bf16x8_kernel, b8, 256, 0, s, (const bf16*)gu, (bf16*)out, I, act, colw, group, n_groups, units, limit, alpha));
        PE_LAUNCH_CHECK();
        return 0;
    }
    if (dtype == PE_F32) PE_TRY(pe_launch(gated_act_kernel<float>, blocks, 256, 0, s, (const float*)gu, (float*)out, I, act, colw, group, n_groups, total, limit, alpha));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(gated_act_kernel<bf16>, blocks, 256, 0, s, (const bf16*)gu, (bf16*)out, I, act, colw, group, n_groups, total, limit, alpha));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- activation of ungated experts, a weight per group of columns
// h [T, I]; out[t, c] = act(h[t, c]) * colw[t, min(c / group, n_groups - 1)], formed in float32 (a zero weight gives an exact zero).
template <typename T>
__global__ void weighted_act_kernel(const T* h, T* out, int I, int act, const float* colw, int group, int n_groups, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, c = idx % I;
        const float w = colw[t * n_groups + min((int)(c / group), n_groups - 1)];
        out[idx] = from_f<T>(w == 0.f ? 0.f : go_act(to_f(h[idx]), act) * w);
    }
}

// bfloat16 with I and group multiples of 8: a thread takes 8 columns of one group with 16-byte accesses, and does not read
// hidden units whose weight is zero.
__global__ void weighted_act_vec_kernel(const bf16* h, bf16* out, int I8, int act, const float* colw, int group8, int n_groups, size_t total8) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I8;
        const int c8 = (int)(idx - t * I8);
        const float w = colw[t * n_groups + min(c8 / group8, n_groups - 1)];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (w != 0.f) {
            v = *reinterpret_cast<const uint4*>(h + idx * 8);
            __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(p[k]);
                p[k] = __floats2bfloat162_rn(go_act(f.x, act) * w, go_act(f.y, act) * w);
            }
        }
        *reinterpret_cast<uint4*>(out + idx * 8) = v;
    }
}

extern "C" int pe_weighted_act(const void* h, void* out, int dtype, int T, int I, int act, const float* colw, int group, int n_groups,
                               void* stream) {
    if (T <= 0 || I <= 0) return 0;
    if (!colw || group <= 0 || n_groups <= 0) return PE_ERR_UNSUPPORTED;
    const size_t total = (size_t)T * I;
    if (dtype == PE_BF16 && I % 8 == 0 && group % 8 == 0 && (((uintptr_t)h | (uintptr_t)out) & 15) == 0) {
        const size_t total8 = total / 8;
        const int vblocks = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
        PE_TRY(pe_launch(weighted_act_vec_kernel, vblocks, 256, 0, (cudaStream_t)stream, (const bf16*)h, (bf16*)out, I / 8, act, colw, group / 8,
                         n_groups, total8));
        PE_LAUNCH_CHECK();
        return 0;
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32) PE_TRY(pe_launch(weighted_act_kernel<float>, blocks, 256, 0, s, (const float*)h, (float*)out, I, act, colw, group, n_groups, total));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(weighted_act_kernel<bf16>, blocks, 256, 0, s, (const bf16*)h, (bf16*)out, I, act, colw, group, n_groups, total));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- the choice of experts
// logits [T, ld] float32: columns 0 .. E-1 are the router's, column E (extra != 0) the logit of a gate for a part that
// every token uses.  weights [T, E + extra] float32: the softmax over the `top` largest logits at their places, zero at
// the others (of equal logits the lower index is taken first); the extra column holds sigmoid(logit).  ids [T, top] int32
// (or null) receives the chosen experts, largest logit first.  A warp a token.
// `over_all` != 0: the weights are the chosen experts' entries of the softmax over all E logits (not renormalised);
// either way they are multiplied by `factor`.  extra == 2: there is no logit for the extra column, which holds 1.
__device__ __forceinline__ void moe_choose(const float* z, int E, int top, int extra, float* w, int* ids, int lane,
                                           int over_all = 0, float factor = 1.0f) {
    for (int e = lane; e < E; e += 32) w[e] = 0.f;
    if (extra && lane == 0) w[E] = extra == 2 ? 1.0f : go_sigmoid(z[E]);
    __syncwarp();
    float zmax = 0.f, sum = 0.f;
    unsigned long long taken_lo = 0ull;                 // the lane's taken places (a lane sees E / 32 <= 64 of them)
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane, i = 0; e < E; e += 32, ++i) {
            if (taken_lo >> i & 1ull) continue;
            const float v = z[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) break;
        if ((at & 31) == lane) taken_lo |= 1ull << (at >> 5);
        if (k == 0) zmax = best;
        const float p = expf(best - zmax);
        sum += p;
        if (lane == 0) { w[at] = p; if (ids) ids[k] = at; }
    }
    __syncwarp();
    if (over_all) {                                     // the denominator runs over every expert (zmax is the largest logit of all)
        float all = 0.f;
        for (int e = lane; e < E; e += 32) all += expf(z[e] - zmax);
        sum = warp_sum(all);
    }
    const float inv = factor / sum;
    for (int e = lane; e < E; e += 32) w[e] *= inv;
}

__global__ void __launch_bounds__(128) moe_route_kernel(const float* logits, int ld, int E, int top, int extra, float* weights,
                                                        int* ids, int T, int over_all, float factor) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    moe_choose(logits + (size_t)t * ld, E, top, extra, weights + (size_t)t * (E + (extra ? 1 : 0)), ids ? ids + (size_t)t * top : nullptr,
               lane, over_all, factor);
}

// The same from the float32 residual stream: the logits are router[e] . (x * rsqrt(mean(x^2) + eps) * norm_w), formed in float32
// by the token's block (the RMS norm in front of the router is part of this kernel), for up to MR_MAX_E experts (+ the extra row).
// norm_w null: the router reads the stream as it is (no norm).
#define MR_MAX_E 256
#define MR_THREADS 128
// A block a token: its four warps share the row (each a quarter of the 16-byte units, so four times the reads are in flight),
// their partial sums meet in shared memory in a fixed order, and the first warp chooses.
__global__ void __launch_bounds__(MR_THREADS) moe_route_stream_kernel(const float* x, const void* norm_w, int nw_dtype, float eps,
                                                                      const float* router, int K, int E, int top, int extra,
                                                                      float* weights, int* ids, int T, int over_all, float factor) {
    pdl_launch_dependents();
    __shared__ float z[MR_MAX_E + 1];
    __shared__ float part[MR_THREADS / 32][8];
    __shared__ float red[33];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = blockIdx.x;
    pdl_wait();
    const float* row = x + (size_t)t * K;
    const int n = E + (extra == 1 ? 1 : 0);
    // VEC (K a multiple of 4, a float32 norm weight, aligned rows): 16-byte reads, four of a thread's reads of the row in flight
    // at once for the sum of squares.
    const bool vec = norm_w && K % 4 == 0 && nw_dtype == PE_F32 && !(((uintptr_t)x | (uintptr_t)router | (uintptr_t)norm_w) & 15);
    float ss = 0.f;
    if (!norm_w) {
    } else if (vec) {
        const float4* row4 = reinterpret_cast<const float4*>(row);
#pragma unroll 4
        for (int k = tid; k < K / 4; k += MR_THREADS) { const float4 v = row4[k]; ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
    } else {
        for (int k = tid; k < K; k += MR_THREADS) ss = fmaf(row[k], row[k], ss);
    }
    const float rstd = norm_w ? 1.0f / sqrtf(block_sum(ss, red) / (float)K + eps) : 1.0f;
    for (int e0 = 0; e0 < n; e0 += 8) {                                     // eight logits at a time: the row is read once for them
        float acc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] = 0.f;
        if (vec) {
            const float4* row4 = reinterpret_cast<const float4*>(row);
            const float4* nw4 = reinterpret_cast<const float4*>(norm_w);
            const float4* r4 = reinterpret_cast<const float4*>(router);
            for (int k = tid; k < K / 4; k += MR_THREADS) {
                float4 xv = row4[k];
                const float4 w = nw4[k];
                xv.x *= w.x; xv.y *= w.y; xv.z *= w.z; xv.w *= w.w;
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (e0 + u < n) {
                        const float4 r = r4[(size_t)(e0 + u) * (K / 4) + k];
                        acc[u] = fmaf(xv.x, r.x, acc[u]); acc[u] = fmaf(xv.y, r.y, acc[u]);
                        acc[u] = fmaf(xv.z, r.z, acc[u]); acc[u] = fmaf(xv.w, r.w, acc[u]);
                    }
            }
        } else {
            for (int k = tid; k < K; k += MR_THREADS) {
                const float xv = norm_w ? row[k] * load_as_f(norm_w, nw_dtype, k) : row[k];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (e0 + u < n) acc[u] = fmaf(xv, router[(size_t)(e0 + u) * K + k], acc[u]);
            }
        }
        __syncthreads();                                                    // the sums of the eight logits before these have been read
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float sum = warp_sum(acc[u]);
            if (lane == 0) part[warp][u] = sum;
        }
        __syncthreads();
        if (tid < 8 && e0 + tid < n) z[e0 + tid] = ((part[0][tid] + part[1][tid]) + (part[2][tid] + part[3][tid])) * rstd;
    }
    __syncthreads();
    if (warp == 0) moe_choose(z, E, top, extra, weights + (size_t)t * (E + (extra ? 1 : 0)), ids ? ids + (size_t)t * top : nullptr, lane,
                              over_all, factor);
}

extern "C" int pe_moe_route_stream(const float* x, const void* norm_w, int nw_dtype, float eps, const float* router, int K, int E,
                                   int top, int extra, float* weights, int* ids, int T, int over_all, float factor, void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > MR_MAX_E || top <= 0 || top > E || K <= 0 || extra < 0 || extra > 2) return PE_ERR_UNSUPPORTED;
    PE_TRY(pe_launch(moe_route_stream_kernel, T, MR_THREADS, 0, (cudaStream_t)stream, x, norm_w, nw_dtype, eps, router, K, E, top, extra,
                     weights, ids, T, over_all, factor));
    PE_LAUNCH_CHECK();
    return 0;
}

extern "C" int pe_moe_route(const float* logits, int ld, int E, int top, int extra, float* weights, int* ids, int T, int over_all,
                            float factor, void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > 2048 || top <= 0 || top > E || extra < 0 || extra > 2) return PE_ERR_UNSUPPORTED;
    PE_TRY(pe_launch(moe_route_kernel, (T + 3) / 4, 128, 0, (cudaStream_t)stream, logits, ld, E, top, extra, weights, ids, T, over_all,
                     factor));
    PE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- the choice of experts among groups, sigmoid scores
// logits [T, ld] float32.  Scores s = sigmoid(logit).  The choice reads c = s + correction (a stored vector [E], or null: zeros):
// the experts form `n_groups` equal runs of neighbours; a run counts the sum of its `group_best` largest c; the `keep` runs that
// count most stay, every other run's c is minus infinity; of what stays the `top` largest c are chosen (of equal numbers the
// lower index first, for runs and for experts).  weights [T, E] float32: factor * s at the chosen places, zero elsewhere;
// ids [T, top] int32 (or null) receives the chosen experts, largest c first.  A warp a token, four tokens a block.
#define MG_MAX_E 1024
#define MG_MAX_GROUPS 64
// The choice itself, by one warp: z [E] the logits, c [E] and gs [n_groups] scratch of the warp.
__device__ __forceinline__ void moe_choose_grouped(const float* z, float* c, float* gs, int E, int top, const void* corr, int corr_dtype,
                                                   int n_groups, int keep, int group_best, float factor, float* w, int* ids, int lane) {
    for (int e = lane; e < E; e += 32) {
        c[e] = go_sigmoid(z[e]) + (corr ? load_as_f(corr, corr_dtype, e) : 0.f);
        w[e] = 0.f;
    }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int per = E / n_groups;
        for (int g = 0; g < n_groups; ++g) {
            unsigned long long taken = 0ull;
            float total = 0.f;
            for (int b = 0; b < group_best && b < per; ++b) {
                float best = -INFINITY;
                int at = 0x7fffffff;
                for (int j = lane, i = 0; j < per; j += 32, ++i) {
                    if (taken >> i & 1ull) continue;
                    const float v = c[g * per + j];
                    if (v > best || (v == best && j < at)) { best = v; at = j; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
                }
                if (at == 0x7fffffff) break;
                if ((at & 31) == lane) taken |= 1ull << (at >> 5);
                total += best;
            }
            if (lane == 0) gs[g] = total;
        }
        __syncwarp();
        // a run that stays is marked in place: its count becomes +infinity
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[g];
                if (v == INFINITY) continue;
                if (v > best || (v == best && g < at) || at == 0x7fffffff) { best = v; at = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
            }
            if (at == 0x7fffffff) break;
            if (lane == 0) gs[at] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    unsigned long long taken = 0ull;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane, i = 0; e < E; e += 32, ++i) {
            if (taken >> i & 1ull) continue;
            const float v = c[e];
            if (v > best || (v == best && e < at) || at == 0x7fffffff) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) break;
        if ((at & 31) == lane) taken |= 1ull << (at >> 5);
        if (lane == 0) { w[at] = factor * go_sigmoid(z[at]); if (ids) ids[k] = at; }
    }
}

__global__ void __launch_bounds__(128) moe_route_grouped_kernel(const float* logits, int ld, int E, int top, const void* corr, int corr_dtype,
                                                                int n_groups, int keep, int group_best, float factor, float* weights,
                                                                int* ids, int T) {
    pdl_launch_dependents();
    __shared__ float s_c[4][MG_MAX_E];
    __shared__ float s_g[4][MG_MAX_GROUPS];
    const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + wi;
    pdl_wait();
    if (t >= T) return;
    moe_choose_grouped(logits + (size_t)t * ld, s_c[wi], s_g[wi], E, top, corr, corr_dtype, n_groups, keep, group_best, factor,
                       weights + (size_t)t * E, ids ? ids + (size_t)t * top : nullptr, lane);
}

// The same from the float32 residual stream with the layer norm in front of the router inside the kernel: the logits are
// router[e] . ((x - mean) / sqrt(var + eps) * norm_w + norm_b), all in float32 (var the mean of the squared deviations, two passes),
// for up to MR_MAX_E experts.  A block a token, as in moe_route_stream_kernel: its four warps share the row, their partial sums meet
// in shared memory in a fixed order, and the first warp chooses.
__global__ void __launch_bounds__(MR_THREADS) moe_route_stream_grouped_kernel(const float* x, const void* norm_w, int nw_dtype, const void* norm_b,
                                                                              int nb_dtype, float eps, const float* router, int K, int E, int top,
                                                                              const void* corr, int corr_dtype, int n_groups, int keep,
                                                                              int group_best, float factor, float* weights, int* ids, int T) {
    pdl_launch_dependents();
    __shared__ float z[MR_MAX_E];
    __shared__ float c[MR_MAX_E];
    __shared__ float gs[MG_MAX_GROUPS];
    __shared__ float part[MR_THREADS / 32][8];
    __shared__ float red[33];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = blockIdx.x;
    pdl_wait();
    const float* row = x + (size_t)t * K;
    const bool vec = K % 4 == 0 && !(((uintptr_t)x | (uintptr_t)router) & 15);
    float s = 0.f;
    if (vec) {
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int k = tid; k < K / 4; k += MR_THREADS) { const float4 v = row4[k]; s += (v.x + v.y) + (v.z + v.w); }
    } else {
        for (int k = tid; k < K; k += MR_THREADS) s += row[k];
    }
    const float mean = block_sum(s, red) / (float)K;
    float v2 = 0.f;
    for (int k = tid; k < K; k += MR_THREADS) { const float d = row[k] - mean; v2 = fmaf(d, d, v2); }
    const float rstd = 1.0f / sqrtf(block_sum(v2, red) / (float)K + eps);
    for (int e0 = 0; e0 < E; e0 += 8) {                                     // eight logits at a time: the row is read once for them
        float acc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] = 0.f;
        if (vec) {
            const float4* row4 = reinterpret_cast<const float4*>(row);
            const float4* r4 = reinterpret_cast<const float4*>(router);
            for (int k = tid; k < K / 4; k += MR_THREADS) {
                float4 xv = row4[k];
                xv.x = fmaf((xv.x - mean) * rstd, load_as_f(norm_w, nw_dtype, 4 * k), load_as_f(norm_b, nb_dtype, 4 * k));
                xv.y = fmaf((xv.y - mean) * rstd, load_as_f(norm_w, nw_dtype, 4 * k + 1), load_as_f(norm_b, nb_dtype, 4 * k + 1));
                xv.z = fmaf((xv.z - mean) * rstd, load_as_f(norm_w, nw_dtype, 4 * k + 2), load_as_f(norm_b, nb_dtype, 4 * k + 2));
                xv.w = fmaf((xv.w - mean) * rstd, load_as_f(norm_w, nw_dtype, 4 * k + 3), load_as_f(norm_b, nb_dtype, 4 * k + 3));
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (e0 + u < E) {
                        const float4 r = r4[(size_t)(e0 + u) * (K / 4) + k];
                        acc[u] = fmaf(xv.x, r.x, acc[u]); acc[u] = fmaf(xv.y, r.y, acc[u]);
                        acc[u] = fmaf(xv.z, r.z, acc[u]); acc[u] = fmaf(xv.w, r.w, acc[u]);
                    }
            }
        } else {
            for (int k = tid; k < K; k += MR_THREADS) {
                const float xv = fmaf((row[k] - mean) * rstd, load_as_f(norm_w, nw_dtype, k), load_as_f(norm_b, nb_dtype, k));
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (e0 + u < E) acc[u] = fmaf(xv, router[(size_t)(e0 + u) * K + k], acc[u]);
            }
        }
        __syncthreads();                                                    // the sums of the eight logits before these have been read
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float sum = warp_sum(acc[u]);
            if (lane == 0) part[warp][u] = sum;
        }
        __syncthreads();
        if (tid < 8 && e0 + tid < E) z[e0 + tid] = (part[0][tid] + part[1][tid]) + (part[2][tid] + part[3][tid]);
    }
    __syncthreads();
    if (warp == 0) moe_choose_grouped(z, c, gs, E, top, corr, corr_dtype, n_groups, keep, group_best, factor, weights + (size_t)t * E,
                                      ids ? ids + (size_t)t * top : nullptr, lane);
}

extern "C" int pe_moe_route_stream_grouped(const float* x, const void* norm_w, int nw_dtype, const void* norm_b, int nb_dtype, float eps,
                                           const float* router, int K, int E, int top, const void* corr, int corr_dtype, int n_groups, int keep,
                                           int group_best, float factor, float* weights, int* ids, int T, void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > MR_MAX_E || top <= 0 || top > E || K <= 0 || !norm_w || !norm_b || n_groups <= 0 || n_groups > MG_MAX_GROUPS || E % n_groups ||
        keep <= 0 || keep > n_groups || group_best <= 0)
        return PE_ERR_UNSUPPORTED;
    PE_TRY(pe_launch(moe_route_stream_grouped_kernel, T, MR_THREADS, 0, (cudaStream_t)stream, x, norm_w, nw_dtype, norm_b, nb_dtype, eps, router, K,
                     E, top, corr, corr_dtype, n_groups, keep, group_best, factor, weights, ids, T));
    PE_LAUNCH_CHECK();
    return 0;
}

extern "C" int pe_moe_route_grouped(const float* logits, int ld, int E, int top, const void* corr, int corr_dtype, int n_groups, int keep,
                                    int group_best, float factor, float* weights, int* ids, int T, void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > MG_MAX_E || top <= 0 || top > E || n_groups <= 0 || n_groups > MG_MAX_GROUPS || E % n_groups || keep <= 0 || keep > n_groups ||
        group_best <= 0 || ld < E)
        return PE_ERR_UNSUPPORTED;
    PE_TRY(pe_launch(moe_route_grouped_kernel, (T + 3) / 4, 128, 0, (cudaStream_t)stream, logits, ld, E, top, corr, corr_dtype, n_groups, keep,
                     group_best, factor, weights, ids, T));
    PE_LAUNCH_CHECK();
    return 0;
}
