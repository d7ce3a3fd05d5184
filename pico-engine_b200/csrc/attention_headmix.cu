// Softmax attention over the paged key/value cache whose weights are mixed across heads before they meet
// the values, with an optional sink in the denominator and an optional window; either dtype, float32 math.
//
//   s_g(i, j) = scale * q_g(i) . k_c(g)(j)                         c(g) = g / (H / G), j visible to i
//   p_g(i, j) = exp(s_g(i, j)) / (exp(sink_g) + sum_j' exp(s_g(i, j')))
//   w_h(i, j) = sum_g mix[h, g] * p_g(i, j)                        o_h(i) = sum_j w_h(i, j) * v_c(h)(j)
//
// Mixing needs the normalised weights of all heads for the same (i, j), and a weight is normalised only
// when its whole row is known, so the keys are passed over twice: the first pass leaves every (query, head)
// its maximum and its sum of exponentials, the second computes the scores again, normalises, mixes and
// multiplies with the values.  Because the second pass knows the final denominators, the contributions of
// different ranges of keys simply add: the keys of a tile may be cut into `splits` ranges that run as blocks
// of their own (a step of single tokens with long contexts has few tiles), summed by a last small kernel in
// the order of the ranges.
//
// A block takes a tile of up to QT consecutive tokens of one sequence and all heads.  Keys are visited in
// blocks of HM_KB = 32 positions that start at multiples of 32, so a position's arithmetic does not depend on
// how its sequence was cut into steps.  Also here: the kernel that norms query and key heads (RMS over the
// head, one weight vector for all heads) and writes keys and values into their cache pages.
#include "common.cuh"

#define HM_KB 32
#define HM_THREADS 256

struct HeadMixArgs {
    const void* q; int q_stride;
    const void* k_pool; const void* v_pool;
    const int* table; int table_stride;
    const int* tok_pos; const int* tok_row;
    const int* tiles; int tile_tokens;        // runs of at most tile_tokens tokens (row, first token, tokens, first position); null: every token alone
    int H, G, D, Dv, window; float scale;
    const void* sink; int sink_dtype;
    const void* mix; int mix_dtype;
    int QT, splits;
    const float* slopes; int keep_first; int v_ld;   // slope_h * (i - j) is taken off a score (null: nothing); the first keep_first keys stay
                                                     // visible behind the window; a value row has v_ld entries of which the first Dv are read
    float* stats;                             // [tile][split][QT][H][2]
    float* opart;                             // [tile][split][QT][H][Dv]
    void* out;                                // [T][H * Dv]
};

struct TileInfo { int row, t0, nq, p0; };

__device__ __forceinline__ bool hm_tile(const HeadMixArgs& a, int qtile, TileInfo& ti) {
    if (a.tiles == nullptr) {
        ti.row = a.tok_row[qtile]; ti.t0 = qtile; ti.nq = 1; ti.p0 = a.tok_pos[qtile];
        return true;
    }
    const int per = a.tile_tokens / a.QT;
    const int* r = a.tiles + 4 * (qtile / per);
    const int off = (qtile % per) * a.QT;
    if (off >= r[2]) return false;
    ti.row = r[0]; ti.t0 = r[1] + off; ti.nq = min(a.QT, r[2] - off); ti.p0 = r[3] + off;
    return true;
}

// PASS 0: maxima and sums.  PASS 1: weights, mixing, values.
template <typename T, int PASS, int NACC>
__global__ void __launch_bounds__(HM_THREADS) headmix_kernel(HeadMixArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int H = a.H, G = a.G, D = a.D, Dv = a.Dv, QT = a.QT, per_kv = H / G;
    const int pitch = max(D, Dv) + 1;
    float* q_s = smem;                                   // [QT][H][D]
    float* kv_s = q_s + (size_t)QT * H * D;              // [G][KB][pitch]
    float* p_s = kv_s + (size_t)G * HM_KB * pitch;       // [H][QT][KB]
    float* w_s = p_s + (size_t)H * QT * HM_KB;           // [H][QT][KB] (PASS 1 with mixing)
    float* m_s = w_s + (PASS == 1 && a.mix ? (size_t)H * QT * HM_KB : 0);   // [QT][H]: running maximum / final maximum
    float* l_s = m_s + QT * H;                           // [QT][H]: running sum / 1 / denominator
    float* mix_s = l_s + QT * H;                         // [H][H]

    TileInfo ti;
    if (!hm_tile(a, blockIdx.x, ti)) return;
    const int split = blockIdx.y, tid = threadIdx.x;
    const int hi = ti.p0 + ti.nq;                        // one past the last visible key
    int lo = (a.window > 0 && ti.p0 - a.window + 1 > 0) ? (ti.p0 - a.window + 1) & ~(HM_KB - 1) : 0;
    // the kept first keys are blocks of their own in front of the window's, unless the window reaches them anyway
    int kept_blocks = (a.window > 0 && a.keep_first > 0) ? (a.keep_first + HM_KB - 1) / HM_KB : 0;
    if (lo <= kept_blocks * HM_KB) { lo = 0; kept_blocks = 0; }
    const int n_blocks = kept_blocks + (hi - lo + HM_KB - 1) / HM_KB;
    const int per_split = (n_blocks + a.splits - 1) / a.splits;
    const int b_begin = split * per_split, b_end = min(n_blocks, b_begin + per_split);
    const int k_end = hi;
    const int* table = a.table + (size_t)ti.row * a.table_stride;
    const T* qg = (const T*)a.q;
    const T* kp = (const T*)a.k_pool;
    const T* vp = (const T*)a.v_pool;

    for (int e = tid; e < QT * H * D; e += HM_THREADS) {
        const int i = e / (H * D), r = e % (H * D);
        q_s[e] = i < ti.nq ? to_f(qg[(size_t)(ti.t0 + i) * a.q_stride + r]) : 0.f;
    }
    if (PASS == 0) {
        for (int e = tid; e < QT * H; e += HM_THREADS) { m_s[e] = -INFINITY; l_s[e] = 0.f; }
    } else {
        // the final maximum and denominator of every (query, head) from the ranges' partial results
        for (int e = tid; e < QT * H; e += HM_THREADS) {
            const int h = e % H;
            const float* st = a.stats + ((size_t)blockIdx.x * a.splits * QT * H + e) * 2;
            float M = a.sink ? load_as_f(a.sink, a.sink_dtype, h) : -INFINITY;
            for (int s = 0; s < a.splits; ++s) M = fmaxf(M, st[(size_t)s * QT * H * 2]);
            float den = a.sink ? expf(load_as_f(a.sink, a.sink_dtype, h) - M) : 0.f;
            for (int s = 0; s < a.splits; ++s) {
                const float ms = st[(size_t)s * QT * H * 2], ls = st[(size_t)s * QT * H * 2 + 1];
                if (ms > -INFINITY) den += ls * expf(ms - M);
            }
            m_s[e] = M;
            l_s[e] = den > 0.f ? 1.0f / den : 0.f;
        }
        if (a.mix) for (int e = tid; e < H * H; e += HM_THREADS) mix_s[e] = load_as_f(a.mix, a.mix_dtype, e);
    }
    float acc[NACC];
#pragma unroll
    for (int r = 0; r < NACC; ++r) acc[r] = 0.f;
    __syncthreads();

    for (int blk = b_begin; blk < b_end; ++blk) {
        const int kb = blk < kept_blocks ? blk * HM_KB : lo + (blk - kept_blocks) * HM_KB;
        const int page = table[kb / PE_PAGE];
        const int in_page = kb % PE_PAGE;
        // keys of the block, all key/value heads
        for (int e = tid; e < G * HM_KB * D; e += HM_THREADS) {
            const int d = e % D, j = (e / D) % HM_KB, c = e / (D * HM_KB);
            float v = 0.f;
            if (page >= 0 && kb + j < k_end) v = to_f(kp[(((size_t)page * G + c) * PE_PAGE + in_page + j) * D + d]);
            kv_s[((size_t)c * HM_KB + j) * pitch + d] = v;
        }
        __syncthreads();
        // scores (PASS 0) or normalised weights (PASS 1) of every (head, query, key)
        for (int e = tid; e < H * QT * HM_KB; e += HM_THREADS) {
            const int j = e % HM_KB, i = (e / HM_KB) % QT, h = e / (HM_KB * QT);
            const int key = kb + j, qpos = ti.p0 + i;
            const bool seen = page >= 0 && i < ti.nq && key < k_end && key <= qpos &&
                              (a.window <= 0 || qpos - key < a.window || key < a.keep_first);
            float s = -INFINITY;
            if (seen) {
                const float* qv = q_s + ((size_t)i * H + h) * D;
                const float* kv = kv_s + ((size_t)(h / per_kv) * HM_KB + j) * pitch;
                float dot = 0.f;
                for (int d = 0; d < D; ++d) dot = fmaf(qv[d], kv[d], dot);
                s = dot * a.scale;
                if (a.slopes) s -= a.slopes[h] * (float)(qpos - key);
            }
            if (PASS == 0) p_s[e] = s;
            else p_s[e] = seen ? expf(s - m_s[i * H + h]) * l_s[i * H + h] : 0.f;
        }
        __syncthreads();
        if (PASS == 0) {
            // a warp per (head, query): the block's maximum and sum join the running ones
            for (int pair = tid / 32; pair < H * QT; pair += HM_THREADS / 32) {
                const int i = pair % QT, h = pair / QT;
                const float s = p_s[(size_t)pair * HM_KB + (tid & 31)];
                const float bm = warp_max(s);
                if (bm > -INFINITY) {
                    const float m_old = m_s[i * H + h], m_new = fmaxf(m_old, bm);
                    const float sum = warp_sum(s > -INFINITY ? expf(s - m_new) : 0.f);
                    if ((tid & 31) == 0) {
                        l_s[i * H + h] = (m_old > -INFINITY ? l_s[i * H + h] * expf(m_old - m_new) : 0.f) + sum;
                        m_s[i * H + h] = m_new;
                    }
                }
            }
            __syncthreads();
            continue;
        }
        // values of the block into the buffer the keys were in; meanwhile the weights are mixed
        for (int e = tid; e < G * HM_KB * Dv; e += HM_THREADS) {
            const int d = e % Dv, j = (e / Dv) % HM_KB, c = e / (Dv * HM_KB);
            float v = 0.f;
            if (page >= 0 && kb + j < k_end) v = to_f(vp[(((size_t)page * G + c) * PE_PAGE + in_page + j) * a.v_ld + d]);
            kv_s[((size_t)c * HM_KB + j) * pitch + d] = v;
        }
        const float* wsrc = p_s;
        if (a.mix) {
            for (int e = tid; e < H * QT * HM_KB; e += HM_THREADS) {
                const int ij = e % (QT * HM_KB), h = e / (QT * HM_KB);
                float w = 0.f;
                for (int g = 0; g < H; ++g) w = fmaf(mix_s[h * H + g], p_s[(size_t)g * QT * HM_KB + ij], w);
                w_s[e] = w;
            }
            wsrc = w_s;
        }
        __syncthreads();
        const int total = H * QT * Dv;
#pragma unroll
        for (int r = 0; r < NACC; ++r) {
            const int e = r * HM_THREADS + tid;
            if (e < total) {
                const int d = e % Dv, hi_ = e / Dv;              // hi_ = h * QT + i
                const float* wv = wsrc + (size_t)hi_ * HM_KB;
                const float* vv = kv_s + ((size_t)((hi_ / QT) / per_kv) * HM_KB) * pitch + d;
                float s = acc[r];
#pragma unroll 8
                for (int j = 0; j < HM_KB; ++j) s = fmaf(wv[j], vv[(size_t)j * pitch], s);
                acc[r] = s;
            }
        }
        __syncthreads();
    }

    if (PASS == 0) {
        float* st = a.stats + (((size_t)blockIdx.x * a.splits + split) * QT * H) * 2;
        for (int e = tid; e < QT * H; e += HM_THREADS) { st[2 * e] = m_s[e]; st[2 * e + 1] = l_s[e]; }
        return;
    }
    const int total = H * QT * Dv;
#pragma unroll
    for (int r = 0; r < NACC; ++r) {
        const int e = r * HM_THREADS + tid;
        if (e < total) {
            const int d = e % Dv, i = (e / Dv) % QT, h = e / (Dv * QT);
            if (a.splits == 1) {
                if (i < ti.nq) ((T*)a.out)[((size_t)(ti.t0 + i) * H + h) * Dv + d] = from_f<T>(acc[r]);
            } else {
                a.opart[(((size_t)blockIdx.x * a.splits + split) * QT + i) * H * Dv + (size_t)h * Dv + d] = acc[r];
            }
        }
    }
}

// The ranges' contributions summed in their order.
template <typename T>
__global__ void headmix_reduce_kernel(HeadMixArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    TileInfo ti;
    if (!hm_tile(a, blockIdx.x, ti)) return;
    const int HD = a.H * a.Dv;
    for (int e = threadIdx.x; e < ti.nq * HD; e += blockDim.x) {
        const int i = e / HD, r = e % HD;
        float s = 0.f;
        for (int sp = 0; sp < a.splits; ++sp) s += a.opart[(((size_t)blockIdx.x * a.splits + sp) * a.QT + i) * HD + r];
        ((T*)a.out)[(size_t)(ti.t0 + i) * HD + r] = from_f<T>(s);
    }
}

static size_t hm_smem_bytes(int H, int G, int D, int Dv, int QT, bool mix) {
    const size_t pitch = (size_t)(D > Dv ? D : Dv) + 1;
    return sizeof(float) * ((size_t)QT * H * D + (size_t)G * HM_KB * pitch + (size_t)(mix ? 2 : 1) * H * QT * HM_KB
                            + 2 * (size_t)QT * H + (size_t)H * H);
}

// The largest tile (a power of two up to `limit`) whose accumulators and shared memory fit; 0: none does.
extern "C" int pe_attention_headmix_tile(int H, int G, int D, int Dv, int mix, int limit) {
    for (int qt = 16; qt >= 1; qt >>= 1) {
        if (qt > limit) continue;
        if ((size_t)H * qt * Dv > (size_t)64 * HM_THREADS) continue;
        if (hm_smem_bytes(H, G, D, Dv, qt, mix != 0) > 200 * 1024) continue;
        return qt;
    }
    return 0;
}

extern "C" long long pe_attention_headmix_scratch_floats(int n_tiles, int splits, int QT, int H, int Dv) {
    return (long long)n_tiles * splits * QT * H * (2 + (splits > 1 ? Dv : 0));
}

template <typename T, int NACC>
static int hm_launch(const HeadMixArgs& a, int n_tiles, size_t smem, cudaStream_t s) {
    PE_TRY(cudaFuncSetAttribute(headmix_kernel<T, 0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PE_TRY(cudaFuncSetAttribute(headmix_kernel<T, 1, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PE_TRY(pe_launch(headmix_kernel<T, 0, 1>, dim3(n_tiles, a.splits), HM_THREADS, smem, s, a));
    PE_LAUNCH_CHECK();
    PE_TRY(pe_launch(headmix_kernel<T, 1, NACC>, dim3(n_tiles, a.splits), HM_THREADS, smem, s, a));
    PE_LAUNCH_CHECK();
    if (a.splits > 1) {
        PE_TRY(pe_launch(headmix_reduce_kernel<T>, n_tiles, 256, 0, s, a));
        PE_LAUNCH_CHECK();
    }
    return 0;
}

extern "C" int pe_attention_headmix(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool, int dtype,
                                    const int* table, int table_stride, const int* tok_pos, const int* tok_row,
                                    const int* tiles, int n_runs, int tile_tokens, int T, int H, int G, int D, int Dv,
                                    int window, float scale, const void* sink, int sink_dtype, const void* mix, int mix_dtype,
                                    int QT, int splits, float* scratch, const float* slopes, int keep_first, int v_ld, void* stream) {
    if (T <= 0) return 0;
    if (v_ld <= 0) v_ld = Dv;
    if (v_ld < Dv || keep_first < 0) return PE_ERR_UNSUPPORTED;
    if (H <= 0 || G <= 0 || H % G || QT < 1 || splits < 1 || splits > 65535 || (tiles && (tile_tokens % QT || n_runs <= 0)))
        return PE_ERR_UNSUPPORTED;
    if ((size_t)H * QT * Dv > (size_t)64 * HM_THREADS) return PE_ERR_UNSUPPORTED;
    const size_t smem = hm_smem_bytes(H, G, D, Dv, QT, mix != nullptr);
    if (smem > 227 * 1024) return PE_ERR_UNSUPPORTED;
    const int n_tiles = tiles ? n_runs * (tile_tokens / QT) : T;
    HeadMixArgs a = {q, q_stride, k_pool, v_pool, table, table_stride, tok_pos, tok_row, tiles, tile_tokens, H, G, D, Dv, window,
                     scale, sink, sink_dtype, mix, mix_dtype, QT, splits, slopes, keep_first, v_ld, scratch,
                     scratch + (size_t)n_tiles * splits * QT * H * 2, out};
    cudaStream_t s = (cudaStream_t)stream;
    const int nacc = (int)(((size_t)H * QT * Dv + HM_THREADS - 1) / HM_THREADS);
    if (dtype == PE_F32) {
        if (nacc <= 4) return hm_launch<float, 4>(a, n_tiles, smem, s);
        if (nacc <= 16) return hm_launch<float, 16>(a, n_tiles, smem, s);
        return hm_launch<float, 64>(a, n_tiles, smem, s);
    }
    if (dtype == PE_BF16) {
        if (nacc <= 4) return hm_launch<bf16, 4>(a, n_tiles, smem, s);
        if (nacc <= 16) return hm_launch<bf16, 16>(a, n_tiles, smem, s);
        return hm_launch<bf16, 64>(a, n_tiles, smem, s);
    }
    return PE_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- query/key norm and the cache write
// qkv [T, H*D + G*D + G*Dv] in the step's dtype.  Query and key heads are normed in place (RMS over the head:
// v / sqrt(mean(v^2) + eps) * w, float32), then keys and values go to their cache pages.  A warp per head.
template <typename T>
__global__ void __launch_bounds__(128) qknorm_store_kernel(T* qkv, int H, int G, int D, int Dv, const void* qw, int qw_dtype,
                                                           const void* kw, int kw_dtype, float eps, const int* tok_pos,
                                                           const int* tok_row, T* k_pool, T* v_pool, const int* table,
                                                           int table_stride, int store) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T* row = qkv + (size_t)t * ((size_t)H * D + (size_t)G * D + (size_t)G * Dv);
    const int pos = tok_pos[t];
    long long page = -1;
    if (store) page = table[(size_t)tok_row[t] * table_stride + pos / PE_PAGE];
    for (int u = warp; u < H + 2 * G; u += 4) {
        if (u < H + G) {                                 // a query or key head
            T* v = row + (size_t)u * D;
            const void* w = u < H ? qw : kw;
            const int wd = u < H ? qw_dtype : kw_dtype;
            float rstd = 1.f;
            if (w) {
                float ss = 0.f;
                for (int d = lane; d < D; d += 32) { const float f = to_f(v[d]); ss = fmaf(f, f, ss); }
                rstd = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
            }
            T* dst = (u >= H && store && page >= 0) ? k_pool + (((size_t)page * G + (u - H)) * PE_PAGE + pos % PE_PAGE) * D : nullptr;
            for (int d = lane; d < D; d += 32) {
                T o = v[d];
                if (w) { o = from_f<T>(to_f(o) * rstd * load_as_f(w, wd, d)); v[d] = o; }
                if (dst) dst[d] = o;
            }
        } else if (store && page >= 0) {                 // a value head
            const int c = u - H - G;
            const T* v = row + (size_t)(H + G) * D + (size_t)c * Dv;
            T* dst = v_pool + (((size_t)page * G + c) * PE_PAGE + pos % PE_PAGE) * Dv;
            for (int d = lane; d < Dv; d += 32) dst[d] = v[d];
        }
    }
}

extern "C" int pe_qknorm_store(void* qkv, int dtype, int T, int H, int G, int D, int Dv, const void* qw, int qw_dtype,
                               const void* kw, int kw_dtype, float eps, const int* tok_pos, const int* tok_row, void* k_pool,
                               void* v_pool, const int* table, int table_stride, int store, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32) PE_TRY(pe_launch(qknorm_store_kernel<float>, T, 128, 0, s, (float*)qkv, H, G, D, Dv, qw, qw_dtype, kw, kw_dtype, eps, tok_pos, tok_row, (float*)k_pool, (float*)v_pool, table, table_stride, store));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(qknorm_store_kernel<bf16>, T, 128, 0, s, (bf16*)qkv, H, G, D, Dv, qw, qw_dtype, kw, kw_dtype, eps, tok_pos, tok_row, (bf16*)k_pool, (bf16*)v_pool, table, table_stride, store));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}
