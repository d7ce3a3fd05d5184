// Attention with mixed heads for bfloat16 in one pass over the keys.
//
// The mixing is linear, so it can follow the product with the values:
//     o_h(i) = sum_j (sum_g mix[h, g] p_g(i, j)) v_c(h)(j) = sum_g mix[h, g] * (sum_j p_g(i, j) v_c(h)(j)).
// The first kernel is therefore flash attention whose every head g keeps an output for EVERY key/value head c,
// O'_g,c = sum_j exp(s_g(i, j) - m) v_c(j), with the running maximum m and the sum l of the exponentials, unnormalised:
// one product Q K^T and G products P V per block of keys, all on the tensor cores (mma.sync m16n8k16, float32
// accumulators, S and P in registers, the C fragment of S reused as the A fragment of P V).  The keys of a tile may be cut
// into ranges that run as blocks of their own and leave partial (m, l, O').  The second kernel merges the ranges,
// puts exp(sink_g) into the denominator, normalises and mixes: out_h = sum_g mix[h, g] O'_g,c(h) / l_g, in float32.
//
// Two row layouts of the 16-row MMA tile:
//   prompt: rows are consecutive tokens of one sequence, a block = 64 tokens (4 warps) of one head and one group
//           of value heads;
//   single tokens: rows are the query heads that share a key/value head (a warp per 16 of them), a block = one
//           token, one key/value head for the keys and one group of value heads.
// A block of keys is one cache page (64 positions): K of the head's key/value head and V of the group's heads are
// copied to shared memory by cp.async (16 bytes a copy, rows beyond the range's end zero-filled), the next page
// while this one is multiplied (two stages).  Head sizes: D a multiple of 16, Dv of 8.
#include "common.cuh"

#define FX_THREADS 128
#define FX_WARPS 4
#define FX_PAD 8

struct FlashMixArgs {
    const bf16* q; int q_stride;
    const bf16* k_pool; const bf16* v_pool;
    const int* table; int table_stride;
    const int* tok_pos; const int* tok_row;
    const int* tiles;                         // prompt: runs of at most 64 tokens (row, first token, tokens, first position); null: single tokens
    int H, G, D, Dv, window; float scale;
    int splits, cg, ngroups;                  // ranges of keys; value heads a block; groups of value heads
    const float* slopes; int keep_first; int v_ld; int v_in_k;   // slope_h * (i - j) is taken off a score (null: nothing); the first keep_first keys stay
                                                     // visible behind the window; a value row has v_ld entries of which the first Dv are read;
                                                     // v_in_k: the values are the front of the one key head's rows and are read from K's copy
    float* pm; float* pl; float* po;          // [T][splits][H], [T][splits][H], [T][splits][H][G][Dv]
    bf16* direct; const float* sink;          // direct != null (one range, no mixing): a head's output is complete in the block that has its
                                              // key/value head: it is normalised (with exp(sink) in the denominator) and written there
};

__device__ __forceinline__ void fx_ldsm_x2(uint32_t (&r)[2], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void fx_ldsm_x2_trans(uint32_t (&r)[2], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void fx_mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// 16 bytes global -> shared without a register in between; `bytes` 0 writes zeros
__device__ __forceinline__ void fx_cp16(void* dst, const void* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fx_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void fx_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

__device__ __forceinline__ float fx_exp2(float v) {          // 2^v; 2^-inf = 0
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ uint32_t fx_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// DKM: most 16-wide steps of the head size; NVM: most 8-wide value tiles a block accumulates (cg * Dv / 8).
// SUB (single tokens whose query heads of a key/value head fill one warp's 16 rows): every warp takes the same rows and a
// quarter of each page's keys (16), and leaves a partial result of its own, as if the range were cut in four once more.
template <int DKM, int NVM, bool SUB>
__global__ void __launch_bounds__(FX_THREADS, (NVM <= 16 && DKM <= 8) ? 3 : 2) flashmix_kernel(FlashMixArgs a) {
    constexpr int NT = SUB ? 2 : 8;                           // tiles of 8 keys a warp takes of a page
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char fx_smem[];
    const int H = a.H, G = a.G, D = a.D, Dv = a.Dv, per_kv = H / G;
    const int kp = D + FX_PAD, vp = Dv + FX_PAD;
    const int vs_ld = a.v_in_k ? kp : vp;                     // entries between two value rows in a stage
    const size_t stage_elems = (size_t)PE_PAGE * kp + (a.v_in_k ? 0 : (size_t)a.cg * PE_PAGE * vp);      // a stage: K [64][kp], V [cg][64][vp]
    bf16* stages = reinterpret_cast<bf16*>(fx_smem);          // two stages: the next page is copied while this one is used
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, split = blockIdx.z;
    const bool prompt = a.tiles != nullptr;
    const int koff = SUB ? warp * 16 : 0;                     // the warp's first key within a page

    // what the block and this warp's 16 rows stand for
    int seq, p_first, p_last, kvh, grp;
    int tok[2], head[2], qpos[2];                             // of this thread's two rows (lane / 4 and lane / 4 + 8)
    bool live[2];
    if (prompt) {
        const int* r = a.tiles + 4 * blockIdx.x;
        const int g = blockIdx.y / a.ngroups;
        grp = blockIdx.y % a.ngroups;
        seq = r[0]; p_first = r[3]; p_last = r[3] + r[2] - 1; kvh = g / per_kv;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int i = warp * 16 + (lane >> 2) + x * 8;
            live[x] = i < r[2]; tok[x] = r[1] + i; head[x] = g; qpos[x] = r[3] + i;
        }
    } else {
        const int t = blockIdx.x;
        kvh = blockIdx.y / a.ngroups;
        grp = blockIdx.y % a.ngroups;
        seq = a.tok_row[t]; p_first = p_last = a.tok_pos[t];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int i = (SUB ? 0 : warp * 16) + (lane >> 2) + x * 8;
            live[x] = i < per_kv; tok[x] = t; head[x] = kvh * per_kv + i; qpos[x] = p_first;
        }
    }
    const int c_lo = grp * a.cg, c_n = min(a.cg, G - c_lo);   // this block's value heads
    const int nvt = Dv / 8, nv = c_n * nvt, dk = D / 16;
    const int hi = p_last + 1;
    int lo = (a.window > 0 && p_first - a.window + 1 > 0) ? (p_first - a.window + 1) & ~(PE_PAGE - 1) : 0;
    // the pages of the kept first keys are visited in front of the window's, unless the window reaches them anyway
    int kept_pages = (a.window > 0 && a.keep_first > 0) ? (a.keep_first + PE_PAGE - 1) / PE_PAGE : 0;
    if (lo <= kept_pages * PE_PAGE) { lo = 0; kept_pages = 0; }
    const int n_pages = kept_pages + (hi - lo + PE_PAGE - 1) / PE_PAGE;
    const int per_split = (n_pages + a.splits - 1) / a.splits;
    const int b_begin = split * per_split, b_end = min(n_pages, b_begin + per_split);
    const int k_end = hi;
    auto page_start = [&](int blk) { return blk < kept_pages ? blk * PE_PAGE : lo + (blk - kept_pages) * PE_PAGE; };
    const int* table = a.table + (size_t)seq * a.table_stride;

    // the queries of this warp's rows as A fragments
    uint32_t qf[DKM][4];
#pragma unroll
    for (int kk = 0; kk < DKM; ++kk) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int rr = x & 1, col = kk * 16 + (lane & 3) * 2 + (x >> 1) * 8;
            qf[kk][x] = (kk < dk && live[rr]) ? *reinterpret_cast<const uint32_t*>(a.q + (size_t)tok[rr] * a.q_stride + (size_t)head[rr] * D + col) : 0u;
        }
    }
    float o[NVM][4];
#pragma unroll
    for (int n = 0; n < NVM; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const float sl2 = a.scale * 1.4426950408889634f;          // scores in units of log2 e
    float slope2[2] = {0.f, 0.f};                             // the rows' distance slopes in the same units
    if (a.slopes) {
#pragma unroll
        for (int x = 0; x < 2; ++x) slope2[x] = live[x] ? a.slopes[head[x]] * 1.4426950408889634f : 0.f;
    }
    const int q_first = prompt ? a.tiles[4 * blockIdx.x + 3] + warp * 16 : p_first;      // the earliest position among this warp's rows
    const bool warp_live = prompt ? (warp * 16 < a.tiles[4 * blockIdx.x + 2]) : (SUB || warp * 16 < per_kv);

    // Copies of one page into a stage.  The page's keys of one key/value head are one contiguous piece of the pool, and so are
    // its values of the group's heads; both go to padded rows in 16-byte units.  A thread's units are `FX_THREADS` apart: their
    // (row, column) advance by fixed steps (no division inside the loop).
    const int per = D >> 3, perv = Dv >> 3;
    const int k_r0 = tid / per, k_c0 = tid % per, k_dr = FX_THREADS / per, k_dc = FX_THREADS % per;
    const int v_r0 = tid / perv, v_c0 = tid % perv, v_dr = FX_THREADS / perv, v_dc = FX_THREADS % perv;
    auto copy_page = [&](int kb, int stage) {
        const int page = table[kb / PE_PAGE];
        const int valid = page >= 0 ? min(PE_PAGE, k_end - kb) : 0;
        bf16* ks = stages + stage * stage_elems;
        bf16* vs = ks + (size_t)PE_PAGE * kp;
        const bf16* ksrc = a.k_pool + (((size_t)max(page, 0) * G + kvh) * PE_PAGE) * D;
        for (int r = k_r0, c = k_c0; r < PE_PAGE;) {
            fx_cp16(ks + (size_t)r * kp + c * 8, ksrc + (size_t)r * D + c * 8, r < valid ? 16 : 0);
            r += k_dr; c += k_dc;
            if (c >= per) { c -= per; ++r; }
        }
        const bf16* vsrc = a.v_pool + (((size_t)max(page, 0) * G + c_lo) * PE_PAGE) * a.v_ld;
        for (int r = v_r0, c = v_c0; !a.v_in_k && r < c_n * PE_PAGE;) {
            fx_cp16(vs + (size_t)r * vp + c * 8, vsrc + (size_t)r * a.v_ld + c * 8, (r & (PE_PAGE - 1)) < valid ? 16 : 0);
            r += v_dr; c += v_dc;
            if (c >= perv) { c -= perv; ++r; }
        }
        fx_commit();
    };
    // where value tile n of this block lies in a stage's V (head n / nvt, columns 8 (n % nvt) ..): a table, not divisions in the loop
    __shared__ int v_off[32];
    if (tid < 32) v_off[tid] = tid < nv ? (tid / nvt) * PE_PAGE * vs_ld + (tid % nvt) * 8 : 0;
    __syncthreads();
    if (b_begin < b_end) copy_page(page_start(b_begin), 0);
    int stage = 0;
#pragma unroll 1
    for (int blk = b_begin; blk < b_end; ++blk, stage ^= 1) {
        const int kb = page_start(blk);
        const int valid = table[kb / PE_PAGE] >= 0 ? min(PE_PAGE, k_end - kb) : 0;
        if (blk + 1 < b_end) { copy_page(page_start(blk + 1), stage ^ 1); fx_wait<1>(); }
        else fx_wait<0>();
        __syncthreads();                                      // this page's copies of all threads have landed
        const bf16* k_s = stages + stage * stage_elems;
        const bf16* v_lane = k_s + (a.v_in_k ? 0 : (size_t)PE_PAGE * kp) + (koff + (lane & 15)) * vs_ld;      // this lane's row of a 16-key step of V
        const bf16* k_lane = k_s + (size_t)(koff + (lane & 7)) * kp + ((lane >> 3) & 1) * 8;
        if (warp_live) {
        // S = Q K^T: NT tiles of 8 keys
        float s[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < DKM; ++kk) {
            if (kk < dk) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    uint32_t bfr[2];
                    fx_ldsm_x2(bfr, k_lane + n * 8 * kp + kk * 16);
                    fx_mma(s[n], qf[kk], bfr);
                }
            }
        }
        // scale (into units of log2 e, so that the exponentials are single ex2 instructions), mask, the rows' new maxima
        float mx[2] = {-INFINITY, -INFINITY};
        if (valid == PE_PAGE && a.window <= 0 && !a.slopes && kb + PE_PAGE - 1 <= q_first) {
            // every key of the page is seen by every row of this warp: nothing to mask
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int x = 0; x < 4; ++x) { s[n][x] *= sl2; mx[x >> 1] = fmaxf(mx[x >> 1], s[n][x]); }
            }
        } else {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int rr = x >> 1, j = koff + n * 8 + (lane & 3) * 2 + (x & 1), key = kb + j;
                    const bool seen = live[rr] && j < valid && key <= qpos[rr] &&
                                      (a.window <= 0 || qpos[rr] - key < a.window || key < a.keep_first);
                    s[n][x] = seen ? s[n][x] * sl2 - slope2[rr] * (float)(qpos[rr] - key) : -INFINITY;
                    mx[rr] = fmaxf(mx[rr], s[n][x]);
                }
            }
        }
        float alpha[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            const float m_new = fmaxf(m[rr], mx[rr]);
            alpha[rr] = (m[rr] > -INFINITY) ? fx_exp2(m[rr] - m_new) : 0.f;
            m[rr] = m_new;
            l[rr] *= alpha[rr];
        }
        const float m0 = m[0] > -INFINITY ? m[0] : 0.f, m1 = m[1] > -INFINITY ? m[1] : 0.f;     // (a row that has seen nothing: exp2(-inf - 0) = 0)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            s[n][0] = fx_exp2(s[n][0] - m0); s[n][1] = fx_exp2(s[n][1] - m0);
            s[n][2] = fx_exp2(s[n][2] - m1); s[n][3] = fx_exp2(s[n][3] - m1);
            l[0] += s[n][0] + s[n][1];
            l[1] += s[n][2] + s[n][3];
        }
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {                      // some row's maximum moved
#pragma unroll
            for (int n = 0; n < NVM; ++n) { o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1]; }
        }
        // O' += P V for every value head of the group
#pragma unroll
        for (int ks = 0; ks < NT / 2; ++ks) {
            uint32_t pf[4] = {fx_pack(s[2 * ks][0], s[2 * ks][1]), fx_pack(s[2 * ks][2], s[2 * ks][3]),
                              fx_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), fx_pack(s[2 * ks + 1][2], s[2 * ks + 1][3])};
#pragma unroll
            for (int n = 0; n < NVM; ++n) {
                if (n < nv) {
                    uint32_t bfr[2];
                    fx_ldsm_x2_trans(bfr, v_lane + v_off[n] + ks * 16 * vs_ld);
                    fx_mma(o[n], pf, bfr);
                }
            }
        }
        }
        __syncthreads();                                      // the stage is free for the page after the next
    }

    if (!warp_live) return;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
    }
    if (a.direct) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int ci = head[rr] / per_kv - c_lo;              // the head's own value head among this block's
            if (!live[rr] || ci < 0 || ci >= c_n) continue;
            float den = l[rr];
            if (a.sink) den += exp2f(fmaf(a.sink[head[rr]], 1.4426950408889634f, -m[rr]));      // (m in powers of two)
            const float inv = den > 0.f ? 1.0f / den : 0.f;
            bf16* dst = a.direct + ((size_t)tok[rr] * H + head[rr]) * Dv;
#pragma unroll
            for (int n = 0; n < NVM; ++n) {
                if (n < nv && n / nvt == ci)
                    *reinterpret_cast<__nv_bfloat162*>(dst + (n % nvt) * 8 + (lane & 3) * 2) = __floats2bfloat162_rn(o[n][rr * 2] * inv, o[n][rr * 2 + 1] * inv);
            }
        }
        return;
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        if (!live[rr]) continue;
        const size_t at = ((size_t)tok[rr] * (SUB ? 4 * a.splits : a.splits) + (SUB ? 4 * split + warp : split)) * H + head[rr];
        if ((lane & 3) == 0 && grp == 0) { a.pm[at] = m[rr] * 0.6931471805599453f; a.pl[at] = l[rr]; }     // the maximum back in natural units
        float* dst = a.po + (at * G + c_lo) * Dv;
#pragma unroll
        for (int n = 0; n < NVM; ++n) {
            if (n < nv) {
                const int ci = n / nvt, nt = n % nvt;
                *reinterpret_cast<float2*>(dst + (size_t)ci * Dv + nt * 8 + (lane & 3) * 2) = make_float2(o[n][rr * 2], o[n][rr * 2 + 1]);
            }
        }
    }
}

// out[t][h] = sum_g mix[h, g] * (sum over ranges of O'_g,c(h) * exp(m - M_g)) / (sum over ranges of l * exp(m - M_g) + exp(sink_g - M_g)).
// A block has R groups of Dv threads (a thread a value column).  With many (range, head) pairs to add (single tokens with
// long contexts: `share` = 1) a block takes one (token, head) and deals the pairs to its groups, whose sums meet in shared
// memory in the order of the groups; with few (prompts) every group takes a head of its own.  A thread's loads do not
// depend on one another; eight are in flight at a time.
__global__ void __launch_bounds__(1024) flashmix_merge_kernel(FlashMixArgs a, const float* sink, const float* mix, bf16* out, int share) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float merge_s[];
    const int t = blockIdx.x, H = a.H, G = a.G, Dv = a.Dv, per_kv = H / G, S = a.splits;
    float* coef = merge_s;                                    // [splits][H]: first the ranges' maxima, then exp(m - M_g) / denominator_g
    float* pl_s = coef + S * H;                               // [splits][H]: the ranges' sums
    float* M_s = pl_s + S * H;                                // [H]
    float* inv_s = M_s + H;                                   // [H]
    float* red = inv_s + H;                                   // [R][Dv]
    for (int e = threadIdx.x; e < S * H; e += blockDim.x) {   // all loads at once, not one after the other
        coef[e] = a.pm[(size_t)t * S * H + e];
        pl_s[e] = a.pl[(size_t)t * S * H + e];
    }
    __syncthreads();
    // a head's maximum and denominator: a warp a head, its lanes dealt the partial results (whole warps only take part)
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int g = wid; wid < n_warps && g < H; g += n_warps) {
        float M = -INFINITY;
        for (int s = lane; s < S; s += 32) M = fmaxf(M, coef[s * H + g]);
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        if (sink) M = fmaxf(M, sink[g]);
        float den = 0.f;
        for (int s = lane; s < S; s += 32) if (coef[s * H + g] > -INFINITY) den += pl_s[s * H + g] * expf(coef[s * H + g] - M);
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        if (sink) den += expf(sink[g] - M);
        if (lane == 0) { M_s[g] = M; inv_s[g] = den > 0.f ? 1.0f / den : 0.f; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < S * H; e += blockDim.x) {
        const int g = e % H;
        coef[e] = coef[e] > -INFINITY ? expf(coef[e] - M_s[g]) * inv_s[g] : 0.f;
    }
    __syncthreads();
    const int R = blockDim.x / Dv, r = threadIdx.x / Dv, d = threadIdx.x % Dv;
    const int h = share ? blockIdx.y : blockIdx.y * R + r;   // this group's head
    const bool on = r < R && h < H;
    float acc = 0.f;
    if (on) {
        const float* po = a.po + (size_t)t * S * H * G * Dv + (size_t)(h / per_kv) * Dv + d;
        const float* mrow = mix ? mix + (size_t)h * H : nullptr;
        const int first = share ? r : 0, step = share ? R : 1;
        if (mix) {
            // pairs (s, g) in the order s-major; g advances by `step` with carry into s (no division in the loop)
            int sg = first / H, g = first % H;
#pragma unroll 8
            for (int p = first; p < S * H; p += step) {
                acc = fmaf(coef[sg * H + g] * mrow[g], po[((size_t)sg * H + g) * G * Dv], acc);
                g += step;
                while (g >= H) { g -= H; ++sg; }
            }
        } else {
#pragma unroll 8
            for (int sg = first; sg < S; sg += step) acc = fmaf(coef[sg * H + h], po[((size_t)sg * H + h) * G * Dv], acc);
        }
    }
    if (!share) {
        if (on) out[((size_t)t * H + h) * Dv + d] = __float2bfloat16_rn(acc);
        return;
    }
    if (on) red[r * Dv + d] = acc;
    __syncthreads();
    if (threadIdx.x < Dv) {
        float sum = 0.f;
        for (int k = 0; k < R; ++k) sum += red[k * Dv + threadIdx.x];
        out[((size_t)t * H + blockIdx.y) * Dv + threadIdx.x] = __float2bfloat16_rn(sum);
    }
}

// Value heads a block accumulates for these sizes (0: the kernel does not take them).
extern "C" int pe_attention_flashmix_group(int H, int G, int D, int Dv) {
    if (H < 1 || G < 1 || H % G || D % 16 || Dv % 8 || D < 16 || D > 256 || Dv < 8 || Dv > 256 || H / G > 16 * FX_WARPS) return 0;
    int cg = (32 * 8) / Dv;                                   // 32 accumulator tiles of 8 columns
    if (cg > G) cg = G;
    return cg;
}

// single != 0: single tokens, whose ranges may be cut in four once more inside a block
extern "C" long long pe_attention_flashmix_scratch_floats(int T, int splits, int H, int G, int Dv, int single) {
    return (long long)T * splits * (single ? 4 : 1) * H * (2 + (long long)G * Dv);
}

template <int DKM, int NVM, bool SUB>
static int fx_launch_as(const FlashMixArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
    PE_TRY(cudaFuncSetAttribute(flashmix_kernel<DKM, NVM, SUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PE_TRY(pe_launch(flashmix_kernel<DKM, NVM, SUB>, grid, FX_THREADS, smem, s, a));
    PE_LAUNCH_CHECK();
    return 0;
}
template <int DKM, int NVM>
static int fx_launch(const FlashMixArgs& a, bool sub, dim3 grid, size_t smem, cudaStream_t s) {
    return sub ? fx_launch_as<DKM, NVM, true>(a, grid, smem, s) : fx_launch_as<DKM, NVM, false>(a, grid, smem, s);
}

extern "C" int pe_attention_flashmix(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                     const int* table, int table_stride, const int* tok_pos, const int* tok_row,
                                     const int* tiles, int n_runs, int T, int H, int G, int D, int Dv, int window, float scale,
                                     const float* sink, const float* mix, int splits, float* scratch, const float* slopes,
                                     int keep_first, int v_ld, void* stream) {
    if (T <= 0) return 0;
    if (v_ld <= 0) v_ld = Dv;
    if (v_ld < Dv || v_ld % 8 || keep_first < 0) return PE_ERR_UNSUPPORTED;
    const int cg = pe_attention_flashmix_group(H, G, D, Dv);
    if (cg == 0 || splits < 1 || splits > 65535 || (tiles && n_runs <= 0)) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15 || (q_stride & 1)) return PE_ERR_UNSUPPORTED;
    const int ngroups = (G + cg - 1) / cg;
    int merge_threads = Dv >= 256 ? Dv : (256 / Dv) * Dv;                          // whole groups of Dv threads
    // single tokens whose heads of a key/value head fill one warp's rows: the four warps share a page's keys (where the merge
    // kernel has room for four times the partial results)
    const bool sub = !tiles && H / G <= 16 && sizeof(float) * (8 * (size_t)H * splits + 2 * (size_t)H + 1024) <= 48 * 1024;
    const int parts = sub ? 4 * splits : splits;              // partial results a (token, head)
    float* pm = scratch;
    float* pl = pm + (size_t)T * parts * H;
    float* po = pl + (size_t)T * parts * H;
    FlashMixArgs a = {(const bf16*)q, q_stride, (const bf16*)k_pool, (const bf16*)v_pool, table, table_stride, tok_pos, tok_row, tiles,
                      H, G, D, Dv, window, scale, splits, cg, ngroups, slopes, keep_first, v_ld, 0, pm, pl, po, nullptr, sink};
    if (parts == 1 && !mix && !(((uintptr_t)out) & 3) && Dv % 2 == 0) a.direct = (bf16*)out;      // no partial results, no merge
    a.v_in_k = (v_pool == k_pool && G == 1 && v_ld == D) ? 1 : 0;                  // one copy of a page serves as keys and values
    const size_t smem = 2 * 2 * ((size_t)PE_PAGE * (D + FX_PAD) + (a.v_in_k ? 0 : (size_t)cg * PE_PAGE * (Dv + FX_PAD)));      // two stages of bfloat16
    const size_t merge_smem = sizeof(float) * (2 * (size_t)H * parts + 2 * (size_t)H + 1024);       // (room for the most threads)
    if (smem > 220 * 1024 || merge_smem > 48 * 1024 || H > 65535) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(tiles ? n_runs : T, (tiles ? H : G) * ngroups, splits);
    const int dk = D / 16, nv = cg * (Dv / 8);
    int rc;
    if (dk <= 4) rc = nv <= 16 ? fx_launch<4, 16>(a, sub, grid, smem, s) : fx_launch<4, 32>(a, sub, grid, smem, s);
    else if (dk <= 8) rc = nv <= 16 ? fx_launch<8, 16>(a, sub, grid, smem, s) : fx_launch<8, 32>(a, sub, grid, smem, s);
    else rc = nv <= 16 ? fx_launch<16, 16>(a, sub, grid, smem, s) : fx_launch<16, 32>(a, sub, grid, smem, s);
    if (rc) return rc;
    if (a.direct) return 0;
    a.splits = parts;                                         // what the merge kernel adds up
    if (parts * (mix ? H : 1) >= 64) merge_threads = (1024 / Dv) * Dv;               // many pairs to add: more groups share them
    const int groups = merge_threads / Dv;
    const int share = (parts * (mix ? H : 1) >= 64 && groups > 1) ? 1 : 0;           // many pairs to add: the groups share a head
    PE_TRY(pe_launch(flashmix_merge_kernel, dim3(T, share ? H : (H + groups - 1) / groups), merge_threads, merge_smem, s, a, sink, mix,
                     (bf16*)out, share));
    PE_LAUNCH_CHECK();
    return 0;
}
