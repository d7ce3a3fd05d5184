// A selective state-space mixer with a scalar decay a head and token: the short causal convolution with silu on its inputs,
// the recurrence, and the gate followed by a norm over groups of channels.  Decays, step sizes, the state, its outputs, the
// gate and the norm are float32 in either engine dtype; only the loads of projections and the store of the result convert.
//
//   dt_t = softplus(dt_raw_t + dt_bias_h)        a_t = exp(-exp(A_log_h) * dt_t)
//   S_t = a_t S_(t-1) + dt_t B_t x_t^T           (S [N, P] a head, B and C shared by the heads of a group)
//   y_t = S_t^T C_t + D_h x_t
//
// The recurrence runs token after token: a block owns (sequence, head, a tile of the P columns); thread (p, ns) keeps rows
// n = ns NR + r (r < NR) of column p in registers (B and C are read from shared memory four rows at a time), the NS threads of a
// column are neighbours in a warp and add their parts of y by shuffles.  Prompts can run as three passes over chunks of 64 tokens.
// A sequence's state lies in its row of the cache's state area in exactly the order the threads hold it,
// element ((h * NR + r) * P + p) * NS + ns, so it is read and written in whole lines; rows n >= N are padding and stay zero.
// NS depends on N alone (the smallest power of two that leaves a thread at most 16 rows), so a model's layout never changes.
#include "common.cuh"

extern "C" void pe_set_pdl(int on) { pe_pdl_enabled() = on ? 1 : 0; }     // (this library's own copy of the switch)

#define SS_TOKENS 8          // tokens whose B, C, x, dt are staged in shared memory at a time

__device__ __forceinline__ float ss_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float ss_softplus(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

// ---------------------------------------------------------------- convolution + silu
// in: columns c_off .. c_off + C - 1 of proj [T, ld] (the step's dtype).  out [T, C] float32:
// silu(bias[c] + sum_j w[c, j] * u_(t - taps + 1 + j)[c]); inputs before the step's first token come from the sequence's state
// (entry k: the input k + 1 places before the next step's first token), inputs before the sequence's start are zero (the state of a
// new sequence is zero).
template <typename T>
__global__ void conv_silu_kernel(const T* proj, int ld, int c_off, int C, int taps, const void* w, int w_dtype, const void* bias,
                                 int b_dtype, const float* state, long long state_stride, const int* tok_row, const int* row_first,
                                 const int* slots, float* out, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const int t = (int)(e / C), c = (int)(e % C);
    const int b = tok_row[t], i = t - row_first[b];              // the token's place within its row's tokens of this step
    const float* st = state + (size_t)slots[b] * state_stride;
    float acc = bias ? load_as_f(bias, b_dtype, c) : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                           // 0: the token itself
        const float v = back <= i ? to_f(proj[(size_t)(t - back) * ld + c_off + c]) : st[(size_t)(back - i - 1) * C + c];
        acc = fmaf(load_as_f(w, w_dtype, (size_t)c * taps + j), v, acc);
    }
    out[e] = ss_silu(acc);
}

// New state from the step's inputs: entry k <- the input of the step's token n - 1 - k, or, where the step brought fewer tokens,
// the old entry k - n.  Entries are rewritten from the oldest to the newest, so an old entry is read before it is overwritten.
template <typename T>
__global__ void conv_state_kernel(const T* proj, int ld, int c_off, int C, int taps, float* state, long long state_stride,
                                  const int* row_first, const int* row_lens, const int* slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int n = row_lens[b], first = row_first[b];
    float* st = state + (size_t)slots[b] * state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x)
        for (int k = taps - 2; k >= 0; --k)
            st[(size_t)k * C + c] = k < n ? to_f(proj[(size_t)(first + n - 1 - k) * ld + c_off + c]) : st[(size_t)(k - n) * C + c];
}

extern "C" int pe_conv_silu(const void* proj, int dtype, int ld, int c_off, int C, int taps, const void* w, int w_dtype, const void* bias,
                            int b_dtype, float* state, long long state_stride, const int* tok_row, const int* row_first,
                            const int* row_lens, const int* slots, float* out, int T, int B, void* stream) {
    if (T <= 0) return 0;
    if (taps < 1 || C <= 0 || c_off < 0 || c_off + C > ld) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * C;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == PE_F32) PE_TRY(pe_launch(conv_silu_kernel<float>, blocks, 256, 0, s, (const float*)proj, ld, c_off, C, taps, w, w_dtype, bias, b_dtype, (const float*)state, state_stride, tok_row, row_first, slots, out, total));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(conv_silu_kernel<bf16>, blocks, 256, 0, s, (const bf16*)proj, ld, c_off, C, taps, w, w_dtype, bias, b_dtype, (const float*)state, state_stride, tok_row, row_first, slots, out, total));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    if (taps > 1) {
        if (dtype == PE_F32) PE_TRY(pe_launch(conv_state_kernel<float>, dim3(B, (C + 255) / 256), 256, 0, s, (const float*)proj, ld, c_off, C, taps, state, state_stride, row_first, row_lens, slots));
        else PE_TRY(pe_launch(conv_state_kernel<bf16>, dim3(B, (C + 255) / 256), 256, 0, s, (const bf16*)proj, ld, c_off, C, taps, state, state_stride, row_first, row_lens, slots));
        PE_LAUNCH_CHECK();
    }
    return 0;
}

// ---------------------------------------------------------------- the recurrence
#define SS_CHUNK 64          // tokens of a chunk in the three-pass way

struct ScanArgs {
    const float* xbc; int xbc_ld;             // [T, inner + 2 G N] float32: x | B | C after the convolution
    const void* proj; int proj_ld, dt_off;    // dt_raw at columns dt_off .. dt_off + H - 1 of proj (the step's dtype)
    const void* dt_bias; int dtb_dtype; const void* a_log; int al_dtype; const void* d_skip; int d_dtype;   // [H] each
    float* state; long long state_stride;     // row slots[b] holds the sequence's state
    const int* row_first; const int* row_lens; const int* slots;
    float* y;                                 // [T, H * P]
    int B, H, P, N, G, NS, NR, NRP, PT;
    float* chunk_state;                       // [chunks][H * NR * P * NS]: a chunk's own contribution, then its incoming state
    float* chunk_decay;                       // [chunks][H]: the product of a chunk's decays
    int max_chunks;
};

extern "C" int pe_state_space_split(int N) {
    int ns = 1;
    while ((N + ns - 1) / ns > 16 && ns < 32) ns *= 2;
    return ns;
}
// float32 numbers of a sequence's state for these sizes (with the padding rows)
extern "C" long long pe_state_space_elems(int H, int P, int N) {
    const int ns = pe_state_space_split(N);
    return (long long)H * ((N + ns - 1) / ns) * ns * P;
}
// Chunks a step of T tokens in B sequences can have at most, and the floats of scratch the three-pass way needs.
extern "C" int pe_state_space_chunks(int T, int B) { return (T + SS_CHUNK - 1) / SS_CHUNK + B; }
extern "C" long long pe_state_space_scratch_floats(int T, int B, int H, int P, int N) {
    return (long long)pe_state_space_chunks(T, B) * (pe_state_space_elems(H, P, N) + H);
}

// Which sequence chunk `c` of the step belongs to, its first packed token and its number of tokens (0: no such chunk).
__device__ __forceinline__ void ss_find_chunk(const int* row_first, const int* row_lens, int B, int c, int& row, int& first, int& count) {
    int base = 0;
    row = -1; first = 0; count = 0;
    for (int b = 0; b < B; ++b) {
        const int n = row_lens[b], nc = (n + SS_CHUNK - 1) / SS_CHUNK;
        if (c < base + nc) {
            const int local = c - base;
            row = b; first = row_first[b] + local * SS_CHUNK;
            count = min(SS_CHUNK, n - local * SS_CHUNK);
            return;
        }
        base += nc;
    }
}

// MODE 0: a sequence's tokens from its stored state; 1: a chunk from zero, leaving its contribution and the product of its decays;
// 2: a chunk from its incoming state, writing outputs.  The recurrence is linear in S (S_end = (prod a) S_in + L), so the three-pass
// way (1, the carry kernel, 2) equals the walk up to float32 rounding.
template <typename T, int NRMAX, int MODE>
__global__ void __launch_bounds__(256, MODE == 0 ? 1 : 3) scan_kernel(ScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float ss_smem[];
    __shared__ int where[3];
    const int h = blockIdx.y, p0 = blockIdx.z * a.PT;
    const int N = a.N, P = a.P, NS = a.NS, NR = a.NR, NRP = a.NRP, PT = a.PT, ROW = NS * NRP;
    const int tid = threadIdx.x, ns = tid % NS, pl = tid / NS, p = p0 + pl;
    const bool on = pl < PT && p < P;
    const int g = h / (a.H / a.G), inner = a.H * P;
    float* Bs = ss_smem;                      // [SS_TOKENS][ROW]: row n = s NR + r at s NRP + r (a thread's rows side by side, padded)
    float* Cs = Bs + SS_TOKENS * ROW;         // [SS_TOKENS][ROW]
    float* xs = Cs + SS_TOKENS * ROW;         // [SS_TOKENS][PT]
    float* dts = xs + SS_TOKENS * PT;         // [SS_TOKENS]: step sizes
    float* das = dts + SS_TOKENS;             // [SS_TOKENS]: decays
    int b, first, n_tok;
    if (MODE == 0) {
        b = blockIdx.x; first = a.row_first[b]; n_tok = a.row_lens[b];
    } else {
        if (tid == 0) { ss_find_chunk(a.row_first, a.row_lens, a.B, blockIdx.x, b, first, n_tok); where[0] = b; where[1] = first; where[2] = n_tok; }
        __syncthreads();
        b = where[0]; first = where[1]; n_tok = where[2];
    }
    if (n_tok <= 0) return;
    const size_t per_head = (size_t)NR * P * NS;
    float* st = nullptr;
    if (MODE == 0) st = a.state + (size_t)a.slots[b] * a.state_stride + (size_t)h * per_head;
    else st = a.chunk_state + ((size_t)blockIdx.x * a.H + h) * per_head;
    float S[NRMAX];
#pragma unroll
    for (int r = 0; r < NRMAX; ++r) S[r] = (MODE != 1 && on && r < NR) ? st[((size_t)r * P + p) * NS + ns] : 0.f;
    const float A = expf(load_as_f(a.a_log, a.al_dtype, h)), Dh = load_as_f(a.d_skip, a.d_dtype, h), dtb = load_as_f(a.dt_bias, a.dtb_dtype, h);
    float decay = 1.f;                                         // MODE 1: the product of the chunk's decays
    const T* proj = (const T*)a.proj;
    // Where a group's B, C, x and raw step sizes are few enough a thread (at most SS_PRE entries of B and of C, one of x), they are
    // fetched into registers while the group before is walked, and go to shared memory after it: the loads' latency lies under the
    // walk.  Entry k of a thread is element e = tid + k blockDim.x of the group every time, so what it stands for is worked out once:
    // code = token << 24 | state row n; -2 a padding place (zero), -1 nothing.
    constexpr int SS_PRE = 6;
    const bool pre = MODE != 0 && SS_TOKENS * ROW <= SS_PRE * (int)blockDim.x && SS_TOKENS * PT <= (int)blockDim.x;   // (the walk of whole rows, which decoding uses, stages as it goes)
    int code[SS_PRE];
    float pb[SS_PRE], pc[SS_PRE], px = 0.f, pdt = 0.f;
    const float* b_col = a.xbc + inner + g * N;                // B of this head's group; C lies G N columns further
    const int c_off = a.G * N;
    const int x_tok = tid / PT, x_col = tid % PT;              // the x entry of this thread
#pragma unroll
    for (int k = 0; k < SS_PRE; ++k) {
        code[k] = -1;
        pb[k] = pc[k] = 0.f;
        const int e = tid + k * (int)blockDim.x;
        if (pre && e < SS_TOKENS * ROW) {
            const int i = e / ROW, w = e % ROW, sidx = w / NRP, r = w % NRP, n = sidx * NR + r;
            code[k] = (r < NR && n < N) ? ((i << 24) | n) : -2;
        }
    }
    auto fetch = [&](int c0) {
        const int nc = min(SS_TOKENS, n_tok - c0);
#pragma unroll
        for (int k = 0; k < SS_PRE; ++k) {
            const int i = code[k] >> 24, n = code[k] & 0xffffff;
            const bool there = code[k] >= 0 && i < nc;
            const float* at = b_col + (size_t)(first + c0 + (there ? i : 0)) * a.xbc_ld + (there ? n : 0);
            pb[k] = there ? at[0] : 0.f;
            if (MODE != 1) pc[k] = there ? at[c_off] : 0.f;
        }
        px = (x_tok < nc && p0 + x_col < P) ? a.xbc[(size_t)(first + c0 + x_tok) * a.xbc_ld + h * P + p0 + x_col] : 0.f;
        pdt = tid < nc ? to_f(proj[(size_t)(first + c0 + tid) * a.proj_ld + a.dt_off + h]) : 0.f;
    };
    if (pre) fetch(0);
    for (int c0 = 0; c0 < n_tok; c0 += SS_TOKENS) {
        const int nc = min(SS_TOKENS, n_tok - c0);
        __syncthreads();                                       // the group before has been walked
        if (pre) {
#pragma unroll
            for (int k = 0; k < SS_PRE; ++k) {
                if (code[k] != -1) {
                    Bs[tid + k * (int)blockDim.x] = pb[k];
                    if (MODE != 1) Cs[tid + k * (int)blockDim.x] = pc[k];
                }
            }
            if (tid < SS_TOKENS * PT) xs[tid] = px;
            if (tid < nc) {
                const float dt = ss_softplus(pdt + dtb);
                dts[tid] = dt;
                das[tid] = expf(-A * dt);
            }
        } else {
        for (int e = tid; e < nc * ROW; e += blockDim.x) {
            const int i = e / ROW, w = e % ROW, s = w / NRP, r = w % NRP, n = s * NR + r;
            const bool there = r < NR && n < N;
            const float* row = a.xbc + (size_t)(first + c0 + i) * a.xbc_ld;
            Bs[e] = there ? row[inner + g * N + n] : 0.f;
            if (MODE != 1) Cs[e] = there ? row[inner + a.G * N + g * N + n] : 0.f;
        }
        for (int e = tid; e < nc * PT; e += blockDim.x) {
            const int i = e / PT, q = e % PT;
            xs[i * PT + q] = p0 + q < P ? a.xbc[(size_t)(first + c0 + i) * a.xbc_ld + h * P + p0 + q] : 0.f;
        }
        if (tid < nc) {
            const float dt = ss_softplus(to_f(proj[(size_t)(first + c0 + tid) * a.proj_ld + a.dt_off + h]) + dtb);
            dts[tid] = dt;
            das[tid] = expf(-A * dt);
        }
        }
        if (pre && c0 + SS_TOKENS < n_tok) fetch(c0 + SS_TOKENS);          // the next group's numbers travel during this walk
        __syncthreads();
        for (int i = 0; i < nc; ++i) {
            const float x = xs[i * PT + (on ? pl : 0)];
            const float da = das[i], dtx = dts[i] * x;
            const float4* B4 = reinterpret_cast<const float4*>(Bs + i * ROW + ns * NRP);
            const float4* C4 = reinterpret_cast<const float4*>(Cs + i * ROW + ns * NRP);
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int r = 0; r < NRMAX; r += 4) {
                if (r < NR) {                                  // rows NR .. of the last four meet zeros of B and C and stay zero
                    const float4 bv = B4[r / 4];
                    S[r + 0] = fmaf(da, S[r + 0], dtx * bv.x); S[r + 1] = fmaf(da, S[r + 1], dtx * bv.y);
                    S[r + 2] = fmaf(da, S[r + 2], dtx * bv.z); S[r + 3] = fmaf(da, S[r + 3], dtx * bv.w);
                    if (MODE != 1) {
                        const float4 cv = C4[r / 4];
                        acc0 = fmaf(S[r + 0], cv.x, acc0); acc1 = fmaf(S[r + 1], cv.y, acc1);
                        acc0 = fmaf(S[r + 2], cv.z, acc0); acc1 = fmaf(S[r + 3], cv.w, acc1);
                    }
                }
            }
            if (MODE == 1) decay *= da;
            else {
                float acc = acc0 + acc1;
                for (int o = 1; o < NS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (on && ns == 0) a.y[(size_t)(first + c0 + i) * inner + h * P + p] = fmaf(Dh, x, acc);
            }
        }
    }
    if (MODE != 2 && on) {
#pragma unroll
        for (int r = 0; r < NRMAX; ++r)
            if (r < NR) st[((size_t)r * P + p) * NS + ns] = S[r];
    }
    if (MODE == 1 && blockIdx.z == 0 && tid == 0) a.chunk_decay[(size_t)blockIdx.x * a.H + h] = decay;
}

// The carry pass: a thread an element of a sequence's state walks the sequence's chunks in order, leaves every chunk its incoming
// state where its own contribution was, and stores the sequence's new state.
__global__ void __launch_bounds__(256) scan_carry_kernel(ScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const size_t per_head = (size_t)a.NR * a.P * a.NS, per = per_head * a.H;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    int base = 0;
    for (int i = 0; i < b; ++i) base += (a.row_lens[i] + SS_CHUNK - 1) / SS_CHUNK;
    const int nc = (a.row_lens[b] + SS_CHUNK - 1) / SS_CHUNK;
    if (nc == 0) return;
    const int h = (int)(e / per_head);
    float* sp = a.state + (size_t)a.slots[b] * a.state_stride + e;
    float carry = *sp;
    for (int c0 = base; c0 < base + nc; c0 += 8) {           // eight chunks' numbers in flight: they do not depend on the carry
        float own[8], dec[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const bool there = c0 + u < base + nc;
            own[u] = there ? a.chunk_state[(size_t)(c0 + u) * per + e] : 0.f;
            dec[u] = there ? a.chunk_decay[(size_t)(c0 + u) * a.H + h] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (c0 + u < base + nc) {
                a.chunk_state[(size_t)(c0 + u) * per + e] = carry;
                carry = fmaf(dec[u], carry, own[u]);
            }
        }
    }
    *sp = carry;
}

template <typename T, int NRMAX>
static int scan_run(const ScanArgs& a, int chunked, int threads, size_t smem, cudaStream_t s) {
    const int tiles = (a.P + a.PT - 1) / a.PT;
    if (!chunked) {
        PE_TRY(pe_launch(scan_kernel<T, NRMAX, 0>, dim3(a.B, a.H, tiles), threads, smem, s, a));
        PE_LAUNCH_CHECK();
        return 0;
    }
    PE_TRY(pe_launch(scan_kernel<T, NRMAX, 1>, dim3(a.max_chunks, a.H, tiles), threads, smem, s, a));
    PE_LAUNCH_CHECK();
    const size_t per = (size_t)a.H * a.NR * a.P * a.NS;
    PE_TRY(pe_launch(scan_carry_kernel, dim3((unsigned)((per + 255) / 256), a.B), 256, 0, s, a));
    PE_LAUNCH_CHECK();
    PE_TRY(pe_launch(scan_kernel<T, NRMAX, 2>, dim3(a.max_chunks, a.H, tiles), threads, smem, s, a));
    PE_LAUNCH_CHECK();
    return 0;
}

extern "C" int pe_state_space_scan(const float* xbc, int xbc_ld, const void* proj, int dtype, int proj_ld, int dt_off, const void* dt_bias,
                                   int dtb_dtype, const void* a_log, int al_dtype, const void* d_skip, int d_dtype, float* state,
                                   long long state_stride, const int* row_first, const int* row_lens, const int* slots, float* y,
                                   int T, int B, int H, int P, int N, int G, int chunked, float* scratch, void* stream) {
    if (B <= 0 || T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || P <= 0 || N <= 0 || N > 512) return PE_ERR_UNSUPPORTED;
    if (chunked && !scratch) return PE_ERR_UNSUPPORTED;
    const int NS = pe_state_space_split(N), NR = (N + NS - 1) / NS, NRP = (NR + 3) / 4 * 4 + 4;
    int PT = 256 / NS;
    if (PT > P) PT = P;
    int threads = ((PT * NS + 31) / 32) * 32;
    ScanArgs a = {xbc, xbc_ld, proj, proj_ld, dt_off, dt_bias, dtb_dtype, a_log, al_dtype, d_skip, d_dtype, state, state_stride,
                  row_first, row_lens, slots, y, B, H, P, N, G, NS, NR, NRP, PT, nullptr, nullptr, 0};
    a.max_chunks = pe_state_space_chunks(T, B);
    a.chunk_state = scratch;
    a.chunk_decay = scratch ? scratch + (size_t)a.max_chunks * pe_state_space_elems(H, P, N) : nullptr;
    const size_t smem = sizeof(float) * ((size_t)SS_TOKENS * (2 * NS * NRP + PT) + 2 * SS_TOKENS);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32) return NR <= 8 ? scan_run<float, 8>(a, chunked, threads, smem, s) : scan_run<float, 16>(a, chunked, threads, smem, s);
    if (dtype == PE_BF16) return NR <= 8 ? scan_run<bf16, 8>(a, chunked, threads, smem, s) : scan_run<bf16, 16>(a, chunked, threads, smem, s);
    return PE_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- gate, then a norm over groups of channels
// y [T, C] float32, the gate z at columns z_off .. of proj [T, ld] (the step's dtype): u = y * silu(z); every run of `group`
// channels of u is divided by sqrt(mean(run^2) + eps) and multiplied by weight[channel]; out [T, C] in the step's dtype.
// A block a (token, run).
template <typename T>
__global__ void __launch_bounds__(256) gate_norm_kernel(const float* y, int C, int group, const T* proj, int ld, int z_off, const void* weight,
                                                        int w_dtype, float eps, T* out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x, c0 = blockIdx.y * group;
    float ss = 0.f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const float u = y[(size_t)t * C + c0 + i] * ss_silu(to_f(proj[(size_t)t * ld + z_off + c0 + i]));
        ss = fmaf(u, u, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)group + eps);
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const float u = y[(size_t)t * C + c0 + i] * ss_silu(to_f(proj[(size_t)t * ld + z_off + c0 + i]));
        out[(size_t)t * C + c0 + i] = from_f<T>(u * rstd * load_as_f(weight, w_dtype, c0 + i));
    }
}

extern "C" int pe_gate_norm(const float* y, int T, int C, int group, const void* proj, int dtype, int ld, int z_off, const void* weight,
                            int w_dtype, float eps, void* out, void* stream) {
    if (T <= 0) return 0;
    if (group <= 0 || C % group || z_off < 0 || z_off + C > ld) return PE_ERR_UNSUPPORTED;
    const int threads = group >= 256 ? 256 : ((group + 31) / 32) * 32;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32) PE_TRY(pe_launch(gate_norm_kernel<float>, dim3(T, C / group), threads, 0, s, y, C, group, (const float*)proj, ld, z_off, weight, w_dtype, eps, (float*)out));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(gate_norm_kernel<bf16>, dim3(T, C / group), threads, 0, s, y, C, group, (const bf16*)proj, ld, z_off, weight, w_dtype, eps, (bf16*)out));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}
