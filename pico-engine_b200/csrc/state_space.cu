// A selective state-space mixer with a scalar decay a head and token: the short causal convolution with silu on its inputs,
// the recurrence, and the gate followed by a norm over groups of channels.  Decays, step sizes, the state, its outputs, the
// gate and the norm are float32 in either engine dtype; only the loads of projections and the store of the result convert.
//
//   dt_t = softplus(dt_raw_t + dt_bias_h)        a_t = exp(-exp(A_log_h) * dt_t)
//   S_t = a_t S_(t-1) + dt_t B_t x_t^T           (S [N, P] a head, B and C shared by the heads of a group)
//   y_t = S_t^T C_t + D_h x_t
//
// The recurrence runs token after token: a block owns (sequence, head, a tile of the P columns); thread (p, ns) keeps rows
// n = ns + NS r (r < NR) of column p in registers, the NS threads of a column are neighbours in a warp and add their parts
// of y by shuffles.  A sequence's state lies in its row of the cache's state area in exactly the order the threads hold it,
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
struct ScanArgs {
    const float* xbc; int xbc_ld;             // [T, inner + 2 G N] float32: x | B | C after the convolution
    const void* proj; int proj_ld, dt_off;    // dt_raw at columns dt_off .. dt_off + H - 1 of proj (the step's dtype)
    const void* dt_bias; int dtb_dtype; const void* a_log; int al_dtype; const void* d_skip; int d_dtype;   // [H] each
    float* state; long long state_stride;     // row slots[b] holds the sequence's state
    const int* row_first; const int* row_lens; const int* slots;
    float* y;                                 // [T, H * P]
    int H, P, N, G, NS, NR, PT;
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

template <typename T, int NRMAX>
__global__ void __launch_bounds__(256) scan_kernel(ScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float ss_smem[];
    const int b = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * a.PT;
    const int N = a.N, P = a.P, NS = a.NS, NR = a.NR, PT = a.PT;
    const int tid = threadIdx.x, ns = tid % NS, pl = tid / NS, p = p0 + pl;
    const bool on = pl < PT && p < P;
    const int g = h / (a.H / a.G), inner = a.H * P;
    float* Bs = ss_smem;                      // [SS_TOKENS][N]
    float* Cs = Bs + SS_TOKENS * N;           // [SS_TOKENS][N]
    float* xs = Cs + SS_TOKENS * N;           // [SS_TOKENS][PT]
    float* dts = xs + SS_TOKENS * PT;         // [SS_TOKENS]: step sizes
    float* das = dts + SS_TOKENS;             // [SS_TOKENS]: decays
    const int n_tok = a.row_lens[b], first = a.row_first[b];
    float* st = a.state + (size_t)a.slots[b] * a.state_stride + (size_t)h * NR * P * NS;
    float S[NRMAX];
#pragma unroll
    for (int r = 0; r < NRMAX; ++r) S[r] = (on && r < NR) ? st[((size_t)r * P + p) * NS + ns] : 0.f;
    const float A = expf(load_as_f(a.a_log, a.al_dtype, h)), Dh = load_as_f(a.d_skip, a.d_dtype, h), dtb = load_as_f(a.dt_bias, a.dtb_dtype, h);
    const T* proj = (const T*)a.proj;
    for (int c0 = 0; c0 < n_tok; c0 += SS_TOKENS) {
        const int nc = min(SS_TOKENS, n_tok - c0);
        __syncthreads();                                       // the chunk before has been walked
        for (int e = tid; e < nc * N; e += blockDim.x) {
            const int i = e / N, n = e % N;
            const float* row = a.xbc + (size_t)(first + c0 + i) * a.xbc_ld;
            Bs[i * N + n] = row[inner + g * N + n];
            Cs[i * N + n] = row[inner + a.G * N + g * N + n];
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
        __syncthreads();
        for (int i = 0; i < nc; ++i) {
            const float x = xs[i * PT + (on ? pl : 0)];
            const float da = das[i], dtx = dts[i] * x;
            const float* Bi = Bs + i * N;
            const float* Ci = Cs + i * N;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < NRMAX; ++r) {
                const int n = ns + NS * r;
                if (r < NR && n < N) {
                    S[r] = fmaf(da, S[r], dtx * Bi[n]);
                    acc = fmaf(S[r], Ci[n], acc);
                }
            }
            for (int o = 1; o < NS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (on && ns == 0) a.y[(size_t)(first + c0 + i) * inner + h * P + p] = fmaf(Dh, x, acc);
        }
    }
    if (on) {
#pragma unroll
        for (int r = 0; r < NRMAX; ++r)
            if (r < NR) st[((size_t)r * P + p) * NS + ns] = S[r];
    }
}

extern "C" int pe_state_space_scan(const float* xbc, int xbc_ld, const void* proj, int dtype, int proj_ld, int dt_off, const void* dt_bias,
                                   int dtb_dtype, const void* a_log, int al_dtype, const void* d_skip, int d_dtype, float* state,
                                   long long state_stride, const int* row_first, const int* row_lens, const int* slots, float* y,
                                   int B, int H, int P, int N, int G, void* stream) {
    if (B <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || P <= 0 || N <= 0 || N > 512) return PE_ERR_UNSUPPORTED;
    const int NS = pe_state_space_split(N), NR = (N + NS - 1) / NS;
    int PT = 256 / NS;
    if (PT > P) PT = P;
    int threads = ((PT * NS + 31) / 32) * 32;
    ScanArgs a = {xbc, xbc_ld, proj, proj_ld, dt_off, dt_bias, dtb_dtype, a_log, al_dtype, d_skip, d_dtype, state, state_stride,
                  row_first, row_lens, slots, y, H, P, N, G, NS, NR, PT};
    const size_t smem = sizeof(float) * ((size_t)SS_TOKENS * (2 * N + PT) + 2 * SS_TOKENS);
    const dim3 grid(B, H, (P + PT - 1) / PT);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32) {
        if (NR <= 8) PE_TRY(pe_launch(scan_kernel<float, 8>, grid, threads, smem, s, a));
        else PE_TRY(pe_launch(scan_kernel<float, 16>, grid, threads, smem, s, a));
    } else if (dtype == PE_BF16) {
        if (NR <= 8) PE_TRY(pe_launch(scan_kernel<bf16, 8>, grid, threads, smem, s, a));
        else PE_TRY(pe_launch(scan_kernel<bf16, 16>, grid, threads, smem, s, a));
    } else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
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
