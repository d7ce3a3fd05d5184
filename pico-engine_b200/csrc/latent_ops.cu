// Small kernels around attention over one low-rank row per position.
//
// A position keeps the row [c | k_rot]: c = rmsnorm(first `rank` entries of W_dkv h) * w (the latent), k_rot = the other R
// entries, turned by the position's angles (one rotated key part for all heads).  A head's plain key is W_uk,h c, so
// q_plain . k_plain = (W_uk,h^T q_plain) . c: with the queries carried into the latent space, attention reads the kept rows as
// they are, as one key/value head of size rank + R whose first `rank` entries are also the value; W_uv,h acts on the result.
//
// The rotation has two layouts: neighbours (2i, 2i+1), or (`halves`) entry i with entry i + rot_dims / 2.
// latent_prepare: a block a token.  Norms and stores c, turns and stores k_rot (into the cache page of the token), and builds the
// token's queries [H][rank + R] from the absorbed plain parts qa [H, T, rank] (null: they are in q_out already) and the turned rotated parts of q.
// head_gate: out[t, h, :] = o[h, t, :] * sigmoid(gate logit of head h) (o comes head-major out of a batched product).
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const T* proj, int ld, int H, int D, int R, int rank, int dkv_off,
                                                             const void* norm_w, int nw_dtype, float eps, const float* freq, int rot_dims,
                                                             const T* qa, int n_tokens, T* q_out, const int* tok_pos, const int* tok_row,
                                                             T* k_pool, const int* table, int table_stride, int store, int halves, const T* q_rows, int q_ld) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = tok_pos[t];
    const T* row = proj + (size_t)t * ld;
    const T* qrow = q_rows ? q_rows + (size_t)t * q_ld : row;      // the queries may lie in rows of their own
    const int W = rank + R;
    T* dst = nullptr;
    if (store) {
        const int page = table[(size_t)tok_row[t] * table_stride + pos / PE_PAGE];
        if (page >= 0) dst = k_pool + ((size_t)page * PE_PAGE + pos % PE_PAGE) * W;
    }
    // the latent row
    float ss = 0.f;
    for (int i = tid; i < rank; i += blockDim.x) { const float f = to_f(row[dkv_off + i]); ss = fmaf(f, f, ss); }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)rank + eps);
    if (dst) for (int i = tid; i < rank; i += blockDim.x) dst[i] = from_f<T>(to_f(row[dkv_off + i]) * rstd * load_as_f(norm_w, nw_dtype, i));
    // pairs: unit u < R / 2 of the key part, then of every head's rotated query part; entries beyond rot_dims pass unchanged
    const int half = R / 2;
    for (int u = tid; u < (H + 1) * half; u += blockDim.x) {
        const int who = u / half, i = u % half;                  // who 0: the key part; who - 1: the query head
        const T* src = who == 0 ? row + dkv_off + rank : qrow + (size_t)(who - 1) * (D + R) + D;
        T* o = who == 0 ? (dst ? dst + rank : nullptr) : q_out + ((size_t)t * H + (who - 1)) * W + rank;
        if (halves) {
            // the other layout: entry i < rot_dims / 2 pairs with entry i + rot_dims / 2; unit i of the R / 2 takes care of one such
            // pair, or, beyond the rotated entries, of the two entries rot_dims + 2 (i - rot_dims / 2) and the next, which stay
            const int rh = rot_dims / 2;
            const int e0 = i < rh ? i : rot_dims + 2 * (i - rh), e1 = i < rh ? i + rh : e0 + 1;
            float a0 = to_f(src[e0]), a1 = to_f(src[e1]);
            if (i < rh) {
                float sn, cs;
                sincosf((float)pos * freq[i], &sn, &cs);
                const float b0 = a0 * cs - a1 * sn, b1 = a1 * cs + a0 * sn;
                a0 = b0; a1 = b1;
            }
            if (o) { o[e0] = from_f<T>(a0); o[e1] = from_f<T>(a1); }
            continue;
        }
        float a0 = to_f(src[2 * i]), a1 = to_f(src[2 * i + 1]);
        if (2 * i + 1 < rot_dims) {
            float sn, cs;
            sincosf((float)pos * freq[i], &sn, &cs);
            const float b0 = a0 * cs - a1 * sn, b1 = a1 * cs + a0 * sn;
            a0 = b0; a1 = b1;
        }
        if (o) { o[2 * i] = from_f<T>(a0); o[2 * i + 1] = from_f<T>(a1); }
    }
    if (R & 1) {                                                 // an odd last entry is never part of a pair
        for (int who = tid; who <= H; who += blockDim.x) {
            const T* src = who == 0 ? row + dkv_off + rank : qrow + (size_t)(who - 1) * (D + R) + D;
            T* o = who == 0 ? (dst ? dst + rank : nullptr) : q_out + ((size_t)t * H + (who - 1)) * W + rank;
            if (o) o[R - 1] = src[R - 1];
        }
    }
    if (!qa) return;                                             // the batched product wrote the carried parts into q_out itself
    for (int e = tid; e < H * rank; e += blockDim.x) {
        const int h = e / rank, i = e % rank;
        q_out[((size_t)t * H + h) * W + i] = qa[((size_t)h * n_tokens + t) * rank + i];
    }
}

extern "C" int pe_latent_prepare(const void* proj, int dtype, int ld, int T, int H, int D, int R, int rank, int dkv_off, const void* norm_w,
                                 int nw_dtype, float eps, const float* freq, int rot_dims, const void* qa, void* q_out, const int* tok_pos,
                                 const int* tok_row, void* k_pool, const int* table, int table_stride, int store, int halves, const void* q_rows, int q_ld,
                                 void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || D <= 0 || R < 0 || rank <= 0 || rot_dims < 0 || rot_dims > R || rot_dims % 2 || dkv_off + rank + R > ld || (q_rows && q_ld < H * (D + R))) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32) PE_TRY(pe_launch(latent_prepare_kernel<float>, T, 256, 0, s, (const float*)proj, ld, H, D, R, rank, dkv_off, norm_w, nw_dtype, eps, freq, rot_dims, (const float*)qa, T, (float*)q_out, tok_pos, tok_row, (float*)k_pool, table, table_stride, store, halves, (const float*)q_rows, q_ld));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(latent_prepare_kernel<bf16>, T, 256, 0, s, (const bf16*)proj, ld, H, D, R, rank, dkv_off, norm_w, nw_dtype, eps, freq, rot_dims, (const bf16*)qa, T, (bf16*)q_out, tok_pos, tok_row, (bf16*)k_pool, table, table_stride, store, halves, (const bf16*)q_rows, q_ld));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

template <typename T>
__global__ void head_gate_kernel(const T* o, const T* proj, int ld, int g_off, int n_tokens, int H, int Dv, T* out, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const int d = (int)(e % Dv), h = (int)((e / Dv) % H);
    const size_t t = e / ((size_t)Dv * H);
    float f = to_f(o[((size_t)h * n_tokens + t) * Dv + d]);
    if (proj) f *= 1.0f / (1.0f + expf(-to_f(proj[t * ld + g_off + h])));
    out[e] = from_f<T>(f);
}

extern "C" int pe_head_gate(const void* o, int dtype, const void* proj, int ld, int g_off, int T, int H, int Dv, void* out, void* stream) {
    if (T <= 0) return 0;
    const size_t total = (size_t)T * H * Dv;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32) PE_TRY(pe_launch(head_gate_kernel<float>, blocks, 256, 0, s, (const float*)o, (const float*)proj, ld, g_off, T, H, Dv, (float*)out, total));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(head_gate_kernel<bf16>, blocks, 256, 0, s, (const bf16*)o, (const bf16*)proj, ld, g_off, T, H, Dv, (bf16*)out, total));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}

// out[t, :C] = rmsnorm(rows[t, off : off + C]) * w: the RMS norm of a run of columns of a product's rows (a low-rank row that the
// next product reads), in float32, stored in the rows' dtype.  A block a token.
template <typename T>
__global__ void __launch_bounds__(128) rmsnorm_cols_kernel(const T* rows, int ld, int off, int C, const void* w, int w_dtype, float eps, T* out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const T* row = rows + (size_t)blockIdx.x * ld + off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) { const float f = to_f(row[i]); ss = fmaf(f, f, ss); }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);
    T* o = out + (size_t)blockIdx.x * C;
    for (int i = threadIdx.x; i < C; i += blockDim.x) o[i] = from_f<T>(to_f(row[i]) * rstd * load_as_f(w, w_dtype, i));
}

extern "C" int pe_rmsnorm_cols(const void* rows, int dtype, int ld, int off, int C, const void* w, int w_dtype, float eps, void* out, int T,
                               void* stream) {
    if (T <= 0) return 0;
    if (C <= 0 || off < 0 || off + C > ld) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == PE_F32) PE_TRY(pe_launch(rmsnorm_cols_kernel<float>, T, 128, 0, s, (const float*)rows, ld, off, C, w, w_dtype, eps, (float*)out));
    else if (dtype == PE_BF16) PE_TRY(pe_launch(rmsnorm_cols_kernel<bf16>, T, 128, 0, s, (const bf16*)rows, ld, off, C, w, w_dtype, eps, (bf16*)out));
    else return PE_ERR_UNSUPPORTED;
    PE_LAUNCH_CHECK();
    return 0;
}
