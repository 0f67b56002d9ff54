// What stands between a fused q,k projection and attention for mixers that normalise q and k over
// the whole projection (all heads at once) and have no value projection: the value of a token is
// its key projection as projected, before the norm.
//
// Per token, in 32-bit:
//   q' = q + b_q, k' = k + b_k                       (rounded to the activation type: this is the projection)
//   V page <- k'
//   q  <- q' / sqrt(mean(q'^2) + eps) * w_q * temp(p)     over all Hq * Dh values of the token
//   K page <- k' / sqrt(mean(k'^2) + eps) * w_k           over all Hkv * Dh values
// temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1): the query grows with the logarithm of the
// position, in steps of `every` tokens (every <= 0: no such factor).
#include "common.cuh"

constexpr int PN_BLOCK = 256;

template <typename TA>
__global__ void __launch_bounds__(PN_BLOCK) proj_norm_kv_kernel(
    TA* __restrict__ qk, int64_t row_stride, int n_q, int n_k, const float* __restrict__ b_q, const float* __restrict__ b_k,
    const float* __restrict__ w_q, const float* __restrict__ w_k, float eps, float temp_coef, int temp_every,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int bt_stride,
    int n_seqs, TA* __restrict__ k_cache, TA* __restrict__ v_cache, int Hkv, int Dh, int page_size, int num_pages, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    TA* q = qk + (int64_t)t * row_stride;
    TA* k = q + n_q;
    const int pos = positions[t];
    const int seq = seq_of_token[t];

    // ---- q: bias, statistics, norm and temperature in place
    float ss = 0.f;
    for (int c = tid; c < n_q; c += PN_BLOCK) {
        const TA x = from_float<TA>(to_float(q[c]) + (b_q ? b_q[c] : 0.f));
        q[c] = x;
        const float xf = to_float(x);
        ss = fmaf(xf, xf, ss);
    }
    ss = block_sum(ss, scratch);
    float r = rsqrtf(ss / (float)n_q + eps);
    if (temp_every > 0) r *= 1.f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
    for (int c = tid; c < n_q; c += PN_BLOCK) q[c] = from_float<TA>(to_float(q[c]) * r * w_q[c]);

    // ---- k: bias, the raw row is the value, the normalised row the key
    int64_t base = -1;
    if (k_cache) {
        if (seq < 0 || seq >= n_seqs) {
            if (tid == 0) imp_report(status, IMP_BAD_SEQUENCE);
        } else if (pos < 0 || pos / page_size >= bt_stride) {
            if (tid == 0) imp_report(status, IMP_BAD_POSITION);
        } else {
            const int page = block_table[(int64_t)seq * bt_stride + pos / page_size];
            if (page < 0 || page >= num_pages) {
                if (tid == 0) imp_report(status, IMP_BAD_PAGE);
            } else {
                base = ((int64_t)page * Hkv * page_size + pos % page_size) * Dh;
            }
        }
    }
    ss = 0.f;
    for (int c = tid; c < n_k; c += PN_BLOCK) {
        const TA x = from_float<TA>(to_float(k[c]) + (b_k ? b_k[c] : 0.f));
        k[c] = x;
        const float xf = to_float(x);
        ss = fmaf(xf, xf, ss);
        if (base >= 0) v_cache[base + (int64_t)(c / Dh) * page_size * Dh + c % Dh] = x;
    }
    ss = block_sum(ss, scratch);
    r = rsqrtf(ss / (float)n_k + eps);
    for (int c = tid; c < n_k; c += PN_BLOCK) {
        const TA x = from_float<TA>(to_float(k[c]) * r * w_k[c]);
        k[c] = x;
        if (base >= 0) k_cache[base + (int64_t)(c / Dh) * page_size * Dh + c % Dh] = x;
    }
}

// qk: [n_tokens, row_stride], q in columns [0, Hq * Dh), k in [Hq * Dh, (Hq + Hkv) * Dh); rewritten in place.
// b_q, b_k (null = none), w_q, w_k: float32.  k_cache, v_cache: [num_pages, Hkv, page_size, Dh] of one layer
// (null: no cache write).
IMP_API int imp_proj_norm_kv_write(void* qk, int64_t row_stride, int n_tokens, int Hq, int Hkv, int Dh, const float* b_q,
                                   const float* b_k, const float* w_q, const float* w_k, float eps, float temp_coef,
                                   int temp_every, const int* positions, const int* seq_of_token, const int* block_table,
                                   int bt_stride, int n_seqs, void* k_cache, void* v_cache, int page_size, int num_pages,
                                   int act_dtype, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(qk && w_q && w_k && positions && seq_of_token, "imp_proj_norm_kv_write: null pointer");
    IMP_CHECK_ARG(Hq > 0 && Hkv > 0 && Dh > 0 && row_stride >= (int64_t)(Hq + Hkv) * Dh, "imp_proj_norm_kv_write: bad sizes");
    IMP_CHECK_ARG(!k_cache || (v_cache && block_table && page_size > 0 && num_pages > 0), "imp_proj_norm_kv_write: bad cache geometry");
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == IMP_F32)
        imp_launch(proj_norm_kv_kernel<float>, dim3(n_tokens), dim3(PN_BLOCK), 0, s, (float*)qk, row_stride, Hq * Dh, Hkv * Dh, b_q,
                   b_k, w_q, w_k, eps, temp_coef, temp_every, positions, seq_of_token, block_table, bt_stride, n_seqs,
                   (float*)k_cache, (float*)v_cache, Hkv, Dh, page_size, num_pages, status);
    else
        imp_launch(proj_norm_kv_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(PN_BLOCK), 0, s, (__nv_bfloat16*)qk, row_stride,
                   Hq * Dh, Hkv * Dh, b_q, b_k, w_q, w_k, eps, temp_coef, temp_every, positions, seq_of_token, block_table,
                   bt_stride, n_seqs, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hkv, Dh, page_size, num_pages, status);
    IMP_RETURN_LAUNCH();
}

// ------------------------------------------------------------------------------------ small helpers
// out = (x + bias) (bias per column, float32), in place allowed; and out = a * x + b * y.
template <typename TA>
__global__ void add_bias_kernel(TA* __restrict__ x, int64_t stride, int n_rows, int n_cols, const float* __restrict__ bias) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t total = (int64_t)n_rows * n_cols;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n_cols;
        const int c = (int)(i - r * n_cols);
        x[r * stride + c] = from_float<TA>(to_float(x[r * stride + c]) + bias[c]);
    }
}

IMP_API int imp_add_bias(void* x, int64_t stride, int n_rows, int n_cols, const float* bias, int dtype, void* stream) {
    if (n_rows == 0 || n_cols == 0) return 0;
    IMP_CHECK_ARG(x && bias, "imp_add_bias: null pointer");
    const int64_t total = (int64_t)n_rows * n_cols;
    const int64_t cap = (int64_t)imp_sm_count() * 16;
    const int grid = (int)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IMP_F32) imp_launch(add_bias_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)x, stride, n_rows, n_cols, bias);
    else imp_launch(add_bias_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (__nv_bfloat16*)x, stride, n_rows, n_cols, bias);
    IMP_RETURN_LAUNCH();
}

template <typename TA>
__global__ void scaled_sum_kernel(TA* out, const TA* x, float a, const TA* y, float b,
                                  const float* __restrict__ col_bias, float bias_scale, int n_cols, int64_t n) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = a * to_float(x[i]);
        if (col_bias) v = fmaf(bias_scale, col_bias[i % n_cols], v);
        if (y) v = fmaf(b, to_float(y[i]), v);
        out[i] = from_float<TA>(v);
    }
}

// out = a * x + b * y (+ bias_scale * col_bias per column), dense [n_rows, n_cols]; y and col_bias may be null;
// out may be x or y.
IMP_API int imp_scaled_sum(void* out, const void* x, float a, const void* y, float b, const float* col_bias, float bias_scale,
                           int n_rows, int n_cols, int dtype, void* stream) {
    const int64_t n = (int64_t)n_rows * n_cols;
    if (n == 0) return 0;
    IMP_CHECK_ARG(out && x, "imp_scaled_sum: null pointer");
    const int64_t cap = (int64_t)imp_sm_count() * 16;
    const int grid = (int)((n + 255) / 256 < cap ? (n + 255) / 256 : cap);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IMP_F32)
        imp_launch(scaled_sum_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)out, (const float*)x, a, (const float*)y, b, col_bias,
                   bias_scale, n_cols, n);
    else
        imp_launch(scaled_sum_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, a,
                   (const __nv_bfloat16*)y, b, col_bias, bias_scale, n_cols, n);
    IMP_RETURN_LAUNCH();
}
