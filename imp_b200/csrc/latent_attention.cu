// The small kernels of latent attention: what happens between its matrix products.
//
// A token's down-projection holds [ query latent (q_rank) | key/value latent (kv_rank) | rotated key part (rot) ].
// latent_prepare: RMS norm (plain weight, eps inside the root) of the two latents, rotation of the key part at the
// token's position, and the cache write: a page holds one vector [kv_rank + rot] per token, the normalised latent
// followed by the rotated key part.  latent_query_rope: the rotated part of every head's query, moved behind that
// head's latent-space query.  Norms, angles and rotations are 32-bit; the rotation pairs entry i with i + dims/2.
#include "common.cuh"

namespace {

constexpr int LP_BLOCK = 128;

template <typename TA>
__global__ void __launch_bounds__(LP_BLOCK) latent_prepare_kernel(
    const TA* __restrict__ proj, int64_t ld, int q_rank, int kv_rank, int rot, const float* __restrict__ wq, const float* __restrict__ wkv,
    float eps, TA* __restrict__ cq, int64_t cq_ld, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rot_dims,
    int max_pos, const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
    int bt_stride, int n_seqs, TA* __restrict__ pages, int page_size, int num_pages, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const TA* row = proj + (int64_t)t * ld;
    // the query latent
    float ss = 0.f;
    for (int i = tid; i < q_rank; i += LP_BLOCK) {
        const float v = to_float(row[i]);
        ss = fmaf(v, v, ss);
    }
    float inv = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int i = tid; i < q_rank; i += LP_BLOCK) cq[(int64_t)t * cq_ld + i] = from_float<TA>(to_float(row[i]) * inv * wq[i]);
    // the key/value latent and the rotated key part go to the token's place in the pages
    const int seq = seq_of_token[t], pos = positions[t];
    if (!pages) return;
    if (seq < 0 || seq >= n_seqs || pos < 0 || pos >= max_pos || pos / page_size >= bt_stride) {
        if (tid == 0) imp_report(status, seq < 0 || seq >= n_seqs ? IMP_BAD_SEQUENCE : IMP_BAD_POSITION);
        return;
    }
    const int page = block_table[(int64_t)seq * bt_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (tid == 0) imp_report(status, IMP_BAD_PAGE);
        return;
    }
    TA* dst = pages + ((int64_t)page * page_size + pos % page_size) * (kv_rank + rot);
    const TA* lat = row + q_rank;
    ss = 0.f;
    for (int i = tid; i < kv_rank; i += LP_BLOCK) {
        const float v = to_float(lat[i]);
        ss = fmaf(v, v, ss);
    }
    inv = rsqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
    for (int i = tid; i < kv_rank; i += LP_BLOCK) dst[i] = from_float<TA>(to_float(lat[i]) * inv * wkv[i]);
    const TA* kr = lat + kv_rank;
    const int half = rot_dims / 2;
    for (int i = tid; i < rot; i += LP_BLOCK) {
        float v = to_float(kr[i]);
        if (i < rot_dims) {
            const int f = i < half ? i : i - half;
            const float c = cos_tab[(int64_t)pos * half + f], s = sin_tab[(int64_t)pos * half + f];
            const float other = to_float(kr[i < half ? i + half : i - half]);
            v = i < half ? v * c - other * s : v * c + other * s;
        }
        dst[kv_rank + i] = from_float<TA>(v);
    }
}

// q [T, H, D + rot] -> out[t, h, kv_rank + i] = rotated q[t, h, D + i]
template <typename TA>
__global__ void latent_query_rope_kernel(const TA* __restrict__ q, int64_t q_ld, int H, int D, int rot, TA* __restrict__ out, int64_t out_ld,
                                         int kv_rank, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rot_dims,
                                         int max_pos, const int* __restrict__ positions, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) imp_report(status, IMP_BAD_POSITION);
        return;
    }
    const int half = rot_dims / 2;
    for (int e = threadIdx.x; e < H * rot; e += blockDim.x) {
        const int h = e / rot, i = e % rot;
        const TA* src = q + (int64_t)t * q_ld + (int64_t)h * (D + rot) + D;
        float v = to_float(src[i]);
        if (i < rot_dims) {
            const int f = i < half ? i : i - half;
            const float c = cos_tab[(int64_t)pos * half + f], s = sin_tab[(int64_t)pos * half + f];
            const float other = to_float(src[i < half ? i + half : i - half]);
            v = i < half ? v * c - other * s : v * c + other * s;
        }
        out[(int64_t)t * out_ld + (int64_t)h * (kv_rank + rot) + kv_rank + i] = from_float<TA>(v);
    }
}

}  // namespace

IMP_API int imp_latent_prepare(const void* proj, int64_t ld, int n_tokens, int q_rank, int kv_rank, int rot, const float* wq,
                               const float* wkv, float eps, void* cq, int64_t cq_ld, const float* cos_tab, const float* sin_tab,
                               int rot_dims, int max_pos, const int* positions, const int* seq_of_token, const int* block_table,
                               int bt_stride, int n_seqs, void* pages, int page_size, int num_pages, int act_dtype, int* status,
                               void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(proj && wq && wkv && cq && cos_tab && sin_tab && positions && seq_of_token, "imp_latent_prepare: null pointer");
    IMP_CHECK_ARG(q_rank > 0 && kv_rank > 0 && rot >= 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0,
                  "imp_latent_prepare: bad sizes (the rotated entries must be even in number and within the rotated part)");
    IMP_CHECK_ARG(!pages || (block_table && page_size > 0 && num_pages > 0), "imp_latent_prepare: bad cache geometry");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (act_dtype == IMP_F32)
        e = imp_launch(latent_prepare_kernel<float>, dim3(n_tokens), dim3(LP_BLOCK), 0, s, (const float*)proj, ld, q_rank, kv_rank, rot, wq,
                       wkv, eps, (float*)cq, cq_ld, cos_tab, sin_tab, rot_dims, max_pos, positions, seq_of_token, block_table, bt_stride,
                       n_seqs, (float*)pages, page_size, num_pages, status);
    else
        e = imp_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(LP_BLOCK), 0, s, (const __nv_bfloat16*)proj, ld, q_rank,
                       kv_rank, rot, wq, wkv, eps, (__nv_bfloat16*)cq, cq_ld, cos_tab, sin_tab, rot_dims, max_pos, positions, seq_of_token,
                       block_table, bt_stride, n_seqs, (__nv_bfloat16*)pages, page_size, num_pages, status);
    if (e != cudaSuccess) {
        imp_set_error("imp_latent_prepare: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

IMP_API int imp_latent_query_rope(const void* q, int64_t q_ld, int n_tokens, int H, int D, int rot, void* out, int64_t out_ld, int kv_rank,
                                  const float* cos_tab, const float* sin_tab, int rot_dims, int max_pos, const int* positions,
                                  int act_dtype, int* status, void* stream) {
    if (n_tokens == 0 || rot == 0) return 0;
    IMP_CHECK_ARG(q && out && cos_tab && sin_tab && positions && H > 0 && D >= 0 && rot > 0 && rot_dims <= rot && rot_dims % 2 == 0,
                  "imp_latent_query_rope: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (act_dtype == IMP_F32)
        e = imp_launch(latent_query_rope_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float*)q, q_ld, H, D, rot, (float*)out, out_ld,
                       kv_rank, cos_tab, sin_tab, rot_dims, max_pos, positions, status);
    else
        e = imp_launch(latent_query_rope_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, s, (const __nv_bfloat16*)q, q_ld, H, D, rot,
                       (__nv_bfloat16*)out, out_ld, kv_rank, cos_tab, sin_tab, rot_dims, max_pos, positions, status);
    if (e != cudaSuccess) {
        imp_set_error("imp_latent_query_rope: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
