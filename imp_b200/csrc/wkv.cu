// The wkv mixer's own kernels: a linear recurrence with a matrix state per head and inputs mixed with the
// previous token's.
//
//   mix_s[t] = x[t] + (x[t-1] - x[t]) * mu_s            s = r, k, v, g, w;  x[-1] is the state's `prev` (zero at a
//                                                        request's start)
//   w[t]     = exp(-exp(d[t] + w0))                      d: the decay's low-rank product, 32-bit
//   o[t]     = (S + diag(u) k[t] v[t]^T)^T r[t]          per head, S [D keys, D values] in 32-bit
//   S        = diag(w[t]) S + k[t] v[t]^T
//   y[t]     = o[t] / sqrt(mean(o[t]^2) + eps) * g_norm * gate[t]     per head
//
// Everything but the projections is 32-bit.  The scan gives 32 value columns of a (sequence, head) to one CTA; a column
// of S is spread over four lanes, each with a quarter of the key rows in registers, so a token costs D/4
// multiply-adds a lane for the read-out, as many for the update, and two shuffles.  Inputs come in chunks of
// 16 tokens through shared memory.  The order of every sum depends on D alone: a token's result is the same bits
// however the prompt is cut and whatever else is in the batch.
#include <algorithm>

#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------ token shift
// out: [5][T, d] of the activation type (r, k, v, g, w).  update_state (steps of single tokens): the token's row
// becomes the state's `prev` in the same pass; otherwise wkv_shift_state_kernel does that afterwards.
template <typename TA>
__global__ void wkv_mix_kernel(const TA* __restrict__ x, int64_t ldx, const float* __restrict__ mu /* [5, d] */, float* __restrict__ prev_state,
                               const int* __restrict__ seq_of_token, const int* __restrict__ q_start, const int* __restrict__ slots, int n_tokens,
                               int n_seqs, int d, TA* __restrict__ out, int update_state, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0 || seq >= n_seqs) {
        if (threadIdx.x == 0) imp_report(status, IMP_BAD_SEQUENCE);
        return;
    }
    const bool first = t == q_start[seq];
    float* prev = prev_state + (int64_t)slots[seq] * d;
    const TA* cur = x + (int64_t)t * ldx;
    const TA* before = first ? nullptr : x + (int64_t)(t - 1) * ldx;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float c = to_float(cur[i]);
        const float p = before ? to_float(before[i]) : prev[i];
        const float diff = p - c;
#pragma unroll
        for (int s = 0; s < 5; ++s) out[((int64_t)s * n_tokens + t) * d + i] = from_float<TA>(fmaf(diff, mu[s * d + i], c));
        if (update_state) prev[i] = c;
    }
}

template <typename TA>
__global__ void wkv_shift_state_kernel(const TA* __restrict__ x, int64_t ldx, float* __restrict__ prev_state, const int* __restrict__ q_start,
                                       const int* __restrict__ slots, int d) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x;
    const int end = q_start[seq + 1];
    if (end <= q_start[seq]) return;
    const TA* last = x + (int64_t)(end - 1) * ldx;
    float* prev = prev_state + (int64_t)slots[seq] * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) prev[i] = to_float(last[i]);
}

template <typename TA> __global__ void tanh_kernel(TA* __restrict__ x, int64_t n) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        x[i] = from_float<TA>(tanhf(to_float(x[i])));
}

// ------------------------------------------------------------------------------------------------- scan
// A CTA owns WKV_COLS value columns of one head's S for one sequence; a column is spread over four lanes, each with a
// contiguous quarter of the key rows in registers.  The token's r, w and k are read from shared memory four at a time.
constexpr int WKV_LANES = 4, WKV_COLS = 32;

template <typename TA, int RPT>
__global__ void __launch_bounds__(WKV_COLS* WKV_LANES) wkv_scan_kernel(const TA* __restrict__ r, const TA* __restrict__ k, const TA* __restrict__ v,
                                                                        int64_t ld, const float* __restrict__ dlog, const float* __restrict__ w0,
                                                                        const float* __restrict__ u, float* __restrict__ state,
                                                                        float* __restrict__ out, const int* __restrict__ q_start,
                                                                        const int* __restrict__ slots, int H, int D, int col_blocks) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int DP = RPT * WKV_LANES;   // D rounded up to the rows the four lanes hold (RPT a multiple of 4)
    constexpr int WKV_CHUNK = RPT > 32 ? 8 : 16;   // three arrays of WKV_CHUNK x DP floats stay under 48 KB
    // row i lives at i + 4 * (i / RPT): the four lanes of a column read 16 bytes each from four different groups of banks
    constexpr int DPP = DP + 4 * WKV_LANES;
    __shared__ __align__(16) float s_r[WKV_CHUNK][DPP], s_k[WKV_CHUNK][DPP], s_w[WKV_CHUNK][DPP];
    __shared__ float s_v[WKV_CHUNK][WKV_COLS], s_b[WKV_CHUNK];
    const int h = blockIdx.x / col_blocks, j0 = (blockIdx.x % col_blocks) * WKV_COLS, seq = blockIdx.y;
    const int t0 = q_start[seq], t1 = q_start[seq + 1];
    if (t1 <= t0) return;
    const int tid = threadIdx.x, j = j0 + tid / WKV_LANES, sub = tid % WKV_LANES, lane = tid & 31, warp = tid >> 5;
    const bool col = j < D;
    float* S = state + (int64_t)slots[seq] * H * D * D * 2 + (int64_t)h * D * D;   // a slot has room for 64-bit words; this path uses half
    float s[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) {
        const int i = sub * RPT + ii;
        s[ii] = (col && i < D) ? S[(int64_t)i * D + j] : 0.f;
    }
    const int64_t hoff = (int64_t)h * D;
    // The next chunk's inputs are asked for before the current chunk's tokens are walked and land in registers meanwhile:
    // a CTA is alone on its SM with four warps, and a chunk read when it is needed would cost more than walking it.
    constexpr int THREADS = WKV_COLS * WKV_LANES;
    constexpr int NIT = WKV_CHUNK * DP / THREADS, NVI = WKV_CHUNK * WKV_COLS / THREADS;
    TA pr[NIT], pk[NIT], pv[NVI];
    float pd[NIT];
    auto prefetch = [&](int c0) {
        const int n = min(WKV_CHUNK, t1 - c0);
#pragma unroll
        for (int it = 0; it < NIT; ++it) {
            const int e = tid + it * THREADS, tt = e / DP, i = e % DP;
            pr[it] = from_float<TA>(0.f), pk[it] = from_float<TA>(0.f), pd[it] = 0.f;
            if (tt < n && i < D) {
                const int64_t at = (int64_t)(c0 + tt) * ld + hoff + i;
                pr[it] = r[at];
                pk[it] = k[at];
                pd[it] = dlog[(int64_t)(c0 + tt) * H * D + hoff + i];
            }
        }
#pragma unroll
        for (int it = 0; it < NVI; ++it) {
            const int e = tid + it * THREADS, tt = e / WKV_COLS, c = e % WKV_COLS;
            pv[it] = (tt < n && j0 + c < D) ? v[(int64_t)(c0 + tt) * ld + hoff + j0 + c] : from_float<TA>(0.f);
        }
    };
    prefetch(t0);
    for (int c0 = t0; c0 < t1; c0 += WKV_CHUNK) {
        const int n = min(WKV_CHUNK, t1 - c0);
        __syncthreads();   // the chunk before has been read
#pragma unroll
        for (int it = 0; it < NIT; ++it) {
            const int e = tid + it * THREADS, tt = e / DP, i = e % DP;
            const int at = i + 4 * (i / RPT);
            s_r[tt][at] = to_float(pr[it]);
            s_k[tt][at] = to_float(pk[it]);
            s_w[tt][at] = i < D ? expf(-expf(pd[it] + w0[hoff + i])) : 1.f;
        }
#pragma unroll
        for (int it = 0; it < NVI; ++it) {
            const int e = tid + it * THREADS;
            s_v[e / WKV_COLS][e % WKV_COLS] = to_float(pv[it]);
        }
        __syncthreads();
        if (c0 + WKV_CHUNK < t1) prefetch(c0 + WKV_CHUNK);
        // the bonus term's sum over the key rows, sum_i r_i u_i k_i: one warp per token, lanes stride the rows
        for (int tt = warp; tt < n; tt += THREADS / 32) {
            float b = 0.f;
            for (int i = lane; i < D; i += 32) b = fmaf(s_r[tt][i + 4 * (i / RPT)] * u[hoff + i], s_k[tt][i + 4 * (i / RPT)], b);
            b = warp_sum(b);
            if (lane == 0) s_b[tt] = b;
        }
        __syncthreads();
        // two tokens a round: both tokens' inputs are asked of shared memory before the first is used (four warps on
        // an SM hide no latency for one another)
        constexpr int NQ = RPT / 4;
        const int base = sub * (RPT + 4);
        auto fetch = [&](int tt, float4 (&R)[NQ], float4 (&W)[NQ], float4 (&K)[NQ], float& vj, float& bb) {
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                R[q] = *reinterpret_cast<const float4*>(&s_r[tt][base + 4 * q]);
                W[q] = *reinterpret_cast<const float4*>(&s_w[tt][base + 4 * q]);
                K[q] = *reinterpret_cast<const float4*>(&s_k[tt][base + 4 * q]);
            }
            vj = s_v[tt][tid / WKV_LANES];
            bb = s_b[tt];
        };
        auto walk = [&](int tt, const float4 (&R)[NQ], const float4 (&W)[NQ], const float4 (&K)[NQ], float vj, float bb) {
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                a0 = fmaf(R[q].x, s[4 * q], a0);
                a1 = fmaf(R[q].y, s[4 * q + 1], a1);
                a0 = fmaf(R[q].z, s[4 * q + 2], a0);
                a1 = fmaf(R[q].w, s[4 * q + 3], a1);
            }
            float o = a0 + a1;
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o = fmaf(vj, bb, o);
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                s[4 * q] = fmaf(W[q].x, s[4 * q], K[q].x * vj);
                s[4 * q + 1] = fmaf(W[q].y, s[4 * q + 1], K[q].y * vj);
                s[4 * q + 2] = fmaf(W[q].z, s[4 * q + 2], K[q].z * vj);
                s[4 * q + 3] = fmaf(W[q].w, s[4 * q + 3], K[q].w * vj);
            }
            if (col && sub == 0) out[(int64_t)(c0 + tt) * H * D + hoff + j] = o;
        };
        for (int tt = 0; tt < n; tt += 2) {
            float4 Ra[NQ], Wa[NQ], Ka[NQ], Rb[NQ], Wb[NQ], Kb[NQ];
            float va, ba, vb, bb;
            const bool two = tt + 1 < n;
            fetch(tt, Ra, Wa, Ka, va, ba);
            fetch(two ? tt + 1 : tt, Rb, Wb, Kb, vb, bb);
            walk(tt, Ra, Wa, Ka, va, ba);
            if (two) walk(tt + 1, Rb, Wb, Kb, vb, bb);
        }
    }
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) {
        const int i = sub * RPT + ii;
        if (col && i < D) S[(int64_t)i * D + j] = s[ii];
    }
}

// The float32 path carries the state, the decay and the read-out in 64-bit.  A state of slowly decaying channels is a sum
// over hundreds of tokens; where a head's read-out nearly cancels (its root mean square a few per cent of the usual), the
// rounding of a 32-bit state, 1e-6 of the state after so many steps, becomes 1e-5 and more of the normalised result.  The
// slot holds the doubles' words, so a prompt cut anywhere continues from the same bits.  Same layout of the work as above,
// without its tuning: this path is the sharper one, not the fast one.
template <int RPT>
__global__ void __launch_bounds__(WKV_COLS* WKV_LANES) wkv_scan_f64_kernel(const float* __restrict__ r, const float* __restrict__ k,
                                                                            const float* __restrict__ v, int64_t ld, const float* __restrict__ dlog,
                                                                            const float* __restrict__ w0, const float* __restrict__ u,
                                                                            float* __restrict__ state, float* __restrict__ out,
                                                                            const int* __restrict__ q_start, const int* __restrict__ slots, int H, int D,
                                                                            int col_blocks) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int DP = RPT * WKV_LANES, CH = 8;
    __shared__ double s_w[CH][DP], s_b[CH];
    __shared__ float s_r[CH][DP], s_k[CH][DP], s_v[CH][WKV_COLS];
    const int h = blockIdx.x / col_blocks, j0 = (blockIdx.x % col_blocks) * WKV_COLS, seq = blockIdx.y;
    const int t0 = q_start[seq], t1 = q_start[seq + 1];
    if (t1 <= t0) return;
    const int tid = threadIdx.x, j = j0 + tid / WKV_LANES, sub = tid % WKV_LANES, lane = tid & 31, warp = tid >> 5;
    const bool col = j < D;
    double* S = reinterpret_cast<double*>(state) + ((int64_t)slots[seq] * H + h) * D * D;
    double s[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) {
        const int i = sub * RPT + ii;
        s[ii] = (col && i < D) ? S[(int64_t)i * D + j] : 0.0;
    }
    const int64_t hoff = (int64_t)h * D;
    for (int c0 = t0; c0 < t1; c0 += CH) {
        const int n = min(CH, t1 - c0);
        __syncthreads();   // the chunk before has been read
        for (int e = tid; e < n * DP; e += blockDim.x) {
            const int tt = e / DP, i = e % DP;
            float rv = 0.f, kv = 0.f;
            double wv = 1.0;
            if (i < D) {
                const int64_t at = (int64_t)(c0 + tt) * ld + hoff + i;
                rv = r[at];
                kv = k[at];
                wv = exp(-exp((double)dlog[(int64_t)(c0 + tt) * H * D + hoff + i] + (double)w0[hoff + i]));
            }
            s_r[tt][i] = rv, s_k[tt][i] = kv, s_w[tt][i] = wv;
        }
        for (int e = tid; e < n * WKV_COLS; e += blockDim.x) {
            const int tt = e / WKV_COLS, c = e % WKV_COLS;
            s_v[tt][c] = j0 + c < D ? v[(int64_t)(c0 + tt) * ld + hoff + j0 + c] : 0.f;
        }
        __syncthreads();
        for (int tt = warp; tt < n; tt += (int)(blockDim.x >> 5)) {
            double b = 0.0;
            for (int i = lane; i < D; i += 32) b = fma((double)s_r[tt][i] * (double)u[hoff + i], (double)s_k[tt][i], b);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) b += __shfl_xor_sync(0xffffffffu, b, o);
            if (lane == 0) s_b[tt] = b;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const double vj = (double)s_v[tt][tid / WKV_LANES];
            double a0 = 0.0, a1 = 0.0;
#pragma unroll
            for (int ii = 0; ii < RPT; ii += 2) {
                a0 = fma((double)s_r[tt][sub * RPT + ii], s[ii], a0);
                a1 = fma((double)s_r[tt][sub * RPT + ii + 1], s[ii + 1], a1);
            }
            double o = a0 + a1;
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o = fma(vj, s_b[tt], o);
#pragma unroll
            for (int ii = 0; ii < RPT; ++ii) s[ii] = fma(s_w[tt][sub * RPT + ii], s[ii], (double)s_k[tt][sub * RPT + ii] * vj);
            if (col && sub == 0) out[(int64_t)(c0 + tt) * H * D + hoff + j] = (float)o;
        }
    }
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) {
        const int i = sub * RPT + ii;
        if (col && i < D) S[(int64_t)i * D + j] = s[ii];
    }
}

// y[t, h, :] = o / sqrt(mean(o^2) + eps) * w * silu(g): one warp per (token, head).
template <typename TA>
__global__ void wkv_output_kernel(TA* __restrict__ y, const float* __restrict__ o, const TA* __restrict__ g, int64_t ldg,
                                  const float* __restrict__ w, float eps, int n_tokens, int H, int D) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item % H);
    const float* orow = o + (t * H + h) * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) ss = fmaf(orow[i], orow[i], ss);
    const float inv = rsqrtf(warp_sum(ss) / (float)D + eps);
    for (int i = lane; i < D; i += 32) {
        const float z = to_float(g[t * ldg + (int64_t)h * D + i]);
        y[(t * H + h) * D + i] = from_float<TA>(orow[i] * inv * w[h * D + i] * (z / (1.f + expf(-z))));
    }
}

template <typename TA, int RPT>
cudaError_t launch_scan(const void* r, const void* k, const void* v, int64_t ld, const float* dlog, const float* w0, const float* u,
                        float* state, float* out, const int* q_start, const int* slots, int n_seqs, int H, int D, cudaStream_t s) {
    // an ordinary dependent: its CTAs hold many registers and would sit on the SMs while the kernels before it run
    const int col_blocks = (D + WKV_COLS - 1) / WKV_COLS;
    if (sizeof(TA) == 4) {
        wkv_scan_f64_kernel<RPT><<<dim3(H * col_blocks, n_seqs), WKV_COLS * WKV_LANES, 0, s>>>((const float*)r, (const float*)k, (const float*)v, ld, dlog, w0, u,
                                                                                             state, out, q_start, slots, H, D, col_blocks);
        return cudaGetLastError();
    }
    wkv_scan_kernel<TA, RPT><<<dim3(H * col_blocks, n_seqs), WKV_COLS * WKV_LANES, 0, s>>>((const TA*)r, (const TA*)k, (const TA*)v, ld, dlog, w0, u, state, out,
                                                                                         q_start, slots, H, D, col_blocks);
    return cudaGetLastError();
}

template <typename TA>
cudaError_t scan_by_size(const void* r, const void* k, const void* v, int64_t ld, const float* dlog, const float* w0, const float* u,
                         float* state, float* out, const int* q_start, const int* slots, int n_seqs, int H, int D, cudaStream_t s) {
    const int rpt = (D + WKV_LANES - 1) / WKV_LANES;
    if (rpt <= 8) return launch_scan<TA, 8>(r, k, v, ld, dlog, w0, u, state, out, q_start, slots, n_seqs, H, D, s);
    if (rpt <= 16) return launch_scan<TA, 16>(r, k, v, ld, dlog, w0, u, state, out, q_start, slots, n_seqs, H, D, s);
    if (rpt <= 24) return launch_scan<TA, 24>(r, k, v, ld, dlog, w0, u, state, out, q_start, slots, n_seqs, H, D, s);
    if (rpt <= 32) return launch_scan<TA, 32>(r, k, v, ld, dlog, w0, u, state, out, q_start, slots, n_seqs, H, D, s);
    return launch_scan<TA, 64>(r, k, v, ld, dlog, w0, u, state, out, q_start, slots, n_seqs, H, D, s);
}

}  // namespace

IMP_API int imp_wkv_max_head_dim() { return 64 * WKV_LANES; }

IMP_API int imp_wkv_mix(const void* x, int64_t ldx, const float* mu, float* prev_state, const int* seq_of_token, const int* q_start,
                        const int* slots, int n_tokens, int n_seqs, int d, void* out, int update_state, int act_dtype, int* status,
                        void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(x && mu && prev_state && seq_of_token && q_start && slots && out && d > 0, "imp_wkv_mix: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = act_dtype == IMP_F32
                        ? imp_launch(wkv_mix_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (const float*)x, ldx, mu, prev_state, seq_of_token,
                                     q_start, slots, n_tokens, n_seqs, d, (float*)out, update_state, status)
                        : imp_launch(wkv_mix_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, s, (const __nv_bfloat16*)x, ldx, mu, prev_state,
                                     seq_of_token, q_start, slots, n_tokens, n_seqs, d, (__nv_bfloat16*)out, update_state, status);
    if (e == cudaSuccess && !update_state)
        e = act_dtype == IMP_F32
                ? imp_launch(wkv_shift_state_kernel<float>, dim3(n_seqs), dim3(256), 0, s, (const float*)x, ldx, prev_state, q_start, slots, d)
                : imp_launch(wkv_shift_state_kernel<__nv_bfloat16>, dim3(n_seqs), dim3(256), 0, s, (const __nv_bfloat16*)x, ldx, prev_state,
                             q_start, slots, d);
    if (e != cudaSuccess) {
        imp_set_error("imp_wkv_mix: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

IMP_API int imp_tanh_inplace(void* x, int64_t n, int dtype, void* stream) {
    if (n == 0) return 0;
    IMP_CHECK_ARG(x && n > 0, "imp_tanh_inplace: bad argument");
    const dim3 grid((unsigned)std::min<int64_t>((n + 255) / 256, 4096));
    cudaError_t e = dtype == IMP_F32 ? imp_launch(tanh_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, (float*)x, n)
                                     : imp_launch(tanh_kernel<__nv_bfloat16>, grid, dim3(256), 0, (cudaStream_t)stream, (__nv_bfloat16*)x, n);
    if (e != cudaSuccess) {
        imp_set_error("imp_tanh_inplace: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// r, k, v: [T, H*D] of the activation type, rows ld apart (three tensors with one stride); dlog: float32 [T, H*D]
// dense; w0: [H*D]; u: [H, D]; state: [slots, H, D, 2 D] float32 words (float32 activations: [slots, H, D, D] doubles; bfloat16:
// the first H*D*D floats of a slot); out: float32 [T, H*D] dense.
IMP_API int imp_wkv_scan(const void* r, const void* k, const void* v, int64_t ld, const float* dlog, const float* w0, const float* u,
                         float* state, float* out, const int* q_start, const int* slots, int n_seqs, int H, int D, int act_dtype,
                         void* stream) {
    if (n_seqs == 0) return 0;
    IMP_CHECK_ARG(r && k && v && dlog && w0 && u && state && out && q_start && slots && H > 0 && D > 0, "imp_wkv_scan: bad argument");
    IMP_CHECK_ARG(D <= imp_wkv_max_head_dim(), "imp_wkv_scan: head size %d above %d", D, imp_wkv_max_head_dim());
    IMP_CHECK_ARG(n_seqs <= 65535, "imp_wkv_scan: too many sequences");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = act_dtype == IMP_F32 ? scan_by_size<float>(r, k, v, ld, dlog, w0, u, state, out, q_start, slots, n_seqs, H, D, s)
                                         : scan_by_size<__nv_bfloat16>(r, k, v, ld, dlog, w0, u, state, out, q_start, slots, n_seqs, H, D, s);
    if (e != cudaSuccess) {
        imp_set_error("imp_wkv_scan: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

IMP_API int imp_wkv_output(void* y, const float* o, const void* g, int64_t ldg, const float* w, float eps, int n_tokens, int H, int D,
                           int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(y && o && g && w && H > 0 && D > 0, "imp_wkv_output: bad argument");
    const int warps = 8;
    const dim3 grid((unsigned)(((int64_t)n_tokens * H + warps - 1) / warps));
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = act_dtype == IMP_F32 ? imp_launch(wkv_output_kernel<float>, grid, dim3(warps * 32), 0, s, (float*)y, o, (const float*)g, ldg,
                                                      w, eps, n_tokens, H, D)
                                         : imp_launch(wkv_output_kernel<__nv_bfloat16>, grid, dim3(warps * 32), 0, s, (__nv_bfloat16*)y, o,
                                                      (const __nv_bfloat16*)g, ldg, w, eps, n_tokens, H, D);
    if (e != cudaSuccess) {
        imp_set_error("imp_wkv_output: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
