// Routing of a mixture of experts, and the sum of the chosen experts' outputs.
//
//   z[t, e]   = x[t] . Wr[e] + b[e]                       32-bit
//   chosen    = the `top` experts with the largest z (the lower index wins a tie)
//   weight    = softmax over the chosen logits only
//   gate[t]   = sigmoid(x[t] . Wg)                         one number per token, for a shared expert (optional)
//   out[t]    = sum_k weight[t, k] * y[place(t, k)] + gate[t] * shared[t]
//
// The expert products run over a list of (token, choice) pairs sorted by expert (see grouped_gemm.cu); moe_sort makes
// that list on the device: seg [E + 1], the token of every list row, and the row of every pair.  Nothing comes back
// to the host, so the launches of a step depend on its sizes alone.
#include "common.cuh"

namespace {

constexpr int ROUTE_BLOCK = 128, ROUTE_MAX_E = 1024, ROUTE_MAX_TOP = 32;

template <typename TA>
__global__ void __launch_bounds__(ROUTE_BLOCK) moe_route_kernel(const TA* __restrict__ x, int64_t ldx, int d, const float* __restrict__ wr,
                                                               const float* __restrict__ br, int E, int top, const float* __restrict__ wg,
                                                               int* __restrict__ idx, float* __restrict__ wts, float* __restrict__ gate) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float sm[];   // x [d], then z [E]
    float* xs = sm;
    float* z = sm + d;
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const TA* row = x + (int64_t)t * ldx;
    for (int i = tid; i < d; i += ROUTE_BLOCK) xs[i] = to_float(row[i]);
    __syncthreads();
    for (int e = warp; e < E + (wg ? 1 : 0); e += ROUTE_BLOCK / 32) {
        const float* w = e < E ? wr + (int64_t)e * d : wg;
        float acc = 0.f;
        for (int i = lane; i < d; i += 32) acc = fmaf(xs[i], w[i], acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            if (e < E) z[e] = acc + (br ? br[e] : 0.f);
            else gate[t] = 1.f / (1.f + expf(-acc));
        }
    }
    __syncthreads();
    if (warp != 0) return;
    // `top` rounds of arg-max over the logits that are left; the lower index wins a tie
    float chosen[ROUTE_MAX_TOP];
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best) best = v, at = e;     // ascending e: the first of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > best || (ov == best && oa < at)) best = ov, at = oa;
        }
        chosen[k] = best;
        if (lane == 0) {
            idx[(int64_t)t * top + k] = at;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float largest = chosen[0];   // the first chosen is the largest
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            chosen[k] = expf(chosen[k] - largest);
            sum += chosen[k];
        }
        for (int k = 0; k < top; ++k) wts[(int64_t)t * top + k] = chosen[k] / sum;
    }
}

// One CTA.  seg[e] .. seg[e + 1]: expert e's rows of the list; row_token[r]: the token of row r; pair_row[p]: the row of
// pair p = t * top + k.  Within an expert the rows follow the pair index, so the list is the same for the same routing.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int n_pairs, int top, int E, int* __restrict__ seg,
                                                        int* __restrict__ row_token, int* __restrict__ pair_row) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ int cnt[];   // [E + 1]
    const int tid = threadIdx.x;
    for (int e = tid; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = tid; p < n_pairs; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int c = cnt[e];
            cnt[e] = run;
            seg[e] = run;
            run += c;
        }
        cnt[E] = run;
        seg[E] = run;
    }
    __syncthreads();
    // every expert's rows in pair order: a warp walks the pairs of one expert at a time
    const int lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    for (int e = warp; e < E; e += n_warps) {
        int at = cnt[e];
        for (int p0 = 0; p0 < n_pairs; p0 += 32) {
            const int p = p0 + lane;
            const bool mine = p < n_pairs && idx[p] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int r = at + __popc(m & ((1u << lane) - 1u));
                row_token[r] = p / top;
                pair_row[p] = r;
            }
            at += __popc(m);
        }
    }
}

template <typename TA>
__global__ void moe_combine_kernel(TA* __restrict__ out, const TA* __restrict__ y, const int* __restrict__ pair_row, const float* __restrict__ wts,
                                   int top, const TA* __restrict__ shared, const float* __restrict__ gate, int d) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t t = blockIdx.x;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) acc = fmaf(wts[t * top + k], to_float(y[(int64_t)pair_row[t * top + k] * d + i]), acc);
        if (shared) acc = fmaf(gate ? gate[t] : 1.f, to_float(shared[t * d + i]), acc);
        out[t * d + i] = from_float<TA>(acc);
    }
}

}  // namespace

// x [T, d] (activation type, rows ldx apart); wr float32 [E, d], br float32 [E] or null; wg float32 [d] or null (then
// gate is not written).  idx int32 [T, top], wts float32 [T, top], gate float32 [T].
IMP_API int imp_moe_route(const void* x, int64_t ldx, int n_tokens, int d, const float* wr, const float* br, int E, int top, const float* wg,
                          int* idx, float* wts, float* gate, int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(x && wr && idx && wts && d > 0 && (!wg || gate), "imp_moe_route: bad argument");
    IMP_CHECK_ARG(E > 0 && E <= ROUTE_MAX_E && top > 0 && top <= E && top <= ROUTE_MAX_TOP,
                  "imp_moe_route: %d experts (at most %d), %d chosen (at most %d and no more than there are)", E, ROUTE_MAX_E, top, ROUTE_MAX_TOP);
    const size_t smem = (size_t)(d + E) * 4;
    IMP_CHECK_ARG(smem <= 200 * 1024, "imp_moe_route: rows of %d values do not fit the shared memory", d);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (act_dtype == IMP_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = imp_launch(moe_route_kernel<float>, dim3(n_tokens), dim3(ROUTE_BLOCK), smem, s, (const float*)x, ldx, d, wr, br, E, top, wg, idx, wts, gate);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = imp_launch(moe_route_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(ROUTE_BLOCK), smem, s, (const __nv_bfloat16*)x, ldx, d, wr, br, E,
                       top, wg, idx, wts, gate);
    }
    if (e != cudaSuccess) {
        imp_set_error("imp_moe_route: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

IMP_API int imp_moe_sort(const int* idx, int n_tokens, int top, int E, int* seg, int* row_token, int* pair_row, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(idx && seg && row_token && pair_row && top > 0 && E > 0 && E <= ROUTE_MAX_E, "imp_moe_sort: bad argument");
    cudaError_t e = imp_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(E + 1) * 4, (cudaStream_t)stream, idx, n_tokens * top, top, E, seg,
                               row_token, pair_row);
    if (e != cudaSuccess) {
        imp_set_error("imp_moe_sort: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// out [T, d] = sum_k wts[t, k] * y[pair_row[t * top + k]] (+ gate[t] * shared[t]); y [T * top, d], all dense.
IMP_API int imp_moe_combine(void* out, const void* y, const int* pair_row, const float* wts, int n_tokens, int top, const void* shared,
                            const float* gate, int d, int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(out && y && pair_row && wts && top > 0 && d > 0, "imp_moe_combine: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = act_dtype == IMP_F32 ? imp_launch(moe_combine_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (float*)out, (const float*)y,
                                                      pair_row, wts, top, (const float*)shared, gate, d)
                                         : imp_launch(moe_combine_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, s, (__nv_bfloat16*)out,
                                                      (const __nv_bfloat16*)y, pair_row, wts, top, (const __nv_bfloat16*)shared, gate, d);
    if (e != cudaSuccess) {
        imp_set_error("imp_moe_combine: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
