// The gated delta rule: a recurrent token mixer with one matrix state S [D, Dv] per head.
//
// Per token and value head h (reading the query / key head h / (H / G)):
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with g in (0, 1) a decay and beta in (0, 1) a step size, both per head and token.  q, k and v come out
// of a short causal convolution over time per channel (taps - 1 earlier inputs are part of a request's
// state) followed by silu; q and k are then unit vectors per head and q carries D^(-1/2).
//
// Four kernels, all 32-bit arithmetic on 32-bit state whatever the activation type:
//   gdr_prepare     one CTA per token: convolution + silu of every channel, unit q and k, beta and decay
//   gdr_conv_state  the last taps - 1 inputs of every sequence of the batch go to its state slot
//   gdr_scan        the recurrence; a CTA owns 32 value columns of one head of one sequence and walks
//                   the sequence's new tokens in order; four lanes share a column, each holding a
//                   quarter of it in registers, so no state travels between tokens but through registers
//   gdr_output      per head: o / rms(o) * w * silu(gate)
// Every column of S evolves independently of the others, which is what the scan kernel's split rests on.
// A token's result depends on the tokens before it only through S and the convolution's inputs, and the
// order of every sum is fixed by the sizes alone: cutting a prompt into portions changes no bit.
#include "common.cuh"

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------------------------- prepare
// proj: [T, ld] activations, columns [q: G*D | k: G*D | v: H*Dv | gate: H*Dv | b: H | a: H].
// conv_w: [C, taps] float32 with C = 2*G*D + H*Dv (the last tap is the current token's).
// conv_state: [slots, taps - 1, C] float32: the inputs of the taps - 1 tokens before the portion.
constexpr int GP_BLOCK = 256;

template <typename TA>
__global__ void __launch_bounds__(GP_BLOCK) gdr_prepare_kernel(
    const TA* __restrict__ proj, int64_t ld, const float* __restrict__ conv_w, int taps, const float* __restrict__ conv_state,
    const int* __restrict__ seq_of_token, const int* __restrict__ q_start, const int* __restrict__ slots, int n_seqs, int G,
    int D, int H, int Dv, const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ qn,
    float* __restrict__ kn, float* __restrict__ vc, float* __restrict__ beta, float* __restrict__ decay, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float ch[];   // [C] channels after convolution and silu
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nqk = G * D, C = 2 * nqk + H * Dv;
    const int seq = seq_of_token[t];
    if (seq < 0 || seq >= n_seqs) {
        if (tid == 0) imp_report(status, IMP_BAD_SEQUENCE);
        return;
    }
    const int start = q_start[seq];
    const int n = t - start;                 // index of the token inside its portion
    const float* st = conv_state + (int64_t)slots[seq] * (taps - 1) * C;
    for (int c = tid; c < C; c += GP_BLOCK) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int idx = n - (taps - 1) + j;
            const float x = idx >= 0 ? to_float(proj[(int64_t)(start + idx) * ld + c]) : st[(int64_t)(taps - 1 + idx) * C + c];
            acc = fmaf(conv_w[(int64_t)c * taps + j], x, acc);
        }
        ch[c] = silu_f(acc);
    }
    __syncthreads();
    // unit q and k per head: a warp per head
    const float q_scale = rsqrtf((float)D);
    for (int hh = warp; hh < 2 * G; hh += GP_BLOCK / 32) {
        const float* x = ch + hh * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(x[d], x[d], ss);
        ss = warp_sum(ss);
        const float r = rsqrtf(ss + 1e-6f) * (hh < G ? q_scale : 1.f);
        float* dst = (hh < G ? qn + (int64_t)t * nqk + hh * D : kn + (int64_t)t * nqk + (hh - G) * D);
        for (int d = lane; d < D; d += 32) dst[d] = x[d] * r;
    }
    for (int c = tid; c < H * Dv; c += GP_BLOCK) vc[(int64_t)t * H * Dv + c] = ch[2 * nqk + c];
    if (tid < H) {
        const TA* row = proj + (int64_t)t * ld + C + H * Dv;
        const float b = to_float(row[tid]), a = to_float(row[H + tid]);
        beta[(int64_t)t * H + tid] = 1.f / (1.f + expf(-b));
        decay[(int64_t)t * H + tid] = expf(-expf(a_log[tid]) * softplus_f(a + dt_bias[tid]));
    }
}

// New state of every sequence in the batch: the inputs of its last taps - 1 tokens (older ones shift down).
template <typename TA>
__global__ void gdr_conv_state_kernel(const TA* __restrict__ proj, int64_t ld, float* __restrict__ conv_state, int taps, int C,
                                      const int* __restrict__ q_start, const int* __restrict__ slots, int n_seqs) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C || seq >= n_seqs) return;
    const int start = q_start[seq], n = q_start[seq + 1] - start;
    if (n <= 0) return;
    float* st = conv_state + (int64_t)slots[seq] * (taps - 1) * C;
    for (int i = 0; i < taps - 1; ++i) {   // ascending: entry i reads entry i + n, never one already rewritten
        const int idx = n - (taps - 1) + i;
        st[(int64_t)i * C + c] = idx >= 0 ? to_float(proj[(int64_t)(start + idx) * ld + c]) : st[(int64_t)(i + n) * C + c];
    }
}

// ---------------------------------------------------------------------------------------- scan
constexpr int GS_COLS = 32;          // value columns per CTA
constexpr int GS_LANES = 4;          // lanes that share a column
constexpr int GS_BLOCK = GS_COLS * GS_LANES;
constexpr int GS_CHUNK = 8;          // tokens whose q and k are staged together

// DPL: key dimensions per lane (D <= 4 * DPL).  Lane r of a column holds dimensions [r * DPL, (r + 1) * DPL).
template <int DPL>
__global__ void __launch_bounds__(GS_BLOCK) gdr_scan_kernel(
    const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vc, const float* __restrict__ beta,
    const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out, const int* __restrict__ q_start,
    const int* __restrict__ slots, int G, int D, int H, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int ROW = DPL + 4;                          // padded so that the four lanes' 16-byte reads miss each other's banks
    __shared__ __align__(16) float k_s[GS_CHUNK][GS_LANES * ROW];
    __shared__ __align__(16) float q_s[GS_CHUNK][GS_LANES * ROW];
    __shared__ float g_s[GS_CHUNK], b_s[GS_CHUNK];
    const int tid = threadIdx.x, r = tid & (GS_LANES - 1);
    const int col = blockIdx.x * GS_COLS + (tid >> 2);
    const int h = blockIdx.y, seq = blockIdx.z;
    const int hk = h / (H / G);
    const int start = q_start[seq], n = q_start[seq + 1] - start;
    if (n <= 0) return;
    const bool live = col < Dv;
    float* S = state + (((int64_t)slots[seq] * H + h) * D) * Dv + col;
    float s[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = r * DPL + i;
        s[i] = (live && d < D) ? S[(int64_t)d * Dv] : 0.f;
    }
    const int nqk = G * D;
    for (int t0 = 0; t0 < n; t0 += GS_CHUNK) {
        const int nt = min(GS_CHUNK, n - t0);
        __syncthreads();
        for (int e = tid; e < nt * GS_LANES * DPL; e += GS_BLOCK) {
            const int tt = e / (GS_LANES * DPL), d = e - tt * (GS_LANES * DPL);
            const int64_t src = (int64_t)(start + t0 + tt) * nqk + hk * D + d;
            const int dst = (d / DPL) * ROW + d % DPL;
            k_s[tt][dst] = d < D ? kn[src] : 0.f;
            q_s[tt][dst] = d < D ? qn[src] : 0.f;
        }
        if (tid < nt) {
            g_s[tid] = decay[(int64_t)(start + t0 + tid) * H + h];
            b_s[tid] = beta[(int64_t)(start + t0 + tid) * H + h];
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const int64_t tok = start + t0 + tt;
            const float g = g_s[tt], b = b_s[tt];
            const float v = live ? vc[tok * H * Dv + (int64_t)h * Dv + col] : 0.f;
            const float4* k4 = reinterpret_cast<const float4*>(&k_s[tt][r * ROW]);
            const float4* q4 = reinterpret_cast<const float4*>(&q_s[tt][r * ROW]);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int i = 0; i < DPL / 4; ++i) {
                const float4 kk = k4[i];
                a0 = fmaf(s[4 * i], kk.x, a0);
                a1 = fmaf(s[4 * i + 1], kk.y, a1);
                a2 = fmaf(s[4 * i + 2], kk.z, a2);
                a3 = fmaf(s[4 * i + 3], kk.w, a3);
            }
            float ks = (a0 + a1) + (a2 + a3);
            ks += __shfl_xor_sync(0xffffffffu, ks, 1);
            ks += __shfl_xor_sync(0xffffffffu, ks, 2);
            const float u = b * (v - g * ks);             // S^T k after the decay is g times S^T k before it
            a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
            for (int i = 0; i < DPL / 4; ++i) {
                const float4 kk = k4[i], qq = q4[i];
                s[4 * i] = fmaf(kk.x, u, g * s[4 * i]);
                s[4 * i + 1] = fmaf(kk.y, u, g * s[4 * i + 1]);
                s[4 * i + 2] = fmaf(kk.z, u, g * s[4 * i + 2]);
                s[4 * i + 3] = fmaf(kk.w, u, g * s[4 * i + 3]);
                a0 = fmaf(s[4 * i], qq.x, a0);
                a1 = fmaf(s[4 * i + 1], qq.y, a1);
                a2 = fmaf(s[4 * i + 2], qq.z, a2);
                a3 = fmaf(s[4 * i + 3], qq.w, a3);
            }
            float o = (a0 + a1) + (a2 + a3);
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (live && r == 0) out[tok * H * Dv + (int64_t)h * Dv + col] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = r * DPL + i;
        if (live && d < D) S[(int64_t)d * Dv] = s[i];
    }
}

// -------------------------------------------------------------------------------------- output
// y[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w * silu(gate[t, h, :]); a warp per (token, head).
template <typename TA>
__global__ void gdr_output_kernel(TA* __restrict__ y, const float* __restrict__ o, const TA* __restrict__ gate, int64_t gate_ld,
                                  const float* __restrict__ w, float eps, int n_tokens, int H, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)n_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const float* x = o + (t * H + h) * Dv;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) ss = fmaf(x[d], x[d], ss);
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)Dv + eps);
    const TA* gt = gate + t * gate_ld + (int64_t)h * Dv;
    TA* dst = y + (t * H + h) * Dv;
    for (int d = lane; d < Dv; d += 32) dst[d] = from_float<TA>(x[d] * r * w[d] * silu_f(to_float(gt[d])));
}

// ------------------------------------------------------------------------------------ launchers
IMP_API int imp_gdr_prepare(const void* proj, int64_t ld, const float* conv_w, int taps, const float* conv_state,
                            const int* seq_of_token, const int* q_start, const int* slots, int n_tokens, int n_seqs, int G, int D,
                            int H, int Dv, const float* a_log, const float* dt_bias, float* qn, float* kn, float* vc, float* beta,
                            float* decay, int act_dtype, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(proj && conv_w && conv_state && seq_of_token && q_start && slots && a_log && dt_bias && qn && kn && vc && beta && decay,
                  "imp_gdr_prepare: null pointer");
    IMP_CHECK_ARG(G > 0 && H > 0 && H % G == 0 && D > 0 && Dv > 0 && taps >= 1 && H <= GP_BLOCK,
                  "imp_gdr_prepare: bad sizes (heads %d over %d key heads, at most %d heads)", H, G, GP_BLOCK);
    const int C = 2 * G * D + H * Dv;
    IMP_CHECK_ARG(ld >= (int64_t)C + H * Dv + 2 * H, "imp_gdr_prepare: the projection's rows are too short");
    const size_t smem = (size_t)C * 4;
    IMP_CHECK_ARG(smem <= 200 * 1024, "imp_gdr_prepare: %d convolution channels do not fit shared memory", C);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
    if (act_dtype == IMP_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(gdr_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            imp_launch(gdr_prepare_kernel<float>, dim3(n_tokens), dim3(GP_BLOCK), smem, s, (const float*)proj, ld, conv_w, taps, conv_state,
                       seq_of_token, q_start, slots, n_seqs, G, D, H, Dv, a_log, dt_bias, qn, kn, vc, beta, decay, status);
    } else {
        if (smem > 48 * 1024)
            e = cudaFuncSetAttribute(gdr_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            imp_launch(gdr_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(GP_BLOCK), smem, s, (const __nv_bfloat16*)proj, ld, conv_w,
                       taps, conv_state, seq_of_token, q_start, slots, n_seqs, G, D, H, Dv, a_log, dt_bias, qn, kn, vc, beta, decay,
                       status);
    }
    if (e != cudaSuccess) {
        imp_set_error("imp_gdr_prepare: %s", cudaGetErrorString(e));
        return (int)e;
    }
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_gdr_conv_state(const void* proj, int64_t ld, float* conv_state, int taps, int C, const int* q_start, const int* slots,
                               int n_seqs, int act_dtype, void* stream) {
    if (n_seqs == 0 || taps <= 1) return 0;
    IMP_CHECK_ARG(proj && conv_state && q_start && slots && C > 0 && n_seqs <= 65535, "imp_gdr_conv_state: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((C + 127) / 128, n_seqs);
    if (act_dtype == IMP_F32)
        imp_launch(gdr_conv_state_kernel<float>, grid, dim3(128), 0, s, (const float*)proj, ld, conv_state, taps, C, q_start, slots, n_seqs);
    else
        imp_launch(gdr_conv_state_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16*)proj, ld, conv_state, taps, C,
                   q_start, slots, n_seqs);
    IMP_RETURN_LAUNCH();
}

// state: [slots, H, D, Dv] float32, updated in place; out: [n_tokens, H * Dv] float32.
IMP_API int imp_gdr_scan(const float* qn, const float* kn, const float* vc, const float* beta, const float* decay, float* state,
                         float* out, const int* q_start, const int* slots, int n_seqs, int G, int D, int H, int Dv, void* stream) {
    if (n_seqs == 0) return 0;
    IMP_CHECK_ARG(qn && kn && vc && beta && decay && state && out && q_start && slots, "imp_gdr_scan: null pointer");
    IMP_CHECK_ARG(G > 0 && H % G == 0 && D > 0 && Dv > 0 && H <= 65535 && n_seqs <= 65535, "imp_gdr_scan: bad sizes");
    if (D > 256) {
        imp_set_error("imp_gdr_scan: key size %d exceeds 256", D);
        return IMP_ERR_UNSUPPORTED;
    }
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((Dv + GS_COLS - 1) / GS_COLS, H, n_seqs);
#define GDR_SCAN(DPL) \
    imp_launch(gdr_scan_kernel<DPL>, grid, dim3(GS_BLOCK), 0, s, qn, kn, vc, beta, decay, state, out, q_start, slots, G, D, H, Dv)
    if (D <= 16) GDR_SCAN(4);
    else if (D <= 32) GDR_SCAN(8);
    else if (D <= 64) GDR_SCAN(16);
    else if (D <= 128) GDR_SCAN(32);
    else GDR_SCAN(64);
#undef GDR_SCAN
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_gdr_output(void* y, const float* o, const void* gate, int64_t gate_ld, const float* w, float eps, int n_tokens, int H,
                           int Dv, int act_dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(y && o && gate && w && H > 0 && Dv > 0, "imp_gdr_output: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t items = (int64_t)n_tokens * H;
    const dim3 grid((unsigned)((items + 7) / 8));
    if (act_dtype == IMP_F32)
        imp_launch(gdr_output_kernel<float>, grid, dim3(256), 0, s, (float*)y, o, (const float*)gate, gate_ld, w, eps, n_tokens, H, Dv);
    else
        imp_launch(gdr_output_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (__nv_bfloat16*)y, o, (const __nv_bfloat16*)gate, gate_ld, w,
                   eps, n_tokens, H, Dv);
    IMP_RETURN_LAUNCH();
}
