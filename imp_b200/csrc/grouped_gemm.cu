// Matrix products over groups:  C_g[r, n] = sum_k A[row(r), a0(g) + k] * W_g[n, k],  one weight matrix per group.
//
// Two ways of saying which rows a group has:
//   uniform    every group has the same M rows (grid.z = group): per-head products, where the head's slice of a
//              row starts a_group_cols * g columns in and the result goes c_group_cols * g columns in;
//   segmented  a list of rows sorted by group, seg[g] .. seg[g + 1] being group g's part of it (device memory, so a
//              launch does not depend on the routing): routed experts.  Row r of the list reads A row a_rows[r]
//              (null: r) and writes C row r.  The grid covers the most tiles any routing can make
//              (rows / BM + groups); a CTA finds its group by walking seg, and leaves if there is no tile for it.
// Optionally two weight matrices per group and the epilogue silu(A Wg^T) * (A Wu^T).
//
// bfloat16: mma.sync m16n8k16 with 32-bit accumulation, 64 x 64 x 64 tiles through a cp.async ring of three or four stages,
// fragments by ldmatrix, four warps.  (Tiles of 128 x 64 and 128 x 128 measured no faster for many rows a group and slower
// for few; skipping the products of 16-row pieces without rows measured slower too.)  float32: FFMA, k ascending in blocks
// of 16 whose sums are added in order, for every output element, so a row's result does not depend on what else is in the batch.
#include <algorithm>

#include "common.cuh"

namespace {

constexpr int GG_BM = 64, GG_BN = 64;

struct GroupedArgs {
    const void* A;
    int64_t lda;
    const int* a_rows;
    int64_t a_group_cols;
    const void* W;
    const void* W2;
    int64_t w_group_stride, ldw;
    void* C;
    int64_t ldc, c_group_cols;
    const int* seg;
    int M, N, K, G;
    int vec;   // rows of A and W start on 16 bytes and K is a multiple of 8 (bfloat16) / 4 (float32)
    int il;    // the gated epilogue's two matrices are one, gate and up rows alternating in runs of 8 (W2 unused)
};

// Row n of the gate (up = false) or up (up = true) matrix inside a group's weight.
__device__ __forceinline__ int64_t gated_row(const GroupedArgs& p, int n, bool up) {
    return p.il ? (int64_t)(n >> 3) * 16 + (n & 7) + (up ? 8 : 0) : n;
}

// Which group and which rows of the list this CTA has; false if it has none.
__device__ __forceinline__ bool find_tile(const GroupedArgs& p, int& g, int& row0, int& row_end, int bm = GG_BM) {
    if (!p.seg) {
        g = blockIdx.z;
        row0 = blockIdx.y * bm;
        row_end = p.M;
        return row0 < row_end;
    }
    int t = blockIdx.y;
    for (int e = 0; e < p.G; ++e) {
        const int a = p.seg[e], b = p.seg[e + 1];
        const int nt = (b - a + bm - 1) / bm;
        if (t < nt) {
            g = e;
            row0 = a + t * bm;
            row_end = b;
            return true;
        }
        t -= nt;
    }
    return false;
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// --------------------------------------------------------------------------------------- bfloat16
constexpr int GB_BK = 64, GB_LD = GB_BK + 8;   // a row of a block is a whole 128-byte line; padded rows: ldmatrix hits 32 different banks

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// rows x 32 bfloat16 of `src` (row r at src_row(r), null rows zero) into a padded tile.  With `vec` the chunks of 8 travel as
// asynchronous 16-byte copies (the caller commits and waits); otherwise element by element.
template <int ROWS, typename RowFn>
__device__ __forceinline__ void load_tile_bf16(__nv_bfloat16 (*tile)[GB_LD], RowFn src_row, int k0, int K, int vec, const void* any_global) {
    const int tid = threadIdx.x;
    if (vec) {
        // ROWS x 8 chunks of 8: four chunks a thread for 64 rows, one for 16
#pragma unroll
        for (int e = 0; e < ROWS / 16; ++e) {
            const int idx = tid + e * 128, r = idx >> 3, c = (idx & 7) * 8;
            const __nv_bfloat16* row = src_row(r);
            const bool there = row && k0 + c < K;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&tile[r][c]);
            const void* src = there ? (const void*)(row + k0 + c) : any_global;   // a copy of zero bytes fills with zeros and reads nothing
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(there ? 16 : 0) : "memory");
        }
    } else {
        for (int idx = tid; idx < ROWS * GB_BK; idx += 128) {
            const int r = idx / GB_BK, c = idx % GB_BK;
            const __nv_bfloat16* row = src_row(r);
            tile[r][c] = (row && k0 + c < K) ? row[k0 + c] : __float2bfloat16_rn(0.f);
        }
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// BM rows a tile: 64 (four warps as 2 x 2, 32 x 32 outputs each) or 16 (four warps side by side, 16 x 16 each: steps of few
// rows a group, where the 64-row tile would spend the tensor pipe and the shared memory on rows that hold nothing).
template <bool SWIGLU, int BM> struct GroupedTile {
    static constexpr int STAGES = SWIGLU ? 3 : 4;
    static constexpr size_t STAGE_ELEMS = (size_t)(BM + GG_BN * (SWIGLU ? 2 : 1)) * GB_LD;
    static constexpr size_t SMEM = STAGES * STAGE_ELEMS * 2;
};

template <bool SWIGLU, int BM>
__global__ void __launch_bounds__(128) grouped_gemm_bf16_kernel(const GroupedArgs p) {
    pdl_wait();
    pdl_launch_dependents();
    using Tile = GroupedTile<SWIGLU, BM>;
    constexpr int GB_STAGES = Tile::STAGES;
    constexpr int WM = BM == 64 ? 32 : 16, WN = BM == 64 ? 32 : 16, MI = WM / 16, NJ = WN / 16;
    int g, row0, row_end;
    if (!find_tile(p, g, row0, row_end, BM)) return;
    extern __shared__ __align__(16) unsigned char gg_smem[];
    typedef __nv_bfloat16(*TilePtr)[GB_LD];
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(gg_smem);
    auto As = [&](int st) { return reinterpret_cast<TilePtr>(ring + st * Tile::STAGE_ELEMS); };
    auto Ws = [&](int st) { return reinterpret_cast<TilePtr>(ring + st * Tile::STAGE_ELEMS + (size_t)BM * GB_LD); };
    auto Us = [&](int st) { return reinterpret_cast<TilePtr>(ring + st * Tile::STAGE_ELEMS + (size_t)(BM + GG_BN) * GB_LD); };
    __shared__ int64_t a_off[BM];   // where each row of the tile starts in A (-1: beyond the group's rows)
    const int n0 = blockIdx.x * GG_BN;
    const __nv_bfloat16* A = (const __nv_bfloat16*)p.A + p.a_group_cols * g;
    const __nv_bfloat16* W = (const __nv_bfloat16*)p.W + p.w_group_stride * g;
    const __nv_bfloat16* U = SWIGLU ? (p.il ? W : (const __nv_bfloat16*)p.W2 + p.w_group_stride * g) : nullptr;
    if (threadIdx.x < BM) {
        const int lr = row0 + threadIdx.x;
        a_off[threadIdx.x] = lr < row_end ? (int64_t)(p.a_rows ? p.a_rows[lr] : lr) * p.lda : -1;
    }
    __syncthreads();
    auto a_row = [&](int r) -> const __nv_bfloat16* { return a_off[r] >= 0 ? A + a_off[r] : nullptr; };
    auto w_row = [&](int r) -> const __nv_bfloat16* { return n0 + r < p.N ? W + gated_row(p, n0 + r, false) * p.ldw : nullptr; };
    auto u_row = [&](int r) -> const __nv_bfloat16* { return n0 + r < p.N ? U + gated_row(p, n0 + r, true) * p.ldw : nullptr; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int wm = BM == 64 ? (warp >> 1) * 32 : 0, wn = BM == 64 ? (warp & 1) * 32 : warp * 16;
    // what a lane hands to ldmatrix: for A (16 rows x 16 k) row lane % 16 at k + 8 * (lane / 16); for W (16 n x 16 k, two
    // 8-column tiles of the product) row lane % 8 + 8 * (lane / 16) at k + 8 * ((lane / 8) % 2)
    const int a_r = lane & 15, a_c = (lane >> 4) * 8;
    const int b_r = (lane & 7) + (lane >> 4) * 8, b_c = ((lane >> 3) & 1) * 8;
    float acc[MI][2 * NJ][4], acu[SWIGLU ? MI : 1][2 * NJ][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < 2 * NJ; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[i][j][e] = 0.f;
                if (SWIGLU) acu[i][j][e] = 0.f;
            }

    const int n_k = (p.K + GB_BK - 1) / GB_BK;
    auto fetch = [&](int kb) {
        if (kb < n_k) {
            const int st = kb % GB_STAGES;
            load_tile_bf16<BM>(As(st), a_row, kb * GB_BK, p.K, p.vec, p.W);
            load_tile_bf16<GG_BN>(Ws(st), w_row, kb * GB_BK, p.K, p.vec, p.W);
            if (SWIGLU) load_tile_bf16<GG_BN>(Us(st), u_row, kb * GB_BK, p.K, p.vec, p.W);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");   // one group per k-block, empty ones included: the wait counts groups
    };
    for (int kb = 0; kb < GB_STAGES - 1; ++kb) fetch(kb);
    for (int kb = 0; kb < n_k; ++kb) {
        asm volatile("cp.async.wait_group %0;" ::"n"(GB_STAGES - 2) : "memory");
        __syncthreads();                 // block kb has landed for everyone, and block kb - 1's stage is free again
        fetch(kb + GB_STAGES - 1);
        const int st = kb % GB_STAGES;
        const TilePtr as = As(st), ws = Ws(st), us = Us(st);
#pragma unroll
        for (int kk = 0; kk < GB_BK; kk += 16) {
            uint32_t a[MI][4];
#pragma unroll
            for (int i = 0; i < MI; ++i) ldmatrix_x4(a[i], &as[wm + i * 16 + a_r][kk + a_c]);
#pragma unroll
            for (int jj = 0; jj < NJ; ++jj) {
                uint32_t b[4];
                ldmatrix_x4(b, &ws[wn + jj * 16 + b_r][kk + b_c]);
                const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
#pragma unroll
                for (int i = 0; i < MI; ++i) {
                    mma_bf16(acc[i][2 * jj], a[i], b0);
                    mma_bf16(acc[i][2 * jj + 1], a[i], b1);
                }
                if (SWIGLU) {
                    ldmatrix_x4(b, &us[wn + jj * 16 + b_r][kk + b_c]);
                    const uint32_t u0[2] = {b[0], b[1]}, u1[2] = {b[2], b[3]};
#pragma unroll
                    for (int i = 0; i < MI; ++i) {
                        mma_bf16(acu[i][2 * jj], a[i], u0);
                        mma_bf16(acu[i][2 * jj + 1], a[i], u1);
                    }
                }
            }
        }
    }
    __nv_bfloat16* C = (__nv_bfloat16*)p.C + p.c_group_cols * g;
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int lr = row0 + wm + i * 16 + gid + half * 8;
            if (lr >= row_end) continue;
            __nv_bfloat16* crow = C + (int64_t)lr * p.ldc;
#pragma unroll
            for (int j = 0; j < 2 * NJ; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = n0 + wn + j * 8 + 2 * tig + e;
                    if (n >= p.N) continue;
                    float v = acc[i][j][half * 2 + e];
                    if (SWIGLU) v = silu_f(v) * acu[i][j][half * 2 + e];   // the activation on the 32-bit sums
                    crow[n] = __float2bfloat16_rn(v);
                }
        }
}

// ---------------------------------------------------------------------------------------- float32
constexpr int GF_BK = 16;

template <bool SWIGLU>
__global__ void __launch_bounds__(256) grouped_gemm_f32_kernel(const GroupedArgs p) {
    pdl_wait();
    pdl_launch_dependents();
    int g, row0, row_end;
    if (!find_tile(p, g, row0, row_end)) return;
    __shared__ float As[GF_BK][GG_BM + 4];
    __shared__ float Ws[GF_BK][GG_BN + 4];
    __shared__ float Us[SWIGLU ? GF_BK : 1][GG_BN + 4];
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * GG_BN;
    const float* A = (const float*)p.A + p.a_group_cols * g;
    const float* W = (const float*)p.W + p.w_group_stride * g;
    const float* U = SWIGLU ? (p.il ? W : (const float*)p.W2 + p.w_group_stride * g) : nullptr;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4], acu[SWIGLU ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.f;
            if (SWIGLU) acu[i][j] = 0.f;
        }
    // the A rows this thread loads, resolved once
    int64_t a_off[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int r = (tid + e * 256) / GF_BK, lr = row0 + r;
        a_off[e] = lr < row_end ? (int64_t)(p.a_rows ? p.a_rows[lr] : lr) * p.lda : -1;
    }
    for (int k0 = 0; k0 < p.K; k0 += GF_BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / GF_BK, kk = idx % GF_BK;
            const int gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (a_off[e] >= 0 && gk < p.K) ? A[a_off[e] + gk] : 0.f;
            Ws[kk][r] = (gn < p.N && gk < p.K) ? W[gated_row(p, gn, false) * p.ldw + gk] : 0.f;
            if (SWIGLU) Us[kk][r] = (gn < p.N && gk < p.K) ? U[gated_row(p, gn, true) * p.ldw + gk] : 0.f;
        }
        __syncthreads();
        // a block's 16 products are summed on their own and then added to the running sum (as in gemm_f32.cu)
        float blk[4][4], blu[SWIGLU ? 4 : 1][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                blk[i][j] = 0.f;
                if (SWIGLU) blu[i][j] = 0.f;
            }
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            float a[4], w[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = Ws[kk][tn + j];
                if (SWIGLU) u[j] = Us[kk][tn + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    blk[i][j] = fmaf(a[i], w[j], blk[i][j]);
                    if (SWIGLU) blu[i][j] = fmaf(a[i], u[j], blu[i][j]);
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[i][j] += blk[i][j];
                if (SWIGLU) acu[i][j] += blu[i][j];
            }
        __syncthreads();
    }
    float* C = (float*)p.C + p.c_group_cols * g;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int lr = row0 + tm + i;
        if (lr >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tn + j;
            if (gn < p.N) C[(int64_t)lr * p.ldc + gn] = SWIGLU ? silu_f(acc[i][j]) * acu[i][j] : acc[i][j];
        }
    }
}

}  // namespace

// A: activations (dtype), rows lda apart.  W (and W2 with swiglu == 1): [G][N, K], groups w_group_stride elements apart,
// rows ldw apart; swiglu == 2: W is [G][2N, K] with gate and up rows alternating in runs of 8 (W2 unused, N a multiple
// of 8).  C: rows ldc apart.  seg == null: uniform groups of M rows each; else the list has M rows in all.
IMP_API int imp_grouped_gemm(void* C, int64_t ldc, int64_t c_group_cols, const void* A, int64_t lda, int64_t a_group_cols,
                             const int* a_rows, const void* W, const void* W2, int64_t w_group_stride, int64_t ldw, const int* seg,
                             int M, int N, int K, int G, int swiglu, int dtype, void* stream) {
    if (M == 0 || N == 0 || G == 0) return 0;
    IMP_CHECK_ARG(C && A && W && M > 0 && N > 0 && K > 0 && G > 0, "imp_grouped_gemm: bad argument");
    IMP_CHECK_ARG(swiglu != 1 || W2, "imp_grouped_gemm: the gated epilogue needs a second weight");
    IMP_CHECK_ARG(swiglu != 2 || N % 8 == 0, "imp_grouped_gemm: interleaved gate and up rows come in runs of 8");
    GroupedArgs p;
    p.A = A, p.lda = lda, p.a_rows = a_rows, p.a_group_cols = a_group_cols;
    p.W = W, p.W2 = W2, p.w_group_stride = w_group_stride, p.ldw = ldw;
    p.C = C, p.ldc = ldc, p.c_group_cols = c_group_cols, p.seg = seg;
    p.M = M, p.N = N, p.K = K, p.G = G;
    p.il = swiglu == 2 ? 1 : 0;
    const int el = dtype == IMP_F32 ? 4 : 2, per16 = 16 / el;
    auto aligned = [&](const void* q) { return q == nullptr || (uintptr_t)q % 16 == 0; };
    p.vec = (K % per16 == 0 && lda % per16 == 0 && ldw % per16 == 0 && a_group_cols % per16 == 0 && w_group_stride % per16 == 0 &&
             aligned(A) && aligned(W) && aligned(W2))
                ? 1
                : 0;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    // few rows a group (a decode step's experts, its per-head products): 16-row tiles
    const int bm = (dtype != IMP_F32 && (seg ? M / G : M) < 16) ? 16 : GG_BM;
    const int row_tiles = seg ? (M + bm - 1) / bm + G : (M + bm - 1) / bm;
    IMP_CHECK_ARG(row_tiles <= 65535 && G <= 65535, "imp_grouped_gemm: too many row tiles or groups for one launch");
    const dim3 grid((N + GG_BN - 1) / GG_BN, row_tiles, seg ? 1 : G);
    if (dtype == IMP_F32) {
        e = swiglu ? imp_launch(grouped_gemm_f32_kernel<true>, grid, dim3(256), 0, s, p) : imp_launch(grouped_gemm_f32_kernel<false>, grid, dim3(256), 0, s, p);
    } else {
        static bool raised = false;
        if (!raised) {
            cudaFuncSetAttribute(grouped_gemm_bf16_kernel<true, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GroupedTile<true, 64>::SMEM);
            cudaFuncSetAttribute(grouped_gemm_bf16_kernel<false, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GroupedTile<false, 64>::SMEM);
            cudaFuncSetAttribute(grouped_gemm_bf16_kernel<true, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GroupedTile<true, 16>::SMEM);
            cudaFuncSetAttribute(grouped_gemm_bf16_kernel<false, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GroupedTile<false, 16>::SMEM);
            raised = true;
        }
        if (bm == 16)
            e = swiglu ? imp_launch(grouped_gemm_bf16_kernel<true, 16>, grid, dim3(128), GroupedTile<true, 16>::SMEM, s, p)
                       : imp_launch(grouped_gemm_bf16_kernel<false, 16>, grid, dim3(128), GroupedTile<false, 16>::SMEM, s, p);
        else
            e = swiglu ? imp_launch(grouped_gemm_bf16_kernel<true, 64>, grid, dim3(128), GroupedTile<true, 64>::SMEM, s, p)
                       : imp_launch(grouped_gemm_bf16_kernel<false, 64>, grid, dim3(128), GroupedTile<false, 64>::SMEM, s, p);
    }
    if (e != cudaSuccess) {
        imp_set_error("imp_grouped_gemm: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// dst[g][c][r] = src[g][r][c]: per-group transposes of small weight matrices, at load time.
template <typename T> __global__ void transpose_groups_kernel(T* __restrict__ dst, const T* __restrict__ src, int R, int Cn) {
    const int64_t base = (int64_t)blockIdx.y * R * Cn;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < (int64_t)R * Cn; i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / Cn), c = (int)(i % Cn);
        dst[base + (int64_t)c * R + r] = src[base + i];
    }
}

IMP_API int imp_transpose_groups(void* dst, const void* src, int G, int R, int Cn, int dtype, void* stream) {
    if (G == 0 || R == 0 || Cn == 0) return 0;
    IMP_CHECK_ARG(dst && src && G > 0 && R > 0 && Cn > 0 && G <= 65535, "imp_transpose_groups: bad argument");
    const dim3 grid((unsigned)std::min<int64_t>(((int64_t)R * Cn + 255) / 256, 1024), G);
    if (dtype == IMP_F32)
        transpose_groups_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((float*)dst, (const float*)src, R, Cn);
    else
        transpose_groups_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, R, Cn);
    IMP_RETURN_LAUNCH();
}
