// Many small matrix products in one launch, accumulated in float32 with plain FMAs:
//   C_g[m, n] = sum_k A_g[m, k] * B_g[n, k]                      (plain)
//   C_g[m, n] = act(sum_k A_g[m, k] * B_g[n, k]) * sum_k A_g[m, k] * B2_g[n, k]      (gated; act silu or tanh-gelu)
// Two ways of saying which rows belong to which group g:
// * uniform: every group has the same M rows; group g's operands start a_gs, b_gs and c_gs elements after group
//   g-1's (a per-head projection reads column block g of a [T, heads * k] activation: a_gs = k, lda = heads * k);
// * ragged: the rows of A are sorted by group (the tokens of a routed feed-forward, sorted by expert); a table made
//   on the device says, tile by tile, which group the tile belongs to and which rows it covers, and
//   ``num_tiles`` how many tiles there are (the grid is sized for the most there can be).  ``row_map`` (optional)
//   sends row r of the product to row row_map[r] of C.
// Every output element adds its K products in the order k = 0 .. K-1, so a row's result depends neither on the
// tile it falls in nor on what else is in the batch.  Operands may be float32 or bfloat16 in any mix.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

__device__ __forceinline__ float act_apply(float g, int act) {
    if (act == 0) return g / (1.0f + expf(-g));
    const float c = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(c));
}

template <typename TA, typename TB, typename TCc, bool GATED>
__global__ void __launch_bounds__(256)
gemm_grouped_kernel(const TA* __restrict__ A, long long lda, long long a_gs,
                    const TB* __restrict__ B, const TB* __restrict__ B2, long long ldb, long long b_gs,
                    TCc* __restrict__ C, long long ldc, long long c_gs,
                    const int* __restrict__ tile_group, const int* __restrict__ tile_row0,
                    const int* __restrict__ tile_row_end, const int* __restrict__ num_tiles,
                    const int* __restrict__ row_map, int M, int N, int K, int act, int b_interleaved) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    __shared__ float Bs2[GATED ? BK : 1][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    int g, m0, m_end;
    if (tile_group != nullptr) {
        if ((int)blockIdx.y >= *num_tiles) return;
        g = tile_group[blockIdx.y]; m0 = tile_row0[blockIdx.y]; m_end = tile_row_end[blockIdx.y];
    } else {
        g = blockIdx.z; m0 = blockIdx.y * BM; m_end = M;
    }
    const int n0 = blockIdx.x * BN;
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const TA* Ag = A + (size_t)g * a_gs;
    const TB* Bg = B + (size_t)g * b_gs;
    const TB* B2g = GATED ? B2 + (size_t)g * b_gs : nullptr;
    float acc[TM][TN], acc2[GATED ? TM : 1][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) { acc[i][j] = 0.f; if constexpr (GATED) acc2[i][j] = 0.f; }

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int gk = k0 + kk;
            float a = 0.f, w = 0.f, w2 = 0.f;
            if (gk < K) {
                if (m0 + r < m_end) a = to_f32<TA>(Ag[(size_t)(m0 + r) * lda + gk]);
                if (n0 + r < N) {
                    // gate and up alternating in blocks of b_interleaved rows: output column n has its gate row at
                    // (n / blk) * 2 blk + n % blk and its up row blk further (B2 = B + blk rows)
                    const int n = n0 + r;
                    const size_t brow = b_interleaved ? (size_t)(n / b_interleaved) * 2 * b_interleaved + (n % b_interleaved) : (size_t)n;
                    w = to_f32<TB>(Bg[brow * ldb + gk]);
                    if constexpr (GATED) w2 = to_f32<TB>(B2g[brow * ldb + gk]);
                }
            }
            As[kk][r] = a;
            Bs[kk][r] = w;
            if constexpr (GATED) Bs2[kk][r] = w2;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN], w2[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) { w[j] = Bs[kk][tx * TN + j]; if constexpr (GATED) w2[j] = Bs2[kk][tx * TN + j]; }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if constexpr (GATED) acc2[i][j] = fmaf(a[i], w2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= m_end) continue;
        const long long row = row_map ? row_map[m] : m;
        TCc* crow = C + (size_t)g * c_gs + (size_t)row * ldc;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if constexpr (GATED) v = act_apply(v, act) * acc2[i][j];
            else if (act == 2) { v = fmaxf(v, 0.f); v = v * v; }     // a plain product with the square of relu behind it
            crow[n] = from_f32<TCc>(v);
        }
    }
}

}  // namespace

// dt codes: 0 = float32, 1 = bfloat16.  B2 null = plain product (``act`` 2: relu(.)^2 of it; else as it is); else gated
// with ``act`` (0 silu, 1 tanh-gelu).
// b_interleaved (gated only) > 0: the gate and up rows of a group alternate in blocks of that many rows in ONE matrix
// (B2 = B + that many rows); 0: B and B2 are matrices of their own.
// Uniform: tile_group null, ``groups`` groups of M rows.  Ragged: the four tile arrays on the device, ``max_tiles`` the
// grid's size, M unused, c_gs and a_gs usually 0.
TFF_API int tff_gemm_grouped(
    const void* A, int a_dt, long long lda, long long a_gs,
    const void* B, const void* B2, int b_dt, long long ldb, long long b_gs,
    void* C, int c_dt, long long ldc, long long c_gs,
    const int* tile_group, const int* tile_row0, const int* tile_row_end, const int* num_tiles, int max_tiles,
    const int* row_map, int groups, int M, int N, int K, int act, int b_interleaved, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || !A || !B || !C) return TFF_ERR_BAD_ARGUMENT;
    dim3 grid;
    if (tile_group) {
        if (!tile_row0 || !tile_row_end || !num_tiles) return TFF_ERR_BAD_ARGUMENT;
        if (max_tiles <= 0) return TFF_OK;
        grid = dim3((N + BN - 1) / BN, max_tiles, 1);
    } else {
        if (M <= 0 || groups <= 0) return TFF_OK;
        if (groups > 65535) return TFF_ERR_UNSUPPORTED;
        grid = dim3((N + BN - 1) / BN, (M + BM - 1) / BM, groups);
    }
    if (grid.y > 65535) return TFF_ERR_UNSUPPORTED;
#define TFF_GG(TA, TB, TCc)                                                                                          \
    do {                                                                                                             \
        if (B2)                                                                                                      \
            return tff_launch_pdl(gemm_grouped_kernel<TA, TB, TCc, true>, grid, dim3(256), 0, stream, (const TA*)A, lda, a_gs, \
                                  (const TB*)B, (const TB*)B2, ldb, b_gs, (TCc*)C, ldc, c_gs, tile_group, tile_row0,   \
                                  tile_row_end, num_tiles, row_map, M, N, K, act, b_interleaved);                                   \
        return tff_launch_pdl(gemm_grouped_kernel<TA, TB, TCc, false>, grid, dim3(256), 0, stream, (const TA*)A, lda, a_gs,   \
                              (const TB*)B, (const TB*)nullptr, ldb, b_gs, (TCc*)C, ldc, c_gs, tile_group, tile_row0, \
                              tile_row_end, num_tiles, row_map, M, N, K, act, b_interleaved);                                       \
    } while (0)
    if (a_dt == 0 && b_dt == 0 && c_dt == 0) TFF_GG(float, float, float);
    if (a_dt == 0 && b_dt == 1 && c_dt == 0) TFF_GG(float, bf16, float);
    if (a_dt == 0 && b_dt == 1 && c_dt == 1) TFF_GG(float, bf16, bf16);
    if (a_dt == 1 && b_dt == 1 && c_dt == 1) TFF_GG(bf16, bf16, bf16);
    if (a_dt == 1 && b_dt == 1 && c_dt == 0) TFF_GG(bf16, bf16, float);
    if (a_dt == 1 && b_dt == 0 && c_dt == 0) TFF_GG(bf16, float, float);
    if (a_dt == 0 && b_dt == 0 && c_dt == 1) TFF_GG(float, float, bf16);
    if (a_dt == 1 && b_dt == 0 && c_dt == 1) TFF_GG(bf16, float, bf16);
#undef TFF_GG
    return TFF_ERR_BAD_ARGUMENT;
}

// Rows a tile of the ragged form covers: the planner of a routed feed-forward cuts each group's rows into tiles of this many.
TFF_API int tff_gemm_grouped_tile_rows() { return BM; }
