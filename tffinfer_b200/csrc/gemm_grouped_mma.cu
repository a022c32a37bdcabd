// The grouped product of gemm_grouped.cu for bfloat16 operands on the tensor cores (mma.sync m16n8k16, float32
// accumulation): C_g[m, n] = sum_k A_g[m, k] * B_g[n, k], uniform or ragged groups, optional row map, as there.
// Tiles of 128 x 128 x 64, eight warps of 32 x 64, operands through a three-stage cp.async ring into padded shared
// memory (rows of 144 bytes: the eight rows of an ldmatrix fall into different banks), fragments by ldmatrix.
// Gated form: B_g holds the gate and up rows of a group alternating in blocks of 64 ([g0..g63 | u0..u63 | g64.. ], the
// layout of the tcgen05 products), a tile of 128 rows of B being one such pair of blocks; a warp then takes 32 gate
// rows and the 32 up rows of the same outputs, so that a thread finds act(gate) and up of an output element four
// accumulator tiles apart; C_g[m, f] = act(gate_f) * up_f has half as many columns as B_g has rows.
// Needs K, lda, ldb and the group strides to be multiples of 8 elements and 16-byte aligned bases (the launcher
// refuses anything else and the caller takes the FMA kernel).  A row's result does not depend on the tile it is in:
// every output element adds its products in the same order of k.
#include "common.cuh"

namespace {

constexpr int MBM = 128, MBN = 128, MBK = 64, LDS = MBK + 8, STAGES = 3, THREADS = 256;
constexpr int CHUNKS = MBK / 8;                          // 16-byte pieces of a tile row
constexpr int SMEM_BYTES = STAGES * (MBM + MBN) * LDS * 2;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float act_of(float g, int act) {
    if (act == 0) return g / (1.0f + expf(-g));
    const float c = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(c));
}

template <typename TCc, bool GATED>
__global__ void __launch_bounds__(THREADS, 2)
gemm_grouped_mma_kernel(const bf16* __restrict__ A, long long lda, long long a_gs,
                        const bf16* __restrict__ B, long long ldb, long long b_gs,
                        TCc* __restrict__ C, long long ldc, long long c_gs,
                        const int* __restrict__ tile_group, const int* __restrict__ tile_row0,
                        const int* __restrict__ tile_row_end, const int* __restrict__ num_tiles,
                        const int* __restrict__ row_map, int M, int N, int K, int act) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* As = (bf16*)smem_raw;                               // [STAGES][MBM][LDS]
    bf16* Bs = As + STAGES * MBM * LDS;                       // [STAGES][MBN][LDS]
    pdl_launch_dependents();
    pdl_wait();
    int g, m0, m_end;
    if (tile_group != nullptr) {
        if ((int)blockIdx.y >= *num_tiles) return;
        g = tile_group[blockIdx.y]; m0 = tile_row0[blockIdx.y]; m_end = tile_row_end[blockIdx.y];
    } else {
        g = blockIdx.z; m0 = blockIdx.y * MBM; m_end = M;
    }
    const int n0 = blockIdx.x * MBN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 1, wn = warp & 1;                  // 4 x 2 warps of 32 x 64
    const bf16* Ag = A + (size_t)g * a_gs;
    const bf16* Bg = B + (size_t)g * b_gs;
    const int kt = (K + MBK - 1) / MBK;

    auto load_stage = [&](int s, int k0) {
#pragma unroll
        for (int i = 0; i < MBM * CHUNKS / THREADS; ++i) {
            const int c = tid + i * THREADS, r = c / CHUNKS, kc = (c % CHUNKS) * 8;
            const bool ka = k0 + kc < K;
            const bool oka = ka && (m0 + r < m_end);
            cp_async16(smem_addr(As + ((size_t)s * MBM + r) * LDS + kc),
                       oka ? (const void*)(Ag + (size_t)(m0 + r) * lda + k0 + kc) : (const void*)Ag, oka ? 16 : 0);
            const bool okb = ka && (n0 + r < N);
            cp_async16(smem_addr(Bs + ((size_t)s * MBN + r) * LDS + kc),
                       okb ? (const void*)(Bg + (size_t)(n0 + r) * ldb + k0 + kc) : (const void*)Bg, okb ? 16 : 0);
        }
    };

    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < kt) load_stage(s, s * MBK);
        cp_commit();
    }
    for (int kb = 0; kb < kt; ++kb) {
        cp_wait<STAGES - 2>();
        __syncthreads();
        const int nk = kb + STAGES - 1;
        if (nk < kt) load_stage(nk % STAGES, nk * MBK);
        cp_commit();
        const bf16* as = As + (size_t)(kb % STAGES) * MBM * LDS;
        const bf16* bs = Bs + (size_t)(kb % STAGES) * MBN * LDS;
#pragma unroll
        for (int kk = 0; kk < MBK; kk += 16) {
            uint32_t a[2][4], b[4][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
                ldsm4(a[mi], smem_addr(as + (size_t)(wm * 32 + mi * 16 + (lane & 15)) * LDS + kk + (lane >> 4) * 8));
#pragma unroll
            for (int nj = 0; nj < 4; ++nj) {
                // rows of B this warp's 16-row slice nj covers: plain 64 in a row; gated 32 gate rows, then their 32 up rows
                const int brow = GATED ? ((nj >> 1) * 64 + wn * 32 + (nj & 1) * 16) : (wn * 64 + nj * 16);
                ldsm4(b[nj], smem_addr(bs + (size_t)(brow + (lane & 7) + (lane >> 4) * 8) * LDS + kk + ((lane >> 3) & 1) * 8));
            }
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int nj = 0; nj < 4; ++nj) {
                    mma16816(acc[mi][2 * nj], a[mi], b[nj][0], b[nj][1]);
                    mma16816(acc[mi][2 * nj + 1], a[mi], b[nj][2], b[nj][3]);
                }
        }
    }
    cp_wait<0>();

#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m0 + wm * 32 + mi * 16 + (lane >> 2) + half * 8;
            if (m >= m_end) continue;
            const long long row = row_map ? row_map[m] : m;
            TCc* crow = C + (size_t)g * c_gs + (size_t)row * ldc;
            if constexpr (GATED) {
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int f = n0 / 2 + wn * 32 + t * 8 + 2 * (lane & 3);
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        if (f + e < N / 2)
                            crow[f + e] = from_f32<TCc>(act_of(acc[mi][t][half * 2 + e], act) * acc[mi][t + 4][half * 2 + e]);
                }
            } else {
#pragma unroll
                for (int nj = 0; nj < 8; ++nj) {
                    const int n = n0 + wn * 64 + nj * 8 + 2 * (lane & 3);
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        if (n + e < N) {
                            float v = acc[mi][nj][half * 2 + e];
                            if (act == 2) { v = fmaxf(v, 0.f); v = v * v; }     // the square of relu behind a plain product
                            crow[n + e] = from_f32<TCc>(v);
                        }
                }
            }
        }
}

}  // namespace

// A and B bfloat16.  gated != 0: B's N rows are gate and up rows alternating in blocks of 64 and C has N / 2 columns.
// c_dt 0 = float32, 1 = bfloat16.  The ragged form's tiles must have been planned with tff_gemm_grouped_mma_tile_rows().
TFF_API int tff_gemm_grouped_mma(
    const void* A, long long lda, long long a_gs, const void* B, long long ldb, long long b_gs,
    void* C, int c_dt, long long ldc, long long c_gs,
    const int* tile_group, const int* tile_row0, const int* tile_row_end, const int* num_tiles, int max_tiles,
    const int* row_map, int groups, int M, int N, int K, int gated, int act, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || !A || !B || !C) return TFF_ERR_BAD_ARGUMENT;
    if ((K & 7) || (lda & 7) || (ldb & 7) || (a_gs & 7) || (b_gs & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) ||
        (gated && (N & 127)))
        return TFF_ERR_UNSUPPORTED;
    dim3 grid;
    if (tile_group) {
        if (!tile_row0 || !tile_row_end || !num_tiles) return TFF_ERR_BAD_ARGUMENT;
        if (max_tiles <= 0) return TFF_OK;
        grid = dim3((N + MBN - 1) / MBN, max_tiles, 1);
    } else {
        if (M <= 0 || groups <= 0) return TFF_OK;
        if (groups > 65535) return TFF_ERR_UNSUPPORTED;
        grid = dim3((N + MBN - 1) / MBN, (M + MBM - 1) / MBM, groups);
    }
    if (grid.y > 65535) return TFF_ERR_UNSUPPORTED;
#define TFF_GM(TCc, G)                                                                                              \
    do {                                                                                                            \
        cudaFuncSetAttribute(gemm_grouped_mma_kernel<TCc, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); \
        return tff_launch_pdl(gemm_grouped_mma_kernel<TCc, G>, grid, dim3(THREADS), (size_t)SMEM_BYTES, stream,     \
                              (const bf16*)A, lda, a_gs, (const bf16*)B, ldb, b_gs, (TCc*)C, ldc, c_gs, tile_group, \
                              tile_row0, tile_row_end, num_tiles, row_map, M, N, K, act);                           \
    } while (0)
    if (c_dt == 0 && gated) TFF_GM(float, true);
    if (c_dt == 0) TFF_GM(float, false);
    if (c_dt == 1 && gated) TFF_GM(bf16, true);
    if (c_dt == 1) TFF_GM(bf16, false);
#undef TFF_GM
    return TFF_ERR_BAD_ARGUMENT;
}

TFF_API int tff_gemm_grouped_mma_tile_rows() { return MBM; }
