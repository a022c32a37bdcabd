// Softmax attention over the paged cache for tiles of packed query rows, computed in float32 with plain FMAs, for
// the geometries and score rules the tensor-core kernels do not take:
//
// * keys of d and values of dv elements, any sizes (d, dv <= 1024 as far as shared memory reaches);
// * values in a plane of their own (cache [pages, layers, 2, kv heads, page, slot]) or, in a cache of ONE plane
//   ([pages, layers, 1, kv heads, page, slot]), the value of a token being the first dv elements of its key: a
//   latent attention, where every query head reads the same small vector per token;
// * visibility: causal, and optionally a sliding window (keys p-window+1 .. p) and/or blocks of ``chunk``
//   positions counted from position 0 of the sequence (key n is seen from p only if n / chunk == p / chunk);
// * score(p, n) = (q . k_n) * scale * temp[h]  -  r1[h] * ln(1 + r2[h] * (p - n)), with per-head float32 arrays temp
//   (null: 1) and r1, r2 (null: no distance term); with ``softcap`` > 0 the scaled product is first squashed to
//   softcap * tanh(. / softcap);
// * the output is multiplied by out_scale and may go to a column block of a wider row (out_ld, out_off).
//
// A tile is ROWS packed rows of one request and one key/value head: row r of the request is (token r / G, query head
// r % G of the G heads that share the key/value head).  Key blocks of KB keys are aligned to absolute positions and a
// row's running maximum and sum only ever see its own visible keys, so a row's result does not depend on the tile it
// is in, on how the prompt was cut or on what else is in the batch.  Keys outside the tile's range are never read
// (pages behind a window may have been given back).
#include "common.cuh"
#include "attention_common.h"
#include <stdlib.h>

namespace {

constexpr int ROWS = 32, KB = 32, THREADS = 256;

struct TileArgs {
    const int* q_start; const int* pos_start; const int* block_table; int table_width;
    long long page_stride, head_stride, v_offset;   // elements; v_offset from a key's slot to the value's (0: the key itself)
    int slot, page_size;
    int nq, nkv, d, dv;
    float scale; int window, chunk;
    float softcap;                                  // > 0: a scaled score s becomes softcap * tanh(s / softcap)
    const float* temp; const float* r1; const float* r2;
    float out_scale; int q_ld, out_ld, out_off;
    int splits; float* part_o; float* part_ml;     // splits > 1: shares of the key range, merged by a second kernel
    // Keys and values of THIS step's tokens in plain rows instead of the cache (tensor-core form only; every request of the
    // step must start at position 0): key n of a request is row q_start + n, head h at columns h*d (values: h*dv).
    const void* k_dense; const void* v_dense; int k_ld, v_ld;
};

template <typename TQ, typename TC, int NC>
__global__ void __launch_bounds__(THREADS)
attention_tile_kernel(const TQ* __restrict__ q, const TC* __restrict__ cache, TQ* __restrict__ out, TileArgs a) {
    extern __shared__ float sm[];
    const int d = a.d, dv = a.dv, G = a.nq / a.nkv;
    const int kstride = d + 1;                                  // odd: lanes that read one column of 16 keys hit 16 banks
    const bool own_v = a.v_offset != 0;
    float* Qs = sm;                                             // [ROWS][d]
    float* Ks = Qs + ROWS * d;                                  // [KB][d + 1]
    float* Vs = Ks + KB * kstride;                              // [KB][dv] when values have a plane of their own
    float* Ps = Vs + (own_v ? KB * dv : 0);                     // [ROWS][KB + 1]
    float* alpha_s = Ps + ROWS * (KB + 1);                      // [ROWS]
    int* row_p = (int*)(alpha_s + ROWS);                        // [ROWS] position, -1 = no such row
    int* row_lo = row_p + ROWS;                                 // [ROWS] first visible key

    pdl_launch_dependents();
    const int b = blockIdx.z, kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = a.q_start[b], q_len = a.q_start[b + 1] - t0, pos0 = a.pos_start[b];
    const int split = blockIdx.x % a.splits;
    const int n_rows = q_len * G, r0 = (blockIdx.x / a.splits) * ROWS;
    if (r0 >= n_rows) return;
    pdl_wait();

    if (tid < ROWS) {
        const int r = r0 + tid;
        int p = -1, lo = 0;
        if (r < n_rows) {
            p = pos0 + r / G;
            if (a.window > 0) lo = max(lo, p - a.window + 1);
            if (a.chunk > 0) lo = max(lo, (p / a.chunk) * a.chunk);
        }
        row_p[tid] = p; row_lo[tid] = lo;
    }
    for (int idx = tid; idx < ROWS * d; idx += THREADS) {
        const int rr = idx / d, i = idx % d, r = r0 + rr;
        float v = 0.f;
        if (r < n_rows) v = to_f32<TQ>(q[(size_t)(t0 + r / G) * a.q_ld + (size_t)(kvh * G + r % G) * d + i]);
        Qs[idx] = v;
    }
    __syncthreads();
    const int last = min(r0 + ROWS, n_rows) - 1;
    const int p_max = pos0 + last / G;
    const int lo_min = row_lo[0];                               // positions rise with the row, and so do the lower ends

    // score phase: thread -> rows 2*ry, 2*ry+1 and keys kx, kx+16;  value phase: the same rows, columns cx + 16*j
    const int ry = tid >> 4, kx = tid & 15, cx = kx;
    const int ra = 2 * ry, rb = 2 * ry + 1;
    const int pa = row_p[ra], pb = row_p[rb], la = row_lo[ra], lb = row_lo[rb];
    const int ha = kvh * G + (r0 + ra) % G, hb = kvh * G + (r0 + rb) % G;
    const float sa = a.scale * (a.temp ? a.temp[ha] : 1.f), sb = a.scale * (a.temp ? a.temp[hb] : 1.f);
    const bool biased = a.r1 != nullptr;
    const float r1a = biased ? a.r1[ha] : 0.f, r2a = biased ? a.r2[ha] : 0.f;
    const float r1b = biased ? a.r1[hb] : 0.f, r2b = biased ? a.r2[hb] : 0.f;
    float oa[NC], ob[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) { oa[j] = 0.f; ob[j] = 0.f; }
    // softmax phase: warp w owns rows 4w .. 4w+3, lane = key of the block
    float m_run[4], l_run[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }
    const int* table = a.block_table + (size_t)b * a.table_width;

    // the tile's key blocks, in equal contiguous shares when the key range is cut (a share may be empty)
    const int kb_first = lo_min / KB, kb_count = p_max / KB - kb_first + 1;
    const int kb_lo = kb_first + (int)((long long)kb_count * split / a.splits);
    const int kb_hi = kb_first + (int)((long long)kb_count * (split + 1) / a.splits);
    for (int k0 = kb_lo * KB; k0 < kb_hi * KB; k0 += KB) {
        // the block's keys (and values) into shared memory as float32; keys outside [lo_min, p_max] are zeros
        for (int kk = warp; kk < KB; kk += THREADS / 32) {
            const int n = k0 + kk;
            const TC* src = nullptr;
            if (n >= lo_min && n <= p_max) {
                const int page = table[n / a.page_size];
                if (page >= 0)
                    src = cache + (size_t)page * a.page_stride + (size_t)kvh * a.head_stride + (size_t)(n % a.page_size) * a.slot;
            }
            for (int i = lane; i < d; i += 32) Ks[kk * kstride + i] = src ? to_f32<TC>(src[i]) : 0.f;
            if (own_v)
                for (int i = lane; i < dv; i += 32) Vs[kk * dv + i] = src ? to_f32<TC>(src[a.v_offset + i]) : 0.f;
        }
        __syncthreads();
        {
            float s00 = 0.f, s01 = 0.f, s10 = 0.f, s11 = 0.f;
            const float* qa = Qs + ra * d; const float* qb = Qs + rb * d;
            const float* ka = Ks + kx * kstride; const float* kb = Ks + (kx + 16) * kstride;
            if (pa >= 0) {                                      // rows rise in pairs: no first row, no second either
#pragma unroll 4
                for (int i = 0; i < d; ++i) {
                    const float x0 = qa[i], x1 = qb[i], y0 = ka[i], y1 = kb[i];
                    s00 = fmaf(x0, y0, s00); s01 = fmaf(x0, y1, s01);
                    s10 = fmaf(x1, y0, s10); s11 = fmaf(x1, y1, s11);
                }
            }
            const int n0 = k0 + kx, n1 = k0 + kx + 16;
            auto score = [&](float dot, float sc, float r1, float r2, int p, int lo, int n) -> float {
                if (p < 0 || n > p || n < lo) return -INFINITY;
                float s = dot * sc;
                if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
                if (biased) s -= r1 * log1pf(r2 * (float)(p - n));
                return s;
            };
            Ps[ra * (KB + 1) + kx] = score(s00, sa, r1a, r2a, pa, la, n0);
            Ps[ra * (KB + 1) + kx + 16] = score(s01, sa, r1a, r2a, pa, la, n1);
            Ps[rb * (KB + 1) + kx] = score(s10, sb, r1b, r2b, pb, lb, n0);
            Ps[rb * (KB + 1) + kx + 16] = score(s11, sb, r1b, r2b, pb, lb, n1);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rr = warp * 4 + i;
            const float s = Ps[rr * (KB + 1) + lane];
            const float m_new = fmaxf(m_run[i], warp_max(s));
            float alpha = 1.f, pr = 0.f;
            if (m_new != -INFINITY) {
                alpha = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_new);
                pr = expf(s - m_new);                           // -inf - finite = -inf -> 0
            }
            l_run[i] = l_run[i] * alpha + warp_sum(pr);
            m_run[i] = m_new;
            Ps[rr * (KB + 1) + lane] = pr;
            if (lane == 0) alpha_s[rr] = alpha;
        }
        __syncthreads();
        {
            const float al_a = alpha_s[ra], al_b = alpha_s[rb];
#pragma unroll
            for (int j = 0; j < NC; ++j) { oa[j] *= al_a; ob[j] *= al_b; }
            const float* vbase = own_v ? Vs : Ks;
            const int vstride = own_v ? dv : kstride;
            for (int kk = 0; kk < KB && pa >= 0; ++kk) {
                const float p0 = Ps[ra * (KB + 1) + kk], p1 = Ps[rb * (KB + 1) + kk];
                const float* v = vbase + kk * vstride;
#pragma unroll
                for (int j = 0; j < NC; ++j) {
                    const int c = cx + 16 * j;
                    if (c < dv) {
                        const float x = v[c];
                        oa[j] = fmaf(p0, x, oa[j]); ob[j] = fmaf(p1, x, ob[j]);
                    }
                }
            }
        }
        __syncthreads();
    }
    // the rows' sums (and maxima) live in the softmax warps: hand them over through shared memory
    float* m_s = Ps;                                            // the scores' buffer is free now
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (lane == 0) { alpha_s[warp * 4 + i] = l_run[i]; m_s[warp * 4 + i] = m_run[i]; }
    __syncthreads();
#pragma unroll
    for (int side = 0; side < 2; ++side) {
        const int rr = side ? rb : ra, r = r0 + rr;
        if (r >= n_rows) continue;
        const int t = t0 + r / G, h = kvh * G + r % G;
        if (a.splits == 1) {
            const float inv = a.out_scale / alpha_s[rr];
            TQ* orow = out + (size_t)t * a.out_ld + a.out_off + (size_t)h * dv;
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const int c = cx + 16 * j;
                if (c < dv) orow[c] = from_f32<TQ>((side ? ob[j] : oa[j]) * inv);
            }
        } else {                                                // this share's unnormalised sums, its maximum and its sum
            const size_t slot = ((size_t)t * a.nq + h) * a.splits + split;
            float* prow = a.part_o + slot * dv;
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const int c = cx + 16 * j;
                if (c < dv) prow[c] = side ? ob[j] : oa[j];
            }
            if (cx == 0) { a.part_ml[2 * slot] = m_s[rr]; a.part_ml[2 * slot + 1] = alpha_s[rr]; }
        }
    }
}

// out[t, h] = out_scale * sum_s w_s o_s / sum_s w_s l_s with w_s = exp(m_s - max m): one warp per (token, head)
template <typename TQ>
__global__ void __launch_bounds__(128)
attention_tile_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, TQ* __restrict__ out,
                            int out_ld, int out_off, long long rows, int nq, int dv, int splits, float out_scale) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 4 + warp;
    if (row >= rows) return;
    pdl_wait();
    const float* ml = part_ml + (size_t)row * splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, ml[2 * s]);
    float L = 0.f;
    for (int s = 0; s < splits; ++s) L += (ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - M)) * ml[2 * s + 1];
    const float inv = out_scale / L;
    TQ* orow = out + (size_t)(row / nq) * out_ld + out_off + (size_t)(row % nq) * dv;
    for (int c = lane; c < dv; c += 32) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float w = ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - M);
            if (w != 0.f) acc = fmaf(w, part_o[((size_t)row * splits + s) * dv + c], acc);
        }
        orow[c] = from_f32<TQ>(acc * inv);
    }
}

template <typename TQ, typename TC>
int launch_tile(const void* q, const void* cache, void* out, const TileArgs& a, int num_requests, int max_q_len,
                int num_tokens, cudaStream_t stream) {
    const int G = a.nq / a.nkv;
    const int tiles = (max_q_len * G + ROWS - 1) / ROWS;
    if (num_requests > 65535 || a.nkv > 65535) return TFF_ERR_UNSUPPORTED;
    const bool own_v = a.v_offset != 0;
    const size_t smem = sizeof(float) * ((size_t)ROWS * a.d + (size_t)KB * (a.d + 1) + (own_v ? (size_t)KB * a.dv : 0) +
                                         (size_t)ROWS * (KB + 1) + ROWS) + sizeof(int) * 2 * ROWS;
    if (smem > 220 * 1024) return TFF_ERR_UNSUPPORTED;
    dim3 grid(tiles * a.splits, a.nkv, num_requests);
#define TFF_TILE(NCV)                                                                                                \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(attention_tile_kernel<TQ, TC, NCV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        const int st = tff_launch_pdl(attention_tile_kernel<TQ, TC, NCV>, grid, dim3(THREADS), smem, stream, (const TQ*)q, \
                                      (const TC*)cache, (TQ*)out, a);                                                \
        if (st != TFF_OK || a.splits == 1) return st;                                                                \
        const long long rows = (long long)num_tokens * a.nq;                                                         \
        return tff_launch_pdl(attention_tile_merge_kernel<TQ>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream, \
                              (const float*)a.part_o, (const float*)a.part_ml, (TQ*)out, a.out_ld, a.out_off, rows,  \
                              a.nq, a.dv, a.splits, a.out_scale);                                                    \
    } while (0)
    if (a.dv <= 64) TFF_TILE(4);
    if (a.dv <= 128) TFF_TILE(8);
    if (a.dv <= 256) TFF_TILE(16);
    if (a.dv <= 512) TFF_TILE(32);
    if (a.dv <= 1024) TFF_TILE(64);
#undef TFF_TILE
    return TFF_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------------------------------
// The same tiles for bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulation): 64 rows x 64 keys, sixteen
// warps.  Q and the key block lie in shared memory as bfloat16 rows padded by 16 bytes (ldmatrix without bank
// conflicts); S = Q K^T by a 4 x 4 grid of warps (16 rows x 16 keys each) goes to shared memory as float32 with scale,
// distance term and mask applied; the softmax warps (four rows each) keep the running maxima and sums in float32 and
// leave the probabilities as bfloat16; O += P V by a 4 x 4 grid of warps (16 rows x a quarter of the value columns
// each), V read through ldmatrix.trans from the key rows themselves (one plane) or from the value block.  Everything
// the float32 kernel above promises about blocks, masks and shares holds here too.
constexpr int MKB = 64, PST = MKB + 8, SST = MKB + 4;

__device__ __forceinline__ uint32_t sm_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int bytes) {     // bytes 0: sixteen zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct MmaGeom { int dpad, kst, vst; };      // padded key size, elements between key rows and between value rows in shared memory

// RG groups of 16 rows (a tile has 16 * RG rows and 4 * RG warps: steps of one token need one group, portions four);
// a warp of the value phase owns 16 rows x NT * 8 columns
template <int NT, int RG>
__global__ void __launch_bounds__(128 * RG)
attention_tile_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, bf16* __restrict__ out, TileArgs a,
                          MmaGeom gm) {
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr int MROWS = 16 * RG, MTHREADS = 128 * RG;
    const int d = a.d, dv = a.dv, G = a.nq / a.nkv;
    const bool dense = a.k_dense != nullptr;
    const bool own_v = a.v_offset != 0 || dense;
    const int kst = gm.kst, vst = gm.vst, dpad = gm.dpad;
    bf16* Qs = (bf16*)smraw;                                    // [MROWS][kst]
    bf16* Ks = Qs + MROWS * kst;                                // [MKB][kst]
    bf16* Vs = own_v ? Ks + MKB * kst : Ks;                     // [MKB][vst]
    bf16* Pb = own_v ? Vs + MKB * vst : Ks + MKB * kst;         // [MROWS][PST] probabilities
    float* Ss = (float*)(Pb + MROWS * PST);                     // [MROWS][SST] scores
    float* alpha_s = Ss + MROWS * SST;                          // [MROWS]
    float* m_fin = alpha_s + MROWS;                             // [MROWS]
    int* row_p = (int*)(m_fin + MROWS);
    int* row_lo = row_p + MROWS;
    const bf16** key_src = (const bf16**)(row_lo + MROWS);     // [MKB] (8-byte aligned: an even number of 4-byte words lies ahead)
    const bf16** val_src = key_src + MKB;                      // [MKB]

    pdl_launch_dependents();
    const int b = blockIdx.z, kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = a.q_start[b], q_len = a.q_start[b + 1] - t0, pos0 = a.pos_start[b];
    const int split = blockIdx.x % a.splits;
    const int n_rows = q_len * G, r0 = (blockIdx.x / a.splits) * MROWS;
    if (r0 >= n_rows) return;
    pdl_wait();

    if (tid < MROWS) {
        const int r = r0 + tid;
        int p = -1, lo = 0;
        if (r < n_rows) {
            p = pos0 + r / G;
            if (a.window > 0) lo = max(lo, p - a.window + 1);
            if (a.chunk > 0) lo = max(lo, (p / a.chunk) * a.chunk);
        }
        row_p[tid] = p; row_lo[tid] = lo;
    }
    const int dch = dpad / 8;                                   // 16-byte pieces of a padded key
    for (int idx = tid; idx < MROWS * dch; idx += MTHREADS) {
        const int rr = idx / dch, c = (idx % dch) * 8, r = r0 + rr;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < n_rows && c < d) v = *(const uint4*)(q + (size_t)(t0 + r / G) * a.q_ld + (size_t)(kvh * G + r % G) * d + c);
        *(uint4*)(Qs + rr * kst + c) = v;
    }
    __syncthreads();
    const int last = min(r0 + MROWS, n_rows) - 1;
    const int p_max = pos0 + last / G;
    const int lo_min = row_lo[0];

    const int rw = warp % RG, cw = warp / RG;                    // 4 x 4 warps: rows rw*16.., keys cw*16.. / columns cw*NT*8..
    const int fr = lane >> 2, fc = 2 * (lane & 3);              // a thread's place in an accumulator tile: rows fr, fr+8; columns fc, fc+1
    const int ra = rw * 16 + fr, rb = ra + 8;
    const int pa = row_p[ra], pb = row_p[rb], la = row_lo[ra], lb = row_lo[rb];
    const int ha = kvh * G + (r0 + ra) % G, hb = kvh * G + (r0 + rb) % G;
    const float sa = a.scale * (a.temp ? a.temp[ha] : 1.f), sb = a.scale * (a.temp ? a.temp[hb] : 1.f);
    const bool biased = a.r1 != nullptr;
    const float r1a = biased ? a.r1[ha] : 0.f, r2a = biased ? a.r2[ha] : 0.f;
    const float r1b = biased ? a.r1[hb] : 0.f, r2b = biased ? a.r2[hb] : 0.f;
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m_run[4], l_run[4];                                   // softmax phase: warp w owns rows 4w .. 4w+3
#pragma unroll
    for (int i = 0; i < 4; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }
    const int* table = a.block_table + (size_t)b * a.table_width;
    const int vch = own_v ? (vst - 8) / 8 : 0;

    const int kb_first = lo_min / MKB, kb_count = p_max / MKB - kb_first + 1;
    const int kb_lo = kb_first + (int)((long long)kb_count * split / a.splits);
    const int kb_hi = kb_first + (int)((long long)kb_count * (split + 1) / a.splits);
    for (int k0 = kb_lo * MKB; k0 < kb_hi * MKB; k0 += MKB) {
        // where the block's keys lie (one thread a key), then the rows in 16-byte pieces, all loads independent
        if (tid < MKB) {
            const int n = k0 + tid;
            const bf16* src = nullptr;
            const bf16* vsrc = nullptr;
            if (n >= lo_min && n <= p_max) {
                if (dense) {
                    src = (const bf16*)a.k_dense + (size_t)(t0 + n - pos0) * a.k_ld + (size_t)kvh * d;
                    vsrc = (const bf16*)a.v_dense + (size_t)(t0 + n - pos0) * a.v_ld + (size_t)kvh * dv;
                } else {
                    const int page = table[n / a.page_size];
                    if (page >= 0) {
                        src = cache + (size_t)page * a.page_stride + (size_t)kvh * a.head_stride + (size_t)(n % a.page_size) * a.slot;
                        vsrc = src + a.v_offset;
                    }
                }
            }
            key_src[tid] = src;
            val_src[tid] = vsrc;
        }
        __syncthreads();
        // asynchronous 16-byte copies straight into shared memory (zero fill where there is no key or the row has
        // ended): all of a thread's copies are in flight at once
        for (int idx = tid; idx < MKB * dch; idx += MTHREADS) {
            const int kk = idx / dch, c = idx % dch;
            const bf16* src = key_src[kk];
            const bool ok = src && c * 8 < d;
            cp_async_16(sm_addr(Ks + kk * kst + c * 8), ok ? (const void*)(src + c * 8) : (const void*)q, ok ? 16 : 0);
        }
        for (int idx = tid; idx < MKB * vch; idx += MTHREADS) {
            const int kk = idx / vch, c = idx % vch;
            const bf16* src = val_src[kk];
            const bool ok = src && c * 8 < dv;
            cp_async_16(sm_addr(Vs + kk * vst + c * 8), ok ? (const void*)(src + c * 8) : (const void*)q, ok ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        {   // S = Q K^T: rows rw*16 .. +16, keys cw*16 .. +16
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t qa = sm_addr(Qs + (rw * 16 + (lane & 15)) * kst + (lane >> 4) * 8);
            const uint32_t ka = sm_addr(Ks + (cw * 16 + (lane & 7) + (lane >> 4) * 8) * kst + ((lane >> 3) & 1) * 8);
            for (int kk = 0; kk < dpad; kk += 16) {
                uint32_t af[4], bfr[4];
                ldsm4(af, qa + kk * 2);
                ldsm4(bfr, ka + kk * 2);
                mma16816(s0, af, bfr[0], bfr[1]);
                mma16816(s1, af, bfr[2], bfr[3]);
            }
            auto score = [&](float dot, float sc, float r1, float r2, int p, int lo, int n) -> float {
                if (p < 0 || n > p || n < lo) return -INFINITY;
                float s = dot * sc;
                if (a.softcap > 0.f) s = a.softcap * attn_tanh(s / a.softcap);
                if (biased) s -= r1 * log1pf(r2 * (float)(p - n));
                return s;
            };
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c0 = cw * 16 + fc + e, c1 = c0 + 8;
                Ss[ra * SST + c0] = score(s0[e], sa, r1a, r2a, pa, la, k0 + c0);
                Ss[rb * SST + c0] = score(s0[2 + e], sb, r1b, r2b, pb, lb, k0 + c0);
                Ss[ra * SST + c1] = score(s1[e], sa, r1a, r2a, pa, la, k0 + c1);
                Ss[rb * SST + c1] = score(s1[2 + e], sb, r1b, r2b, pb, lb, k0 + c1);
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rr = warp * 4 + i;
            const float x0 = Ss[rr * SST + lane], x1 = Ss[rr * SST + lane + 32];
            const float m_new = fmaxf(m_run[i], warp_max(fmaxf(x0, x1)));
            float alpha = 1.f, p0 = 0.f, p1 = 0.f;
            if (m_new != -INFINITY) {
                alpha = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_new);
                p0 = expf(x0 - m_new); p1 = expf(x1 - m_new);
            }
            l_run[i] = l_run[i] * alpha + warp_sum(p0 + p1);
            m_run[i] = m_new;
            Pb[rr * PST + lane] = __float2bfloat16_rn(p0);
            Pb[rr * PST + lane + 32] = __float2bfloat16_rn(p1);
            if (lane == 0) alpha_s[rr] = alpha;
        }
        __syncthreads();
        {   // O += P V: rows rw*16 .. +16, columns cw*NT*8 .. + NT*8
            const float al_a = alpha_s[ra], al_b = alpha_s[rb];
#pragma unroll
            for (int j = 0; j < NT; ++j) { o[j][0] *= al_a; o[j][1] *= al_a; o[j][2] *= al_b; o[j][3] *= al_b; }
            const uint32_t pa_addr = sm_addr(Pb + (rw * 16 + (lane & 15)) * PST + (lane >> 4) * 8);
            const uint32_t va = sm_addr(Vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * vst + cw * NT * 8 + (lane >> 4) * 8);
#pragma unroll
            for (int kk = 0; kk < MKB; kk += 16) {
                uint32_t af[4];
                ldsm4(af, pa_addr + kk * 2);
#pragma unroll
                for (int j2 = 0; j2 < NT / 2; ++j2) {
                    uint32_t bfr[4];
                    ldsm4t(bfr, va + (kk * vst + j2 * 16) * 2);
                    mma16816(o[2 * j2], af, bfr[0], bfr[1]);
                    mma16816(o[2 * j2 + 1], af, bfr[2], bfr[3]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (lane == 0) { alpha_s[warp * 4 + i] = l_run[i]; m_fin[warp * 4 + i] = m_run[i]; }
    __syncthreads();
#pragma unroll
    for (int side = 0; side < 2; ++side) {
        const int rr = side ? rb : ra, r = r0 + rr;
        if (r >= n_rows) continue;
        const int t = t0 + r / G, h = kvh * G + r % G;
        if (a.splits == 1) {
            const float inv = a.out_scale / alpha_s[rr];
            bf16* orow = out + (size_t)t * a.out_ld + a.out_off + (size_t)h * dv;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = cw * NT * 8 + j * 8 + fc + e;
                    if (c < dv) orow[c] = __float2bfloat16_rn(o[j][side * 2 + e] * inv);
                }
        } else {
            const size_t slot = ((size_t)t * a.nq + h) * a.splits + split;
            float* prow = a.part_o + slot * dv;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = cw * NT * 8 + j * 8 + fc + e;
                    if (c < dv) prow[c] = o[j][side * 2 + e];
                }
            if (cw == 0 && fc == 0) { a.part_ml[2 * slot] = m_fin[rr]; a.part_ml[2 * slot + 1] = alpha_s[rr]; }
        }
    }
}

static bool tile_mma_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("TFFINFER_TILE_MMA"); v = (e && e[0] == '0') ? 0 : 1; }
    return v != 0;
}

// Launches the tensor-core form if the sizes allow it; TFF_ERR_UNSUPPORTED otherwise (the caller takes the float32 form).
int launch_tile_mma(const void* q, const void* cache, void* out, const TileArgs& a, int num_requests, int max_q_len,
                    int num_tokens, cudaStream_t stream) {
    const int G = a.nq / a.nkv;
    const bool dense = a.k_dense != nullptr;
    const bool own_v = a.v_offset != 0 || dense;
    if (!tile_mma_enabled() || (a.d & 7) || (a.q_ld & 7) || ((uintptr_t)q & 15) || (own_v && (a.dv & 7)) || a.dv > 512)
        return TFF_ERR_UNSUPPORTED;
    if (dense ? ((a.k_ld & 7) || (a.v_ld & 7) || ((uintptr_t)a.k_dense & 15) || ((uintptr_t)a.v_dense & 15))
              : ((a.slot & 7) || (a.page_stride & 7) || (a.v_offset & 7) || ((uintptr_t)cache & 15)))
        return TFF_ERR_UNSUPPORTED;
    if (num_requests > 65535 || a.nkv > 65535) return TFF_ERR_UNSUPPORTED;
    int nt = 2;
    while (nt * 32 < a.dv) nt *= 2;                              // value columns per warp: nt * 8, four warps across
    MmaGeom gm;
    gm.dpad = (a.d + 15) / 16 * 16;
    gm.kst = (own_v ? gm.dpad : max(gm.dpad, nt * 32)) + 8;
    gm.vst = own_v ? nt * 32 + 8 : gm.kst;
    const int rows_most = max_q_len * G;
    const int rg = rows_most <= 16 ? 1 : (rows_most <= 32 ? 2 : 4);
    const int MROWS = 16 * rg;
    const size_t smem = 2 * ((size_t)(MROWS + MKB) * gm.kst + (own_v ? (size_t)MKB * gm.vst : 0) + (size_t)MROWS * PST) +
                        4 * ((size_t)MROWS * SST + 2 * MROWS) + 4 * 2 * MROWS + 2 * 8 * MKB;
    if (smem > 220 * 1024) return TFF_ERR_UNSUPPORTED;
    const int tiles = (rows_most + MROWS - 1) / MROWS;
    dim3 grid(tiles * a.splits, a.nkv, num_requests);
#define TFF_TMMA(NTV)                                                                                                \
    do {                                                                                                             \
        if (rg == 1) TFF_TMMA_RG(NTV, 1);                                                                            \
        if (rg == 2) TFF_TMMA_RG(NTV, 2);                                                                            \
        TFF_TMMA_RG(NTV, 4);                                                                                         \
    } while (0)
#define TFF_TMMA_RG(NTV, RGV)                                                                                        \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(attention_tile_mma_kernel<NTV, RGV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        const int st = tff_launch_pdl(attention_tile_mma_kernel<NTV, RGV>, grid, dim3(128 * RGV), smem, stream, (const bf16*)q, \
                                      (const bf16*)cache, (bf16*)out, a, gm);                                        \
        if (st != TFF_OK || a.splits == 1) return st;                                                                \
        const long long rows = (long long)num_tokens * a.nq;                                                         \
        return tff_launch_pdl(attention_tile_merge_kernel<bf16>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream, \
                              (const float*)a.part_o, (const float*)a.part_ml, (bf16*)out, a.out_ld, a.out_off, rows, \
                              a.nq, a.dv, a.splits, a.out_scale);                                                    \
    } while (0)
    if (nt == 2) TFF_TMMA(2);
    if (nt == 4) TFF_TMMA(4);
    if (nt == 8) TFF_TMMA(8);
    TFF_TMMA(16);
#undef TFF_TMMA
#undef TFF_TMMA_RG
}

}  // namespace

// q [tokens, q_ld] with head h at columns h*d; the cache pointer is the start of the layer's share of the pool (the
// layer's offset already added); ``planes`` 2: values in the second plane of a page, 1: the value is the first dv
// elements of the key's slot.  is_bf16: q, out and the cache are bfloat16, else float32.  splits > 1: every tile's key
// range in that many shares (float32 workspaces part_o [tokens*nq, splits, dv] and part_ml [tokens*nq, splits, 2]) and a
// merge kernel; for steps of few rows behind long contexts, which would otherwise be a handful of CTAs.  k_dense / v_dense
// (bfloat16 [tokens, k_ld] / [tokens, v_ld], both or neither): the keys and values of this step's tokens in plain rows
// instead of the cache, for steps whose requests all start at position 0.
TFF_API int tff_attention_tile(
    const void* q, int is_bf16, int q_ld, const int* q_start, const int* pos_start, const int* block_table,
    int table_width, const void* cache, long long page_stride, int planes, int page_size, int slot,
    void* out, int out_ld, int out_off, int num_requests, int max_q_len, int nq, int nkv, int d, int dv, float scale,
    int window, int chunk, const float* temp, const float* r1, const float* r2, float out_scale,
    int num_tokens, int splits, float* part_o, float* part_ml,
    const void* k_dense, const void* v_dense, int k_ld, int v_ld, float softcap, cudaStream_t stream) {
    if (num_requests <= 0 || max_q_len <= 0) return TFF_OK;
    if ((k_dense == nullptr) != (v_dense == nullptr)) return TFF_ERR_BAD_ARGUMENT;
    if (k_dense) { planes = 2; slot = d > dv ? d : dv; page_size = 1; }      // no cache is read: any consistent geometry
    if (nq <= 0 || nkv <= 0 || nq % nkv || d <= 0 || dv <= 0 || slot < d || page_size <= 0 || window < 0 || chunk < 0 ||
        (planes != 1 && planes != 2) || (planes == 2 && slot < dv) || (planes == 1 && dv > d) || ((r1 == nullptr) != (r2 == nullptr)))
        return TFF_ERR_BAD_ARGUMENT;
    TileArgs a;
    a.q_start = q_start; a.pos_start = pos_start; a.block_table = block_table; a.table_width = table_width;
    a.page_stride = page_stride; a.head_stride = (long long)page_size * slot;
    a.v_offset = planes == 2 ? (long long)nkv * page_size * slot : 0;
    a.slot = slot; a.page_size = page_size; a.nq = nq; a.nkv = nkv; a.d = d; a.dv = dv; a.scale = scale;
    a.softcap = softcap > 0.f ? softcap : 0.f;
    a.window = window; a.chunk = chunk; a.temp = temp; a.r1 = r1; a.r2 = r2; a.out_scale = out_scale;
    a.q_ld = q_ld; a.out_ld = out_ld; a.out_off = out_off;
    if (splits < 1 || (splits > 1 && (!part_o || !part_ml))) return TFF_ERR_BAD_ARGUMENT;
    a.splits = splits; a.part_o = part_o; a.part_ml = part_ml;
    a.k_dense = k_dense; a.v_dense = v_dense; a.k_ld = k_ld; a.v_ld = v_ld;
    if (k_dense) {                                   // the tensor-core form or nothing
        if (!is_bf16) return TFF_ERR_UNSUPPORTED;
        return launch_tile_mma(q, cache, out, a, num_requests, max_q_len, num_tokens, stream);
    }
    if (is_bf16) {
        const int st = launch_tile_mma(q, cache, out, a, num_requests, max_q_len, num_tokens, stream);
        if (st != TFF_ERR_UNSUPPORTED) return st;
        return launch_tile<bf16, bf16>(q, cache, out, a, num_requests, max_q_len, num_tokens, stream);
    }
    return launch_tile<float, float>(q, cache, out, a, num_requests, max_q_len, num_tokens, stream);
}
