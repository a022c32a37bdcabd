// The small kernels around a routed feed-forward (mixture of experts); the experts' products are gemm_grouped.cu.
//
//   route    per token: z = W_r h in float32 (one warp per expert, a fixed order of additions), s = sigmoid(z) or
//            softmax(z) over all outputs (or z itself, the chosen then weighted by a softmax among themselves; z may
//            carry a bias), choice scores s + correction, optionally only the experts of the best
//            ``keep`` of ``groups`` groups of neighbours (a group's score is its best choice score), the ``top`` experts
//            of largest choice score (the lower index wins a tie), weights s, optionally renormalised to sum 1; writes
//            the pair (token, k) -> (expert, weight) and counts the pairs of every expert.  The last router outputs may
//            be identity experts (output = weight * input): their pairs get expert -1, no row in the experts' products,
//            and the combine kernel adds them from the input rows
//   plan     one block: the experts' row ranges in the sorted order, the tile table of the grouped product (tiles of
//            ``tile_rows`` rows that never span two experts), and the counters back to zero for the next call
//   gather   per pair: its place among its expert's rows (an atomic cursor: the order within an expert is not fixed,
//            but a row's result does not depend on its place), row_map[place] = pair, and the expert's input row
//            x[place] = w * h[token] (weight on the input) or h[token]
//   combine  per token: residual[t] += sum_k y[t * top + k] (times the weight when it multiplies the output), in
//            the order k = 0 .. top-1
#include "common.cuh"

namespace {

constexpr int ROUTE_TOK = 4;                   // tokens a block of moe_route_kernel, one warp each for the choice
constexpr int ROUTE_THREADS = 256;

template <typename TH, typename TW>
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const TH* __restrict__ h, const TW* __restrict__ w_router, const float* __restrict__ bias, int T, int W, int E,
                 int top, int renormalize, int softmax_scores, const float* __restrict__ correction, int groups, int keep, int num_real,
                 int* __restrict__ pair_expert, float* __restrict__ pair_weight, int* __restrict__ counts) {
    // A block takes ROUTE_TOK tokens: the router's rows are read once for all of them (2,048 tokens re-read a 64 KB router
    // 2,048 times otherwise), every token keeps sums of its own, and behind the products warp i does token i's choice.
    extern __shared__ float sm[];              // per token W floats (its row) and 3 E: the scores, the choice scores, groups
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * ROUTE_TOK, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt = min(ROUTE_TOK, T - t0);
    float* rows = sm;                          // [ROUTE_TOK][W]
    float* scores = sm + (size_t)ROUTE_TOK * W;   // [ROUTE_TOK][3 E]
    if ((W & 7) == 0 && ((size_t)h & 15) == 0) {           // eight elements a load (sixteen bytes of bfloat16)
        for (int v = threadIdx.x; v < nt * (W >> 3); v += ROUTE_THREADS) {
            const int k = v / (W >> 3), i = (v - k * (W >> 3)) << 3;
            float* dst = rows + (size_t)k * W + i;
            const TH* src = h + (size_t)(t0 + k) * W + i;
            if constexpr (sizeof(TH) == 2) {
                const uint4 raw = *reinterpret_cast<const uint4*>(src);
                const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 a = __bfloat1622float2(p2[0]), b = __bfloat1622float2(p2[1]);
                const float2 c = __bfloat1622float2(p2[2]), d = __bfloat1622float2(p2[3]);
                *reinterpret_cast<float4*>(dst) = make_float4(a.x, a.y, b.x, b.y);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(c.x, c.y, d.x, d.y);
            } else {
                *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
                *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
            }
        }
    } else {
        for (int k = 0; k < nt; ++k)
            for (int i = threadIdx.x; i < W; i += ROUTE_THREADS) rows[(size_t)k * W + i] = to_f32<TH>(h[(size_t)(t0 + k) * W + i]);
    }
    for (int k = nt; k < ROUTE_TOK; ++k)
        for (int i = threadIdx.x; i < W; i += ROUTE_THREADS) rows[(size_t)k * W + i] = 0.f;
    __syncthreads();
    // A warp an output; a lane takes eight neighbouring elements a load where the rows allow it (16-byte loads, several in
    // flight), else one.  Either way the order of a dot product's additions is fixed by W alone.
    const bool wide = (W & 7) == 0 && ((size_t)w_router & 15) == 0;
    for (int e = warp; e < E; e += ROUTE_THREADS / 32) {
        const TW* wr = w_router + (size_t)e * W;
        float acc[ROUTE_TOK];
#pragma unroll
        for (int k = 0; k < ROUTE_TOK; ++k) acc[k] = 0.f;
        if (wide) {
#pragma unroll 4
            for (int i = lane * 8; i < W; i += 256) {
                float w8[8];
                if constexpr (sizeof(TW) == 2) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(wr + i);
                    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                    for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(p2[k]); w8[2 * k] = f.x; w8[2 * k + 1] = f.y; }
                } else {
                    const float4 a = *reinterpret_cast<const float4*>(wr + i), b = *reinterpret_cast<const float4*>(wr + i + 4);
                    w8[0] = a.x; w8[1] = a.y; w8[2] = a.z; w8[3] = a.w; w8[4] = b.x; w8[5] = b.y; w8[6] = b.z; w8[7] = b.w;
                }
#pragma unroll
                for (int k = 0; k < ROUTE_TOK; ++k) {
                    const float* row = rows + (size_t)k * W + i;
                    const float4 r0 = *reinterpret_cast<const float4*>(row), r1 = *reinterpret_cast<const float4*>(row + 4);
                    float a = acc[k];
                    a = fmaf(r0.x, w8[0], a); a = fmaf(r0.y, w8[1], a); a = fmaf(r0.z, w8[2], a); a = fmaf(r0.w, w8[3], a);
                    a = fmaf(r1.x, w8[4], a); a = fmaf(r1.y, w8[5], a); a = fmaf(r1.z, w8[6], a); a = fmaf(r1.w, w8[7], a);
                    acc[k] = a;
                }
            }
        } else {
            for (int i = lane; i < W; i += 32) {
                const float wv = to_f32<TW>(wr[i]);
#pragma unroll
                for (int k = 0; k < ROUTE_TOK; ++k) acc[k] = fmaf(rows[(size_t)k * W + i], wv, acc[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < ROUTE_TOK; ++k) {
            const float z = warp_sum(acc[k]) + (bias ? bias[e] : 0.f);
            if (lane == 0) scores[(size_t)k * 3 * E + e] = softmax_scores ? z : 1.0f / (1.0f + expf(-z));
        }
    }
    __syncthreads();
    if (warp >= nt) return;                    // warp i: token t0 + i
    const int t = t0 + warp;
    float* score = scores + (size_t)warp * 3 * E;
    float* choice = score + E;
    float* gbest = choice + E;
    if (softmax_scores == 1) {                 // over all router outputs, in an order that E alone fixes
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, score[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float x = expf(score[e] - m); score[e] = x; sum += x; }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < E; e += 32) score[e] = score[e] / sum;
        __syncwarp();
    }
    for (int e = lane; e < E; e += 32) choice[e] = score[e] + (correction ? correction[e] : 0.f);
    __syncwarp();
    if (groups > 1 && keep < groups) {         // only the experts of the ``keep`` groups with the best member stay
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY;
            for (int j = 0; j < per; ++j) b = fmaxf(b, choice[g * per + j]);
            gbest[g] = b;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY; int arg = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float s = gbest[g];
                if (!isnan(s) && (arg == 0x7fffffff || s > best)) { best = s; arg = g; }   // kept groups are NaN
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
            }
            if (lane == 0 && arg != 0x7fffffff) gbest[arg] = __int_as_float(0x7fc00000);   // NaN marks a kept group
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (!isnan(gbest[e / per])) choice[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY; int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float s = choice[e];
            if (s > best) { best = s; arg = e; }      // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        const float wgt = arg != 0x7fffffff ? score[arg] : 0.f;   // the weight is the score without the correction
        if (lane == 0) {
            // an identity expert (index >= num_real) has no rows among the experts' products: -1
            pair_expert[(size_t)t * top + k] = (arg == 0x7fffffff || arg >= num_real) ? -1 : arg;
            pair_weight[(size_t)t * top + k] = wgt;
            if (arg != 0x7fffffff) {
                if (arg < num_real) atomicAdd(&counts[arg], 1);
                choice[arg] = -INFINITY;              // taken
            }
        }
        total += wgt;
        __syncwarp();
    }
    if (softmax_scores == 2) {                 // the scores are the logits themselves: softmax over the chosen ones only
        if (lane == 0) {
            float* pw = pair_weight + (size_t)t * top;
            float m = -INFINITY, sum = 0.f;
            for (int k = 0; k < top; ++k) m = fmaxf(m, pw[k]);
            for (int k = 0; k < top; ++k) { pw[k] = expf(pw[k] - m); sum += pw[k]; }
            for (int k = 0; k < top; ++k) pw[k] /= sum;
        }
        return;
    }
    if (renormalize && lane == 0)
        for (int k = 0; k < top; ++k) pair_weight[(size_t)t * top + k] /= total;
}

// pad_rows > 0: every expert's rows start at a multiple of pad_rows (= tile_rows): the sorted order then consists of
// whole tiles of one expert each, and lane_group[row / pad_rows] names it (-1: a tile nobody uses), which is what the
// grouped tcgen05 product reads.
__global__ void moe_plan_kernel(int* __restrict__ counts, int E, int tile_rows, int* __restrict__ cursor,
                                int* __restrict__ tile_group, int* __restrict__ tile_row0, int* __restrict__ tile_row_end,
                                int* __restrict__ num_tiles, int pad_rows, int* __restrict__ lane_group, int lane_tiles) {
    pdl_launch_dependents();
    pdl_wait();
    if (lane_group)
        for (int i = threadIdx.x; i < lane_tiles; i += blockDim.x) lane_group[i] = -1;
    __syncthreads();
    if (threadIdx.x != 0) return;
    int off = 0, n = 0;
    for (int e = 0; e < E; ++e) {
        const int c = counts[e];
        counts[e] = 0;
        if (pad_rows > 0) off = (off + pad_rows - 1) / pad_rows * pad_rows;
        cursor[e] = off;
        for (int r = off; r < off + c; r += tile_rows) {
            tile_group[n] = e; tile_row0[n] = r; tile_row_end[n] = off + c; ++n;
            if (lane_group) lane_group[r / pad_rows] = e;
        }
        off += c;
    }
    *num_tiles = n;
}

template <typename TH>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const TH* __restrict__ h, int W, int top, const int* __restrict__ pair_expert,
                  const float* __restrict__ pair_weight, int weight_on_input, int* __restrict__ cursor,
                  int* __restrict__ row_map, int* __restrict__ place_of_pair, TH* __restrict__ x) {
    __shared__ int place_s;
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x;
    const int expert = pair_expert[pair];
    if (expert < 0) {                                 // an identity expert: no row among the experts' products
        if (threadIdx.x == 0 && place_of_pair) place_of_pair[pair] = -1;
        return;
    }
    if (threadIdx.x == 0) {
        place_s = atomicAdd(&cursor[expert], 1);
        row_map[place_s] = pair;
        if (place_of_pair) place_of_pair[pair] = place_s;
    }
    __syncthreads();
    const int place = place_s;
    const float w = weight_on_input ? pair_weight[pair] : 1.f;
    const TH* src = h + (size_t)(pair / top) * W;
    TH* dst = x + (size_t)place * W;
    for (int i = threadIdx.x; i < W; i += 128) dst[i] = from_f32<TH>(w * to_f32<TH>(src[i]));
}

template <typename TH>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, int W, int top, const float* __restrict__ pair_weight,
                   int weight_on_output, const int* __restrict__ place_of_pair, float* __restrict__ residual,
                   float* __restrict__ out, const int* __restrict__ pair_expert, const TH* __restrict__ h) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int i = blockIdx.y * 256 + threadIdx.x;
    if (i >= W) return;
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
        const size_t pair = (size_t)t * top + k;              // y in (token, rank) order, or in the sorted order
        if (pair_expert && pair_expert[pair] < 0) {           // an identity expert: the weight times the input itself
            acc = fmaf(pair_weight[pair], to_f32<TH>(h[(size_t)t * W + i]), acc);
            continue;
        }
        const float w = weight_on_output ? pair_weight[pair] : 1.f;
        acc = fmaf(w, y[(place_of_pair ? (size_t)place_of_pair[pair] : pair) * W + i], acc);
    }
    const size_t at = (size_t)t * W + i;
    out[at] = residual ? residual[at] + acc : acc;
}

}  // namespace

// E router outputs, of which the last E - num_real are identity experts (pair_expert -1).  softmax_scores: the scores are
// softmax(z) over all E outputs instead of sigmoid(z); 2: the scores are the logits z, and the weights of the chosen are the
// softmax over the chosen logits alone.  bias [E] float32 or null: added to the router's product.  correction [E] float32 or null: added to the scores for the
// choice only.  groups > 1 with keep < groups: E / groups neighbours form a group, and only the ``keep`` groups whose best
// choice score is largest can be chosen from.
TFF_API int tff_moe_route(const void* h, int h_dt, const void* w_router, int w_dt, const float* bias, int T, int W, int E, int top,
                          int renormalize, int softmax_scores, const float* correction, int groups, int keep,
                          int num_real, int* pair_expert, float* pair_weight, int* counts, cudaStream_t stream) {
    if (T <= 0) return TFF_OK;
    if (W <= 0 || E <= 0 || top <= 0 || top > E || !h || !w_router || num_real < 0 || num_real > E)
        return TFF_ERR_BAD_ARGUMENT;
    if (groups > 1 && (E % groups != 0 || keep <= 0 || keep > groups || top > keep * (E / groups))) return TFF_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)ROUTE_TOK * (W + 3 * E) * sizeof(float);
    if (smem > 200 * 1024) return TFF_ERR_UNSUPPORTED;
#define TFF_ROUTE(TH, TW)                                                                                             \
    do {                                                                                                              \
        if (smem > 48 * 1024)                                                                                         \
            cudaFuncSetAttribute(moe_route_kernel<TH, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        return tff_launch_pdl(moe_route_kernel<TH, TW>, dim3((T + ROUTE_TOK - 1) / ROUTE_TOK), dim3(ROUTE_THREADS), smem, stream, (const TH*)h, \
                              (const TW*)w_router, bias, T, W, E, top, renormalize, softmax_scores, correction, groups, keep, \
                              num_real, pair_expert, pair_weight, counts);         \
    } while (0)
    if (h_dt == 0 && w_dt == 0) TFF_ROUTE(float, float);
    if (h_dt == 0 && w_dt == 1) TFF_ROUTE(float, bf16);
    if (h_dt == 1 && w_dt == 1) TFF_ROUTE(bf16, bf16);
    if (h_dt == 1 && w_dt == 0) TFF_ROUTE(bf16, float);
#undef TFF_ROUTE
    return TFF_ERR_BAD_ARGUMENT;
}

TFF_API int tff_moe_plan(int* counts, int E, int tile_rows, int* cursor, int* tile_group, int* tile_row0,
                         int* tile_row_end, int* num_tiles, int pad_rows, int* lane_group, int lane_tiles,
                         cudaStream_t stream) {
    if (E <= 0 || tile_rows <= 0 || pad_rows < 0 || (pad_rows > 0 && pad_rows != tile_rows) || (lane_group && pad_rows <= 0))
        return TFF_ERR_BAD_ARGUMENT;
    return tff_launch_pdl(moe_plan_kernel, dim3(1), dim3(128), 0, stream, counts, E, tile_rows, cursor, tile_group,
                          tile_row0, tile_row_end, num_tiles, pad_rows, lane_group, lane_tiles);
}

TFF_API int tff_moe_gather(const void* h, int h_dt, int pairs, int W, int top, const int* pair_expert,
                           const float* pair_weight, int weight_on_input, int* cursor, int* row_map,
                           int* place_of_pair, void* x, cudaStream_t stream) {
    if (pairs <= 0) return TFF_OK;
    if (h_dt == 0)
        return tff_launch_pdl(moe_gather_kernel<float>, dim3(pairs), dim3(128), 0, stream, (const float*)h, W, top,
                              pair_expert, pair_weight, weight_on_input, cursor, row_map, place_of_pair, (float*)x);
    return tff_launch_pdl(moe_gather_kernel<bf16>, dim3(pairs), dim3(128), 0, stream, (const bf16*)h, W, top,
                          pair_expert, pair_weight, weight_on_input, cursor, row_map, place_of_pair, (bf16*)x);
}

// pair_expert (null: every pair has a row in y) and h [T, W] (h_dt 0 float32, 1 bfloat16): pairs whose expert is -1 are
// identity experts and add pair_weight * h[t]; pair_weight must then be given.
TFF_API int tff_moe_combine(const float* y, int T, int W, int top, const float* pair_weight, int weight_on_output,
                            const int* place_of_pair, float* residual, float* out, const int* pair_expert,
                            const void* h, int h_dt, cudaStream_t stream) {
    if (T <= 0) return TFF_OK;
    if (pair_expert && (!h || !pair_weight)) return TFF_ERR_BAD_ARGUMENT;
    dim3 grid(T, (W + 255) / 256);
    if (h_dt == 1)
        return tff_launch_pdl(moe_combine_kernel<bf16>, grid, dim3(256), 0, stream, y, W, top, pair_weight, weight_on_output,
                              place_of_pair, residual, out, pair_expert, (const bf16*)h);
    return tff_launch_pdl(moe_combine_kernel<float>, grid, dim3(256), 0, stream, y, W, top, pair_weight, weight_on_output,
                          place_of_pair, residual, out, pair_expert, (const float*)h);
}
