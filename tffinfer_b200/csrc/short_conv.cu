// A short causal convolution over time on the channels of a merged projection, with the RMS norm of whole column
// segments behind it, and the per-request state that carries the convolution across steps.
//
//   proj[t] = [seg 0 | seg 1 | seg 2 | rest]      float32 rows of the step's tokens (a product's accumulators)
//   y[t, c] = sum_j w[c, j] * u[t - (taps - 1) + j, c]       j = 0 .. taps-1, u = proj, zeros before position 0
//   out[t, seg] = y[t, seg] / sqrt(mean(y[t, seg]^2) + eps) * g_seg        for segments that have a norm weight
//   out[t, rest] = proj[t, rest]
//
// The taps-1 rows of u that precede a request's first token of this step come from state[slot] ([taps-1, C] float32,
// C = the segments' channels together, the oldest row first); a request whose first token is at position 0 reads
// zeros instead.  The engine clears a slot when position 0 arrives, so both are the same; the kernel does not rely
// on it.  A second kernel, launched behind the first, leaves the request's last taps-1 rows of u in the slot and,
// where the rows are an accumulator buffer that is kept at zero between uses, clears them.
// Sums of squares are added in an order that depends on the row's width alone.
#include "common.cuh"

namespace {

constexpr int MAX_SEGS = 3;
constexpr int MAX_TAPS = 8;

struct ConvSegs {
    int n;
    int off[MAX_SEGS];            // first column of the segment in a row of proj / out and in a row of the state
    int width[MAX_SEGS];
    const float* w[MAX_SEGS];     // [width, taps] or null: the segment passes as it is
    const float* norm[MAX_SEGS];  // [width] or null: no norm
};

__global__ void __launch_bounds__(256)
short_conv_norm_kernel(const float* __restrict__ proj, int ld, float* __restrict__ out, ConvSegs segs, int taps, int C,
                       const float* __restrict__ state, const int* __restrict__ positions,
                       const int* __restrict__ tok_req, const int* __restrict__ q_start,
                       const int* __restrict__ slots, float eps) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int b = tok_req[t];
    const int pos = positions[t];
    const int i_in = t - q_start[b];                       // the token's place in its request's portion
    const float* st = state + (size_t)slots[b] * (taps - 1) * C;
    for (int s = 0; s < segs.n; ++s) {
        const int off = segs.off[s], width = segs.width[s];
        float ss = 0.f;
        for (int c = threadIdx.x; c < width; c += 256) {
            float y;
            if (segs.w[s]) {
                y = 0.f;
                const float* wc = segs.w[s] + (size_t)c * taps;
                for (int j = 0; j < taps; ++j) {
                    const int back = taps - 1 - j;           // how many tokens before this one
                    if (back > pos) continue;                // before the sequence's start
                    float u;
                    if (back <= i_in) u = proj[(size_t)(t - back) * ld + off + c];
                    else u = st[(size_t)(taps - 1 - (back - i_in)) * C + off + c];
                    y = fmaf(wc[j], u, y);
                }
            } else {
                y = proj[(size_t)t * ld + off + c];
            }
            out[(size_t)t * ld + off + c] = y;
            ss = fmaf(y, y, ss);
        }
        if (segs.norm[s]) {                                  // uniform over the block
            ss = block_sum<256>(ss, red);
            const float rs = rsqrtf(ss / (float)width + eps);
            for (int c = threadIdx.x; c < width; c += 256)   // a thread reads back what it wrote itself
                out[(size_t)t * ld + off + c] = (out[(size_t)t * ld + off + c] * rs) * segs.norm[s][c];
            __syncthreads();                                 // red is used again
        }
    }
    for (int c = C + threadIdx.x; c < ld; c += 256) out[(size_t)t * ld + c] = proj[(size_t)t * ld + c];
}

// grid (requests, column blocks of 256).  A thread owns one column of one request: it moves the state up by the
// portion's length (oldest first, so nothing is overwritten before it is read), fills the rest from the portion's last
// rows, and clears the portion's rows of that column when asked to.
__global__ void __launch_bounds__(256)
short_conv_state_kernel(float* __restrict__ proj, int ld, int clear, int taps, int C, float* __restrict__ state,
                        const int* __restrict__ q_start, const int* __restrict__ pos_start,
                        const int* __restrict__ slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= ld) return;
    const int q0 = q_start[b], n = q_start[b + 1] - q0;
    if (c < C && n > 0) {
        float* st = state + (size_t)slots[b] * (taps - 1) * C + c;
        const bool fresh = pos_start[b] == 0;
        for (int s = 0; s < taps - 1; ++s) {
            const int i = n - (taps - 1) + s;               // the row of the portion that ends up at place s
            float v;
            if (i >= 0) v = proj[(size_t)(q0 + i) * ld + c];
            else v = fresh ? 0.f : st[(size_t)(s + n) * C];
            st[(size_t)s * C] = v;
        }
    }
    if (clear)
        for (int i = 0; i < n; ++i) proj[(size_t)(q0 + i) * ld + c] = 0.f;
}

// x[t, k, :] += table[row(t), :] for every copy k, with row(t) = (prev * mul_prev + tok * mul_cur) mod buckets, prev
// the token before t in its request (from the step's tokens, or from state[slot] for a portion's first token), and
// row ``buckets`` for a request's token at position 0.
template <typename TW>
__global__ void __launch_bounds__(128)
pair_embed_kernel(const int* __restrict__ tokens, const int* __restrict__ positions, const int* __restrict__ tok_req,
                  const int* __restrict__ q_start, const int* __restrict__ slots, const int* __restrict__ state,
                  const TW* __restrict__ table, int buckets, long long mul_prev, long long mul_cur,
                  float* __restrict__ x, int copies, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = tok_req[t];
    long long row = buckets;
    if (positions[t] > 0) {
        const long long prev = t > q_start[b] ? tokens[t - 1] : state[slots[b]];
        row = (prev * mul_prev + (long long)tokens[t] * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const TW* src = table + (size_t)row * W;
    float* dst = x + (size_t)t * copies * W;
    for (int i = threadIdx.x; i < W; i += 128) {
        const float v = to_f32<TW>(src[i]);
        for (int k = 0; k < copies; ++k) dst[(size_t)k * W + i] += v;
    }
}

__global__ void last_token_kernel(const int* __restrict__ tokens, const int* __restrict__ q_start,
                                  const int* __restrict__ slots, int* __restrict__ state, int num_requests) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= num_requests) return;
    const int q1 = q_start[b + 1];
    if (q1 > q_start[b]) state[slots[b]] = tokens[q1 - 1];
}

// Two neighbouring elements in one store (the address is a multiple of the pair's size).
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// One q or k head of conv_finish_kernel, by one warp: (y * rs) * w for every element (w null: y as it is), the first
// 2 * half elements rotated, stored to dst.  src, w, cos_s, sin_s are shared memory.  pairs: two elements a lane and
// store (every size involved is even and dst is aligned for it).
template <typename T>
__device__ __forceinline__ void finish_head(T* __restrict__ dst, const float* src, const float* w, float rs,
                                            const float* cos_s, const float* sin_s, int half, int d, int interleaved,
                                            bool pairs, int lane) {
    auto val = [&](int i) { return w ? (src[i] * rs) * w[i] : src[i]; };
    if (pairs && !interleaved) {
        for (int i = lane * 2; i < half; i += 64) {
            const float a0 = val(i), a1 = val(i + 1), b0 = val(i + half), b1 = val(i + half + 1);
            const float c0 = cos_s[i], c1 = cos_s[i + 1], s0 = sin_s[i], s1 = sin_s[i + 1];
            store_pair(dst + i, a0 * c0 - b0 * s0, a1 * c1 - b1 * s1);
            store_pair(dst + i + half, b0 * c0 + a0 * s0, b1 * c1 + a1 * s1);
        }
    } else {
        for (int i = lane; i < half; i += 32) {
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            const float a = val(ia), bb = val(ib);
            const float sn = sin_s[i], cs = cos_s[i];
            const float ra = a * cs - bb * sn, rb = bb * cs + a * sn;
            if (pairs) store_pair(dst + ia, ra, rb);           // interleaved: the two are neighbours
            else { dst[ia] = from_f32<T>(ra); dst[ib] = from_f32<T>(rb); }
        }
    }
    if (pairs) for (int i = 2 * half + lane * 2; i < d; i += 64) store_pair(dst + i, val(i), val(i + 1));
    else for (int i = 2 * half + lane; i < d; i += 32) dst[i] = from_f32<T>(val(i));
}

// The convolution and the norms above and what lies between them and the token mixing, in one pass over a token's row:
// one block a token keeps the convolved q, k and v of the token in shared memory (C floats), norms q and k there, rotates
// the first rot_dims dimensions of every q and k head by the token's position (pairs (2i, 2i+1) or (i, i + rot_dims/2),
// angle float(position) * freq[i], cos and sin times ``magnitude``), stores q to q_out [T, nq*d], k and v to the token's
// slot of the paged cache ([pages, layers, 2, kv heads, page, dc]) and sigmoid(proj[t, gate_off + h]) to gate_out.  The
// float32 row of convolved values is never written to memory.  proj is only read: short_conv_state runs behind it.
// Here the convolution's weights are TRANSPOSED, segs.w[s] = [taps, width], so that one load brings a tap's weights of
// four neighbouring channels.  A block waits for memory as seldom as it can: everything that does not depend on
// anything computed here is loaded ahead of the first wait (all taps of a thread's channels, the norm weights, which go
// to shared memory beside the channels, the page number, the gates); behind the sums of squares only shared memory is read.
// MT: the most taps this instance holds in registers (4 or MAX_TAPS).
template <typename TQ, typename TC, int MT>
__global__ void __launch_bounds__(256, MT <= 4 ? 4 : 2)
conv_finish_kernel(const float* __restrict__ proj, int ld, ConvSegs segs, int taps, int C,
                   const float* __restrict__ state, const int* __restrict__ positions, const int* __restrict__ tok_req,
                   const int* __restrict__ q_start, const int* __restrict__ slots, float eps,
                   TQ* __restrict__ q_out, const float* __restrict__ freq, int rot_dims, float magnitude, int interleaved,
                   const int* __restrict__ block_table, int table_width, TC* __restrict__ cache, KvLayout L, int layer,
                   int dc, int gate_off, float* __restrict__ gate_out, int nq, int nkv, int d, int dv, int pairs) {
    extern __shared__ float y_s[];          // C channels, the norm weights of q and k, 32 for the sums, cos and sin
    const int NW = segs.off[2];             // q and k lie first
    float* nw_s = y_s + C;
    float* red = nw_s + NW;
    float* cos_s = red + 32;
    float* sin_s = cos_s + (rot_dims >> 1);
    __shared__ float rs_s[MAX_SEGS];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = tok_req[t];
    const int pos = positions[t];
    const int i_in = t - q_start[b];
    const int slot_no = slots[b];
    const int page = block_table[(size_t)b * table_width + pos / L.page_size];
    if (gate_out)
        for (int h = threadIdx.x; h < nq; h += 256)
            gate_out[(size_t)t * nq + h] = 1.0f / (1.0f + expf(-proj[(size_t)t * ld + gate_off + h]));
    for (int i = threadIdx.x; i < (rot_dims >> 1); i += 256) {   // the token's angles once, for all heads
        float sn, cs;
        sincosf((float)pos * freq[i], &sn, &cs);
        cos_s[i] = cs * magnitude; sin_s[i] = sn * magnitude;
    }
    const float* st = state + (size_t)slot_no * (taps - 1) * C;
    // Four neighbouring channels a thread in ONE pass over all three segments when every border is a multiple of four.
    bool flat = ((ld | C | segs.off[1] | segs.off[2]) & 3) == 0 && (((size_t)proj | (size_t)state) & 15) == 0;
    for (int s = 0; s < 3; ++s) flat = flat && (((size_t)segs.w[s] | (size_t)segs.norm[s]) & 15) == 0;
    if (flat) {
        float ss0 = 0.f, ss1 = 0.f;
        for (int c = threadIdx.x * 4; c < C; c += 1024) {
            const int s = c >= segs.off[2] ? 2 : (c >= segs.off[1] ? 1 : 0);
            const int cs = c - segs.off[s];
            float4 y;
            if (segs.norm[s]) *reinterpret_cast<float4*>(nw_s + c) = *reinterpret_cast<const float4*>(segs.norm[s] + cs);
            if (segs.w[s]) {
                float4 u[MT], w[MT];
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    u[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    w[j] = u[j];
                    const int back = taps - 1 - j;
                    if (j < taps && back <= pos) {               // zeros before the sequence's start
                        const float* src = back <= i_in ? proj + (size_t)(t - back) * ld + c
                                                        : st + (size_t)(taps - 1 - (back - i_in)) * C + c;
                        u[j] = *reinterpret_cast<const float4*>(src);
                        w[j] = *reinterpret_cast<const float4*>(segs.w[s] + (size_t)j * segs.width[s] + cs);
                    }
                }
                y = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    y.x = fmaf(w[j].x, u[j].x, y.x);
                    y.y = fmaf(w[j].y, u[j].y, y.y);
                    y.z = fmaf(w[j].z, u[j].z, y.z);
                    y.w = fmaf(w[j].w, u[j].w, y.w);
                }
            } else {
                y = *reinterpret_cast<const float4*>(proj + (size_t)t * ld + c);
            }
            *reinterpret_cast<float4*>(y_s + c) = y;
            float ss = y.x * y.x;
            ss = fmaf(y.y, y.y, ss); ss = fmaf(y.z, y.z, ss); ss = fmaf(y.w, y.w, ss);
            if (s == 0) ss0 += ss; else if (s == 1) ss1 += ss;
        }
        if (segs.norm[0]) ss0 = block_sum<256>(ss0, red);      // uniform over the block
        if (segs.norm[1]) { __syncthreads(); ss1 = block_sum<256>(ss1, red); }
        if (threadIdx.x == 0) {
            rs_s[0] = segs.norm[0] ? rsqrtf(ss0 / (float)segs.width[0] + eps) : 1.f;
            rs_s[1] = segs.norm[1] ? rsqrtf(ss1 / (float)segs.width[1] + eps) : 1.f;
            rs_s[2] = 1.f;
        }
    } else {
        for (int s = 0; s < segs.n; ++s) {
            const int off = segs.off[s], width = segs.width[s];
            float ss = 0.f;
            for (int c = threadIdx.x; c < width; c += 256) {
                float y;
                if (segs.norm[s]) nw_s[off + c] = segs.norm[s][c];
                if (segs.w[s]) {
                    y = 0.f;
                    for (int j = 0; j < taps; ++j) {
                        const int back = taps - 1 - j;
                        if (back > pos) continue;
                        const float u = back <= i_in ? proj[(size_t)(t - back) * ld + off + c]
                                                     : st[(size_t)(taps - 1 - (back - i_in)) * C + off + c];
                        y = fmaf(segs.w[s][(size_t)j * width + c], u, y);
                    }
                } else {
                    y = proj[(size_t)t * ld + off + c];
                }
                y_s[off + c] = y;
                ss = fmaf(y, y, ss);
            }
            if (segs.norm[s]) {                                  // uniform over the block
                ss = block_sum<256>(ss, red);
                if (threadIdx.x == 0) rs_s[s] = rsqrtf(ss / (float)width + eps);
                __syncthreads();                                 // red is used again
            } else if (threadIdx.x == 0) {
                rs_s[s] = 1.f;
            }
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = rot_dims >> 1;
    for (int head = warp; head < nq + 2 * nkv; head += 8) {
        const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
        TC* slot = nullptr;
        if (!is_q) {
            if (page < 0) continue;                           // no page: the host never schedules this
            const int kvh = is_k ? head - nq : head - nq - nkv;
            slot = cache + (size_t)page * L.page_stride + (size_t)layer * L.layer_stride + (is_k ? 0 : L.kv_stride) +
                   (size_t)kvh * L.head_stride + (size_t)(pos % L.page_size) * dc;
        }
        if (!is_q && !is_k) {                                 // a value head: as it left the convolution
            const float* src = y_s + segs.off[2] + (size_t)(head - nq - nkv) * dv;
            if (pairs) for (int i = lane * 2; i < dv; i += 64) store_pair(slot + i, src[i], src[i + 1]);
            else for (int i = lane; i < dv; i += 32) slot[i] = from_f32<TC>(src[i]);
            continue;
        }
        const int s = is_q ? 0 : 1;
        const int col = segs.off[s] + (is_q ? head * d : (head - nq) * d);
        const float* w = segs.norm[s] ? nw_s + col : nullptr;
        if (is_q) finish_head<TQ>(q_out + (size_t)t * nq * d + (size_t)head * d, y_s + col, w, rs_s[0], cos_s, sin_s, half,
                                  d, interleaved, pairs != 0, lane);
        else finish_head<TC>(slot, y_s + col, w, rs_s[1], cos_s, sin_s, half, d, interleaved, pairs != 0, lane);
    }
}

// y = act(x) elementwise: 2 = the square of relu.  clear: x is set to zero behind the read (an accumulator buffer).
template <typename TI, typename TO>
__global__ void unary_act_kernel(TI* x, TO* y, long long n, int act, int clear) {   // x and y may be one buffer
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = to_f32<TI>(x[i]);
    if (clear) x[i] = from_f32<TI>(0.f);
    if (act == 2) { v = fmaxf(v, 0.f); v = v * v; }
    y[i] = from_f32<TO>(v);
}

}  // namespace

// seg_off / seg_width / seg_w / seg_norm: arrays of num_segs (<= 3) entries; the segments lie one behind the other
// from column 0 and their widths add up to C <= ld.  state [slots, taps-1, C] float32.
TFF_API int tff_short_conv_norm(const float* proj, int ld, float* out, int num_segs, const int* seg_width,
                                const float* const* seg_w, const float* const* seg_norm, int taps, float eps,
                                const float* state, const int* positions, const int* tok_req, const int* q_start,
                                const int* slots, int num_tokens, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (!proj || !out || num_segs <= 0 || num_segs > MAX_SEGS || taps < 1 || taps > MAX_TAPS) return TFF_ERR_BAD_ARGUMENT;
    ConvSegs segs;
    segs.n = num_segs;
    int C = 0;
    for (int s = 0; s < MAX_SEGS; ++s) {
        segs.off[s] = C;
        segs.width[s] = s < num_segs ? seg_width[s] : 0;
        segs.w[s] = s < num_segs ? seg_w[s] : nullptr;
        segs.norm[s] = s < num_segs ? seg_norm[s] : nullptr;
        if (s < num_segs && seg_width[s] <= 0) return TFF_ERR_BAD_ARGUMENT;
        C += segs.width[s];
    }
    if (C > ld || (taps > 1 && !state)) return TFF_ERR_BAD_ARGUMENT;
    short_conv_norm_kernel<<<num_tokens, 256, 0, stream>>>(proj, ld, out, segs, taps, C, state, positions, tok_req,
                                                           q_start, slots, eps);
    return tff_launch_status();
}

// short_conv_norm and qkv_finish in one kernel, for three segments q (nq*d), k (nkv*d), v (nkv*dv) with a paged cache;
// seg_w are the convolution's weights TRANSPOSED, [taps, width]:
// q_dt, cache_dt: 0 = float32, 1 = bfloat16.  TFF_ERR_UNSUPPORTED when a token's channels do not fit shared memory.
TFF_API int tff_conv_finish(const float* proj, int ld, const float* const* seg_w, const float* const* seg_norm, int taps,
                            float eps, const float* state, const int* positions, const int* tok_req, const int* q_start,
                            const int* slots, void* q_out, int q_dt, const float* freq, int rot_dims, float magnitude,
                            int interleaved, const int* block_table, int table_width, void* cache, int cache_dt,
                            int cache_layers, int layer, int page_size, int dc, int gate_off, float* gate_out,
                            int num_tokens, int nq, int nkv, int d, int dv, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (!proj || !q_out || !cache || !block_table || taps < 1 || taps > MAX_TAPS || nq <= 0 || nkv <= 0 || d <= 0 || dv <= 0 ||
        rot_dims < 0 || rot_dims > d || (rot_dims & 1) || page_size <= 0 || dc < d || dc < dv)
        return TFF_ERR_BAD_ARGUMENT;
    if ((rot_dims > 0 && !freq) || (taps > 1 && !state) || (gate_out && gate_off < 0)) return TFF_ERR_BAD_ARGUMENT;
    ConvSegs segs;
    segs.n = 3;
    const int widths[3] = {nq * d, nkv * d, nkv * dv};
    int C = 0;
    for (int s = 0; s < 3; ++s) {
        segs.off[s] = C; segs.width[s] = widths[s]; segs.w[s] = seg_w[s]; segs.norm[s] = s < 2 ? seg_norm[s] : nullptr;
        C += widths[s];
    }
    if (C > ld || (gate_out && gate_off + nq > ld)) return TFF_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)(C + widths[0] + widths[1] + 32 + rot_dims) * sizeof(float);
    if (smem > 200 * 1024) return TFF_ERR_UNSUPPORTED;
    // two elements a store where every head, rotated part and cache row starts on an even element of an aligned buffer
    const int pairs = (((rot_dims >> 1) | d | dv | dc) & 1) == 0 && (((size_t)q_out | (size_t)cache) & 7) == 0 ? 1 : 0;
    const KvLayout L = make_kv_layout(cache_layers, nkv, page_size, dc);
#define TFF_CF(TQ, TC, MT)                                                                                               \
    do {                                                                                                              \
        if (smem > 48 * 1024 &&                                                                                       \
            cudaFuncSetAttribute(conv_finish_kernel<TQ, TC, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
            return TFF_ERR_LAUNCH;                                                                                    \
        return tff_launch_pdl(conv_finish_kernel<TQ, TC, MT>, dim3(num_tokens), dim3(256), smem, stream, proj, ld, segs, taps, C, \
            state, positions, tok_req, q_start, slots, eps, (TQ*)q_out, freq, rot_dims, magnitude, interleaved, block_table,  \
            table_width, (TC*)cache, L, layer, dc, gate_off, gate_out, nq, nkv, d, dv, pairs);                           \
    } while (0)
    if (taps <= 4) {
        if (q_dt == 0 && cache_dt == 0) TFF_CF(float, float, 4);
        if (q_dt == 1 && cache_dt == 1) TFF_CF(bf16, bf16, 4);
        if (q_dt == 0 && cache_dt == 1) TFF_CF(float, bf16, 4);
    } else {
        if (q_dt == 0 && cache_dt == 0) TFF_CF(float, float, MAX_TAPS);
        if (q_dt == 1 && cache_dt == 1) TFF_CF(bf16, bf16, MAX_TAPS);
        if (q_dt == 0 && cache_dt == 1) TFF_CF(float, bf16, MAX_TAPS);
    }
#undef TFF_CF
    return TFF_ERR_BAD_ARGUMENT;
}

TFF_API int tff_short_conv_state(float* proj, int ld, int clear, int taps, int C, float* state, const int* q_start,
                                 const int* pos_start, const int* slots, int num_requests, cudaStream_t stream) {
    if (num_requests <= 0 || (taps <= 1 && !clear)) return TFF_OK;
    if (!proj || C > ld || taps > MAX_TAPS || (taps > 1 && !state)) return TFF_ERR_BAD_ARGUMENT;
    dim3 grid(num_requests, (ld + 255) / 256);
    return tff_launch_pdl(short_conv_state_kernel, grid, dim3(256), 0, stream, proj, ld, clear, taps, taps > 1 ? C : 0, state,
                          q_start, pos_start, slots);
}

TFF_API int tff_pair_embed(const int* tokens, const int* positions, const int* tok_req, const int* q_start,
                           const int* slots, int* state, const void* table, int table_is_bf16, int buckets,
                           long long mul_prev, long long mul_cur, float* x, int copies, int W, int num_tokens,
                           int num_requests, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (!state || !table || !x || buckets <= 0 || copies <= 0 || W <= 0) return TFF_ERR_BAD_ARGUMENT;
    int st;
    if (table_is_bf16)
        st = tff_launch_pdl(pair_embed_kernel<bf16>, dim3(num_tokens), dim3(128), 0, stream, tokens, positions, tok_req,
                            q_start, slots, (const int*)state, (const bf16*)table, buckets, mul_prev, mul_cur, x, copies, W);
    else
        st = tff_launch_pdl(pair_embed_kernel<float>, dim3(num_tokens), dim3(128), 0, stream, tokens, positions, tok_req,
                            q_start, slots, (const int*)state, (const float*)table, buckets, mul_prev, mul_cur, x, copies, W);
    if (st != TFF_OK) return st;
    return tff_launch_pdl(last_token_kernel, dim3((num_requests + 127) / 128), dim3(128), 0, stream, tokens, q_start,
                          slots, state, num_requests);
}

// x_dt, y_dt: 0 = float32, 1 = bfloat16 (float32 -> bfloat16, or the same type on both sides; in place is fine).
TFF_API int tff_unary_act(void* x, int x_dt, void* y, int y_dt, long long n, int act, int clear, cudaStream_t stream) {
    if (n <= 0) return TFF_OK;
    if (act != 2 || (clear && x == y)) return TFF_ERR_BAD_ARGUMENT;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (x_dt == 1 && y_dt == 1)
        return tff_launch_pdl(unary_act_kernel<bf16, bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, (bf16*)y, n, act, clear);
    if (x_dt == 0 && y_dt == 1)
        return tff_launch_pdl(unary_act_kernel<float, bf16>, dim3(blocks), dim3(256), 0, stream, (float*)x, (bf16*)y, n, act, clear);
    if (x_dt == 0 && y_dt == 0)
        return tff_launch_pdl(unary_act_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (float*)x, (float*)y, n, act, clear);
    return TFF_ERR_BAD_ARGUMENT;
}
