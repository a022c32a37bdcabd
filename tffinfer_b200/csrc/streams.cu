// A residual that is several streams (hyper-connections), with layer scale: one kernel does what lies
// between two sublayers.  x holds S float32 copies of the residual per token, [rows, S, W].
//
//   write (when y is given):  x'[t] = sum_s mix[s, t] x[s] + out[t] * (scale * y),  all t from the old x[s]
//   read  (when h is given):  u = sum_s in[s] x'[s];  h = u * rsqrt(mean(u^2) + eps) * w
//
// y may be cleared behind the read (it is then one of the accumulator buffers that split products add into).
// mix, out, in are float32 [S, S], [S], [S]; a null pointer stands for the identity matrix, ones, ones, so
// S = 1 with null pointers is the plain pre-norm residual with layer scale.  scale and w may be null (ones).
// One CTA per row; a thread owns columns and holds the S values of a column in registers, so the update
// is in place.  Every sum runs over s in ascending order and the row's sum of squares is reduced in an order that
// depends on W alone: a row's result does not depend on what else is in the batch.
// With row_index, CTA r works on row row_index[r] (both parts) and h is written to row r; the row's new streams
// feed h and are not stored (a row may be listed twice): the last sublayer's write and the model's final norm only
// ever matter at the rows whose logits are wanted, and the streams live for one step.
#include "common.cuh"

namespace {

constexpr int MOST_STREAMS = 16;

// four consecutive outputs in one store
template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// MAX_STREAMS: the register arrays' size, the smallest of 4, 8, 16 that holds S
template <typename TO, int NT, int MAX_STREAMS>
__global__ void __launch_bounds__(NT)
stream_step_kernel(float* __restrict__ x, int S, int W,
                   float* __restrict__ y, int clear_y, const float* __restrict__ scale,
                   const float* __restrict__ mix, const float* __restrict__ outw,
                   const float* __restrict__ inw, const float* __restrict__ w, float eps,
                   const int* __restrict__ row_index, TO* __restrict__ h, float* __restrict__ total,
                   const float* __restrict__ bias) {
    extern __shared__ __align__(16) float u_row[];   // W floats: the combined row, kept between the two passes
    __shared__ float red[32];
    __shared__ float c_mix[MAX_STREAMS * MAX_STREAMS], c_out[MAX_STREAMS], c_in[MAX_STREAMS];
    static_assert(MAX_STREAMS * MAX_STREAMS <= NT * 4, "the coefficients are loaded in a few passes");
    pdl_launch_dependents();
    // the coefficients and the row index are older than the kernel ahead
    for (int e = threadIdx.x; e < S * S; e += NT) c_mix[e] = mix ? mix[e] : ((e / S == e % S) ? 1.f : 0.f);
    if (threadIdx.x < S) {
        c_out[threadIdx.x] = outw ? outw[threadIdx.x] : 1.f;
        c_in[threadIdx.x] = inw ? inw[threadIdx.x] : 1.f;
    }
    const int r = blockIdx.x;
    const int row = row_index ? row_index[r] : r;
    __syncthreads();
    pdl_wait();
    float* xr = x + (size_t)row * S * W;
    float* yr = y ? y + (size_t)row * W : nullptr;
    const bool store_x = row_index == nullptr;       // chosen rows: the new streams feed h and are not kept
    float ss = 0.f;
    // four columns a thread at a time (16-byte accesses) when the rows allow it; which path runs depends on W and
    // the buffers' alignment alone, so a row's sums are always added in the same order
    const bool vec = MAX_STREAMS <= 8 && (W & 3) == 0 &&
                     (((uintptr_t)x | (uintptr_t)y | (uintptr_t)scale | (uintptr_t)total | (uintptr_t)bias) & 15) == 0;
    if (vec) {
        const int W4 = W >> 2;
        for (int i = threadIdx.x; i < W4; i += NT) {
            float4 v[MAX_STREAMS];
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                v[s] = s < S ? reinterpret_cast<const float4*>(xr + (size_t)s * W)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (yr) {
                float4 ys = reinterpret_cast<const float4*>(yr)[i];
                if (clear_y) reinterpret_cast<float4*>(yr)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (scale) {
                    const float4 g = reinterpret_cast<const float4*>(scale)[i];
                    ys.x *= g.x; ys.y *= g.y; ys.z *= g.z; ys.w *= g.w;
                }
                float4 n[MAX_STREAMS];
#pragma unroll
                for (int t = 0; t < MAX_STREAMS; ++t) {
                    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int s = 0; s < MAX_STREAMS; ++s)
                        if (s < S && t < S) {
                            const float m = c_mix[s * S + t];
                            a.x = fmaf(m, v[s].x, a.x); a.y = fmaf(m, v[s].y, a.y);
                            a.z = fmaf(m, v[s].z, a.z); a.w = fmaf(m, v[s].w, a.w);
                        }
                    const float o = t < S ? c_out[t] : 0.f;
                    n[t] = make_float4(fmaf(o, ys.x, a.x), fmaf(o, ys.y, a.y), fmaf(o, ys.z, a.z), fmaf(o, ys.w, a.w));
                }
#pragma unroll
                for (int t = 0; t < MAX_STREAMS; ++t)
                    if (t < S) { v[t] = n[t]; if (store_x && !bias) reinterpret_cast<float4*>(xr + (size_t)t * W)[i] = n[t]; }
            }
            if (bias) {                               // a vector added to every stream, behind the write
                const float4 bv = reinterpret_cast<const float4*>(bias)[i];
#pragma unroll
                for (int t = 0; t < MAX_STREAMS; ++t)
                    if (t < S) {
                        v[t].x += bv.x; v[t].y += bv.y; v[t].z += bv.z; v[t].w += bv.w;
                        if (store_x) reinterpret_cast<float4*>(xr + (size_t)t * W)[i] = v[t];
                    }
            }
            if (h || total) {
                float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s)
                    if (s < S) {
                        const float m = c_in[s];
                        u.x = fmaf(m, v[s].x, u.x); u.y = fmaf(m, v[s].y, u.y);
                        u.z = fmaf(m, v[s].z, u.z); u.w = fmaf(m, v[s].w, u.w);
                    }
                reinterpret_cast<float4*>(u_row)[i] = u;
                ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(u.z, u.z, ss); ss = fmaf(u.w, u.w, ss);
                if (total) reinterpret_cast<float4*>(total + (size_t)r * W)[i] = u;
            }
        }
        if (!h) return;
        ss = block_sum<NT>(ss, red);
        const float rs = rsqrtf(ss / (float)W + eps);
        TO* o = h + (size_t)r * W;
        const bool wvec = (((uintptr_t)w) & 15) == 0 && (((uintptr_t)o) & (sizeof(TO) == 2 ? 7 : 15)) == 0;
        for (int i = threadIdx.x; i < W4; i += NT) {  // a thread reads back what it wrote itself
            const float4 u = reinterpret_cast<const float4*>(u_row)[i];
            float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
            if (w) g = wvec ? reinterpret_cast<const float4*>(w)[i] : make_float4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
            if (wvec) {
                store4<TO>(o + 4 * i, (u.x * rs) * g.x, (u.y * rs) * g.y, (u.z * rs) * g.z, (u.w * rs) * g.w);
            } else {
                o[4 * i] = from_f32<TO>((u.x * rs) * g.x); o[4 * i + 1] = from_f32<TO>((u.y * rs) * g.y);
                o[4 * i + 2] = from_f32<TO>((u.z * rs) * g.z); o[4 * i + 3] = from_f32<TO>((u.w * rs) * g.w);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += NT) {
        float v[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) v[s] = s < S ? xr[(size_t)s * W + i] : 0.f;
        if (yr) {
            const float ys = scale ? yr[i] * scale[i] : yr[i];
            if (clear_y) yr[i] = 0.f;
            float n[MAX_STREAMS];
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s) if (s < S && t < S) a = fmaf(c_mix[s * S + t], v[s], a);
                n[t] = t < S ? fmaf(c_out[t], ys, a) : 0.f;
            }
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) if (t < S) { v[t] = n[t]; if (store_x && !bias) xr[(size_t)t * W + i] = n[t]; }
        }
        if (bias) {
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) if (t < S) { v[t] += bias[i]; if (store_x) xr[(size_t)t * W + i] = v[t]; }
        }
        if (h || total) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s) if (s < S) u = fmaf(c_in[s], v[s], u);
            u_row[i] = u;
            ss = fmaf(u, u, ss);
            if (total) total[(size_t)r * W + i] = u;
        }
    }
    if (!h) return;
    ss = block_sum<NT>(ss, red);
    const float rs = rsqrtf(ss / (float)W + eps);
    TO* o = h + (size_t)r * W;
    for (int i = threadIdx.x; i < W; i += NT) {       // a thread reads back what it wrote itself
        const float g = w ? w[i] : 1.f;
        o[i] = from_f32<TO>((u_row[i] * rs) * g);
    }
}

// out[t, c, :] = E[token[t], :] * scale for c < copies: the embedding output as the start of every stream.
template <typename TW>
__global__ void embed_streams_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                     float* __restrict__ out, int hidden, int vocab, float scale, int copies) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (size_t)t * copies * hidden;
    const bool bad = tok < 0 || tok >= vocab;            // never a wrong row: poison instead
    const TW* row = table + (size_t)(bad ? 0 : tok) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = bad ? __int_as_float(0x7fc00000) : to_f32<TW>(row[i]) * scale;
        for (int c = 0; c < copies; ++c) o[(size_t)c * hidden + i] = v;
    }
}

}  // namespace

// x [rows_total, S, W] float32 (updated in place when y is given); y [rows_total, W] float32 or null;
// h [rows, W] of the activation type or null; total [rows, W] float32 or null (the combined row itself).
// clear_y != 0: the rows of y that were read are set to zero (y is then an accumulator buffer that the next split
// product adds into).  bias [W] float32 or null: added to every stream behind the write, ahead of the read.
TFF_API int tff_stream_step(float* x, int S, int W, float* y, int clear_y, const float* scale, const float* mix,
                            const float* outw, const float* inw, const float* w, float eps, const int* row_index,
                            void* h, int h_is_bf16, float* total, int rows, const float* bias, cudaStream_t stream) {
    if (rows <= 0) return TFF_OK;
    if (!x || S <= 0 || W <= 0) return TFF_ERR_BAD_ARGUMENT;
    if (S > MOST_STREAMS) return TFF_ERR_UNSUPPORTED;
    const size_t smem = (size_t)W * sizeof(float);
    if (smem > 96 * 1024) return TFF_ERR_UNSUPPORTED;
#define TFF_STREAM_LAUNCH(TO, NT)                                                                              \
    do {                                                                                                       \
        if (S <= 4) TFF_STREAM_LAUNCH_S(TO, NT, 4);                                                            \
        if (S <= 8) TFF_STREAM_LAUNCH_S(TO, NT, 8);                                                            \
        TFF_STREAM_LAUNCH_S(TO, NT, 16);                                                                       \
    } while (0)
#define TFF_STREAM_LAUNCH_S(TO, NT, MS)                                                                        \
    do {                                                                                                       \
        auto kern = stream_step_kernel<TO, NT, MS>;                                                            \
        if (smem > 48 * 1024) {                                                                                \
            static bool configured = false;                                                                    \
            if (!configured) {                                                                                 \
                if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess) \
                    return TFF_ERR_LAUNCH;                                                                     \
                configured = true;                                                                             \
            }                                                                                                  \
        }                                                                                                      \
        return tff_launch_pdl(kern, dim3(rows), dim3(NT), smem, stream, x, S, W, y, clear_y, scale, mix, outw, inw, w, \
                              eps, row_index, (TO*)h, total, bias);                                                  \
    } while (0)
    if (W >= 1024) {
        if (h_is_bf16) TFF_STREAM_LAUNCH(bf16, 256);
        TFF_STREAM_LAUNCH(float, 256);
    }
    if (h_is_bf16) TFF_STREAM_LAUNCH(bf16, 64);
    TFF_STREAM_LAUNCH(float, 64);
#undef TFF_STREAM_LAUNCH
#undef TFF_STREAM_LAUNCH_S
}

TFF_API int tff_embed_streams(const int* tokens, const void* table, int table_is_bf16, float* out, int num_tokens,
                              int hidden, int vocab, float scale, int copies, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (hidden <= 0 || vocab <= 0 || copies <= 0) return TFF_ERR_BAD_ARGUMENT;
    const int nt = hidden >= 1024 ? 256 : 128;
    if (table_is_bf16)
        return tff_launch_pdl(embed_streams_kernel<bf16>, dim3(num_tokens), dim3(nt), 0, stream, tokens,
                              (const bf16*)table, out, hidden, vocab, scale, copies);
    return tff_launch_pdl(embed_streams_kernel<float>, dim3(num_tokens), dim3(nt), 0, stream, tokens,
                          (const float*)table, out, hidden, vocab, scale, copies);
}
