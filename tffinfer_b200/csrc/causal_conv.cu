// A short causal convolution over time with a bias and an activation, on a block of columns of a projection's float32
// rows, and the per-request rows that carry it from one step to the next:
//
//     y[t, c] = act( bias[c] + sum_j w[c, j] * u[t - (taps - 1) + j, c] )      j = 0 .. taps-1, zeros ahead of position 0
//
// u = columns col0 .. col0 + C of ``proj`` [T, ld]; y goes to ``out`` [T, C] float32.  The taps-1 rows of u ahead of a
// request's first token of the step come from its slot: state + slot * slot_stride + state_off holds [taps-1, C]
// float32, the oldest row first.  A tap that reaches back beyond position 0 reads zero, whatever the slot holds.
// The second kernel, launched behind the first, leaves a request's last taps-1 rows of u in its slot (older rows move
// up when the portion is shorter than that).  In a step in which every request brings one token the first kernel does
// that itself (``update_state``): the thread of a channel has read all of the channel's rows before it writes them.
// act: 0 none, 1 silu.
#include "common.cuh"

namespace {

constexpr int CONV_MAX_TAPS = 16;

__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* __restrict__ proj, int ld, int col0, int C, const float* __restrict__ w,
                   const float* __restrict__ bias, int taps, int act, float* __restrict__ state,
                   long long slot_stride, long long state_off, const int* __restrict__ positions,
                   const int* __restrict__ tok_req, const int* __restrict__ q_start, const int* __restrict__ slots,
                   float* __restrict__ out, int update_state) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= C) return;
    const int b = tok_req[t], pos = positions[t];
    const int i_in = t - q_start[b];                        // the token's place in its request's portion
    float* st = state ? state + (size_t)slots[b] * slot_stride + state_off : nullptr;
    float wc[CONV_MAX_TAPS];
    for (int j = 0; j < taps; ++j) wc[j] = w[(size_t)c * taps + j];
    float y = bias ? bias[c] : 0.f;
    pdl_wait();
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                      // how many tokens before this one
        if (back > pos) continue;                           // ahead of the sequence's start
        const float u = __ldcg(back <= i_in ? proj + (size_t)(t - back) * ld + col0 + c       // past the first-level cache:
                                            : st + (size_t)(taps - 1 - (back - i_in)) * C + c);   // kernels ahead wrote these
        y = fmaf(wc[j], u, y);
    }
    if (act == 1) y = y / (1.f + expf(-y));
    out[(size_t)t * C + c] = y;
    if (update_state && taps > 1) {                         // the request's one token: its rows move up by one
        for (int i = 0; i + 2 < taps; ++i) st[(size_t)i * C + c] = __ldcg(st + (size_t)(i + 1) * C + c);
        st[(size_t)(taps - 2) * C + c] = __ldcg(proj + (size_t)t * ld + col0 + c);
    }
}

__global__ void __launch_bounds__(256)
causal_conv_state_kernel(const float* __restrict__ proj, int ld, int col0, int C, int taps, float* __restrict__ state,
                         long long slot_stride, long long state_off, const int* __restrict__ q_start,
                         const int* __restrict__ slots) {
    pdl_launch_dependents();
    const int b = blockIdx.x;
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= C) return;
    const int t0 = q_start[b], n = q_start[b + 1] - t0, keep = taps - 1;
    if (n <= 0) return;
    float* st = state + (size_t)slots[b] * slot_stride + state_off;
    pdl_wait();
    for (int i = 0; i < keep; ++i) {                        // row i of the new state: the token keep - i before the next one
        const int from_end = keep - i;                      // 1 = the portion's last token
        st[(size_t)i * C + c] = __ldcg(from_end <= n ? proj + (size_t)(t0 + n - from_end) * ld + col0 + c
                                                     : st + (size_t)(i + n) * C + c);       // an older row moves up (i + n > i)
    }
}

}  // namespace

TFF_API int tff_causal_conv(const float* proj, int ld, int col0, int C, const float* w, const float* bias, int taps,
                            int act, float* state, long long slot_stride, long long state_off,
                            const int* positions, const int* tok_req, const int* q_start, const int* slots, float* out,
                            int num_tokens, int update_state, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (!proj || !w || !out || C <= 0 || col0 < 0 || col0 + C > ld || taps < 1 || taps > CONV_MAX_TAPS ||
        (taps > 1 && !state) || act < 0 || act > 1)
        return TFF_ERR_BAD_ARGUMENT;
    return tff_launch_pdl(causal_conv_kernel, dim3(num_tokens, (C + 255) / 256), dim3(256), 0, stream, proj, ld, col0, C, w,
                          bias, taps, act, state, slot_stride, state_off, positions, tok_req, q_start, slots, out, update_state);
}

TFF_API int tff_causal_conv_state(const float* proj, int ld, int col0, int C, int taps, float* state, long long slot_stride,
                                  long long state_off, const int* q_start, const int* slots, int num_requests,
                                  cudaStream_t stream) {
    if (num_requests <= 0 || taps <= 1) return TFF_OK;
    if (!proj || !state || C <= 0 || col0 < 0 || col0 + C > ld || taps > CONV_MAX_TAPS) return TFF_ERR_BAD_ARGUMENT;
    return tff_launch_pdl(causal_conv_state_kernel, dim3(num_requests, (C + 255) / 256), dim3(256), 0, stream, proj, ld,
                          col0, C, taps, state, slot_stride, state_off, q_start, slots);
}
