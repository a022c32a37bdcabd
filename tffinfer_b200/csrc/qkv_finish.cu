// What lies between a mixer's merged projection and its token mixing, for mixers whose rotation is not the
// table-driven whole-head rotate-half one of elementwise.cu: one warp per (token, head) of the projection row
//   proj[t] = [q (nq*d) | k (nkv*d) | v (nkv*dv) | ... ]      float32 accumulators or the activation type
// * q and k: the first rot_dims dimensions of a head are rotated by the token's position, the rest pass.  The angle
//   of pair i is float(position) * freq[i] (one float32 product; freq is an array of rot_dims/2 frequencies, so any
//   rescaling of them is the caller's), cos and sin are multiplied by ``magnitude``.  Pairs are (2i, 2i+1)
//   (interleaved) or (i, i + rot_dims/2) (halves).  k is then multiplied by k_scale.
// * ``bias`` (float32, laid out like the row's q | k | v columns, or null) is added to q, k and v ahead of everything else;
//   with ``unit_eps`` > 0 every q and k head is divided, after the rotation, by its root mean square
//   sqrt(mean(x^2) + unit_eps) (an RMS norm without a weight).
// * q goes to q_out [T, nq*d]; k to the token's slot of the paged cache or, without a cache, to k_out [T, nkv*d].
// * v: value mixing across layers.  v_mode 0: as it is.  1: the layer is the source, its values are also kept,
//   unrounded, in v_share [T, nkv*dv] float32.  2: v <- (1 - lambda) v + lambda v_share[t], lambda a float32 scalar on
//   the device.  The (mixed) v goes to the token's slot of the cache; without a cache v is left where it is.
// * head gates: gate_out[t, h] = sigmoid(proj[t, gate_off + h]) for the nq query heads, when gate_out is given.
// With ``clear_input`` every element of the row that the kernel has consumed is set to zero behind the read (q, k,
// the gates, and v where there is a cache to take it): the row is then an accumulator buffer that the next split
// product adds into.
// The cache is [pages, layers, 2, kv heads, page, dc] with dc >= max(d, dv): keys use the first d elements of a
// slot, values the first dv.
// Everything is computed in float32; only the stores round.
#include "common.cuh"

namespace {

template <typename TIN, typename TQ, typename TC>
__global__ void __launch_bounds__(128)
qkv_finish_kernel(TIN* __restrict__ proj, int clear_input, int ld, TQ* __restrict__ q_out, float* __restrict__ k_out,
                  const float* __restrict__ freq, int rot_dims, float magnitude, int interleaved, float k_scale,
                  const int* __restrict__ positions, const int* __restrict__ tok_req,
                  const int* __restrict__ block_table, int table_width,
                  TC* __restrict__ cache, KvLayout L, int layer, int dc,
                  int v_mode, float* __restrict__ v_share, const float* __restrict__ lambda,
                  int gate_off, float* __restrict__ gate_out,
                  int nq, int nkv, int d, int dv, const float* __restrict__ bias, float unit_eps) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    const int head = blockIdx.x * 4 + warp;
    const int heads = nq + 2 * nkv + (gate_out ? 1 : 0);
    if (head >= heads) return;
    const int pos = positions[t];
    pdl_wait();
    TIN* row = proj + (size_t)t * ld;
    const TIN zero = from_f32<TIN>(0.f);
    if (head == nq + 2 * nkv) {                                   // the head gates of this token
        for (int h = lane; h < nq; h += 32) {
            const float g = to_f32<TIN>(row[gate_off + h]);
            if (clear_input) row[gate_off + h] = zero;
            gate_out[(size_t)t * nq + h] = 1.0f / (1.0f + expf(-g));
        }
        return;
    }
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    TC* slot = nullptr;
    if (!is_q && cache != nullptr) {
        const int kvh = is_k ? head - nq : head - nq - nkv;
        const int page = block_table[(size_t)tok_req[t] * table_width + pos / L.page_size];
        if (page < 0) return;                                     // no page: the host never schedules this
        slot = cache + (size_t)page * L.page_stride + (size_t)layer * L.layer_stride + (is_k ? 0 : L.kv_stride) +
               (size_t)kvh * L.head_stride + (size_t)(pos % L.page_size) * dc;
    }
    if (!is_q && !is_k) {                                         // a value head
        const int kvh = head - nq - nkv;
        TIN* src = row + (size_t)(nq + nkv) * d + (size_t)kvh * dv;
        const float* vb = bias ? bias + (size_t)(nq + nkv) * d + (size_t)kvh * dv : nullptr;
        if (!slot && v_mode != 1) return;                         // nobody takes the values here: they stay in the row
        float* share = v_share ? v_share + (size_t)t * nkv * dv + (size_t)kvh * dv : nullptr;
        const float lam = v_mode == 2 ? *lambda : 0.f;
        for (int i = lane; i < dv; i += 32) {
            float v = to_f32<TIN>(src[i]) + (vb ? vb[i] : 0.f);
            if (clear_input && slot) src[i] = zero;
            if (v_mode == 1) share[i] = v;
            else if (v_mode == 2) v = (1.0f - lam) * v + lam * share[i];
            if (slot) slot[i] = from_f32<TC>(v);
        }
        return;
    }
    TIN* src = row + (size_t)head * d;                            // q heads, then k heads, all of size d
    const float* hb = bias ? bias + (size_t)head * d : nullptr;
    const int half = rot_dims >> 1;
    float ks = is_q ? 1.f : k_scale;
    if (unit_eps > 0.f) {                                         // the head's mean square behind the rotation, first
        float ss = 0.f;
        for (int i = lane; i < half; i += 32) {
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            const float a = to_f32<TIN>(src[ia]) + (hb ? hb[ia] : 0.f), b = to_f32<TIN>(src[ib]) + (hb ? hb[ib] : 0.f);
            float s, c;
            sincosf((float)pos * freq[i], &s, &c);
            s *= magnitude; c *= magnitude;
            const float ra = a * c - b * s, rb = b * c + a * s;
            ss = fmaf(ra, ra, ss); ss = fmaf(rb, rb, ss);
        }
        for (int i = 2 * half + lane; i < d; i += 32) {
            const float a = to_f32<TIN>(src[i]) + (hb ? hb[i] : 0.f);
            ss = fmaf(a, a, ss);
        }
        ss = warp_sum(ss);
        ks *= rsqrtf(ss / (float)d + unit_eps);
    }
    for (int i = lane; i < half; i += 32) {
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        const float a = to_f32<TIN>(src[ia]) + (hb ? hb[ia] : 0.f), b = to_f32<TIN>(src[ib]) + (hb ? hb[ib] : 0.f);
        if (clear_input) { src[ia] = zero; src[ib] = zero; }      // this lane alone reads these two
        float s, c;
        sincosf((float)pos * freq[i], &s, &c);
        s *= magnitude; c *= magnitude;
        const float ra = (a * c - b * s) * ks, rb = (b * c + a * s) * ks;
        if (is_q) {
            q_out[(size_t)t * nq * d + (size_t)head * d + ia] = from_f32<TQ>(ra);
            q_out[(size_t)t * nq * d + (size_t)head * d + ib] = from_f32<TQ>(rb);
        } else if (slot) {
            slot[ia] = from_f32<TC>(ra); slot[ib] = from_f32<TC>(rb);
        } else {
            k_out[(size_t)t * nkv * d + (size_t)(head - nq) * d + ia] = ra;
            k_out[(size_t)t * nkv * d + (size_t)(head - nq) * d + ib] = rb;
        }
    }
    for (int i = 2 * half + lane; i < d; i += 32) {
        const float a = (to_f32<TIN>(src[i]) + (hb ? hb[i] : 0.f)) * ks;
        if (clear_input) src[i] = zero;
        if (is_q) q_out[(size_t)t * nq * d + (size_t)head * d + i] = from_f32<TQ>(a);
        else if (slot) slot[i] = from_f32<TC>(a);
        else k_out[(size_t)t * nkv * d + (size_t)(head - nq) * d + i] = a;
    }
}

}  // namespace

// in_dt, q_dt, cache_dt: 0 = float32, 1 = bfloat16.  bias: float32 [nq*d + nkv*d + nkv*dv] or null; unit_eps: 0 = no norm.  q_out has q_dt; the cache cache_dt; k_out and v_share are float32.
TFF_API int tff_qkv_finish(
    void* proj, int in_dt, int clear_input, int ld, void* q_out, int q_dt, float* k_out,
    const float* freq, int rot_dims, float magnitude, int interleaved, float k_scale,
    const int* positions, const int* tok_req, const int* block_table, int table_width,
    void* cache, int cache_dt, int cache_layers, int layer, int page_size, int dc,
    int v_mode, float* v_share, const float* lambda, int gate_off, float* gate_out,
    int num_tokens, int nq, int nkv, int d, int dv, const float* bias, float unit_eps, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || rot_dims < 0 || rot_dims > d || (rot_dims & 1) || !proj || !q_out)
        return TFF_ERR_BAD_ARGUMENT;
    if (rot_dims > 0 && !freq) return TFF_ERR_BAD_ARGUMENT;
    if (cache && (!block_table || page_size <= 0 || dc < d || dc < dv)) return TFF_ERR_BAD_ARGUMENT;
    if (!cache && !k_out) return TFF_ERR_BAD_ARGUMENT;
    if ((v_mode == 1 || v_mode == 2) && !v_share) return TFF_ERR_BAD_ARGUMENT;
    if (v_mode == 2 && !lambda) return TFF_ERR_BAD_ARGUMENT;
    if (v_mode < 0 || v_mode > 2) return TFF_ERR_BAD_ARGUMENT;
    if (gate_out && gate_off < 0) return TFF_ERR_BAD_ARGUMENT;
    const KvLayout L = make_kv_layout(cache_layers, nkv, page_size > 0 ? page_size : 1, dc > 0 ? dc : 1);
    const int heads = nq + 2 * nkv + (gate_out ? 1 : 0);
    dim3 grid((heads + 3) / 4, num_tokens);
#define TFF_FIN(TIN, TQ, TC)                                                                                       \
    return tff_launch_pdl(qkv_finish_kernel<TIN, TQ, TC>, grid, dim3(128), 0, stream, (TIN*)proj, clear_input, ld, (TQ*)q_out, \
                          k_out, freq, rot_dims, magnitude, interleaved, k_scale, positions, tok_req, block_table,   \
                          table_width, (TC*)cache, L, layer, dc, v_mode, v_share, lambda, gate_off, gate_out, nq,     \
                          nkv, d, dv, bias, unit_eps)
    if (in_dt == 0 && q_dt == 0 && cache_dt == 0) TFF_FIN(float, float, float);
    if (in_dt == 0 && q_dt == 1 && cache_dt == 1) TFF_FIN(float, bf16, bf16);
    if (in_dt == 0 && q_dt == 0 && cache_dt == 1) TFF_FIN(float, float, bf16);
    if (in_dt == 1 && q_dt == 1 && cache_dt == 1) TFF_FIN(bf16, bf16, bf16);
#undef TFF_FIN
    return TFF_ERR_BAD_ARGUMENT;
}
