// A linear recurrence over a matrix state per head, with a decay that is read from the input at every token:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T          S [K, V] float32, a_t in (0, 1] on the K rows
//     o_t = S_t^T q_t (+ skip_h * v_t)
//
// It is the token mixing of gated linear attention (a decay per key channel) and of a selective state space (Mamba-2:
// one decay per head and token, q = C, k = dt * B, v = x).  How a_t is made is a mode of the kernel:
//   0  dec holds ln a per channel                          a = exp(dec[t, h, c])
//   1  dec holds a raw gate per channel                    a = sigmoid(dec[t, h, c] + dec_bias[h, c]) ^ inv_tau
//   2  dec holds a raw step size per head                  dt = softplus(dec[t, h] + dec_bias[h]),
//                                                          a = exp(-exp(rate_log[h]) * dt) on all rows, k <- dt * k
// Several heads may share one q and one k (``share`` heads a group).  All inputs are float32 rows (a product's
// accumulators), all arithmetic is float32, and a request's tokens are walked in order, whatever the step holds
// besides: a result does not depend on how a prompt was cut or on the batch.  The state of (slot, head) lies at
// state + slot * slot_stride + state_off + head * K * V; a request whose first token of the step is at position 0
// starts from zeros without reading its slot.
//
// One block of 128 threads owns VS = 128 / KS columns of one head of one request: thread (column, ks) keeps KPT rows
// of its column in registers, the K rows of a column being dealt to KS lanes of one warp (KS a power of two), whose
// partial sums of o meet by shuffles.  Tokens are staged eight at a time in shared memory (q, k and the decay of
// the head, the block's columns of v), the decays computed by the loading threads.
//
// A second kernel finishes such a mixer's output: RMS norm over groups of columns with a weight, and a silu gate ahead
// of the norm or behind it.
#include "common.cuh"

namespace {

constexpr int REC_THREADS = 128;
constexpr int REC_TOKENS = 8;       // tokens staged at a time
constexpr int REC_PAD = 4;          // floats between the row groups of two lanes: keeps 16-byte reads off one bank

struct RecArgs {
    const float* q; int q_ld, q_off;
    const float* k; int k_ld, k_off;
    const float* v; int v_ld, v_off;
    const float* dec; int dec_ld, dec_off;
    const float* dec_bias; const float* rate_log; const float* skip;
    int mode; float inv_tau, q_scale;
    float* state; long long slot_stride, state_off;
    const int* q_start; const int* pos_start; const int* slots;
    float* out; int out_ld;
    int H, K, V, share, KS;
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <int KPT>
__global__ void __launch_bounds__(REC_THREADS)
linear_recurrence_kernel(RecArgs a) {
    extern __shared__ __align__(16) float rec_smem[];
    pdl_launch_dependents();
    const int KS = a.KS, cpw = 32 / KS, VS = REC_THREADS / KS;
    const int RW = KS * (KPT + REC_PAD);                    // floats of one staged vector
    float* q_s = rec_smem;
    float* k_s = q_s + REC_TOKENS * RW;
    float* d_s = k_s + REC_TOKENS * RW;
    float* v_s = d_s + REC_TOKENS * RW;                     // [REC_TOKENS][VS]
    float* dt_s = v_s + REC_TOKENS * VS;                    // [REC_TOKENS][2]: step size, decay (mode 2)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int vc = warp * cpw + lane % cpw, ks = lane / cpw;
    const int head = blockIdx.y, b = blockIdx.z;
    const int v0 = blockIdx.x * VS, vcol = v0 + vc;
    const bool active = vcol < a.V;
    const int K = a.K, V = a.V;
    const int t0 = a.q_start[b], n = a.q_start[b + 1] - t0;
    if (n <= 0) return;
    const int grp = head / a.share;
    float* st = a.state + (size_t)a.slots[b] * a.slot_stride + a.state_off + (size_t)head * K * V;
    const bool fresh = a.pos_start[b] == 0;
    const float skip = a.skip ? a.skip[head] : 0.f;
    const float rate = a.mode == 2 ? expf(a.rate_log[head]) : 0.f;
    pdl_wait();
    float S[KPT];
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
        const int r = ks * KPT + j;
        S[j] = (!fresh && active && r < K) ? st[(size_t)r * V + vcol] : 0.f;
    }
    for (int base = 0; base < n; base += REC_TOKENS) {
        const int nb = min(REC_TOKENS, n - base);
        __syncthreads();                                    // the tokens staged before have been used
        if (a.mode == 2 && tid < nb) {
            const float raw = a.dec[(size_t)(t0 + base + tid) * a.dec_ld + a.dec_off + head] + a.dec_bias[head];
            const float dt = softplus_f(raw);
            dt_s[2 * tid] = dt;
            dt_s[2 * tid + 1] = expf(-rate * dt);
        }
        if (a.mode == 2) __syncthreads();
        for (int i = tid; i < nb * KS * KPT; i += REC_THREADS) {
            const int tt = i / (KS * KPT), r = i % (KS * KPT);
            const int at = tt * RW + (r / KPT) * (KPT + REC_PAD) + r % KPT;
            float qq = 0.f, kk = 0.f, dd = 1.f;
            if (r < K) {
                const size_t t = (size_t)(t0 + base + tt);
                qq = a.q[t * a.q_ld + a.q_off + grp * K + r] * a.q_scale;
                kk = a.k[t * a.k_ld + a.k_off + grp * K + r];
                if (a.mode == 2) { kk *= dt_s[2 * tt]; dd = dt_s[2 * tt + 1]; }
                else {
                    const float raw = a.dec[t * a.dec_ld + a.dec_off + head * K + r];
                    dd = a.mode == 0 ? expf(raw) : expf(log_sigmoid_f(raw + a.dec_bias[head * K + r]) * a.inv_tau);
                }
            }
            q_s[at] = qq; k_s[at] = kk; d_s[at] = dd;
        }
        for (int i = tid; i < nb * VS; i += REC_THREADS) {
            const int tt = i / VS, c = i % VS;
            v_s[i] = (v0 + c < V) ? a.v[(size_t)(t0 + base + tt) * a.v_ld + a.v_off + head * V + v0 + c] : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nb; ++tt) {
            const float vv = v_s[tt * VS + vc];
            const float4* q4 = reinterpret_cast<const float4*>(q_s + tt * RW + ks * (KPT + REC_PAD));
            const float4* k4 = reinterpret_cast<const float4*>(k_s + tt * RW + ks * (KPT + REC_PAD));
            const float4* d4 = reinterpret_cast<const float4*>(d_s + tt * RW + ks * (KPT + REC_PAD));
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < KPT / 4; ++j) {
                const float4 qv = q4[j], kv = k4[j], dv = d4[j];
                S[4 * j + 0] = fmaf(S[4 * j + 0], dv.x, kv.x * vv); acc = fmaf(S[4 * j + 0], qv.x, acc);
                S[4 * j + 1] = fmaf(S[4 * j + 1], dv.y, kv.y * vv); acc = fmaf(S[4 * j + 1], qv.y, acc);
                S[4 * j + 2] = fmaf(S[4 * j + 2], dv.z, kv.z * vv); acc = fmaf(S[4 * j + 2], qv.z, acc);
                S[4 * j + 3] = fmaf(S[4 * j + 3], dv.w, kv.w * vv); acc = fmaf(S[4 * j + 3], qv.w, acc);
            }
            for (int o = cpw; o < 32; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (ks == 0 && active)
                a.out[(size_t)(t0 + base + tt) * a.out_ld + head * V + vcol] = fmaf(skip, vv, acc);
        }
    }
    if (active) {
#pragma unroll
        for (int j = 0; j < KPT; ++j) {
            const int r = ks * KPT + j;
            if (r < K) st[(size_t)r * V + vcol] = S[j];
        }
    }
}

// out[t, out_off + c] = out_scale * y[c], c over ``width`` columns in groups of ``gs``:
//   gate_first 0:  y = o / rms_group(o) * w[c % wlen] * silu(g[c])
//   gate_first 1:  u = o * silu(g[c]),  y = u / rms_group(u) * w[c % wlen]
// o float32 [T, width]; g the columns g_off .. of the float32 rows ``gate`` (ld g_ld).  One block a token, a warp a
// group at a time; a group's sum of squares is added in an order that gs alone fixes.  With ``clear`` the columns
// clear_lo .. clear_hi of the token's row of ``gate`` are set to zero behind the reads (an accumulator buffer that
// the next split product adds into).
template <typename TO>
__global__ void __launch_bounds__(256)
gated_norm_kernel(const float* __restrict__ o, int width, int gs, float* __restrict__ gate, int g_ld, int g_off,
                  const float* __restrict__ w, int wlen, float eps, int gate_first, TO* __restrict__ out, int out_ld,
                  int out_off, float out_scale, int clear, int clear_lo, int clear_hi) {
    pdl_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* orow = o + (size_t)t * width;
    float* grow = gate + (size_t)t * g_ld;
    TO* dst = out + (size_t)t * out_ld + out_off;
    pdl_wait();
    for (int g = warp; g < width / gs; g += 8) {
        const int c0 = g * gs;
        float ss = 0.f;
        for (int c = c0 + lane; c < c0 + gs; c += 32) {
            float u = orow[c];
            if (gate_first) { const float z = grow[g_off + c]; u *= z / (1.f + expf(-z)); }
            ss = fmaf(u, u, ss);
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)gs + eps);
        for (int c = c0 + lane; c < c0 + gs; c += 32) {
            const float z = grow[g_off + c];
            const float sg = z / (1.f + expf(-z));
            float y = orow[c];
            y = gate_first ? (y * sg) * inv * w[c % wlen] : (y * inv) * w[c % wlen] * sg;
            dst[c] = from_f32<TO>(y * out_scale);
        }
    }
    if (clear) {
        __syncthreads();
        for (int c = clear_lo + threadIdx.x; c < clear_hi; c += 256) grow[c] = 0.f;
    }
}

}  // namespace

// q, k, v, dec: float32 rows of the step's tokens with leading dimensions and column offsets of their own (they may be
// column blocks of one projection).  out float32 [T, out_ld], head h at columns h*V.  mode, dec_bias, rate_log, skip as
// described at the top of the file.
TFF_API int tff_linear_recurrence(
    const float* q, int q_ld, int q_off, const float* k, int k_ld, int k_off, const float* v, int v_ld, int v_off,
    const float* dec, int dec_ld, int dec_off, const float* dec_bias, const float* rate_log, const float* skip,
    int mode, float inv_tau, float q_scale, float* state, long long slot_stride, long long state_off,
    const int* q_start, const int* pos_start, const int* slots, float* out, int out_ld,
    int num_requests, int H, int K, int V, int share, cudaStream_t stream) {
    if (num_requests <= 0) return TFF_OK;
    if (!q || !k || !v || !dec || !state || !out || !q_start || !pos_start || !slots || H <= 0 || K <= 0 || V <= 0 ||
        share <= 0 || H % share || mode < 0 || mode > 2 || (mode >= 1 && !dec_bias) || (mode == 2 && !rate_log))
        return TFF_ERR_BAD_ARGUMENT;
    if (K > 1024) return TFF_ERR_UNSUPPORTED;
    const int KPT = K <= 32 ? 8 : (K <= 64 ? 16 : 32);
    int KS = 1;
    while (KS * KPT < K) KS <<= 1;
    RecArgs a;
    a.q = q; a.q_ld = q_ld; a.q_off = q_off; a.k = k; a.k_ld = k_ld; a.k_off = k_off; a.v = v; a.v_ld = v_ld; a.v_off = v_off;
    a.dec = dec; a.dec_ld = dec_ld; a.dec_off = dec_off; a.dec_bias = dec_bias; a.rate_log = rate_log; a.skip = skip;
    a.mode = mode; a.inv_tau = inv_tau; a.q_scale = q_scale; a.state = state; a.slot_stride = slot_stride;
    a.state_off = state_off; a.q_start = q_start; a.pos_start = pos_start; a.slots = slots; a.out = out; a.out_ld = out_ld;
    a.H = H; a.K = K; a.V = V; a.share = share; a.KS = KS;
    const int VS = REC_THREADS / KS;
    const size_t smem = (size_t)(REC_TOKENS * (3 * KS * (KPT + REC_PAD) + VS) + 2 * REC_TOKENS) * sizeof(float);
    dim3 grid((V + VS - 1) / VS, H, num_requests);
#define TFF_REC(N)                                                                                                   \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(linear_recurrence_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tff_launch_pdl(linear_recurrence_kernel<N>, grid, dim3(REC_THREADS), smem, stream, a);               \
    } while (0)
    if (KPT == 8) TFF_REC(8);
    if (KPT == 16) TFF_REC(16);
    TFF_REC(32);
#undef TFF_REC
}

// out_dt: 0 = float32, 1 = bfloat16.
TFF_API int tff_gated_norm(const float* o, int width, int gs, float* gate, int g_ld, int g_off, const float* w, int wlen,
                           float eps, int gate_first, void* out, int out_dt, int out_ld, int out_off, float out_scale,
                           int clear, int clear_lo, int clear_hi, int num_tokens, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (!o || !gate || !w || !out || width <= 0 || gs <= 0 || width % gs || wlen <= 0 || !(eps > 0.f) ||
        (clear && (clear_lo < 0 || clear_hi > g_ld || clear_lo > clear_hi)))
        return TFF_ERR_BAD_ARGUMENT;
    if (out_dt == 1)
        return tff_launch_pdl(gated_norm_kernel<bf16>, dim3(num_tokens), dim3(256), 0, stream, o, width, gs, gate, g_ld,
                              g_off, w, wlen, eps, gate_first, (bf16*)out, out_ld, out_off, out_scale, clear, clear_lo,
                              clear_hi);
    return tff_launch_pdl(gated_norm_kernel<float>, dim3(num_tokens), dim3(256), 0, stream, o, width, gs, gate, g_ld,
                          g_off, w, wlen, eps, gate_first, (float*)out, out_ld, out_off, out_scale, clear, clear_lo,
                          clear_hi);
}
