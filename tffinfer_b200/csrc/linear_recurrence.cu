// A linear recurrence over a matrix state per head, with a decay that is read from the input at every token:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T          S [K, V] float32, a_t in (0, 1] on the K rows
//     o_t = S_t^T q_t (+ skip_h * v_t)
//
// It is the token mixing of gated linear attention (a decay per key channel) and of a selective state space (Mamba-2:
// one decay per head and token, q = C, k = dt * B, v = x).  How a_t is made is a mode of the first kernel, which turns the
// raw rows into decay factors once for all blocks of the second:
//   0  dec holds ln a per channel                          a = exp(dec[t, h, c])
//   1  dec holds a raw gate per channel                    a = sigmoid(dec[t, h, c] + dec_bias[h, c]) ^ inv_tau
//   2  dec holds a raw step size per head                  dt = softplus(dec[t, h] + dec_bias[h]),
//                                                          a = exp(-exp(rate_log[h]) * dt) on all rows, k_t v_t^T times dt
// (modes 0 and 1 leave a [T, H * K] tensor of factors, mode 2 a [T, H, 2] tensor of (dt, a).)
// Several heads may share one q and one k (``share`` heads a group).  All inputs are float32 rows (a product's
// accumulators), all arithmetic is float32, and a request's tokens are walked in order, whatever the step holds
// besides: a result does not depend on the batch, and on how a prompt was cut only in its last bits (a portion of more
// than a segment's tokens is joined from segments, below).  The state of (slot, head) lies at
// state + slot * slot_stride + state_off + head * K * V; a request whose first token of the step is at position 0
// starts from zeros without reading its slot.
//
// One block of 128 threads owns VS = 128 / KS columns of one head of one request: thread (column, ks) keeps KPT rows
// of its column in registers, the K rows of a column being dealt to KS lanes of one warp (KS a power of two).  Tokens
// are staged up to eight at a time in shared memory (q, k and the factors of the head, the block's columns of v), two
// buffers: by asynchronous copies of 16 bytes where every row allows them, so that the copies of the next batch run
// while the batch at hand is worked on, by plain loads otherwise.
// Within a batch every thread keeps its partial sums of o of all the batch's tokens; they meet across the KS lanes by
// shuffles once a batch, eight independent chains side by side.
//
// Every kernel here is launched with programmatic dependent launch and reads what the kernels ahead wrote past the
// first-level cache (16-byte asynchronous copies, ld.global.cg): a block that became resident before those kernels had
// finished can find a line there that is older than their writes, and the wait does not drop it.  (The factors kernel
// read its rows through that cache at first: decode steps replayed as CUDA graphs then went wrong, the same way every
// time, and right again when it was launched plainly or read past the cache.)
//
// A further kernel finishes such a mixer's output: RMS norm over groups of columns with a weight, and a silu gate ahead
// of the norm or behind it; another sets columns of an accumulator buffer back to zero.
#include "common.cuh"

namespace {

constexpr int REC_THREADS = 128;
constexpr int REC_TOKENS = 8;       // most tokens staged at a time
constexpr int REC_SEGMENT = 256;    // tokens of a segment of a long portion
constexpr int REC_PAD = 4;          // floats between the row groups of two lanes: keeps 16-byte reads off one bank

struct RecArgs {
    const float* q; int q_ld, q_off;
    const float* k; int k_ld, k_off;
    const float* v; int v_ld, v_off;
    const float* fac;                // [T, H * K] factors, or [T, H, 2] (dt, factor) when ``scalar``
    const float* skip;
    int scalar; float q_scale;
    float* state; long long slot_stride, state_off;
    const int* q_start; const int* pos_start; const int* slots;
    float* out; int out_ld;
    int H, K, V, share, KS, TB, kk_shift;      // TB tokens a batch; KS * KPT = 1 << kk_shift
    int wide;                                  // every staged row starts on 16 bytes and is whole pieces of four floats
    int nseg, seg_len;                         // long portions: a request's tokens in nseg segments of seg_len, side by side
    float* seg_state;                          // [requests * nseg, H, K, V]: what a segment leaves, started from zero (seg > 0)
    float* seg_prod;                           // [T, H * K] or [T, H]: the product of the factors from the segment's start
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_f32x4(float* smem, const float* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// fac[t, c] for c < H * K (modes 0, 1), or fac[t, h] = (dt, a) (mode 2): one thread an element.
__global__ void __launch_bounds__(256)
decay_factors_kernel(const float* __restrict__ dec, int dec_ld, int dec_off, const float* __restrict__ dec_bias,
                     const float* __restrict__ rate_log, int mode, float inv_tau, float* __restrict__ fac, int per_token,
                     long long total) {
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const long long t = i / per_token;
    const int c = (int)(i - t * per_token);
    const float b = mode >= 1 ? dec_bias[c] : 0.f;
    const float rate = mode == 2 ? expf(rate_log[c]) : 0.f;
    pdl_wait();
    const float raw = __ldcg(dec + t * dec_ld + dec_off + c);
    if (mode == 2) {
        const float dt = softplus_f(raw + b);
        fac[2 * i] = dt;
        fac[2 * i + 1] = expf(-rate * dt);
    } else {
        fac[i] = mode == 0 ? expf(raw) : expf(log_sigmoid_f(raw + b) * inv_tau);
    }
}

template <int KPT>
__global__ void __launch_bounds__(REC_THREADS)
linear_recurrence_kernel(RecArgs a) {
    extern __shared__ __align__(16) float rec_smem[];
    pdl_launch_dependents();
    const int KS = a.KS, cpw = 32 / KS, VS = REC_THREADS / KS, TB = a.TB;
    const int KK = KS * KPT;
    const int RW = KS * (KPT + REC_PAD);                    // floats of one staged vector
    const int vec = a.scalar ? 2 : 3;                       // staged vectors a token: q, k and, per channel, the factors
    const int BUF = TB * (vec * RW + VS + 4);               // floats of one buffer: [q | k | (factors)] [v] [dt, factor] (16-byte multiples)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int vc = warp * cpw + lane % cpw, ks = lane / cpw;
    const int head = blockIdx.y, b = blockIdx.z / a.nseg, seg = blockIdx.z - b * a.nseg;
    const int v0 = blockIdx.x * VS, vcol = v0 + vc;
    const bool active = vcol < a.V;
    const int K = a.K, V = a.V;
    const int t_req = a.q_start[b], n_req = a.q_start[b + 1] - t_req;
    const int t0 = t_req + seg * a.seg_len;                  // this block's tokens: segment ``seg`` of the request's portion
    const int n = min(a.seg_len, n_req - seg * a.seg_len);
    if (n <= 0) return;
    const int grp = head / a.share;
    float* st = a.nseg > 1 ? a.seg_state + ((size_t)blockIdx.z * a.H + head) * K * V
                           : a.state + (size_t)a.slots[b] * a.slot_stride + a.state_off + (size_t)head * K * V;
    const float* st_in = a.state + (size_t)a.slots[b] * a.slot_stride + a.state_off + (size_t)head * K * V;
    const bool fresh = a.pos_start[b] == 0 || seg > 0;       // a later segment starts from zero: the scan joins them
    const bool prods = a.nseg > 1 && blockIdx.x == 0 && vc == 0;     // one column's lanes also keep the factors' running product
    float cum[KPT];
#pragma unroll
    for (int j = 0; j < KPT; ++j) cum[j] = 1.f;
    const float skip = a.skip ? a.skip[head] : 0.f;
    // rows beyond K and tokens beyond a short batch are never copied: q and k zero and factors one there, for good
    for (int i = tid; i < 2 * BUF; i += REC_THREADS) {
        const int j = i % BUF;
        rec_smem[i] = (!a.scalar && j >= 2 * TB * RW && j < 3 * TB * RW) ? 1.f : 0.f;
    }
    __syncthreads();
    const float* qp = a.q + a.q_off + grp * K;
    const float* kp = a.k + a.k_off + grp * K;
    const float* fp = a.fac + (a.scalar ? 2 * head : head * K);
    const int f_ld = a.scalar ? 2 * a.H : a.H * K;
    const float* vp = a.v + a.v_off + head * V + v0;
    auto stage = [&](int base, int which) {                 // asynchronous copies of the batch that starts at ``base``
        float* buf = rec_smem + which * BUF;
        const int nb = min(TB, n - base);
        if (a.wide) {                                       // rows and columns in pieces of four floats, 16 bytes a copy
            for (int i = tid; i < nb << (a.kk_shift - 2); i += REC_THREADS) {
                const int tt = i >> (a.kk_shift - 2), r = (i & (KK / 4 - 1)) * 4;
                if (r < K) {
                    const size_t t = (size_t)(t0 + base + tt);
                    const int at = tt * RW + (r / KPT) * (KPT + REC_PAD) + r % KPT;
                    cp_async_f32x4(buf + at, qp + t * a.q_ld + r);
                    cp_async_f32x4(buf + TB * RW + at, kp + t * a.k_ld + r);
                    if (!a.scalar) cp_async_f32x4(buf + 2 * TB * RW + at, fp + t * f_ld + r);
                }
            }
            float* vs = buf + vec * TB * RW;
            for (int i = tid; i < nb * (VS / 4); i += REC_THREADS) {
                const int tt = i / (VS / 4), c = (i - tt * (VS / 4)) * 4;
                if (v0 + c < V) cp_async_f32x4(vs + tt * VS + c, vp + (size_t)(t0 + base + tt) * a.v_ld + c);
            }
        } else {
            for (int i = tid; i < nb << a.kk_shift; i += REC_THREADS) {
                const int tt = i >> a.kk_shift, r = i & (KK - 1);
                if (r < K) {
                    const size_t t = (size_t)(t0 + base + tt);
                    const int at = tt * RW + (r / KPT) * (KPT + REC_PAD) + r % KPT;
                    buf[at] = __ldcg(qp + t * a.q_ld + r);
                    buf[TB * RW + at] = __ldcg(kp + t * a.k_ld + r);
                    if (!a.scalar) buf[2 * TB * RW + at] = __ldcg(fp + t * f_ld + r);
                }
            }
            float* vs = buf + vec * TB * RW;
            for (int i = tid; i < nb * VS; i += REC_THREADS) {
                const int tt = i / VS, c = i - tt * VS;
                if (v0 + c < V) vs[i] = __ldcg(vp + (size_t)(t0 + base + tt) * a.v_ld + c);
            }
        }
        cp_async_commit();
    };
    // Copies of 16 bytes go past the first-level cache.  Smaller ones do not, and a block that became resident before
    // the kernels ahead had finished may find there a line that another block of its SM read when the address still held
    // something else: what is not copied 16 bytes at a time is therefore read past that cache into a register, a batch
    // ahead, and put into the buffer by its reader.
    float fac_next = 0.f;
    auto fetch_scalar = [&](int base) {
        if (a.scalar && tid < 2 * min(TB, n - base))
            fac_next = __ldcg(fp + (size_t)(t0 + base + (tid >> 1)) * f_ld + (tid & 1));
    };
    pdl_wait();
    stage(0, 0);                                            // in flight together with the state
    fetch_scalar(0);
    float S[KPT];
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
        const int r = ks * KPT + j;
        S[j] = (!fresh && active && r < K) ? __ldcg(st_in + (size_t)r * V + vcol) : 0.f;
    }
    int which = 0;
    for (int base = 0; base < n; base += TB, which ^= 1) {
        const int nb = min(TB, n - base);
        if (a.scalar && tid < 2 * nb) rec_smem[which * BUF + vec * TB * RW + TB * VS + tid] = fac_next;
        if (base + TB < n) { stage(base + TB, which ^ 1); fetch_scalar(base + TB); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();                                    // this batch has landed for every thread
        const float* buf = rec_smem + which * BUF;
        const float* vs = buf + vec * TB * RW;
        float acc[REC_TOKENS], vraw[REC_TOKENS];
#pragma unroll
        for (int tt = 0; tt < REC_TOKENS; ++tt) {
            acc[tt] = 0.f; vraw[tt] = 0.f;
            if (tt < nb) {
                const float4* q4 = reinterpret_cast<const float4*>(buf + tt * RW + ks * (KPT + REC_PAD));
                const float4* k4 = reinterpret_cast<const float4*>(buf + TB * RW + tt * RW + ks * (KPT + REC_PAD));
                vraw[tt] = vs[tt * VS + vc];
                float a0 = 0.f, a1 = 0.f;
                if (a.scalar) {
                    const float dt = vs[TB * VS + 2 * tt], d = vs[TB * VS + 2 * tt + 1];
                    const float vv = vraw[tt] * dt;         // k_t (dt v_t)^T: the step size on the value's side
                    if (prods && ks == 0) { cum[0] *= d; a.seg_prod[(size_t)(t0 + base + tt) * a.H + head] = cum[0]; }
#pragma unroll
                    for (int j = 0; j < KPT / 4; ++j) {
                        const float4 qv = q4[j], kv = k4[j];
                        S[4 * j + 0] = fmaf(S[4 * j + 0], d, kv.x * vv); a0 = fmaf(S[4 * j + 0], qv.x, a0);
                        S[4 * j + 1] = fmaf(S[4 * j + 1], d, kv.y * vv); a1 = fmaf(S[4 * j + 1], qv.y, a1);
                        S[4 * j + 2] = fmaf(S[4 * j + 2], d, kv.z * vv); a0 = fmaf(S[4 * j + 2], qv.z, a0);
                        S[4 * j + 3] = fmaf(S[4 * j + 3], d, kv.w * vv); a1 = fmaf(S[4 * j + 3], qv.w, a1);
                    }
                } else {
                    const float4* d4 = reinterpret_cast<const float4*>(buf + 2 * TB * RW + tt * RW + ks * (KPT + REC_PAD));
                    const float vv = vraw[tt];
                    if (prods) {
                        float* pr = a.seg_prod + (size_t)(t0 + base + tt) * a.H * K + head * K + ks * KPT;
#pragma unroll
                        for (int j = 0; j < KPT; ++j) {
                            cum[j] *= reinterpret_cast<const float*>(d4)[j];
                            if (ks * KPT + j < K) pr[j] = cum[j];
                        }
                    }
#pragma unroll
                    for (int j = 0; j < KPT / 4; ++j) {
                        const float4 qv = q4[j], kv = k4[j], dv = d4[j];
                        S[4 * j + 0] = fmaf(S[4 * j + 0], dv.x, kv.x * vv); a0 = fmaf(S[4 * j + 0], qv.x, a0);
                        S[4 * j + 1] = fmaf(S[4 * j + 1], dv.y, kv.y * vv); a1 = fmaf(S[4 * j + 1], qv.y, a1);
                        S[4 * j + 2] = fmaf(S[4 * j + 2], dv.z, kv.z * vv); a0 = fmaf(S[4 * j + 2], qv.z, a0);
                        S[4 * j + 3] = fmaf(S[4 * j + 3], dv.w, kv.w * vv); a1 = fmaf(S[4 * j + 3], qv.w, a1);
                    }
                }
                acc[tt] = a0 + a1;
            }
        }
        for (int o = cpw; o < 32; o <<= 1) {
#pragma unroll
            for (int tt = 0; tt < REC_TOKENS; ++tt) acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], o);
        }
        if (ks == 0 && active) {
#pragma unroll
            for (int tt = 0; tt < REC_TOKENS; ++tt)
                if (tt < nb)
                    a.out[(size_t)(t0 + base + tt) * a.out_ld + head * V + vcol] = fmaf(skip, vraw[tt], acc[tt] * a.q_scale);
        }
        __syncthreads();                                    // the buffer may be filled again
    }
    if (active) {
#pragma unroll
        for (int j = 0; j < KPT; ++j) {
            const int r = ks * KPT + j;
            if (r < K) st[(size_t)r * V + vcol] = S[j];
        }
    }
}

// Long portions run as segments side by side, every segment but a request's first from a zero state.  What joins them:
// with E_s the true state behind segment s, U_s what segment s left from zero and P_t the product of the factors from
// the segment's start up to token t,  E_s = P_(last token of s) * E_(s-1) + U_s  (scan, one thread a state element, in
// place in seg_state, the last one to the request's slot), and every token of a segment s > 0 still lacks
// o_t += (q_t * P_t)^T E_(s-1)  (apply).  No factor is ever divided by, so nothing overflows; a product that has
// run down to zero has simply forgotten what came before.
__global__ void __launch_bounds__(256)
segment_scan_kernel(RecArgs a) {
    pdl_launch_dependents();
    const int b = blockIdx.z, head = blockIdx.y;
    const int e = blockIdx.x * 256 + threadIdx.x;            // element r * V + v of the head's state
    const int K = a.K, V = a.V;
    const int t_req = a.q_start[b], n_req = a.q_start[b + 1] - t_req;
    if (e >= K * V || n_req <= 0) return;
    const int r = e / V;
    const int segs = (n_req + a.seg_len - 1) / a.seg_len;
    pdl_wait();
    float* U = a.seg_state + ((size_t)b * a.nseg * a.H + head) * K * V + e;
    const size_t seg_stride = (size_t)a.H * K * V;
    float E = __ldcg(U);
    for (int s = 1; s < segs; ++s) {
        const size_t last = (size_t)t_req + min(n_req, (s + 1) * a.seg_len) - 1;
        const float P = __ldcg(a.scalar ? a.seg_prod + last * a.H + head : a.seg_prod + last * a.H * K + head * K + r);
        E = fmaf(P, E, __ldcg(U + s * seg_stride));
        U[s * seg_stride] = E;
    }
    a.state[(size_t)a.slots[b] * a.slot_stride + a.state_off + (size_t)head * K * V + e] = E;
}

constexpr int APPLY_TOKENS = 8;      // most tokens staged at a time by the apply kernel

template <int KPT>
__global__ void __launch_bounds__(REC_THREADS)
segment_apply_kernel(RecArgs a, int tokens_a_block) {
    extern __shared__ __align__(16) float rec_smem[];       // [TB][KS * (KPT + REC_PAD)]: q_t * P_t, laid out as q is staged above
    pdl_launch_dependents();
    const int KS = a.KS, cpw = 32 / KS, VS = REC_THREADS / KS;
    const int KK = KS * KPT, RW = KS * (KPT + REC_PAD);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int vc = warp * cpw + lane % cpw, ks = lane / cpw;
    const int per_seg = (a.seg_len + tokens_a_block - 1) / tokens_a_block;
    const int head = blockIdx.y;
    const int zb = blockIdx.z / per_seg, part = blockIdx.z - zb * per_seg;       // zb: (request, segment >= 1)
    const int b = zb / (a.nseg - 1), seg = zb - b * (a.nseg - 1) + 1;
    const int vcol = blockIdx.x * VS + vc;
    const bool active = vcol < a.V;
    const int K = a.K, V = a.V;
    const int t_req = a.q_start[b], n_req = a.q_start[b + 1] - t_req;
    const int first = seg * a.seg_len + part * tokens_a_block;
    const int n = min(min(tokens_a_block, a.seg_len - part * tokens_a_block), n_req - first);
    if (n <= 0) return;
    const int grp = head / a.share;
    pdl_wait();
    const float* E = a.seg_state + (((size_t)b * a.nseg + seg - 1) * a.H + head) * K * V;
    float S[KPT];
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
        const int r = ks * KPT + j;
        S[j] = (active && r < K) ? __ldcg(E + (size_t)r * V + vcol) : 0.f;
    }
    const float* qp = a.q + a.q_off + grp * K;
    const float* pp = a.scalar ? a.seg_prod + head : a.seg_prod + head * K;
    const int p_ld = a.scalar ? a.H : a.H * K;
    const int TB = a.TB;                                    // tokens a batch: a thread stages at most eight products
    float rq[APPLY_TOKENS], rp[APPLY_TOKENS];
    auto fetch = [&](int base) {                            // q and P of the batch at ``base``: loads in flight together
        const int nb = min(TB, n - base);
#pragma unroll
        for (int j = 0; j < APPLY_TOKENS; ++j) {
            const int i = tid + j * REC_THREADS;
            const int tt = i >> a.kk_shift, r = i & (KK - 1);
            const bool on = tt < nb && r < K;
            const size_t t = (size_t)t_req + first + base + (on ? tt : 0);
            rq[j] = on ? __ldcg(qp + t * a.q_ld + r) : 0.f;
            rp[j] = on ? __ldcg(pp + t * p_ld + (a.scalar ? 0 : r)) : 0.f;
        }
    };
    fetch(0);
    for (int base = 0; base < n; base += TB) {
        const int nb = min(TB, n - base);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < APPLY_TOKENS; ++j) {
            const int i = tid + j * REC_THREADS;
            const int tt = i >> a.kk_shift, r = i & (KK - 1);
            if (tt < TB) rec_smem[tt * RW + (r / KPT) * (KPT + REC_PAD) + r % KPT] = rq[j] * rp[j];
        }
        __syncthreads();
        if (base + TB < n) fetch(base + TB);                // in flight while this batch is worked on
        float acc[APPLY_TOKENS];
#pragma unroll
        for (int tt = 0; tt < APPLY_TOKENS; ++tt) {
            float a0 = 0.f, a1 = 0.f;
            if (tt < nb) {
                const float4* q4 = reinterpret_cast<const float4*>(rec_smem + tt * RW + ks * (KPT + REC_PAD));
#pragma unroll
                for (int j = 0; j < KPT / 4; ++j) {
                    const float4 qv = q4[j];
                    a0 = fmaf(S[4 * j + 0], qv.x, a0); a1 = fmaf(S[4 * j + 1], qv.y, a1);
                    a0 = fmaf(S[4 * j + 2], qv.z, a0); a1 = fmaf(S[4 * j + 3], qv.w, a1);
                }
            }
            acc[tt] = a0 + a1;
        }
        for (int o = cpw; o < 32; o <<= 1) {
#pragma unroll
            for (int tt = 0; tt < APPLY_TOKENS; ++tt) acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], o);
        }
        if (ks == 0 && active) {
#pragma unroll
            for (int tt = 0; tt < APPLY_TOKENS; ++tt)
                if (tt < nb) {
                    float* dst = a.out + ((size_t)t_req + first + base + tt) * a.out_ld + head * V + vcol;
                    *dst = __ldcg(dst) + acc[tt] * a.q_scale;
                }
        }
    }
}

// out[t, out_off + c] = out_scale * y[c], c over ``width`` columns in groups of ``gs``:
//   gate_first 0:  y = o / rms_group(o) * w[c % wlen] * silu(g[c])
//   gate_first 1:  u = o * silu(g[c]),  y = u / rms_group(u) * w[c % wlen]
// o float32 [T, width]; g the columns g_off .. of the float32 rows ``gate`` (ld g_ld).  A warp works on a group at a time
// (WIDE false: blockIdx.y picks eight groups of a token) or, for groups of 512 columns and more, a whole block (WIDE
// true: blockIdx.y is the group); either way a group's sum of squares is added in an order that gs alone fixes.  With
// ``clear`` the columns clear_lo .. clear_hi of the token's row of ``gate`` are set to zero by a kernel of its own
// behind this one (an accumulator buffer that the next split product adds into).
template <typename TO, bool WIDE>
__global__ void __launch_bounds__(256)
gated_norm_kernel(const float* __restrict__ o, int width, int gs, const float* __restrict__ gate, int g_ld, int g_off,
                  const float* __restrict__ w, int wlen, float eps, int gate_first, TO* __restrict__ out, int out_ld,
                  int out_off, float out_scale) {
    __shared__ float red[32];
    pdl_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* orow = o + (size_t)t * width;
    const float* grow = gate + (size_t)t * g_ld + g_off;
    TO* dst = out + (size_t)t * out_ld + out_off;
    const int g = WIDE ? blockIdx.y : blockIdx.y * 8 + warp;
    const int first = WIDE ? threadIdx.x : lane, step = WIDE ? 256 : 32;
    pdl_wait();
    if (!WIDE && g >= width / gs) return;
    const int c0 = g * gs;
    float ss = 0.f;
    for (int c = c0 + first; c < c0 + gs; c += step) {
        float u = __ldcg(orow + c);
        if (gate_first) { const float z = __ldcg(grow + c); u *= z / (1.f + expf(-z)); }
        ss = fmaf(u, u, ss);
    }
    ss = WIDE ? block_sum<256>(ss, red) : warp_sum(ss);
    const float inv = rsqrtf(ss / (float)gs + eps);
    for (int c = c0 + first; c < c0 + gs; c += step) {
        const float z = __ldcg(grow + c);
        const float sg = z / (1.f + expf(-z));
        float y = __ldcg(orow + c);
        y = gate_first ? (y * sg) * inv * w[c % wlen] : (y * inv) * w[c % wlen] * sg;
        dst[c] = from_f32<TO>(y * out_scale);
    }
}

__global__ void __launch_bounds__(256)
clear_columns_kernel(float* __restrict__ rows, int ld, int lo, int hi) {
    pdl_launch_dependents();
    float* row = rows + (size_t)blockIdx.x * ld;
    pdl_wait();
    for (int c = lo + threadIdx.x; c < hi; c += 256) row[c] = 0.f;
}

}  // namespace

// q, k, v, dec: float32 rows of the step's tokens with leading dimensions and column offsets of their own (they may be
// column blocks of one projection).  out float32 [T, out_ld], head h at columns h*V.  mode, dec_bias, rate_log, skip as
// described at the top of the file.  ``factors``: float32 workspace of num_tokens * H * K elements (modes 0, 1) or
// num_tokens * H * 2 (mode 2), followed, when the longest portion ``max_q_len`` exceeds a segment, by what
// tff_linear_recurrence_workspace counts for the segments' products and states.
TFF_API int tff_linear_recurrence(
    const float* q, int q_ld, int q_off, const float* k, int k_ld, int k_off, const float* v, int v_ld, int v_off,
    const float* dec, int dec_ld, int dec_off, const float* dec_bias, const float* rate_log, const float* skip,
    int mode, float inv_tau, float q_scale, float* state, long long slot_stride, long long state_off,
    const int* q_start, const int* pos_start, const int* slots, float* out, int out_ld, float* factors,
    int num_tokens, int num_requests, int max_q_len, int H, int K, int V, int share, cudaStream_t stream) {
    if (num_requests <= 0 || num_tokens <= 0) return TFF_OK;
    if (!q || !k || !v || !dec || !state || !out || !factors || !q_start || !pos_start || !slots || H <= 0 || K <= 0 ||
        V <= 0 || share <= 0 || H % share || mode < 0 || mode > 2 || (mode >= 1 && !dec_bias) || (mode == 2 && !rate_log))
        return TFF_ERR_BAD_ARGUMENT;
    if (K > 1024) return TFF_ERR_UNSUPPORTED;
    const int per_token = mode == 2 ? H : H * K;
    const long long total = (long long)num_tokens * per_token;
    int st = tff_launch_pdl(decay_factors_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, dec, dec_ld,
                            dec_off, dec_bias, rate_log, mode, inv_tau, factors, per_token, total);
    if (st != TFF_OK) return st;
    // Rows a thread (8, 16 or 32) against lanes a column (KS): few rows a thread make more blocks (a block owns 128 / KS
    // columns of a head), which a step of few requests and heads needs; many rows a thread read the state in longer runs.
    // The widest that still gives every SM four blocks is taken, the narrowest that K allows otherwise.
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int nseg = max_q_len > REC_SEGMENT ? (max_q_len + REC_SEGMENT - 1) / REC_SEGMENT : 1;
    int KPT = 0, KS = 0;
    for (int kpt = 32; kpt >= 8; kpt >>= 1) {
        int ks = 1;
        while (ks * kpt < K) ks <<= 1;
        if (ks > 32) break;
        KPT = kpt; KS = ks;
        const long long blocks = (long long)((V + REC_THREADS / ks - 1) / (REC_THREADS / ks)) * H * num_requests * nseg;
        if (blocks >= 4LL * sms) break;
    }
    if (KPT == 0) return TFF_ERR_UNSUPPORTED;
    RecArgs a;
    a.q = q; a.q_ld = q_ld; a.q_off = q_off; a.k = k; a.k_ld = k_ld; a.k_off = k_off; a.v = v; a.v_ld = v_ld; a.v_off = v_off;
    a.fac = factors; a.skip = skip; a.scalar = mode == 2 ? 1 : 0; a.q_scale = q_scale;
    a.state = state; a.slot_stride = slot_stride; a.state_off = state_off;
    a.q_start = q_start; a.pos_start = pos_start; a.slots = slots; a.out = out; a.out_ld = out_ld;
    a.H = H; a.K = K; a.V = V; a.share = share; a.KS = KS;
    a.nseg = nseg; a.seg_len = nseg > 1 ? REC_SEGMENT : 0x3fffffff;
    a.seg_prod = factors + total * (mode == 2 ? 2 : 1);
    a.seg_state = a.seg_prod + total;
    const int KK = KS * KPT;
    a.kk_shift = 0;
    while ((1 << a.kk_shift) < KK) ++a.kk_shift;
    a.TB = 1024 / KK;                                       // a buffer holds at most 1024 rows of a staged vector
    if (a.TB > REC_TOKENS) a.TB = REC_TOKENS;
    if (max_q_len > 0 && a.TB > max_q_len) a.TB = max_q_len;       // steps of single tokens: buffers of one token
    const int VS = REC_THREADS / KS;
    auto on16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    a.wide = (K % 4 == 0 && V % 4 == 0 && VS % 4 == 0 && q_ld % 4 == 0 && k_ld % 4 == 0 && v_ld % 4 == 0 && q_off % 4 == 0 &&
              k_off % 4 == 0 && v_off % 4 == 0 && on16(q) && on16(k) && on16(v) && on16(factors)) ? 1 : 0;
    const size_t smem = 2 * (size_t)a.TB * ((a.scalar ? 2 : 3) * KS * (KPT + REC_PAD) + VS + 4) * sizeof(float);
    dim3 grid((V + VS - 1) / VS, H, num_requests * nseg);
    const size_t asmem = (size_t)a.TB * KS * (KPT + REC_PAD) * sizeof(float);
    const int apply_tokens = 64;                            // tokens a block of the apply kernel adds to
    dim3 agrid((V + VS - 1) / VS, H, num_requests * (nseg - 1) * ((REC_SEGMENT + apply_tokens - 1) / apply_tokens));
#define TFF_REC(N)                                                                                                   \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(linear_recurrence_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        st = tff_launch_pdl(linear_recurrence_kernel<N>, grid, dim3(REC_THREADS), smem, stream, a);                 \
        if (st != TFF_OK || nseg == 1) return st;                                                                    \
        st = tff_launch_pdl(segment_scan_kernel, dim3((K * V + 255) / 256, H, num_requests), dim3(256), 0, stream, a); \
        if (st != TFF_OK) return st;                                                                                 \
        if (asmem > 48 * 1024)                                                                                       \
            cudaFuncSetAttribute(segment_apply_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)asmem);  \
        return tff_launch_pdl(segment_apply_kernel<N>, agrid, dim3(REC_THREADS), asmem, stream, a, apply_tokens);    \
    } while (0)
    if (KPT == 8) TFF_REC(8);
    if (KPT == 16) TFF_REC(16);
    TFF_REC(32);
#undef TFF_REC
}

// Floats of the workspace tff_linear_recurrence wants for a step of num_tokens tokens in num_requests requests whose
// longest portion is max_q_len.
TFF_API long long tff_linear_recurrence_workspace(int num_tokens, int num_requests, int max_q_len, int H, int K, int V, int mode) {
    const long long per_token = mode == 2 ? H : (long long)H * K;
    long long need = (long long)num_tokens * per_token * (mode == 2 ? 2 : 1);
    if (max_q_len > REC_SEGMENT) {
        const long long nseg = (max_q_len + REC_SEGMENT - 1) / REC_SEGMENT;
        need += (long long)num_tokens * per_token + (long long)num_requests * nseg * H * K * V;
    }
    return need;
}

// out_dt: 0 = float32, 1 = bfloat16.
TFF_API int tff_gated_norm(const float* o, int width, int gs, float* gate, int g_ld, int g_off, const float* w, int wlen,
                           float eps, int gate_first, void* out, int out_dt, int out_ld, int out_off, float out_scale,
                           int clear, int clear_lo, int clear_hi, int num_tokens, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (!o || !gate || !w || !out || width <= 0 || gs <= 0 || width % gs || wlen <= 0 || !(eps > 0.f) ||
        (clear && (clear_lo < 0 || clear_hi > g_ld || clear_lo > clear_hi)))
        return TFF_ERR_BAD_ARGUMENT;
    const bool wide = gs >= 512;
    const dim3 grid(num_tokens, wide ? width / gs : (width / gs + 7) / 8);
    int st;
#define TFF_GN(TO, WIDE)                                                                                              \
    st = tff_launch_pdl(gated_norm_kernel<TO, WIDE>, grid, dim3(256), 0, stream, o, width, gs, (const float*)gate, g_ld, \
                        g_off, w, wlen, eps, gate_first, (TO*)out, out_ld, out_off, out_scale)
    if (out_dt == 1) { if (wide) TFF_GN(bf16, true); else TFF_GN(bf16, false); }
    else { if (wide) TFF_GN(float, true); else TFF_GN(float, false); }
#undef TFF_GN
    if (st != TFF_OK || !clear || clear_hi <= clear_lo) return st;
    return tff_launch_pdl(clear_columns_kernel, dim3(num_tokens), dim3(256), 0, stream, gate, g_ld, clear_lo, clear_hi);
}
