// Internal interfaces shared by the attention translation units.
#pragma once
#include <cuda_runtime.h>

// What some designs add to softmax attention; all off = plain attention.
//   softcap  > 0: a score s (after the scale) becomes softcap * tanh(s / softcap)
//   sink     != 0: the softmax's denominator has one more term, a key that has no value; its score (not scaled, not
//                 capped) is sink_val[head] (float32 [nq]) or, with sink_val null, 0
//   gate     float32 [tokens, nq]: the output of head h of token t is multiplied by gate[t, h] (null: by 1)
struct AttnExtra {
    float softcap;
    int sink;
    const float* gate;
    const float* sink_val;
};

#ifdef __CUDACC__
// tanh from one exponential and one division: 1 - 2 / (1 + 2^(2 x log2 e)); absolute error near 1e-7, so that a
// capped score keeps the accuracy of an uncapped one (tanh.approx is good to 5e-4 only, times the cap).
__device__ __forceinline__ float attn_tanh(float x) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 2.885390081777927f));
    return 1.0f - __fdividef(2.0f, 1.0f + e);
}
// The sink's score of a head in units of log2.
__device__ __forceinline__ float attn_sink_log2(const float* sink_val, int head) {
    return sink_val ? sink_val[head] * 1.4426950408889634f : 0.f;
}
// A scaled score in units of log2: with a cap, softcap * tanh(s * scale / softcap) * log2(e).
__device__ __forceinline__ float attn_score_log2(float raw, float scale_log2, float scale_over_cap, float cap_log2) {
    return cap_log2 > 0.f ? attn_tanh(raw * scale_over_cap) * cap_log2 : raw * scale_log2;
}
#endif

// Decode kernel (attention_decode.cu): at most 16 packed query rows per (request, kv head),
// keys streamed by TMA.  Writes ``out`` when num_splits == 1, else the partial results.
int tff_attention_decode_launch(
    const void* q, const int* q_start, const int* pos_start, const int* req_ids, const int* block_table, int table_width,
    const void* cache, long long cache_pages, int cache_layers, int layer, int page_size,
    void* out, float* part_o, float* part_ml, int num_requests, int max_q_len, int num_splits,
    int nq, int nkv, int d, float scale, int window, AttnExtra extra, cudaStream_t stream);

// Prompt-portion kernel (attention_prefill.cu): 128 packed rows per CTA on tcgen05, keys by TMA.
int tff_attention_prefill_launch(
    const void* q, const int* q_start, const int* pos_start, const int* req_ids, const int* block_table, int table_width,
    const void* cache, long long cache_pages, int cache_layers, int layer, int page_size,
    void* out, int num_requests, int max_q_len, int nq, int nkv, int d, float scale, int window, AttnExtra extra,
    cudaStream_t stream);
