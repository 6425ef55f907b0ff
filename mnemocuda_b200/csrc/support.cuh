// Host-side launchers of the support kernels (support.cu), shared with the decode path (decode.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace mb200 {

struct AttnParams {
    const float *q;              // [n_heads_q][128] fp32, normalised and rotated
    const __half *kv_k, *kv_v;   // this layer's cache: [position][kv head][128] fp16
    float *out;                  // [n_heads_q][128]
    int n_kv_heads, gqa;         // gqa = query heads per KV head
    int seq_len;                 // positions to attend to ...
    const int *pos_ptr;          // ... or, when given, *pos_ptr + 1 (position kept in device memory)
    float scale;
    float *part;                 // [query-head block][chunk][16][128] partial weighted sums
    float *ml;                   // [query-head block][chunk][2][16] running max (log2 domain) and sum
    int *tickets;                // [query-head block], zero between launches
};

void support_init();
int attn_chunks_for(int n_kv_heads, int gqa, int max_slots);
size_t attn_workspace_bytes(int n_kv_heads, int gqa);
int launch_attn_decode(const float *q, const void *kv_k, const void *kv_v, float *out, int n_heads_q, int n_kv_heads,
                       int seq_len, const int *pos_ptr, float scale, void *workspace, cudaStream_t stream);
void launch_rms_norm(const float *in, const float *w, float *out, float *res_out, int n, float eps, cudaStream_t stream);
void launch_rope_table(float *cos_out, float *sin_out, int head_dim, const int *pos_ptr, int pos, float theta,
                       cudaStream_t stream);
void launch_qk_norm_rope_store(float *q, const float *k, const float *v, const float *wq, const float *wk,
                               const float *cos_t, const float *sin_t, void *kv_k, void *kv_v, int n_q, int n_k,
                               int head_dim, float eps, const int *pos_ptr, int pos, cudaStream_t stream);
void launch_embed_q4k(const void *table, float *out, const int *token_ptr, int token, int hidden, int row_bytes,
                      cudaStream_t stream);
void launch_embed_q3k(const void *table, float *out, const int *token_ptr, int token, int hidden, int row_bytes,
                      cudaStream_t stream);  // other_types.cu
void launch_argmax(const float *logits, int n, int *result, int *pos_ptr, cudaStream_t stream);
void launch_argmax_pair(const float *logits, int n, int index_offset, float *pair_out, cudaStream_t stream);
void launch_argmax_merge(const float *pairs, int n, int *result, int *pos_ptr, cudaStream_t stream);

}  // namespace mb200
