/*
 * mnemo_oracle.h -- CPU restatement (plain C, fp32 with fp64 reference sums) of the
 * reference's quantized-weight hot path.
 *
 * THIS IS TEST INFRASTRUCTURE. It is the checker for the CUDA library and the
 * timed CPU baseline of the benchmark; nothing on the product path may call it.
 *
 * Every function names the reference file:line it follows (paths are relative
 * to the reference project: src/kernels.cu, src/forward.c,
 * tools/validate_dequant.py).
 *
 * Parity pin: the reference ships no golden vectors for this path; the dequant
 * routines here are pinned by equality (==, not a tolerance) against
 * tools/validate_dequant.py's dequant_q4k_cuda_style / dequant_q6k_reference
 * and against gguf.quants.dequantize on seeded blocks (tests/golden/). Q5_K and
 * Q8_0 are pinned the same way against dequant_q5k_cuda_style /
 * dequant_q8_0_cuda_style; RMSNorm and RoPE against the numpy replicas in
 * tools/validate_rope_norm.py. Q3_K has no counterpart in the validator:
 * its parity is UNPINNED on the CPU (it is checked against the reference's
 * compiled kernel on the GPU by tests/test_gpu_vs_reference_kernels.py).
 */
#ifndef MNEMO_ORACLE_H
#define MNEMO_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MO_Q4K_BLOCK_BYTES 144
#define MO_Q6K_BLOCK_BYTES 210
#define MO_QK_K 256

/* ---- helpers: kernels.cu:41-53 ------------------------------------------ */
float mo_f16_to_f32(uint16_t h);
uint16_t mo_f32_to_f16(float f); /* round-to-nearest-even, used by generators and the GEMM oracle */
void mo_get_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m);

/* ---- integer unpack (bit-exact contract) -------------------------------- */
/* Q4_K block -> d, dmin (as f16 bit patterns), sc[8], m[8], q[256] in 0..15.
 * Layout: kernels.cu:20-25; weight order: validate_dequant.py:92-113. */
void mo_unpack_q4k_block(const uint8_t *blk, uint16_t *d_bits, uint16_t *dmin_bits,
                         uint8_t sc[8], uint8_t m[8], uint8_t q[256]);
/* Q6_K block -> d (f16 bits), scales[16], q[256] in -32..31.
 * Layout: kernels.cu:27-32; order: validate_dequant.py:286-317, kernels.cu:455-484. */
void mo_unpack_q6k_block(const uint8_t *blk, uint16_t *d_bits, int8_t scales[16], int8_t q[256]);

/* ---- dequant: validate_dequant.py:68-115 and :253-319 ------------------- */
void mo_dequant_q4k(const uint8_t *w, int n_rows, int n_cols, float *out /*[n_rows][n_cols]*/);
void mo_dequant_q6k(const uint8_t *w, int n_rows, int n_cols, float *out);

/* ---- matvecs (fp32 result; y64 optional fp64 accumulation, may be NULL) --
 * abs_dot (optional) receives sum_c |w_rc * x_c| per row, the scale of the
 * per-element error bound. */
void mo_matvec_q4k(const uint8_t *w, const float *x, float *y, double *y64, double *abs_dot,
                   int n_rows, int n_cols);                          /* kernels.cu:66-145  */
void mo_matvec_q4k_add(const uint8_t *w, const float *x, const float *residual, float *y,
                       double *y64, int n_rows, int n_cols);         /* kernels.cu:149-199 */
void mo_matvec_q4k_qkv(const uint8_t *wq, const uint8_t *wk, const uint8_t *wv, const float *x,
                       float *q, float *k, float *v, int q_rows, int kv_rows,
                       int n_cols);                                  /* kernels.cu:205-274 */
void mo_matvec_q4k_dual(const uint8_t *wa, const uint8_t *wb, const float *x, float *ya, float *yb,
                        int n_rows, int n_cols);                     /* kernels.cu:278-354 */
void mo_matvec_q4k_scaled_add(const uint8_t *w, const float *x, float *y, int n_rows, int n_cols,
                              float scale);                          /* kernels.cu:358-415 */
void mo_matvec_q6k(const uint8_t *w, const float *x, float *y, double *y64, double *abs_dot,
                   int n_rows, int n_cols);                          /* kernels.cu:427-491 */
void mo_matvec_f32(const float *w, const float *x, float *y, int n_rows,
                   int n_cols);                                      /* kernels.cu:859-880 (lane-strided partials + shfl_down tree) */
void mo_matvec_f32_f64(const float *w, const float *x, double *y, int n_rows, int n_cols);

/* ---- elementwise: kernels.cu:677-688, :980-988 -------------------------- */
void mo_swiglu(const float *gate, const float *up, float *out, int n);
void mo_scaled_add(float *out, const float *x, float scale, int n);

/* ---- router select: kernels.cu:993-1057 --------------------------------- */
/* Same candidate order and replace-the-minimum slot rule, so the output
 * order of indices is the reference's. k <= 16. */
void mo_topk_softmax(const float *scores, int *indices, float *weights, int n_experts, int k);

/* ---- expert composition: forward.c:1122-1142; block: forward.c:810-823,875,1114 */
/* expert blob = [gate Q4_K EFFxH][up Q4_K EFFxH][down (Q6_K: type 14 | Q4_K: type 12) HxEFF] */
void mo_expert_fwd(const uint8_t *expert, size_t gate_sz, size_t up_sz, int H, int EFF,
                   int down_type, float weight, const float *x, float *moe_out /* += */);
/* moe_out = sum over the k routed experts; out = moe_out + residual.
 * indices/weights (length k) are outputs too. */
void mo_moe_block(const float *router_w /*[NE][H]*/, const uint8_t *experts, size_t expert_stride,
                  size_t gate_sz, size_t up_sz, int down_type, int NE, int K, int H, int EFF,
                  const float *x, const float *residual, float *out, int *indices,
                  float *weights);

/* ---- GEMM oracle: out[t][n] = sum_k dequant(W)[n][k] * f16(X[t][k]) ------- */
/* The reference's int8 GEMM (gemm_q4k.cu:201-266) is an unvalidated experiment;
 * the semantics asked of the tensor-core path are fp32 dequant(W) . X. */
void mo_gemm_q4k_f16(const uint8_t *w, const uint16_t *x_f16 /*[M][K]*/, float *out /*[M][N]*/,
                     int M, int N, int K);
void mo_gemm_q6k_f16(const uint8_t *w, const uint16_t *x_f16, float *out, int M, int N, int K);

/* ---- support operators of a decode step (computed in double, rounded once) ---- */
void mo_rms_norm(const float *x, const float *w, float *out, int n, float eps);       /* kernels.cu:692-749; validate_rope_norm.py:47-59 */
void mo_rms_norm_heads(const float *x, const float *w, float *out, int head_dim, int n_heads,
                       float eps);                                                       /* kernels.cu:754-780, 1196-1219 */
void mo_rope(float *vec, int n_heads, int head_dim, int pos, float theta);              /* kernels.cu:818-852; validate_rope_norm.py:168-197 */
void mo_f32_to_f16_array(const float *in, uint16_t *out, int n);                        /* kernels.cu:1309-1326 */
void mo_attention_f16kv(const float *q, const uint16_t *kv_k, const uint16_t *kv_v, float *out, int n_heads_q,
                        int head_dim, int n_kv_heads, int seq_len, int gqa_ratio,
                        float scale);                                                    /* kernels.cu:1550-1660 */
void mo_residual_add(const float *a, const float *b, float *out, int n);                /* kernels.cu:784-793 */
void mo_embedding_q4k(const uint8_t *table, int token, int hidden, float *out);         /* forward.c:1189-1229 */
int mo_argmax(const float *logits, int n);                                              /* kernels.cu:2048-2071 */

/* ---- other GGUF types of the reference's matvec() switch (forward.c:160-173): 8 = Q8_0 (kernels.cu:644-673),
 * 11 = Q3_K (:497-575), 13 = Q5_K (:578-640); 12 / 14 as above. Returns -1 for an unknown type. */
int mo_dequant_type(int type, const uint8_t *w, int n_rows, int n_cols, float *out);
int mo_matvec_type(int type, const uint8_t *w, const float *x, float *y, double *y64, double *abs_dot, int n_rows,
                   int n_cols);
/* ---- INT8 KV cache: kernels.cu:1339-1376 (store), :1382-1480 (attention) ---- */
void mo_f32_to_int8_kv(const float *in, int8_t *out, float *scales, int head_dim, int n_kv_heads);
void mo_attention_int8kv(const float *q, const int8_t *kv_k, const int8_t *kv_v, const float *k_scales,
                         const float *v_scales, float *out, int n_heads_q, int head_dim, int n_kv_heads, int seq_len,
                         int gqa_ratio, float scale);

/* temperature + top-p sampling: kernels.cu:2073-2174 (sums in double; see the .c file) */
int mo_sample_top_p(const float *logits, int n, float temperature, float top_p, unsigned long long seed);

int mo_num_threads(void);
void mo_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
