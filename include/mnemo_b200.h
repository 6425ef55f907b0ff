/*
 * mnemo_b200.h -- C ABI of libmnemo_b200.so: sm_100a kernels for the quantized
 * weight hot path of MnemoCUDA (GGUF Q4_K / Q6_K dequant-matvec for decode, the
 * Q4_K tensor-core GEMM for prefill, and its grouped per-expert form).
 *
 * Part 1 exports the reference's own kernel entry points under their own
 * names and signatures, so the reference's forward.c / engine.c link against
 * this library unchanged. The reference has no header for them: forward.c
 * re-declares each one by hand (src/forward.c:24-152); the definitions being
 * replaced are cited per function (paths relative to the reference project).
 *
 * Conventions (same as the reference): every pointer is a device pointer owned
 * by the caller; the library allocates nothing in these calls and keeps no
 * pointer beyond the call; the caller selects the device; any stream may be
 * passed, including one that is being captured into a CUDA graph; Part-1
 * functions return void and report launch errors on stderr. Weights are raw
 * GGUF blocks, row-major, ceil(n_cols/256) blocks per row, rows contiguous.
 * Q4_K tensors must start on a 16-byte boundary (the reference aligns resident
 * tensors to 256 B, src/engine.c:874, and expert parts to multiples of 144 B);
 * Q6_K tensors need 2-byte alignment only.
 *
 * Not exported: cuda_gemm_q4k / cuda_quantize_mmq_q8_1 (src/gemm_q4k.cu:272-324, 360-364), the reference's
 * env-gated int8 mma.sync experiment (batch 1 only, never validated, src/forward.c:683-698). An engine that
 * still calls them keeps the reference's gemm_q4k.o for those two symbols; the tensor-core
 * path of this library is mb200_gemm_q4k_f16 / mb200_moe_prefill below. Likewise the other GGUF types'
 * GDN kernels, the gated norm and the cache-statistics kernels stay with the reference's kernels.o.
 *
 * Part 2 (mb200_*) are additions that return a status code.
 */
#ifndef MNEMO_B200_H
#define MNEMO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifndef __CUDA_RUNTIME_API_H__
#ifndef __DRIVER_TYPES_H__
typedef struct CUstream_st *cudaStream_t;
#endif
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ===================== Part 1: the reference's kernel ABI ===================== */

/* One-time setup (shared-memory opt-in, status word). Replaces src/kernels.cu:2217-2240;
 * called by the engine at load (src/engine.c:1203-1207). Safe to call more than once. */
void cuda_kernels_init(void);

/* y = W x, W Q4_K [n_rows x n_cols]. Replaces src/kernels.cu:1071-1079 (kernel :66-145). */
void cuda_matvec_q4k(const void *weights, const float *x, float *y, int n_rows, int n_cols,
                     cudaStream_t stream);

/* y = W x + residual. Replaces src/kernels.cu:1094-1102 (kernel :149-199). */
void cuda_matvec_q4k_add(const void *weights, const float *x, const float *residual, float *y,
                         int n_rows, int n_cols, cudaStream_t stream);

/* q,k,v = Wq x, Wk x, Wv x in one launch. Replaces src/kernels.cu:1081-1092 (kernel :205-274). */
void cuda_matvec_q4k_qkv(const void *w_q, const void *w_k, const void *w_v, const float *x,
                         float *out_q, float *out_k, float *out_v, int q_rows, int kv_rows,
                         int n_cols, cudaStream_t stream);

/* ya = A x, yb = B x (same shape, shared x). Replaces src/kernels.cu:1104-1113 (kernel :278-354). */
void cuda_matvec_q4k_dual(const void *wa, const void *wb, const float *x, float *ya, float *yb,
                          int n_rows, int n_cols, cudaStream_t stream);

/* y += scale * (W x). Replaces src/kernels.cu:1115-1124 (kernel :358-415). */
void cuda_matvec_q4k_scaled_add(const void *weights, const float *x, float *y, int n_rows,
                                int n_cols, float scale, cudaStream_t stream);

/* y = W x, W Q6_K. Replaces src/kernels.cu:1126-1135 (kernel :427-491). */
void cuda_matvec_q6k(const void *weights, const float *x, float *y, int n_rows, int n_cols,
                     cudaStream_t stream);

/* y = W x, W fp32 row-major (the router). Replaces src/kernels.cu:1275-1281 (kernel :859-880). */
void cuda_matvec_f32(const float *weights, const float *x, float *y, int n_rows, int n_cols,
                     cudaStream_t stream);

/* top-k of n_experts scores + softmax over the k kept scores; k <= 16. Output
 * slot order is the reference's. Replaces src/kernels.cu:1301-1305 (kernel :993-1057). */
void cuda_topk_softmax(const float *scores, int *indices, float *weights, int n_experts, int k,
                       cudaStream_t stream);

/* out = silu(gate) * up. Replaces src/kernels.cu:1170-1176 (kernel :677-688). */
void cuda_swiglu(const float *gate, const float *up, float *out, int n, cudaStream_t stream);

/* out += scale * x. Replaces src/kernels.cu:1293-1299 (kernel :980-988). */
void cuda_scaled_add(float *out, const float *x, float scale, int n, cudaStream_t stream);

/* ---- support operators of a decode step (same names and signatures as the reference) ----
 * Not part of the quantized-weight hot path, but a decode token needs them between the
 * matvecs, and the reference's forward.c / engine.c import them (src/forward.c:24-152). */

/* out = in * weight / sqrt(mean(in^2) + eps). Replaces src/kernels.cu:1187-1193 (kernel :692-722). */
void cuda_rms_norm(const float *input, const float *weight, float *output, int n, float eps,
                   cudaStream_t stream);
/* Same, and copies the input to residual_output. Replaces src/kernels.cu:1178-1185 (kernel :725-749). */
void cuda_rms_norm_residual(const float *input, const float *weight, float *normed_output,
                            float *residual_output, int n, float eps, cudaStream_t stream);
/* RMSNorm of each of n_heads vectors of head_dim with one shared weight. Replaces src/kernels.cu:1221-1227. */
void cuda_rms_norm_batched(const float *input, const float *weight, float *output, int head_dim,
                           int n_heads, float eps, cudaStream_t stream);
/* In-place per-head RMSNorm of q (n_q heads) and k (n_k heads). Replaces src/kernels.cu:1229-1236 (kernel :1196-1219). */
void cuda_rms_norm_qk(float *q, float *k, const float *q_weight, const float *k_weight, int head_dim,
                      int n_q, int n_k, float eps, cudaStream_t stream);
/* Half-split rotary embedding of q and k at `pos`, in place; angles and their sine / cosine are evaluated
 * in double precision (as tools/validate_rope_norm.py:168-197 does). Replaces src/kernels.cu:1256-1273
 * (kernel :818-852); unlike the reference wrapper it copies nothing lazily, so the first call is legal
 * during stream capture. */
void cuda_rope(float *q, float *k, int head_dim, int pos, float theta, int n_heads_q, int n_heads_k,
               cudaStream_t stream);
/* fp32 -> fp16 (round to nearest even): the KV-cache store. Replace src/kernels.cu:1314-1333. */
void cuda_f32_to_f16(const float *in, void *out, int n, cudaStream_t stream);
void cuda_f32_to_f16_dual(const float *a, const float *b, void *oa, void *ob, int n, cudaStream_t stream);
/* Decode attention of one token over an fp16 KV cache laid out [position][kv head][head_dim]:
 * out[h] = softmax_p(scale * q[h] . K[p][h / gqa_ratio]) V[p][h / gqa_ratio], p < seq_len.
 * Replaces src/kernels.cu:1662-1671 (kernel :1550-1660). head_dim 128 runs on tensor cores with all
 * query heads of a KV head in one CTA and the positions split over the SMs (the partial results pass
 * through a workspace inside the library image, about 2 MB per device); other head sizes (<= 1024)
 * run a plain kernel. q, the cache and out must be 16-byte aligned for the fast path. */
void cuda_attention_f16kv(const void *q, const void *kv_k, const void *kv_v, float *out, int n_heads_q,
                          int head_dim, int n_kv_heads, int seq_len, int gqa_ratio, float scale,
                          cudaStream_t stream);
/* out = a + b. Replaces src/kernels.cu:1238-1244 (kernel :784-793). */
void cuda_residual_add(const float *a, const float *b, float *out, int n, cudaStream_t stream);
/* output[0..hidden_size) = dequantised row token_id of a Q4_K table (w = d*sc*q - dmin*m, products and
 * difference rounded separately as in tools/validate_dequant.py:68-115). Replaces src/kernels.cu:2192-2198
 * (kernel :1901-1951, whose nibble indexing differs from the reference's own matvec, validator and CPU
 * fallback src/forward.c:1189-1229; this follows the latter three). */
void cuda_embedding_lookup_q4k(const void *embd_table, float *output, int token_id, int hidden_size,
                               int row_bytes, cudaStream_t stream);
/* The other weight types of the reference's matvec() switch (src/forward.c:160-173): y = dequant(W) x with
 * W in Q8_0 (34-byte blocks of 32), Q5_K (176-byte blocks of 256) or Q3_K (110-byte blocks of 256). Bit layouts are
 * the reference kernels' (src/kernels.cu:644-673, 578-640, 497-575), which for Q5_K's fifth bits and Q3_K's scale
 * high bits are not the GGUF specification's. Replace src/kernels.cu:1159-1168, 1137-1146, 1148-1157. weights must be
 * 2-byte aligned; n_cols up to about 32k. */
void cuda_matvec_q8_0(const void *weights, const float *x, float *y, int n_rows, int n_cols, cudaStream_t stream);
void cuda_matvec_q5k(const void *weights, const float *x, float *y, int n_rows, int n_cols, cudaStream_t stream);
void cuda_matvec_q3k(const void *weights, const float *x, float *y, int n_rows, int n_cols, cudaStream_t stream);
/* Dequantised row token_id of a Q3_K table. Replaces src/kernels.cu:2200-2206 (kernel :1955-2030). */
void cuda_embedding_lookup_q3k(const void *embd_table, float *output, int token_id, int hidden_size,
                               int row_bytes, cudaStream_t stream);
/* INT8 KV cache: per head, scale = absmax / 127 and q = clamp(rint(v * 127 / absmax), -127, 127), both divisions
 * correctly rounded (the reference builds with fast-math, so its quotient can differ in the last place).
 * Replace src/kernels.cu:1484-1491 (kernel :1339-1376) and :1526-1534 (kernel :1493-1524). */
void cuda_f32_to_int8_kv(const float *in, void *out, float *scales, int head_dim, int n_kv_heads,
                         cudaStream_t stream);
void cuda_f32_to_int8_kv_dual(const float *k, const float *v, void *out_k, void *out_v, float *k_scales,
                              float *v_scales, int head_dim, int n_kv_heads, cudaStream_t stream);
/* Decode attention over the INT8 cache ([position][kv head][head_dim] int8, scales [position][kv head]).
 * Replaces src/kernels.cu:1536-1546 (kernel :1382-1480). head_dim 128 with 4 or 8 | gqa_ratio shares each
 * K / V read among the query heads of a CTA and splits the positions over the SMs (partials pass through a
 * workspace inside the library image); anything else runs one CTA per query head. */
void cuda_attention_int8kv(const float *q, const void *kv_k, const void *kv_v, const float *k_scales,
                           const float *v_scales, float *out, int n_heads_q, int head_dim, int n_kv_heads,
                           int seq_len, int gqa_ratio, float scale, cudaStream_t stream);
/* Sampling of one token. temperature <= 0: *d_result = argmax(logits), ties resolved as the reference's scan does
 * (src/kernels.cu:2048-2071). temperature > 0: softmax with temperature and top-p nucleus sampling with the
 * reference's candidate rule (the eight most probable tokens of every residue class mod 256), its xoroshiro128+
 * draw from rng_state and its walk over the nucleus (src/kernels.cu:2073-2174); the same token as the reference
 * unless the cut or the draw falls within float rounding of a boundary (the reference is built with fast-math and
 * adds the probabilities in another order). Two launches; scratch inside the library image, so calls on one
 * device must not overlap. Replaces :2208-2215. */
void cuda_sample_token(const float *logits, int vocab_size, float temperature, float top_p,
                       unsigned long long rng_state, int *d_result, cudaStream_t stream);
/* Addresses of the RoPE, KV-store and attention kernels, whose parameter order is the reference's, for a
 * caller that patches graph nodes by parameter index (src/forward.c:1295-1297, 636-661). Replace src/kernels.cu:2243-2245. */
void *cuda_get_rope_kernel_ptr(void);
void *cuda_get_f16dual_kernel_ptr(void);
void *cuda_get_attn_f16kv_kernel_ptr(void);

/* ===================== Part 2: additions (status-returning) ===================== */

enum {
    MB200_OK = 0,
    MB200_ERR_ARG = 1,       /* bad size / alignment / null pointer: nothing was launched */
    MB200_ERR_LAUNCH = 2,    /* the CUDA runtime refused a launch */
    MB200_ERR_TIMEOUT = 3,   /* a kernel gave up on a bounded wait (see mb200_device_error) */
    MB200_ERR_UNSUPPORTED = 4
};

int mb200_init(void);
/* First failure recorded since the last call to mb200_clear_status (0 = none). */
int mb200_last_status(void);
const char *mb200_last_status_where(void);
void mb200_clear_status(void);
/* Synchronises the device and returns the device-side error word (0 = no kernel gave up on a wait). */
int mb200_device_error(void);
/* Zeroes the current device's error word in stream order, so that later checks report new failures only. */
int mb200_clear_device_error(cudaStream_t stream);

/* Programmatic dependent launch for the streaming matvec kernels. 0 (default): plain
 * launches. 1: each kernel may start while the previous kernel of the stream is still
 * draining; it requests its first weight tiles at once and waits for that kernel only
 * before it reads x or writes y. Use 1 only when no weight tensor is written by the
 * kernel immediately upstream in the same stream (weights loaded once, as the engine
 * does at load time, satisfy this). Returns the previous setting. */
int mb200_set_pdl(int enabled);

/* act = silu(Wg x) * (Wu x): the expert gate+up pair with SwiGLU in the epilogue
 * (reference sequence src/forward.c:1128-1131: matvec_q4k_dual then swiglu). */
int mb200_matvec_q4k_dual_swiglu(const void *w_gate, const void *w_up, const float *x, float *act,
                                 int n_rows, int n_cols, cudaStream_t stream);

/* y += scale * (W x), W Q6_K (reference sequence src/forward.c:1137-1140: matvec_q6k then scaled_add). */
int mb200_matvec_q6k_scaled_add(const void *weights, const float *x, float *y, int n_rows,
                                int n_cols, float scale, cudaStream_t stream);

/* y = W RMSNorm(x): the norm (x * norm_w / sqrt(mean(x^2) + eps), src/kernels.cu:692-722) folded into the matvec's
 * staging of x -- every CTA reads x once anyway, adds up x^2 itself and normalises on the way to shared memory,
 * so the reference's norm kernel and the round trip of the normalised vector through memory
 * (src/forward.c:672-676, 687-720) disappear. n_cols <= 4608. The two-tensor form is the decode path's Q and K. */
int mb200_norm_matvec_q4k(const void *weights, const float *x, const float *norm_w, float eps, float *y, int n_rows,
                          int n_cols, cudaStream_t stream);
int mb200_norm_matvec_q6k(const void *weights, const float *x, const float *norm_w, float eps, float *y, int n_rows,
                          int n_cols, cudaStream_t stream);
int mb200_norm_matvec2_q4k(const void *wa, float *ya, int rows_a, const void *wb, float *yb, int rows_b, const float *x,
                           const float *norm_w, float eps, int n_cols, cudaStream_t stream);
/* The decode path's three projections in one launch: Q and K in Q4_K, V in Q6_K (the Q4_K_M layout), sharing x.
 * norm_w NULL = x is used as it is. Replaces the three launches of src/forward.c:688-704. */
int mb200_norm_matvec_qkv(const void *wq, float *q, int q_rows, const void *wk, float *k, const void *wv, float *v,
                          int kv_rows, const float *x, const float *norm_w, float eps, int n_cols,
                          cudaStream_t stream);

/* ---- decode-time MoE block with the routed expert ids kept on the device ----
 * The reference copies the k routed ids to the host and synchronises in every layer
 * (src/forward.c:849-882) before issuing 3-4 launches per expert (src/forward.c:1122-1142).
 * These three calls do the block in three launches with no host round trip; ids and
 * weights stay in device memory (they are outputs of the first call and inputs of the others).
 * An expert blob is [gate Q4_K EFF x H][up Q4_K EFF x H][down H x EFF], expert e at
 * experts + e * expert_stride (src/forward.c:1127-1136). */

/* Bytes of scratch mb200_router_topk / mb200_moe_block need: a ticket counter, the logits, and
 * (16-byte aligned, at the end) 64 bytes of barrier counters for mb200_moe_block. */
size_t mb200_router_scratch_bytes(int n_experts);

/* logits = router_w x (fp32 [n_experts x n_cols], src/kernels.cu:859-880), then the
 * reference's top-k + softmax (src/kernels.cu:993-1057), in one launch. scratch: 16-byte
 * aligned device memory of mb200_router_scratch_bytes(n_experts) bytes whose first word is zero
 * before the first call (each call leaves it zero); the logits can be read from it at byte 32. */
int mb200_router_topk(const float *router_w, const float *x, void *scratch, int *indices,
                      float *weights, int n_experts, int n_cols, int k, cudaStream_t stream);

/* Same operation and results as mb200_router_topk, for callers that have no device memory to
 * give and cannot get any: an engine that has already handed every free byte to its expert
 * cache and KV cache at load time, or a serving loop that runs under a no-allocation rule
 * once warm-up is over. This entry point has no counterpart in the reference. The ticket and
 * logits live in an array inside the library image instead (about 4 KB, held on each device
 * that loads the library until the process exits), so n_experts is limited to 1024; larger
 * values are refused with MB200_ERR_UNSUPPORTED. Nothing is allocated or freed by the call.
 * cuda_kernels_init() / mb200_init() look up the array's device address for the device that is current
 * when they run; on a device they were not called for, the first call here does the lookup (the device
 * must be current), so make that first call before starting any stream capture. All calls on a device share the one
 * array: calls whose kernels can overlap on the GPU (different streams) race on it -- serialise
 * them or use mb200_router_topk with separate scratch buffers. */
int mb200_router_topk_static(const float *router_w, const float *x, int *indices, float *weights,
                             int n_experts, int n_cols, int k, cudaStream_t stream);

/* act[s][r] = silu(gate_e[r].x) * (up_e[r].x), e = ids[s], for the n_slots routed experts;
 * act is [n_slots][EFF]. Slots with ids[s] < 0 are skipped (their rows of act are not written). (src/forward.c:1128-1131 per expert.) */
int mb200_moe_gate_up(const void *experts, size_t expert_stride, size_t gate_off, size_t up_off,
                      const int *ids, int n_slots, const float *x, float *act, int EFF, int H,
                      cudaStream_t stream);

/* y[r] = (residual ? residual[r] : y[r]) + sum_s wts[s] * (down_e[r] . act[s]), slots added in
 * order; down_type 14 = Q6_K, 12 = Q4_K (src/forward.c:1133-1141, and the zero + residual add
 * around the expert loop: src/forward.c:875,1114). */
int mb200_moe_down(const void *experts, size_t expert_stride, size_t down_off, int down_type,
                   const int *ids, const float *wts, int n_slots, const float *act,
                   const float *residual, float *y, int H, int EFF, cudaStream_t stream);

/* Expert-sharded forms (this replaces the reference's layer-split hand-off, src/engine.c:761-775,
 * src/forward.c:1555-1581): the device holds experts [expert_lo, expert_lo + expert_cnt) of the
 * layer, `experts` points at expert_lo's blob, and routed slots whose id falls outside that range
 * are skipped without reading anything. ids are the router's global ids (the router is replicated).
 * mb200_moe_down_local adds only the local experts; the caller sums the partial results of all
 * devices (NCCL all-reduce) -- pass the residual on one device and NULL with a zeroed y elsewhere. */
int mb200_moe_gate_up_local(const void *experts, size_t expert_stride, size_t gate_off, size_t up_off,
                            const int *ids, int n_slots, int expert_lo, int expert_cnt, const float *x,
                            float *act, int EFF, int H, cudaStream_t stream);
int mb200_moe_down_local(const void *experts, size_t expert_stride, size_t down_off, int down_type,
                         const int *ids, const float *wts, int n_slots, int expert_lo, int expert_cnt,
                         const float *act, const float *residual, float *y, int H, int EFF,
                         cudaStream_t stream);

/* The whole block: out = residual + sum over the k routed experts. ids/wts: [k] (outputs); act: [k][EFF]
 * (workspace); scratch: mb200_router_scratch_bytes(n_experts) bytes, 16-byte aligned, zeroed once and then
 * left to this function. Where the shape allows it (see mb200_moe_experts_fused; in addition n_experts
 * <= 32 k and <= 512) this is ONE cooperative launch that also does the routing: every CTA computes one
 * router row, the CTAs meet at a device-wide barrier, and each CTA runs the top-k itself. Otherwise the
 * router kernel is followed by the fused expert kernel, or by the two separate expert kernels. The
 * results do not depend on which form runs beyond the rounding of the router's dot products. */
int mb200_moe_block(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz,
                    size_t up_sz, int down_type, int n_experts, int k, int H, int EFF,
                    const float *x, const float *residual, float *out, int *ids, float *wts,
                    float *act, void *scratch, cudaStream_t stream);

/* Gate/up + SwiGLU, down projections, weighted sum and residual add of the routed experts in ONE
 * cooperative launch (the two phases are separated by a device-wide barrier inside the kernel, and the
 * down-projection weights stream in while the CTAs meet). Same arguments and results as
 * mb200_moe_gate_up_local followed by mb200_moe_down_local; the expert range [expert_lo, expert_lo +
 * expert_cnt) is what this device holds at `experts` (0, INT_MAX for all). `sync`: 32 bytes (four
 * 64-bit words), 8-byte aligned, zero before the first use and owned by this call sequence afterwards
 * (arrival counters that only grow; after MB200_ERR_TIMEOUT they must be zeroed again).
 * Covers H a multiple of 2048 with 12 % (H / 2048) == 0, EFF a multiple of 512 whose column groups
 * divide 12, at most 8 slots, 16-byte aligned tensors; returns MB200_ERR_UNSUPPORTED -- and launches
 * nothing -- otherwise. mb200_moe_block uses it when it applies (the tail of its scratch is the
 * barrier state) and falls back to the two separate kernels when not, or after mb200_set_fused(0).
 * The first call in a process should be made outside stream capture. */
int mb200_moe_experts_fused(const void *experts, size_t expert_stride, size_t gate_off, size_t up_off,
                            size_t down_off, int down_type, const int *ids, const float *wts, int n_slots,
                            int expert_lo, int expert_cnt, const float *x, float *act,
                            const float *residual, float *y, int H, int EFF, void *sync,
                            cudaStream_t stream);
/* How mb200_moe_block runs the block: 0 = router kernel + two expert kernels, 1 = router kernel + fused
 * expert kernel, 2 = one launch that also routes. Forms that do not cover a shape fall back to the next. */
void mb200_set_fused(int mode);

/* mb200_moe_block for a device that holds only experts [expert_lo, expert_lo + expert_cnt) of the layer at
 * `experts` (expert-sharded engines): the routing is done in full (the router is replicated), slots routed
 * to other devices are skipped, `out` receives this device's partial sum (pass the residual on one device
 * and zeros on the others, then all-reduce). No counterpart in the reference, which shards by layers. */
int mb200_moe_block_local(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz,
                          size_t up_sz, int down_type, int n_experts, int expert_lo, int expert_cnt, int k,
                          int H, int EFF, const float *x, const float *residual, float *out, int *ids,
                          float *wts, float *act, void *scratch, cudaStream_t stream);

/* The expert-sharded block WITH its all-reduce, in the same launch: the warp that finishes a row of the down
 * projection stores this rank's partial value into the receive cells of every rank of `comm` (mb200_comm_create;
 * plain 8-byte stores over NVLink, value and sequence tag together), and once a CTA's rows are out it collects the
 * other ranks' values of the same rows (bounded wait -> MB200_ERR_TIMEOUT in the device error word) and writes
 * out = sum over the ranks in rank order: identical bits on every rank, the same bits as mb200_moe_block_local
 * followed by mb200_push_allreduce, one launch and one kernel tail less. `residual` may be null (pass it on one rank).
 * norm_w != NULL folds the RMSNorm of x in (as mb200_moe_block_norm). Every rank of the communicator must make the
 * call, in the same order relative to its other collectives. Only the one-launch form has it: returns
 * MB200_ERR_UNSUPPORTED, with nothing launched, where that form does not cover the shape or after
 * mb200_set_fused(0 / 1); the caller then uses the two calls named above. */
int mb200_moe_block_push(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz, size_t up_sz,
                         int down_type, int n_experts, int expert_lo, int expert_cnt, int k, int H, int EFF,
                         const float *x, const float *norm_w, float norm_eps, const float *residual, float *out, int *ids,
                         float *wts, float *act, void *scratch, void *comm, cudaStream_t stream);

/* mb200_moe_block_local on RMSNorm(x) (the pre-FFN norm of src/forward.c:810, folded in): norm_w [H], eps; in the
 * one-launch form the router and the gate/up products normalise x on the fly, the other forms run a norm
 * kernel into normed_scratch [H] first. norm_w NULL = x is used as given. */
int mb200_moe_block_norm(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz, size_t up_sz,
                         int down_type, int n_experts, int expert_lo, int expert_cnt, int k, int H, int EFF,
                         const float *x, const float *norm_w, float norm_eps, float *normed_scratch,
                         const float *residual, float *out, int *ids, float *wts, float *act, void *scratch,
                         cudaStream_t stream);

/* The block for a caller that keeps the hidden state in HOST memory: host_x_res = [x | residual], 2*H floats;
 * host_out receives H floats. dev_io is 3*H floats of device memory the caller lends. With page-locked (pinned,
 * mapped) host buffers no copy engine is involved: a one-CTA kernel reads x and the residual across PCIe into
 * dev_io, the block writes its H result floats straight into host_out, and a last one-thread kernel raises a word
 * in host memory that the call spins on; the launches of a call are kept as an instantiated graph per argument
 * set (64 most recent), so a repeated call is one graph launch. With pageable buffers: one copy in, the block, one
 * copy out, a stream synchronisation. Either way the work is complete and the result in host_out when the call
 * returns (mb200_moe_block_local's arguments; expert_cnt 0 = all experts are here). One host call at a time per
 * device; not to be called while the stream is being captured by the caller (it then takes plain launches). The reference's engine moves
 * hidden vectors through the host the same way when peer access is unavailable (src/forward.c:1573-1578). */
int mb200_moe_block_host(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz,
                         size_t up_sz, int down_type, int n_experts, int expert_lo, int expert_cnt, int k, int H,
                         int EFF, const float *host_x_res, float *host_out, float *dev_io, int *ids, float *wts,
                         float *act, void *scratch, cudaStream_t stream);

/* ---- prefill GEMM on tcgen05 tensor cores ----
 * out[t][n] = sum_k f16(X[t][k]) * dequant(W)[n][k]; X fp16 [M x K] row-major (16-byte aligned),
 * W Q4_K / Q6_K [N x K] as for the matvecs, out fp32 [M x N]; K a multiple of 256. Weights are
 * dequantised in fp32 and rounded to fp16 for the tensor core, accumulation is fp32.
 * The reference's counterpart is its int8 mma.sync experiment (src/gemm_q4k.cu:272-324, used at
 * batch 1 only, src/forward.c:683-698); prefill proper is token-serial there (src/forward.c:1783-1830). */
int mb200_gemm_q4k_f16(const void *w, const void *x_f16, float *out, int M, int N, int K,
                       cudaStream_t stream);
int mb200_gemm_q6k_f16(const void *w, const void *x_f16, float *out, int M, int N, int K,
                       cudaStream_t stream);

/* ---- grouped per-expert GEMM: the MoE block for a batch of tokens (prefill) ----
 * For every token t and slot s with e = ids[t][s] >= 0:
 *   y[t] = (residual ? residual[t] : 0) + sum_s wts[t][s] * Wdown_e . SwiGLU(Wgate_e x_t, Wup_e x_t)
 * (the per-token sequence of src/forward.c:1122-1142 applied to a batch; the reference has no batched
 * form: its prefill runs the decode path token by token, src/forward.c:1783-1830). The routed pairs
 * are sorted by expert on the device, each expert's gate|up (one [2*EFF x H] Q4_K matrix) and down
 * ([H x EFF], Q6_K = 14 or Q4_K = 12) run as tcgen05 GEMMs on its token slice in two grouped
 * launches, slots are added in slot order. x is fp16 [M][H]; ids/wts are [M][k] on the device.
 * workspace: mb200_moe_prefill_workspace_bytes() bytes, 256-byte aligned, contents don't matter.
 * max_tokens_per_expert sizes the launches (0 = M, always safe); if an expert receives more tokens
 * than that, the device error word is set (mb200_device_error) and y is incomplete. */
size_t mb200_moe_prefill_workspace_bytes(int M, int k, int H, int EFF, int n_experts);
int mb200_moe_prefill(const void *experts, size_t expert_stride, size_t gate_sz, size_t up_sz, int down_type,
                      int n_experts, int k, int H, int EFF, const void *x_f16, const int *ids,
                      const float *wts, const float *residual, float *y, int M, int max_tokens_per_expert,
                      void *workspace, cudaStream_t stream);

/* ---- whole-token decode (the op order of src/forward.c:1635-1707 and :604-1117, no host round trip) ----
 * The caller owns every buffer: weights, KV cache, workspace, token / position / logits. Nothing is
 * allocated here. Tensor types are GGUF ids: 0 = fp32, 8 = Q8_0, 11 = Q3_K, 12 = Q4_K, 13 = Q5_K, 14 = Q6_K
 * (projections and lm_head: any of them; experts: Q4_K gate / up with a Q4_K or Q6_K down; embedding: Q4_K or Q3_K). */
typedef struct mb200_layer_weights {
    const float *attn_norm;          /* [hidden] */
    const void *wq, *wk, *wv, *wo;   /* [n_heads*head_dim x hidden], [n_kv_heads*head_dim x hidden] x2, [hidden x n_heads*head_dim] */
    int wq_type, wk_type, wv_type, wo_type;
    const float *q_norm, *k_norm;    /* [head_dim] each, or NULL for a model without q/k norm */
    const float *ffn_norm;           /* [hidden] */
    const float *router;             /* fp32 [n_experts x hidden] */
    const void *experts;             /* blob of expert expert_lo, then the following ones (expert_stride apart) */
    void *kv_k, *kv_v;               /* this layer's fp16 cache, [ctx_len][n_kv_heads][head_dim] each */
    /* This layer's expert blob layout where it differs from the model's (a Q4_K_M file mixes Q4_K and Q6_K down
     * projections from layer to layer; the reference derives the layout per layer file, src/forward.c:867-872).
     * expert_stride 0 = the model's expert_stride / gate_sz / up_sz / down_type. */
    size_t expert_stride, gate_sz, up_sz;
    int down_type;
} mb200_layer_weights;

typedef struct mb200_decode_model {
    int n_layers, hidden, n_heads, n_kv_heads, head_dim, n_experts, top_k, moe_inter, vocab, ctx_len;
    float rms_eps, rope_theta;
    int down_type, embd_type, lm_head_type;
    size_t expert_stride, gate_sz, up_sz;   /* expert blob = [gate][up][down] (src/forward.c:1127-1136) */
    int expert_lo, expert_cnt;              /* experts held on this device (0, 0 = all) */
    const mb200_layer_weights *layers;      /* host array [n_layers] */
    const void *token_embd;                 /* [vocab x hidden], embd_type 12 (Q4_K) or 11 (Q3_K) */
    const float *output_norm;               /* [hidden] */
    const void *lm_head;                    /* [vocab x hidden], lm_head_type (a sharded rank: its rows, see below) */
    /* A rank of a model sharded over devices describes ITS SHARD above (n_heads / n_kv_heads = the heads it
     * holds, wq / wk / wv / kv_k / kv_v = their rows, wo = rows [o_row0, o_row0 + o_rows) of the output
     * projection, lm_head = rows [lm_row0, lm_row0 + lm_rows)) and fills these in; all zero = not sharded. */
    int n_heads_total;                      /* query heads of the whole model (width of the O projection's input) */
    int o_row0, o_rows, lm_row0, lm_rows;
} mb200_decode_model;

/* Bytes of device workspace a model needs (256-byte aligned; zero it once before the first token:
 * it holds barrier / ticket counters that the kernels keep consistent afterwards). 0 = bad model. */
size_t mb200_decode_workspace_bytes(const mb200_decode_model *m);
/* The hidden state inside the workspace, fp32 [hidden] (input and output of mb200_decode_layer). */
float *mb200_decode_hidden(const mb200_decode_model *m, void *workspace);
/* One token: embedding of *d_token, all layers at position *d_pos, final norm, lm_head into d_logits
 * [vocab], greedy sample into *d_token, *d_pos += 1. d_token / d_pos are device ints, read and written
 * by kernels only, so a CUDA graph captured around this call decodes one more token on every replay.
 * = mb200_decode_begin, mb200_decode_layer for each layer, mb200_decode_finish (which a caller that
 * shards the model over devices issues itself, with its collectives in between). */
int mb200_decode_step(const mb200_decode_model *m, void *workspace, int *d_token, int *d_pos, float *d_logits,
                      cudaStream_t stream);
int mb200_decode_begin(const mb200_decode_model *m, void *workspace, const int *d_token, const int *d_pos,
                       cudaStream_t stream);
int mb200_decode_layer(const mb200_decode_model *m, int layer, void *workspace, const int *d_pos,
                       cudaStream_t stream);
int mb200_decode_finish(const mb200_decode_model *m, void *workspace, float *d_logits, int *d_token, int *d_pos,
                        cudaStream_t stream);
/* The layer in three pieces for a model sharded over devices (this replaces the reference's layer-range split,
 * src/engine.c:761-775): attention over the rank's heads -> attn_local [n_heads * head_dim]; [all-gather];
 * the rank's rows of the output projection + residual -> hidden_rows [o_rows]; [all-gather into the hidden
 * state, mb200_decode_hidden]; the rank's experts (+ the residual on the rank that passes add_residual) ->
 * out [hidden]; [all-reduce into the hidden state]. Then the rank's rows of the lm_head with the best
 * (logit, vocabulary index) pair of those rows in best_pair[2] (the index as int bits); [all-gather of the
 * pairs]; mb200_decode_pick writes the token and advances the position. The collectives are the caller's
 * (mb200_push_allgather / mb200_push_allreduce, or NCCL). */
int mb200_decode_layer_attn(const mb200_decode_model *m, int layer, void *workspace, const int *d_pos, float *attn_local,
                            cudaStream_t stream);
int mb200_decode_layer_oproj(const mb200_decode_model *m, int layer, void *workspace, const float *attn_full,
                             float *hidden_rows, cudaStream_t stream);
int mb200_decode_layer_moe(const mb200_decode_model *m, int layer, void *workspace, int add_residual, float *out,
                           cudaStream_t stream);
/* mb200_decode_layer_moe followed by the all-reduce over `comm` into `out`: one launch where mb200_moe_block_push
 * applies, else the block into `partial` [hidden] and mb200_push_allreduce. */
int mb200_decode_layer_moe_reduce(const mb200_decode_model *m, int layer, void *workspace, int add_residual,
                                  float *partial, float *out, void *comm, cudaStream_t stream);
int mb200_decode_logits_local(const mb200_decode_model *m, void *workspace, float *logits_rows, float *best_pair,
                              cudaStream_t stream);
int mb200_decode_pick(const float *pairs, int n_pairs, int *d_token, int *d_pos, cudaStream_t stream);

/* ---- push collectives over NVLink peer memory (one process per GPU) ----
 * These replace the reference's only inter-GPU traffic, the hidden-vector copy at a layer-range boundary
 * (src/forward.c:1555-1581, src/engine.c:1238-1262), for a model whose matvec rows and experts are sharded
 * over the GPUs: the pieces are 16-32 KB, so the collectives are latency-bound, and every rank stores its
 * piece straight into every peer's receive buffer (plain 8-byte peer stores, each carrying the collective's
 * sequence number beside the value, so no fence or flag follows), and the receiver sums (all-reduce, in rank
 * order: deterministic and identical on all ranks) or concatenates (all-gather) the pieces as they land. All ranks must issue the same sequence of collectives on a comm.
 * A wait that is not satisfied within ~2 s raises the device error word (MB200_ERR_TIMEOUT) and the kernel
 * returns; nothing hangs. Legal inside stream capture (the sequence number lives in device memory).
 *
 * Set-up (not capturable): each rank calls mb200_comm_alloc (cudaMalloc + zero + CUDA IPC handle), the 64-byte
 * handles of all ranks are exchanged by the caller (MPI, torch.distributed, a file ...), and
 * mb200_comm_create opens the peers' buffers. ipc_handles_64 = world * 64 bytes, rank order. */
size_t mb200_comm_buffer_bytes(int world, size_t max_floats);
int mb200_comm_alloc(int world, size_t max_floats, void **dev_ptr, void *ipc_handle_64);
int mb200_comm_create(int rank, int world, size_t max_floats, void *local_ptr, const void *ipc_handles_64,
                      void **comm_out);
/* The same for ONE process that drives all GPUs itself (the reference engine's model, src/forward.c:606):
 * bases[q] = rank q's buffer (mb200_comm_buffer_bytes bytes, zeroed, on device q with peer access enabled
 * from the device of `rank`); one comm per rank. */
int mb200_comm_create_ptrs(int rank, int world, size_t max_floats, void *const *bases, void **comm_out);
void mb200_comm_destroy(void *comm, int free_local);
/* out[i] = sum over ranks q = 0..world-1 of in_q[i]; n <= max_floats. */
int mb200_push_allreduce(void *comm, const float *in, float *out, int n, cudaStream_t stream);
/* out[q * n_per_rank + i] = in_q[i] (equal-sized pieces). */
int mb200_push_allgather(void *comm, const float *in, float *out, int n_per_rank, cudaStream_t stream);

/* Seeded synthetic tensors written on the device (benchmark workloads). */
int mb200_fill_q4k(void *dst, size_t n_blocks, uint64_t seed, cudaStream_t stream);
int mb200_fill_q6k(void *dst, size_t n_blocks, uint64_t seed, cudaStream_t stream);
/* Blocks [first_block, first_block + n_blocks) of the same stream (a shard of a tensor gets the bytes it has in the whole). */
int mb200_fill_q4k_at(void *dst, size_t first_block, size_t n_blocks, uint64_t seed, cudaStream_t stream);
int mb200_fill_q6k_at(void *dst, size_t first_block, size_t n_blocks, uint64_t seed, cudaStream_t stream);
int mb200_fill_normal_f32(float *dst, size_t n, uint64_t seed, float scale, cudaStream_t stream);
int mb200_fill_normal_f16(void *dst, size_t n, uint64_t seed, float scale, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MNEMO_B200_H */
