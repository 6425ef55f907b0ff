// Whole-token decode: the op order of the reference's forward_pass_sample / forward_layer
// (src/forward.c:1635-1707, 604-1117) issued against this library's kernels, with nothing
// returning to the host inside a token:
//   * every expert is resident, the routed ids stay on the device (the reference copies them
//     to the host and synchronises in every layer, src/forward.c:849-882);
//   * the token id and the position live in device memory: the embedding, RoPE, the KV store
//     and the attention read them there and the sampler writes the next token and advances
//     the position, so ONE captured CUDA graph is replayed token after token with no node
//     patched (the reference patches three kernel nodes per layer per token,
//     src/forward.c:636-662).
// Per layer: RMSNorm -> Q,K (one launch) and V matvecs -> q/k norm + RoPE + KV store (one
// launch) -> attention -> O projection + residual -> RMSNorm -> MoE block (one launch where
// the fused kernel covers the shape) -- 8 launches against the reference's ~45.
// The library allocates nothing: every buffer is inside the caller's workspace.
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "support.cuh"

namespace mb200 {
void qkv_q4k_q6k(const void *wq, float *q, int q_rows, const void *wk, float *k, const void *wv, float *v, int kv_rows,
                 const float *x, int n_cols, const float *norm_w, float norm_eps, cudaStream_t stream, const char *where);
void q4k_matvec2(const void *wa, float *ya, int rows_a, const void *wb, float *yb, int rows_b, const float *x,
                 int n_cols, cudaStream_t stream, const char *where, const float *norm_w, float norm_eps);

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Workspace {
    size_t hidden, normed, q, k, v, attn, rope, ids, wts, act, scratch, attn_ws, zero, total;
};

Workspace layout(const mb200_decode_model &m)
{
    Workspace w{};
    size_t o = 0;
    auto take = [&](size_t bytes) {
        const size_t at = o;
        o = align_up(o + bytes, 256);
        return at;
    };
    const size_t H = m.hidden, QD = (size_t)m.n_heads * m.head_dim, KD = (size_t)m.n_kv_heads * m.head_dim;
    // counters first: the caller zeroes the workspace once, these must start at zero
    w.scratch = take(mb200_router_scratch_bytes(m.n_experts));
    w.attn_ws = take(attn_workspace_bytes(m.n_kv_heads, m.n_heads / (m.n_kv_heads > 0 ? m.n_kv_heads : 1)));
    w.zero = take(H * 4);  // stays zero: the "residual" of a rank that must not add one
    w.hidden = take(H * 4);
    w.normed = take(H * 4);
    w.q = take(QD * 4);
    w.k = take(KD * 4);
    w.v = take(KD * 4);
    w.attn = take(QD * 4);
    w.rope = take((size_t)m.head_dim * 4);  // cos[head_dim / 2], sin[head_dim / 2]
    w.ids = take((size_t)m.top_k * 4);
    w.wts = take((size_t)m.top_k * 4);
    w.act = take((size_t)m.top_k * m.moe_inter * 4);
    w.total = o;
    return w;
}

int check_model(const mb200_decode_model *m)
{
    if (!m || !m->layers || m->n_layers < 1 || m->hidden < 1 || m->n_heads < 1 || m->n_kv_heads < 1 ||
        m->head_dim < 2 || (m->head_dim & 1) || m->n_heads % m->n_kv_heads || m->top_k < 1 || m->top_k > 16 ||
        m->n_experts < 1 || m->moe_inter < 1 || m->ctx_len < 1)
        return MB200_ERR_ARG;
    if (m->head_dim != 128) return MB200_ERR_UNSUPPORTED;  // the tensor-core attention kernel's head size
    return MB200_OK;
}

// The reference's matvec() type switch (src/forward.c:160-173) for the types on this path.
int matvec(const void *w, int type, const float *x, float *y, int rows, int cols, cudaStream_t s)
{
    switch (type) {
        case 0: cuda_matvec_f32(static_cast<const float *>(w), x, y, rows, cols, s); return MB200_OK;
        case 12: cuda_matvec_q4k(w, x, y, rows, cols, s); return MB200_OK;
        case 14: cuda_matvec_q6k(w, x, y, rows, cols, s); return MB200_OK;
        case 8: cuda_matvec_q8_0(w, x, y, rows, cols, s); return MB200_OK;
        case 11: cuda_matvec_q3k(w, x, y, rows, cols, s); return MB200_OK;
        case 13: cuda_matvec_q5k(w, x, y, rows, cols, s); return MB200_OK;
        default: return MB200_ERR_UNSUPPORTED;
    }
}

constexpr int kNormFoldMax = 4608;  // widest vector the matvecs' fused RMSNorm takes (one round of loads per CTA)

// A matvec on RMSNorm(x): folded into the matvec for the quantized types, norm kernel + matvec otherwise.
int matvec_norm(const void *w, int type, const float *x, const float *norm_w, float eps, float *normed_tmp, float *y,
                int rows, int cols, cudaStream_t s)
{
    if (!norm_w) return matvec(w, type, x, y, rows, cols, s);
    if (type == 12) return mb200_norm_matvec_q4k(w, x, norm_w, eps, y, rows, cols, s);
    if (type == 14) return mb200_norm_matvec_q6k(w, x, norm_w, eps, y, rows, cols, s);
    launch_rms_norm(x, norm_w, normed_tmp, nullptr, cols, eps, s);
    return matvec(w, type, normed_tmp, y, rows, cols, s);
}

struct Bufs {
    float *hidden, *normed, *q, *k, *v, *attn, *cos_t, *sin_t;
};
Bufs bufs(const mb200_decode_model &m, uint8_t *ws, const Workspace &W)
{
    Bufs b;
    b.hidden = reinterpret_cast<float *>(ws + W.hidden);
    b.normed = reinterpret_cast<float *>(ws + W.normed);
    b.q = reinterpret_cast<float *>(ws + W.q);
    b.k = reinterpret_cast<float *>(ws + W.k);
    b.v = reinterpret_cast<float *>(ws + W.v);
    b.attn = reinterpret_cast<float *>(ws + W.attn);
    b.cos_t = reinterpret_cast<float *>(ws + W.rope);
    b.sin_t = b.cos_t + m.head_dim / 2;
    return b;
}

// Steps 1-6 of forward_layer (src/forward.c:670-768): norm, Q/K/V projections, q/k norm + RoPE + KV store,
// attention -- over the heads this descriptor holds (all of them, or a rank's share). attn_out: [n_heads * head_dim].
int run_attention(const mb200_decode_model &m, const mb200_layer_weights &L, uint8_t *ws, const Workspace &W,
                  const int *d_pos, float *attn_out, cudaStream_t s)
{
    const Bufs B = bufs(m, ws, W);
    const int H = m.hidden, QD = m.n_heads * m.head_dim, KD = m.n_kv_heads * m.head_dim;
    int rc;
    // 1 + 2. pre-attention norm and the Q, K, V projections. The norm is folded into the matvecs' staging of x
    // (each CTA normalises the vector it reads anyway) where the width allows: no norm kernel, no `normed` round
    // trip. The residual stays in `hidden`: the O projection adds it back in place.
    const bool fold = H <= kNormFoldMax && (L.wv_type == 12 || L.wv_type == 14);
    if (!fold) launch_rms_norm(B.hidden, L.attn_norm, B.normed, nullptr, H, m.rms_eps, s);
    const float *x = fold ? B.hidden : B.normed;
    const float *nw = fold ? L.attn_norm : nullptr;
    if (L.wq_type == 12 && L.wk_type == 12 && L.wv_type == 14) {  // the Q4_K_M layout: one launch for all three
        qkv_q4k_q6k(L.wq, B.q, QD, L.wk, B.k, L.wv, B.v, KD, x, H, nw, m.rms_eps, s, "mb200_decode: Q,K,V projection");
    } else {
        if (L.wq_type == 12 && L.wk_type == 12) {
            q4k_matvec2(L.wq, B.q, QD, L.wk, B.k, KD, x, H, s, "mb200_decode: Q,K projection", nw, m.rms_eps);
        } else {
            if ((rc = matvec_norm(L.wq, L.wq_type, x, nw, m.rms_eps, B.normed, B.q, QD, H, s)) != MB200_OK) return rc;
            if ((rc = matvec_norm(L.wk, L.wk_type, x, nw, m.rms_eps, B.normed, B.k, KD, H, s)) != MB200_OK) return rc;
        }
        if ((rc = matvec_norm(L.wv, L.wv_type, x, nw, m.rms_eps, B.normed, B.v, KD, H, s)) != MB200_OK) return rc;
    }
    // 3-5. q/k norm, RoPE, fp16 KV store at the position
    launch_qk_norm_rope_store(B.q, B.k, B.v, L.q_norm, L.k_norm, B.cos_t, B.sin_t, L.kv_k, L.kv_v, m.n_heads,
                              m.n_kv_heads, m.head_dim, m.rms_eps, d_pos, 0, s);
    // 6. attention over positions 0..pos
    return launch_attn_decode(B.q, L.kv_k, L.kv_v, attn_out, m.n_heads, m.n_kv_heads, 0, d_pos,
                              1.0f / sqrtf(static_cast<float>(m.head_dim)), ws + W.attn_ws, s);
}

// Step 7: rows [row0, row0 + rows) of hidden = Wo[rows] . attn + hidden[rows] (L.wo points at the first of those rows).
int run_oproj(const mb200_decode_model &m, const mb200_layer_weights &L, uint8_t *ws, const Workspace &W,
              const float *attn_full, int qd_total, int row0, int rows, float *out_rows, cudaStream_t s)
{
    const Bufs B = bufs(m, ws, W);
    if (L.wo_type == 12) {
        cuda_matvec_q4k_add(L.wo, attn_full, B.hidden + row0, out_rows, rows, qd_total, s);
        return MB200_OK;
    }
    const int rc = matvec(L.wo, L.wo_type, attn_full, B.normed, rows, qd_total, s);
    if (rc != MB200_OK) return rc;
    cuda_residual_add(B.normed, B.hidden + row0, out_rows, rows, s);
    return MB200_OK;
}

// Steps 8-13: pre-FFN norm, router, top-k, the routed experts held here, weighted sum (+ residual if asked).
int run_moe(const mb200_decode_model &m, const mb200_layer_weights &L, uint8_t *ws, const Workspace &W, bool with_residual,
            float *out, cudaStream_t s)
{
    const Bufs B = bufs(m, ws, W);
    const int H = m.hidden;
    const float *res = B.hidden;
    if (!with_residual) {  // another rank adds the residual: this one contributes its experts only
        float *zero = reinterpret_cast<float *>(ws + W.zero);
        res = zero;
    }
    // the pre-FFN norm is folded into the one-launch block where that form applies (else it runs as a kernel inside)
    const bool own = L.expert_stride != 0;  // this layer's own blob layout
    return mb200_moe_block_norm(L.router, L.experts, own ? L.expert_stride : m.expert_stride, own ? L.gate_sz : m.gate_sz,
                                own ? L.up_sz : m.up_sz, own ? L.down_type : m.down_type, m.n_experts,
                                m.expert_lo, m.expert_cnt > 0 ? m.expert_cnt : 0x7fffffff, m.top_k, H, m.moe_inter,
                                B.hidden, L.ffn_norm, m.rms_eps, B.normed, res, out, reinterpret_cast<int *>(ws + W.ids),
                                reinterpret_cast<float *>(ws + W.wts), reinterpret_cast<float *>(ws + W.act),
                                ws + W.scratch, s);
}

int run_layer(const mb200_decode_model &m, const mb200_layer_weights &L, uint8_t *ws, const Workspace &W,
              const int *d_pos, cudaStream_t s)
{
    const Bufs B = bufs(m, ws, W);
    int rc = run_attention(m, L, ws, W, d_pos, B.attn, s);
    if (rc != MB200_OK) return rc;
    rc = run_oproj(m, L, ws, W, B.attn, m.n_heads * m.head_dim, 0, m.hidden, B.hidden, s);
    if (rc != MB200_OK) return rc;
    return run_moe(m, L, ws, W, true, B.hidden, s);
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" {

size_t mb200_decode_workspace_bytes(const mb200_decode_model *m)
{
    if (check_model(m) != MB200_OK) return 0;
    return layout(*m).total;
}

float *mb200_decode_hidden(const mb200_decode_model *m, void *workspace)
{
    if (check_model(m) != MB200_OK || !workspace) return nullptr;
    return reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + layout(*m).hidden);
}

int mb200_decode_begin(const mb200_decode_model *m, void *workspace, const int *d_token, const int *d_pos,
                       cudaStream_t stream)
{
    int rc = check_model(m);
    if (rc != MB200_OK) return rc;
    if (!workspace || !d_token || !d_pos || !m->token_embd) return MB200_ERR_ARG;
    if (m->embd_type != 12 && m->embd_type != 11) return MB200_ERR_UNSUPPORTED;  // src/forward.c:1176-1187
    const Workspace W = layout(*m);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    mb200_clear_status();
    if (m->embd_type == 12)
        launch_embed_q4k(m->token_embd, reinterpret_cast<float *>(ws + W.hidden), d_token, 0, m->hidden,
                         (m->hidden + 255) / 256 * kQ4KBlock, stream);
    else
        launch_embed_q3k(m->token_embd, reinterpret_cast<float *>(ws + W.hidden), d_token, 0, m->hidden,
                         (m->hidden + 255) / 256 * 110, stream);
    float *cos_t = reinterpret_cast<float *>(ws + W.rope);
    launch_rope_table(cos_t, cos_t + m->head_dim / 2, m->head_dim, d_pos, 0, m->rope_theta, stream);
    if (cudaGetLastError() != cudaSuccess) return MB200_ERR_LAUNCH;
    return mb200_last_status();
}

int mb200_decode_layer(const mb200_decode_model *m, int layer, void *workspace, const int *d_pos, cudaStream_t stream)
{
    int rc = check_model(m);
    if (rc != MB200_OK) return rc;
    if (!workspace || !d_pos || layer < 0 || layer >= m->n_layers) return MB200_ERR_ARG;
    mb200_clear_status();
    rc = run_layer(*m, m->layers[layer], static_cast<uint8_t *>(workspace), layout(*m), d_pos, stream);
    if (rc != MB200_OK) return rc;
    if (cudaGetLastError() != cudaSuccess) return MB200_ERR_LAUNCH;
    return mb200_last_status();
}

// ---- the same layer in three pieces, for a model sharded over devices ----
int mb200_decode_layer_attn(const mb200_decode_model *m, int layer, void *workspace, const int *d_pos, float *attn_local,
                            cudaStream_t stream)
{
    int rc = check_model(m);
    if (rc != MB200_OK) return rc;
    if (!workspace || !d_pos || !attn_local || layer < 0 || layer >= m->n_layers) return MB200_ERR_ARG;
    mb200_clear_status();
    rc = run_attention(*m, m->layers[layer], static_cast<uint8_t *>(workspace), layout(*m), d_pos, attn_local, stream);
    if (rc != MB200_OK) return rc;
    if (cudaGetLastError() != cudaSuccess) return MB200_ERR_LAUNCH;
    return mb200_last_status();
}

int mb200_decode_layer_oproj(const mb200_decode_model *m, int layer, void *workspace, const float *attn_full,
                             float *hidden_rows, cudaStream_t stream)
{
    int rc = check_model(m);
    if (rc != MB200_OK) return rc;
    if (!workspace || !attn_full || !hidden_rows || layer < 0 || layer >= m->n_layers) return MB200_ERR_ARG;
    const int total_heads = m->n_heads_total > 0 ? m->n_heads_total : m->n_heads;
    const int rows = m->o_rows > 0 ? m->o_rows : m->hidden;
    if (m->o_row0 < 0 || m->o_row0 + rows > m->hidden) return MB200_ERR_ARG;
    mb200_clear_status();
    rc = run_oproj(*m, m->layers[layer], static_cast<uint8_t *>(workspace), layout(*m), attn_full,
                   total_heads * m->head_dim, m->o_row0, rows, hidden_rows, stream);
    if (rc != MB200_OK) return rc;
    if (cudaGetLastError() != cudaSuccess) return MB200_ERR_LAUNCH;
    return mb200_last_status();
}

int mb200_decode_layer_moe(const mb200_decode_model *m, int layer, void *workspace, int add_residual, float *out,
                           cudaStream_t stream)
{
    int rc = check_model(m);
    if (rc != MB200_OK) return rc;
    if (!workspace || !out || layer < 0 || layer >= m->n_layers) return MB200_ERR_ARG;
    mb200_clear_status();
    rc = run_moe(*m, m->layers[layer], static_cast<uint8_t *>(workspace), layout(*m), add_residual != 0, out, stream);
    if (rc != MB200_OK) return rc;
    if (cudaGetLastError() != cudaSuccess) return MB200_ERR_LAUNCH;
    return mb200_last_status();
}

int mb200_decode_layer_moe_reduce(const mb200_decode_model *m, int layer, void *workspace, int add_residual,
                                  float *partial, float *out, void *comm, cudaStream_t stream)
{
    int rc = check_model(m);
    if (rc != MB200_OK) return rc;
    if (!workspace || !out || !partial || !comm || layer < 0 || layer >= m->n_layers) return MB200_ERR_ARG;
    mb200_clear_status();
    {   // the block and its all-reduce in one launch, where that form exists
        const mb200_layer_weights &L = m->layers[layer];
        uint8_t *ws = static_cast<uint8_t *>(workspace);
        const Workspace W = layout(*m);
        const Bufs B = bufs(*m, ws, W);
        const bool own = L.expert_stride != 0;
        rc = mb200_moe_block_push(L.router, L.experts, own ? L.expert_stride : m->expert_stride, own ? L.gate_sz : m->gate_sz,
                                  own ? L.up_sz : m->up_sz, own ? L.down_type : m->down_type, m->n_experts, m->expert_lo,
                                  m->expert_cnt > 0 ? m->expert_cnt : 0x7fffffff, m->top_k, m->hidden, m->moe_inter, B.hidden,
                                  L.ffn_norm, m->rms_eps, add_residual ? B.hidden : nullptr, out,
                                  reinterpret_cast<int *>(ws + W.ids), reinterpret_cast<float *>(ws + W.wts),
                                  reinterpret_cast<float *>(ws + W.act), ws + W.scratch, comm, stream);
        if (rc == MB200_OK) return cudaGetLastError() == cudaSuccess ? mb200_last_status() : MB200_ERR_LAUNCH;
        if (rc != MB200_ERR_UNSUPPORTED && rc != MB200_ERR_LAUNCH) return rc;
        (void)cudaGetLastError();
    }
    rc = run_moe(*m, m->layers[layer], static_cast<uint8_t *>(workspace), layout(*m), add_residual != 0, partial, stream);
    if (rc != MB200_OK) return rc;
    rc = mb200_push_allreduce(comm, partial, out, m->hidden, stream);
    if (rc != MB200_OK) return rc;
    if (cudaGetLastError() != cudaSuccess) return MB200_ERR_LAUNCH;
    return mb200_last_status();
}

int mb200_decode_logits_local(const mb200_decode_model *m, void *workspace, float *logits_rows, float *best_pair,
                              cudaStream_t stream)
{
    int rc = check_model(m);
    if (rc != MB200_OK) return rc;
    if (!workspace || !logits_rows || !best_pair || !m->output_norm || !m->lm_head) return MB200_ERR_ARG;
    const int rows = m->lm_rows > 0 ? m->lm_rows : m->vocab;
    if (rows < 1 || m->lm_row0 < 0) return MB200_ERR_ARG;
    const Workspace W = layout(*m);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    float *hidden = reinterpret_cast<float *>(ws + W.hidden), *normed = reinterpret_cast<float *>(ws + W.normed);
    mb200_clear_status();
    if ((rc = matvec_norm(m->lm_head, m->lm_head_type, hidden, m->hidden <= kNormFoldMax ? m->output_norm : nullptr,
                          m->rms_eps, normed, logits_rows, rows, m->hidden, stream)) != MB200_OK)
        return rc;
    launch_argmax_pair(logits_rows, rows, m->lm_row0, best_pair, stream);
    if (cudaGetLastError() != cudaSuccess) return MB200_ERR_LAUNCH;
    return mb200_last_status();
}

int mb200_decode_pick(const float *pairs, int n_pairs, int *d_token, int *d_pos, cudaStream_t stream)
{
    if (!pairs || n_pairs < 1 || !d_token) return MB200_ERR_ARG;
    launch_argmax_merge(pairs, n_pairs, d_token, d_pos, stream);
    return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

int mb200_decode_finish(const mb200_decode_model *m, void *workspace, float *d_logits, int *d_token, int *d_pos,
                        cudaStream_t stream)
{
    int rc = check_model(m);
    if (rc != MB200_OK) return rc;
    if (!workspace || !d_logits || !d_token || !m->output_norm || !m->lm_head || m->vocab < 1) return MB200_ERR_ARG;
    const Workspace W = layout(*m);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    float *hidden = reinterpret_cast<float *>(ws + W.hidden), *normed = reinterpret_cast<float *>(ws + W.normed);
    mb200_clear_status();
    if ((rc = matvec_norm(m->lm_head, m->lm_head_type, hidden, m->hidden <= kNormFoldMax ? m->output_norm : nullptr,
                          m->rms_eps, normed, d_logits, m->vocab, m->hidden, stream)) != MB200_OK)
        return rc;
    launch_argmax(d_logits, m->vocab, d_token, d_pos, stream);
    if (cudaGetLastError() != cudaSuccess) return MB200_ERR_LAUNCH;
    return mb200_last_status();
}

int mb200_decode_step(const mb200_decode_model *m, void *workspace, int *d_token, int *d_pos, float *d_logits,
                      cudaStream_t stream)
{
    int rc = mb200_decode_begin(m, workspace, d_token, d_pos, stream);
    if (rc != MB200_OK) return rc;
    for (int l = 0; l < m->n_layers; l++)
        if ((rc = mb200_decode_layer(m, l, workspace, d_pos, stream)) != MB200_OK) return rc;
    return mb200_decode_finish(m, workspace, d_logits, d_token, d_pos, stream);
}

}  // extern "C"
