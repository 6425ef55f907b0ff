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
void q4k_matvec2(const void *wa, float *ya, int rows_a, const void *wb, float *yb, int rows_b, const float *x,
                 int n_cols, cudaStream_t stream, const char *where);

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Workspace {
    size_t hidden, normed, q, k, v, attn, rope, ids, wts, act, scratch, attn_ws, total;
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
        default: return MB200_ERR_UNSUPPORTED;
    }
}

int run_layer(const mb200_decode_model &m, const mb200_layer_weights &L, uint8_t *ws, const Workspace &W,
              const int *d_pos, cudaStream_t s)
{
    float *hidden = reinterpret_cast<float *>(ws + W.hidden), *normed = reinterpret_cast<float *>(ws + W.normed);
    float *q = reinterpret_cast<float *>(ws + W.q), *k = reinterpret_cast<float *>(ws + W.k);
    float *v = reinterpret_cast<float *>(ws + W.v), *attn = reinterpret_cast<float *>(ws + W.attn);
    float *cos_t = reinterpret_cast<float *>(ws + W.rope), *sin_t = cos_t + m.head_dim / 2;
    const int H = m.hidden, QD = m.n_heads * m.head_dim, KD = m.n_kv_heads * m.head_dim;
    int rc;
    // 1. pre-attention norm (the residual stays in `hidden`: the O projection adds it back in place)
    launch_rms_norm(hidden, L.attn_norm, normed, nullptr, H, m.rms_eps, s);
    // 2. Q, K, V projections
    if (L.wq_type == 12 && L.wk_type == 12) {
        q4k_matvec2(L.wq, q, QD, L.wk, k, KD, normed, H, s, "mb200_decode: Q,K projection");
    } else {
        if ((rc = matvec(L.wq, L.wq_type, normed, q, QD, H, s)) != MB200_OK) return rc;
        if ((rc = matvec(L.wk, L.wk_type, normed, k, KD, H, s)) != MB200_OK) return rc;
    }
    if ((rc = matvec(L.wv, L.wv_type, normed, v, KD, H, s)) != MB200_OK) return rc;
    // 3-5. q/k norm, RoPE, fp16 KV store at the position
    launch_qk_norm_rope_store(q, k, v, L.q_norm, L.k_norm, cos_t, sin_t, L.kv_k, L.kv_v, m.n_heads, m.n_kv_heads,
                              m.head_dim, m.rms_eps, d_pos, 0, s);
    // 6. attention over positions 0..pos
    rc = launch_attn_decode(q, L.kv_k, L.kv_v, attn, m.n_heads, m.n_kv_heads, 0, d_pos,
                            1.0f / sqrtf(static_cast<float>(m.head_dim)), ws + W.attn_ws, s);
    if (rc != MB200_OK) return rc;
    // 7. output projection + residual
    if (L.wo_type == 12) {
        cuda_matvec_q4k_add(L.wo, attn, hidden, hidden, H, QD, s);
    } else {
        if ((rc = matvec(L.wo, L.wo_type, attn, normed, H, QD, s)) != MB200_OK) return rc;
        cuda_residual_add(normed, hidden, hidden, H, s);
    }
    // 8. pre-FFN norm, 9-13. router, top-k, routed experts, weighted sum + residual
    launch_rms_norm(hidden, L.ffn_norm, normed, nullptr, H, m.rms_eps, s);
    return mb200_moe_block_local(L.router, L.experts, m.expert_stride, m.gate_sz, m.up_sz, m.down_type, m.n_experts,
                                 m.expert_lo, m.expert_cnt > 0 ? m.expert_cnt : 0x7fffffff, m.top_k, H, m.moe_inter,
                                 normed, hidden, hidden, reinterpret_cast<int *>(ws + W.ids),
                                 reinterpret_cast<float *>(ws + W.wts), reinterpret_cast<float *>(ws + W.act),
                                 ws + W.scratch, s);
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
    if (m->embd_type != 12) return MB200_ERR_UNSUPPORTED;
    const Workspace W = layout(*m);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    mb200_clear_status();
    launch_embed_q4k(m->token_embd, reinterpret_cast<float *>(ws + W.hidden), d_token, 0, m->hidden,
                     (m->hidden + 255) / 256 * kQ4KBlock, stream);
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
    launch_rms_norm(hidden, m->output_norm, normed, nullptr, m->hidden, m->rms_eps, stream);
    if ((rc = matvec(m->lm_head, m->lm_head_type, normed, d_logits, m->vocab, m->hidden, stream)) != MB200_OK) return rc;
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
