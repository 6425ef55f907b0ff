// The Q, K (Q4_K) and V (Q6_K) projections of a decoded token in ONE launch: a Q4_K_M file stores V in
// Q6_K, so the reference's three-tensor kernel (cuda_matvec_q4k_qkv, src/kernels.cu:196-268) does not
// apply and its engine issues three launches (src/forward.c:688-704). Here the SMs are divided between
// the two block types in proportion to their bytes and each CTA runs the streaming body of its type
// (stream_matvec.cuh: stream_pair_kernel). All three share x; with a norm weight vector the RMSNorm of x
// is folded into each CTA's staging of it.
#include "q4k_policy.cuh"
#include "q6k_policy.cuh"

namespace mb200 {

void q4k_matvec2(const void *wa, float *ya, int rows_a, const void *wb, float *yb, int rows_b, const float *x,
                 int n_cols, cudaStream_t stream, const char *where, const float *norm_w, float norm_eps);

void qkv_q4k_q6k(const void *wq, float *q, int q_rows, const void *wk, float *k, const void *wv, float *v, int kv_rows,
                 const float *x, int n_cols, const float *norm_w, float norm_eps, cudaStream_t stream, const char *where)
{
    stream::Params A{}, B{};
    A.norm_w = B.norm_w = norm_w;
    A.norm_eps = B.norm_eps = norm_eps;
    A.seg[0] = {static_cast<const uint8_t *>(wq), q, q_rows, 0};
    A.seg[1] = {static_cast<const uint8_t *>(wk), k, kv_rows, 0};
    A.nseg = 2;
    B.seg[0] = {static_cast<const uint8_t *>(wv), v, kv_rows, 0};
    B.nseg = 1;
    A.x = B.x = x;
    A.n_cols = B.n_cols = n_cols;
    A.mode = B.mode = stream::kStore;
    if (stream::launch_pair<Q4, Q6>(A, B, stream, where)) return;
    // an empty or unsupported half: the single launches report what is wrong with it
    q4k_matvec2(wq, q, q_rows, wk, k, kv_rows, x, n_cols, stream, where, norm_w, norm_eps);
    if (norm_w)
        mb200_norm_matvec_q6k(wv, x, norm_w, norm_eps, v, kv_rows, n_cols, stream);
    else
        cuda_matvec_q6k(wv, x, v, kv_rows, n_cols, stream);
}

void pair_init()
{
    // the shared-memory opt-in of the pair kernel, per device, outside any stream capture
    static bool done[kMaxDevices] = {false};
    const int dev = current_device();
    if (done[dev]) return;
    cudaFuncSetAttribute(stream::stream_pair_kernel<Q4, Q6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    done[dev] = true;
}

}  // namespace mb200

using namespace mb200;

extern "C" int mb200_norm_matvec_qkv(const void *wq, float *q, int q_rows, const void *wk, float *k, const void *wv,
                                     float *v, int kv_rows, const float *x, const float *norm_w, float eps, int n_cols,
                                     cudaStream_t stream)
{
    if (!wq || !wk || !wv || !q || !k || !v || !x || q_rows < 1 || kv_rows < 1 || n_cols <= 0) return MB200_ERR_ARG;
    mb200_clear_status();
    qkv_q4k_q6k(wq, q, q_rows, wk, k, wv, v, kv_rows, x, n_cols, norm_w, eps, stream, "mb200_norm_matvec_qkv");
    return mb200_last_status();
}
