// Q4_K dequant-matvec family for decode (batch 1), sm_100a: every Q4_K entry
// point of the reference kernel ABI (plain / +residual / QKV / dual / scaled-add)
// plus the gate+up+SwiGLU fusion, all on the streaming skeleton of
// stream_matvec.cuh.
//
// Arithmetic: the activation vector is split once per CTA into two int8 levels
// per 32-column group, x ~= s*(q1 + q2/254). Nibbles are masked four at a time
// (low: w & 0x0F0F0F0F, high: w & 0xF0F0F0F0 = 16*nibble) and multiplied with
// dp4a -- exact integer dot products -- then scaled in fp32:
//   row.x = sum_sub  d*sc*(s*I/254) - dmin*m*sum(x)
// which is the reference's w = d*sc*q - dmin*m (src/kernels.cu:98-136) with the
// products re-associated. Integer fields (scales, mins, nibbles) are exact.
//
// Lane mapping: 4 lanes per super-block (lane g owns qs[32g..32g+31], i.e.
// sub-blocks 2g and 2g+1), 8 super-blocks per warp pass.
#include "q4k_policy.cuh"

namespace mb200 {
namespace {

using stream::Params;

}  // namespace

void q4k_init() { stream::init_attrs<Q4>(); }
int pdl_enabled() { return stream::pdl_mode(); }

// Two Q4_K tensors of different heights that share x, one launch (the decode path's Q and K projections;
// the reference's three-tensor form, cuda_matvec_q4k_qkv, needs V to be Q4_K too, which Q4_K_M files are not).
void q4k_matvec2(const void *wa, float *ya, int rows_a, const void *wb, float *yb, int rows_b, const float *x,
                 int n_cols, cudaStream_t stream, const char *where, const float *norm_w, float norm_eps)
{
    Params P{};
    P.norm_w = norm_w;
    P.norm_eps = norm_eps;
    P.seg[0] = {static_cast<const uint8_t *>(wa), ya, rows_a, 0};
    P.seg[1] = {static_cast<const uint8_t *>(wb), yb, rows_b, 0};
    P.nseg = 2;
    P.x = x;
    P.n_cols = n_cols;
    P.mode = stream::kStore;
    stream::launch<Q4>(P, stream, where);
}

void moe_gate_up_q4k(const void *experts, size_t stride, size_t gate_off, size_t up_off, const int *ids, int n_slots,
                     int expert_lo, int expert_cnt, const float *x, float *act, int EFF, int H, cudaStream_t stream,
                     const char *where)
{
    Params P{};
    P.seg[0].y = act;
    P.nseg = 1;
    P.x = x;
    P.n_cols = H;
    P.mode = stream::kMoeGateUp;
    P.ids = ids;
    P.ebase = static_cast<const uint8_t *>(experts);
    P.estride = stride;
    P.off_a = gate_off;
    P.off_b = up_off;
    P.n_slots = n_slots;
    P.expert_lo = expert_lo;
    P.expert_cnt = expert_cnt;
    P.erows = EFF;
    stream::launch<Q4>(P, stream, where);
}

void moe_down_q4k(const void *experts, size_t stride, size_t down_off, const int *ids, const float *wts, int n_slots,
                  int expert_lo, int expert_cnt, const float *act, const float *residual, float *y, int H, int EFF,
                  cudaStream_t stream, const char *where)
{
    Params P{};
    P.seg[0].y = y;
    P.nseg = 1;
    P.x = act;
    P.x_stride = EFF;
    P.residual = residual;
    P.n_cols = EFF;
    P.mode = stream::kMoeDown;
    P.ids = ids;
    P.wts = wts;
    P.ebase = static_cast<const uint8_t *>(experts);
    P.estride = stride;
    P.off_a = down_off;
    P.n_slots = n_slots;
    P.expert_lo = expert_lo;
    P.expert_cnt = expert_cnt;
    P.erows = H;
    stream::launch<Q4>(P, stream, where);
}

}  // namespace mb200

using namespace mb200;

extern "C" {

void cuda_matvec_q4k(const void *weights, const float *x, float *y, int n_rows, int n_cols,
                     cudaStream_t stream)
{
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(weights), y, n_rows, 0};
    P.nseg = 1;
    P.x = x;
    P.n_cols = n_cols;
    P.mode = stream::kStore;
    stream::launch<Q4>(P, stream, "cuda_matvec_q4k");
}

void cuda_matvec_q4k_add(const void *weights, const float *x, const float *residual, float *y,
                         int n_rows, int n_cols, cudaStream_t stream)
{
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(weights), y, n_rows, 0};
    P.nseg = 1;
    P.x = x;
    P.residual = residual;
    P.n_cols = n_cols;
    P.mode = stream::kAddResidual;
    stream::launch<Q4>(P, stream, "cuda_matvec_q4k_add");
}

void cuda_matvec_q4k_qkv(const void *w_q, const void *w_k, const void *w_v, const float *x,
                         float *out_q, float *out_k, float *out_v, int q_rows, int kv_rows,
                         int n_cols, cudaStream_t stream)
{
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(w_q), out_q, q_rows, 0};
    P.seg[1] = {static_cast<const uint8_t *>(w_k), out_k, kv_rows, 0};
    P.seg[2] = {static_cast<const uint8_t *>(w_v), out_v, kv_rows, 0};
    P.nseg = 3;
    P.x = x;
    P.n_cols = n_cols;
    P.mode = stream::kStore;
    stream::launch<Q4>(P, stream, "cuda_matvec_q4k_qkv");
}

void cuda_matvec_q4k_dual(const void *wa, const void *wb, const float *x, float *ya, float *yb,
                          int n_rows, int n_cols, cudaStream_t stream)
{
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(wa), ya, n_rows, 0};
    P.seg[1] = {static_cast<const uint8_t *>(wb), yb, n_rows, 0};
    P.nseg = 2;
    P.x = x;
    P.n_cols = n_cols;
    P.mode = stream::kStore;
    stream::launch<Q4>(P, stream, "cuda_matvec_q4k_dual");
}

void cuda_matvec_q4k_scaled_add(const void *weights, const float *x, float *y, int n_rows,
                                int n_cols, float scale, cudaStream_t stream)
{
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(weights), y, n_rows, 0};
    P.nseg = 1;
    P.x = x;
    P.scale = scale;
    P.n_cols = n_cols;
    P.mode = stream::kScaledAdd;
    stream::launch<Q4>(P, stream, "cuda_matvec_q4k_scaled_add");
}

int mb200_norm_matvec_q4k(const void *weights, const float *x, const float *norm_w, float eps, float *y, int n_rows,
                          int n_cols, cudaStream_t stream)
{
    if (!weights || !x || !norm_w || !y || n_rows < 0 || n_cols <= 0) return MB200_ERR_ARG;
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(weights), y, n_rows, 0};
    P.nseg = 1;
    P.x = x;
    P.norm_w = norm_w;
    P.norm_eps = eps;
    P.n_cols = n_cols;
    P.mode = stream::kStore;
    mb200_clear_status();
    stream::launch<Q4>(P, stream, "mb200_norm_matvec_q4k");
    return mb200_last_status();
}

int mb200_norm_matvec2_q4k(const void *wa, float *ya, int rows_a, const void *wb, float *yb, int rows_b, const float *x,
                           const float *norm_w, float eps, int n_cols, cudaStream_t stream)
{
    if (!wa || !wb || !ya || !yb || !x || !norm_w || rows_a < 0 || rows_b < 0 || n_cols <= 0) return MB200_ERR_ARG;
    mb200_clear_status();
    q4k_matvec2(wa, ya, rows_a, wb, yb, rows_b, x, n_cols, stream, "mb200_norm_matvec2_q4k", norm_w, eps);
    return mb200_last_status();
}

int mb200_set_pdl(int enabled)
{
    const int prev = stream::pdl_mode();
    stream::pdl_mode() = enabled ? 1 : 0;
    return prev;
}

int mb200_matvec_q4k_dual_swiglu(const void *w_gate, const void *w_up, const float *x, float *act,
                                 int n_rows, int n_cols, cudaStream_t stream)
{
    if (!w_gate || !w_up || !x || !act || n_rows < 0 || n_cols <= 0) return MB200_ERR_ARG;
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(w_gate), act, n_rows, 0};
    P.seg[1] = {static_cast<const uint8_t *>(w_up), act, n_rows, 0};
    P.nseg = 2;
    P.x = x;
    P.n_cols = n_cols;
    P.mode = stream::kSwiGLU;
    mb200_clear_status();
    stream::launch<Q4>(P, stream, "mb200_matvec_q4k_dual_swiglu");
    return mb200_last_status();
}

}  // extern "C"

#ifdef MB200_TRACE
extern "C" void mb200_trace_read(void *dst)
{
    cudaMemcpyFromSymbol(dst, mb200::stream::g_trace, sizeof(long long) * mb200::kSMs * 2 * 48, 0,
                         cudaMemcpyDeviceToDevice);
}
#endif
