// Q6_K dequant-matvec for decode (V projection, expert down projection, lm_head),
// sm_100a, on the streaming skeleton of stream_matvec.cuh.
//
// Q6_K super-blocks are 210 bytes, so only 2-byte alignment can be assumed for
// anything inside the tensor. The bulk copy moves the enclosing 16-byte-aligned
// span of a tile and lanes read their fields from shared memory as aligned
// words + funnel shift.
//
// Lane mapping: 4 lanes per super-block. Lane (hh = half 0/1, jj = 0/1) owns
// positions l = 16jj..16jj+15 of half hh: 16 bytes of ql[64hh..], 16 bytes of
// ql[64hh+32..] and 16 bytes of qh[32hh..] give its 64 weights (4 sixteen-groups
// x 16 columns): q = lo4 | hi2 << 4 rebuilt as bytes, dp4a against the two int8
// levels of x, weight = d * scale * (q - 32)
// (reference src/kernels.cu:455-484, tools/validate_dequant.py:286-317).
#include "q6k_policy.cuh"

namespace mb200 {
namespace {

using stream::Params;

}  // namespace

void q6k_init() { stream::init_attrs<Q6>(); }

void moe_down_q6k(const void *experts, size_t stride, size_t down_off, const int *ids, const float *wts, int n_slots,
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
    stream::launch<Q6>(P, stream, where);
}

}  // namespace mb200

using namespace mb200;

extern "C" {

void cuda_matvec_q6k(const void *weights, const float *x, float *y, int n_rows, int n_cols,
                     cudaStream_t stream)
{
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(weights), y, n_rows, 0};
    P.nseg = 1;
    P.x = x;
    P.n_cols = n_cols;
    P.mode = stream::kStore;
    stream::launch<Q6>(P, stream, "cuda_matvec_q6k");
}

int mb200_norm_matvec_q6k(const void *weights, const float *x, const float *norm_w, float eps, float *y, int n_rows,
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
    stream::launch<Q6>(P, stream, "mb200_norm_matvec_q6k");
    return mb200_last_status();
}

int mb200_matvec_q6k_scaled_add(const void *weights, const float *x, float *y, int n_rows,
                                int n_cols, float scale, cudaStream_t stream)
{
    if (!weights || !x || !y || n_rows < 0 || n_cols <= 0) return MB200_ERR_ARG;
    Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(weights), y, n_rows, 0};
    P.nseg = 1;
    P.x = x;
    P.scale = scale;
    P.n_cols = n_cols;
    P.mode = stream::kScaledAdd;
    mb200_clear_status();
    stream::launch<Q6>(P, stream, "mb200_matvec_q6k_scaled_add");
    return mb200_last_status();
}

}  // extern "C"

#ifdef MB200_TRACE
extern "C" void mb200_trace_read_q6k(void *dst)
{
    cudaMemcpyFromSymbol(dst, mb200::stream::g_trace, sizeof(long long) * mb200::kSMs * 2 * 48, 0,
                         cudaMemcpyDeviceToDevice);
}
#endif
