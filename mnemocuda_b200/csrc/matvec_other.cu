// Q8_0 / Q5_K / Q3_K matvecs on the streaming skeleton (other_policies.cuh): for whole 256-column blocks and
// tensors at the type's alignment. Ragged widths and odd addresses take the row-per-warp kernels of other_types.cu.
#include "other_policies.cuh"

namespace mb200 {

namespace {
template <class F>
bool stream_plain(const void *w, const float *x, float *y, int n_rows, int n_cols, cudaStream_t stream, const char *where)
{
    if (n_cols % 256 != 0 || n_cols > F::kMaxCols || (reinterpret_cast<uintptr_t>(w) & (F::kBaseAlign - 1))) return false;
    stream::Params P{};
    P.seg[0] = {static_cast<const uint8_t *>(w), y, n_rows, 0};
    P.nseg = 1;
    P.x = x;
    P.n_cols = n_cols;
    P.mode = stream::kStore;
    stream::launch<F>(P, stream, where);
    return true;
}
}  // namespace

bool stream_matvec_q8_0(const void *w, const float *x, float *y, int n_rows, int n_cols, cudaStream_t s)
{
    return stream_plain<Q8>(w, x, y, n_rows, n_cols, s, "cuda_matvec_q8_0");
}
bool stream_matvec_q5k(const void *w, const float *x, float *y, int n_rows, int n_cols, cudaStream_t s)
{
    return stream_plain<Q5>(w, x, y, n_rows, n_cols, s, "cuda_matvec_q5k");
}
bool stream_matvec_q3k(const void *w, const float *x, float *y, int n_rows, int n_cols, cudaStream_t s)
{
    return stream_plain<Q3>(w, x, y, n_rows, n_cols, s, "cuda_matvec_q3k");
}

void other_types_init()
{
    stream::init_attrs<Q8>();
    stream::init_attrs<Q5>();
    stream::init_attrs<Q3>();
}

}  // namespace mb200
