// The small fp32 operators of the reference kernel ABI: router matvec, top-k +
// softmax, SwiGLU, scaled add.
#include <cstdio>

#include "common.cuh"
#include "topk.cuh"

namespace mb200 {
namespace {

// ---- y = W x, W fp32 row-major (reference src/kernels.cu:859-880) -------------
// One CTA of 4 warps per row; every lane issues all of its 16-byte loads before
// the first add, so a 16 KB router row is a single round trip to memory.
constexpr int kF32Threads = 128;

__global__ void __launch_bounds__(kF32Threads) matvec_f32_kernel(const float *__restrict__ w,
                                                                 const float *__restrict__ x,
                                                                 float *__restrict__ y, int n_rows,
                                                                 int n_cols, int vec_ok)
{
    __shared__ float red[kF32Threads / 32];
    const int row = blockIdx.x;
    const float *wr = w + (size_t)row * n_cols;
    float acc = 0.0f;
    if (vec_ok) {
        const float4 *w4 = reinterpret_cast<const float4 *>(wr);
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        const int n4 = n_cols >> 2;
        for (int i0 = threadIdx.x; i0 < n4; i0 += kF32Threads * 8) {
            float4 a[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * kF32Threads;
                a[u] = i < n4 ? __ldcs(w4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * kF32Threads;
                if (i < n4) {
                    const float4 b = __ldcg(x4 + i);
                    acc = fmaf(a[u].x, b.x, acc);
                    acc = fmaf(a[u].y, b.y, acc);
                    acc = fmaf(a[u].z, b.z, acc);
                    acc = fmaf(a[u].w, b.w, acc);
                }
            }
        }
    } else {
        for (int c = threadIdx.x; c < n_cols; c += kF32Threads) acc = fmaf(wr[c], x[c], acc);
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) y[row] = (red[0] + red[1]) + (red[2] + red[3]);
}

__global__ void __launch_bounds__(32) topk_softmax_kernel(const float *__restrict__ scores,
                                                          int *__restrict__ indices,
                                                          float *__restrict__ weights, int n_experts,
                                                          int k)
{
    __shared__ TopkShared sh;
    topk_softmax_warp(scores, indices, weights, n_experts, k, sh);
}

__global__ void swiglu_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                              float *__restrict__ out, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = gate[i];
    out[i] = g / (1.0f + expf(-g)) * up[i];
}

__global__ void scaled_add_kernel(float *__restrict__ out, const float *__restrict__ x, float scale,
                                  int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] += scale * x[i];
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" {

void cuda_matvec_f32(const float *weights, const float *x, float *y, int n_rows, int n_cols,
                     cudaStream_t stream)
{
    if (n_rows <= 0 || n_cols <= 0) return;
    const int vec_ok = (n_cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(weights) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    matvec_f32_kernel<<<n_rows, kF32Threads, 0, stream>>>(weights, x, y, n_rows, n_cols, vec_ok);
    MB200_CHECK_LAUNCH("cuda_matvec_f32");
}

void cuda_topk_softmax(const float *scores, int *indices, float *weights, int n_experts, int k,
                       cudaStream_t stream)
{
    if (k < 1 || k > 16) {
        fprintf(stderr, "[mnemo_b200] cuda_topk_softmax: k=%d outside 1..16\n", k);
        set_status(MB200_ERR_ARG, "cuda_topk_softmax");
        return;
    }
    topk_softmax_kernel<<<1, 32, 0, stream>>>(scores, indices, weights, n_experts, k);
    MB200_CHECK_LAUNCH("cuda_topk_softmax");
}

void cuda_swiglu(const float *gate, const float *up, float *out, int n, cudaStream_t stream)
{
    if (n <= 0) return;
    swiglu_kernel<<<(n + 255) / 256, 256, 0, stream>>>(gate, up, out, n);
    MB200_CHECK_LAUNCH("cuda_swiglu");
}

void cuda_scaled_add(float *out, const float *x, float scale, int n, cudaStream_t stream)
{
    if (n <= 0) return;
    scaled_add_kernel<<<(n + 255) / 256, 256, 0, stream>>>(out, x, scale, n);
    MB200_CHECK_LAUNCH("cuda_scaled_add");
}

}  // extern "C"
