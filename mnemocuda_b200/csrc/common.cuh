// Shared device/host helpers for the sm_100a kernels: status codes, mbarrier +
// bulk-copy (TMA 1-D) wrappers with bounded waits, fp16 and Q4_K/Q6_K field decode.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mnemo_b200.h"

namespace mb200 {

constexpr int kQ4KBlock = 144;
constexpr int kQ6KBlock = 210;
constexpr int kSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// ---- library-wide status --------------------------------------------------
// The reference wrappers return void (errors are printed: kernels.cu:1062-1067).
// Ours record the first failure here as well so a caller can poll it.
void set_status(int code, const char *where);
int *device_error_word();  // device int, non-zero after a kernel gave up on a wait

#define MB200_CHECK_LAUNCH(where)                                                        \
    do {                                                                                 \
        cudaError_t e__ = cudaGetLastError();                                            \
        if (e__ != cudaSuccess) {                                                        \
            fprintf(stderr, "[mnemo_b200] launch error in %s: %s\n", where,              \
                    cudaGetErrorString(e__));                                            \
            mb200::set_status(MB200_ERR_LAUNCH, where);                                  \
        }                                                                                \
    } while (0)

// ---- small device helpers ---------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Butterfly over the low log2(width) lane bits only (width: power of two <= 32).
__device__ __forceinline__ float group_sum(float v, int width)
{
    for (int o = width >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float h2f_lo(uint32_t packed)
{
    return __half2float(__ushort_as_half(static_cast<unsigned short>(packed & 0xFFFFu)));
}
__device__ __forceinline__ float h2f_hi(uint32_t packed)
{
    return __half2float(__ushort_as_half(static_cast<unsigned short>(packed >> 16)));
}

// 4 x (u8 * s8) + c, exact.
__device__ __forceinline__ int dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
    return d;
}

// ---- mbarrier + bulk async copy (global -> shared::cta), all waits bounded ----
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Returns false if the phase did not complete within the iteration budget
// (each try_wait already blocks for a hardware time slice).
constexpr uint32_t kWaitBudget = 1u << 20;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kWaitBudget; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// 1-D bulk copy; src and dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                         uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- Q4_K scale/min pair decode (reference src/kernels.cu:45-53) -------------
// a,b,c = the three little-endian words of scales[12]; g = 0..3 selects
// sub-blocks (2g, 2g+1). Returns sc pair / m pair packed as two bytes each.
__device__ __forceinline__ void q4k_scale_pair(uint32_t a, uint32_t b, uint32_t c, int g,
                                               uint32_t &sc2, uint32_t &m2)
{
    const int sh = (g & 1) * 16;
    const uint32_t as = a >> sh, bs = b >> sh, cs = c >> sh;
    if (g < 2) {
        sc2 = as & 0x3F3Fu;
        m2 = bs & 0x3F3Fu;
    } else {
        sc2 = (cs & 0x0F0Fu) | ((as >> 2) & 0x3030u);
        m2 = ((cs >> 4) & 0x0F0Fu) | ((bs >> 2) & 0x3030u);
    }
}

// ---- activation split shared by the Q4_K and Q6_K streaming kernels ----------
// x[c] ~= s1[c/32] * (q1[c] + q2[c]/254) with q1, q2 int8: two exact dp4a dot
// products then recover sum(q*x) to ~1e-5 relative (|error| <= max|x|/64516 per
// 32-column group). xsum holds exact fp32 sums of x over SUM_COLS columns (for
// the terms that multiply sum(x): Q4_K's -dmin*m, Q6_K's -32 offset).
// Columns outside the matrix are stored as zero. GROUP4: a group of 4 columns
// counts only if all four are < n_cols (the Q4_K kernels' tail rule,
// reference src/kernels.cu:124,131); otherwise per column (Q6_K, :474).
// kpad is a multiple of 256; all threads of the CTA call this.
template <int THREADS, int SUM_COLS, bool GROUP4>
__device__ __forceinline__ void quantize_x(const float *__restrict__ x, int n_cols, int kpad,
                                           int8_t *q1, int8_t *q2, float *s1, float *xsum)
{
    static_assert(SUM_COLS == 16 || SUM_COLS == 8, "sum granularity");
    const int lane = threadIdx.x & 31;
    for (int c0 = threadIdx.x * 4; c0 < kpad; c0 += THREADS * 4) {
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const bool in = GROUP4 ? (c0 + 3) < n_cols : (c0 + i) < n_cols;
            v[i] = in ? __ldg(x + c0 + i) : 0.0f;
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        float sum = (v[0] + v[1]) + (v[2] + v[3]);
        // 8 lanes = 32 columns share a scale
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if (SUM_COLS == 16) sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float sc = amax * (1.0f / 127.0f);
        const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
        uint32_t p1 = 0, p2 = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float a = fminf(fmaxf(rintf(v[i] * inv), -127.0f), 127.0f);
            const float r = fmaf(-a, sc, v[i]);
            const float b = fminf(fmaxf(rintf(r * inv * 254.0f), -127.0f), 127.0f);
            p1 |= (static_cast<uint32_t>(static_cast<int>(a)) & 0xFFu) << (8 * i);
            p2 |= (static_cast<uint32_t>(static_cast<int>(b)) & 0xFFu) << (8 * i);
        }
        reinterpret_cast<uint32_t *>(q1)[c0 >> 2] = p1;
        reinterpret_cast<uint32_t *>(q2)[c0 >> 2] = p2;
        if ((lane & 7) == 0) s1[c0 >> 5] = sc;
        if (SUM_COLS == 16) {
            if ((lane & 3) == 0) xsum[c0 >> 4] = sum;
        } else {
            if ((lane & 1) == 0) xsum[c0 >> 3] = sum;
        }
    }
}

}  // namespace mb200
