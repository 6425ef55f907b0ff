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
constexpr int kSMs = 148;      // B200: 2 dies x 74 SMs; used where no device is known yet (fills, table sizes)
constexpr int kMaxDevices = 64;  // per-device host-side state is kept in arrays of this length

// ---- library-wide status --------------------------------------------------
// The reference wrappers return void (errors are printed: kernels.cu:1062-1067).
// Ours record the first failure here as well so a caller can poll it.
void set_status(int code, const char *where);
int *device_error_word();  // device int, non-zero after a kernel gave up on a wait
// Ordinal of the current device, clamped to [0, kMaxDevices). Function attributes (the shared-memory
// opt-in) and symbol addresses are per device, and one process may drive several devices (the
// reference engine does: src/forward.c:606), so every "done once" flag is indexed by this.
int current_device();
int device_sms();          // SM count of the current device (grids of the persistent kernels)

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
constexpr uint32_t kWaitBudget = 1u << 16;  // x a few microseconds per try_wait: a fraction of a second
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
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

}  // namespace mb200
