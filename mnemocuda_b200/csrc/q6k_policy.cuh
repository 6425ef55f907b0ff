// Q6_K policy of the streaming matvec skeleton (shared by the plain matvec
// kernels and the fused expert kernel).
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
#pragma once
#include "stream_matvec.cuh"

namespace mb200 {
namespace {

// 16 bytes starting at any byte address in shared memory -> four words
__device__ __forceinline__ void lds16(const uint8_t *p, uint32_t (&w)[4])
{
    const uint32_t a = smem_u32(p);
    const uint32_t base = a & ~3u;
    const uint32_t sh = (a & 3u) * 8u;
    uint32_t t[5];
#pragma unroll
    for (int i = 0; i < 5; i++) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(t[i]) : "r"(base + 4 * i));
#pragma unroll
    for (int i = 0; i < 4; i++) w[i] = __funnelshift_r(t[i], t[i + 1], sh);
}
// 8 bytes -> two words
__device__ __forceinline__ void lds8(const uint8_t *p, uint32_t &w0, uint32_t &w1)
{
    const uint32_t a = smem_u32(p);
    const uint32_t base = a & ~3u;
    const uint32_t sh = (a & 3u) * 8u;
    uint32_t a0, a1, a2;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(a0) : "r"(base));
    asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(a1) : "r"(base));
    asm volatile("ld.shared.u32 %0, [%1+8];" : "=r"(a2) : "r"(base));
    w0 = __funnelshift_r(a0, a1, sh);
    w1 = __funnelshift_r(a1, a2, sh);
}

struct Q6 {
    static constexpr int kBlockBytes = kQ6KBlock;
    static constexpr int kLanesPerBlock = 4;
    static constexpr float kByteCost = 2.0f;  // relative consumer time per weight byte (splits a shared launch)
    static constexpr int kG = 8;
    static constexpr int kSumCols = 16;
    static constexpr bool kGroup4Tail = false;  // per-element tail, reference src/kernels.cu:474
    static constexpr int kBaseAlign = 2;
    static constexpr int kTileTargetBytes = 30720;
    static constexpr int kMaxCols = 16384;
    // x staging: 16 words per lane slot; slot = 4 * block-column + 2 * half + jj; word = 4g + i
    static constexpr int kXWords = 16;
    static constexpr int kSlotsPerBlock = 4;
    __device__ static __forceinline__ int xslot(int c0) { return ((c0 >> 8) << 2) + (((c0 >> 7) & 1) << 1) + ((c0 >> 4) & 1); }
    __device__ static __forceinline__ int xword(int c0) { return (((c0 >> 5) & 3) << 2) + ((c0 >> 2) & 3); }

    struct XRegs {
        uint32_t q1[16], q2[16];  // [4g + i]: columns 32g + 16jj + 4i .. +3 of the lane's half
        float k[4];               // s1 / 254 per sixteen-group g
        float sx32[4];            // 32 * sum of x over the lane's 16 columns of group g
    };

    __device__ static __forceinline__ void load_xregs(XRegs &xr, const uint8_t *smem, const stream::Layout &L,
                                                      int bpr, int col, int sub, bool valid)
    {
        const int hh = sub >> 1, jj = sub & 1;
        const int c0 = col * 256 + hh * 128 + jj * 16;  // first column of the lane in group 0
        const int pitch = kSlotsPerBlock * bpr + 1;
        const uint32_t *q1 = reinterpret_cast<const uint32_t *>(smem + L.xq1) + col * 4 + sub;
        const uint32_t *q2 = reinterpret_cast<const uint32_t *>(smem + L.xq2) + col * 4 + sub;
        const float *s1 = reinterpret_cast<const float *>(smem + L.xs1);
        const float *xs = reinterpret_cast<const float *>(smem + L.xsum);
#pragma unroll
        for (int w = 0; w < 16; w++) {
            xr.q1[w] = valid ? q1[w * pitch] : 0u;
            xr.q2[w] = valid ? q2[w * pitch] : 0u;
        }
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const int c = c0 + 32 * g;
            xr.k[g] = valid ? s1[c >> 5] * (1.0f / 254.0f) : 0.0f;
            xr.sx32[g] = valid ? 32.0f * xs[c >> 4] : 0.0f;
        }
    }

    // One lane's 64 weights of one super-block of one row: positions l = 16jj..16jj+15 of half hh,
    // in the four sixteen-groups g (g = 0,1: low nibbles of ql[64hh..], ql[64hh+32..]; g = 2,3: their high nibbles).
    __device__ static __forceinline__ float block_dot(const uint8_t *blk, int sub, const XRegs &xr)
    {
        const int hh = sub >> 1, jj = sub & 1;
        uint32_t A[4], B[4], H[4], S[2];
        lds16(blk + 64 * hh + 16 * jj, A);
        lds16(blk + 64 * hh + 32 + 16 * jj, B);
        lds16(blk + 128 + 32 * hh + 16 * jj, H);
        lds8(blk + 192 + 8 * hh, S[0], S[1]);
        unsigned short d_bits;
        asm volatile("ld.shared.u16 %0, [%1+208];" : "=h"(d_bits) : "r"(smem_u32(blk)));
        const float d = __half2float(__ushort_as_half(d_bits));

        int i1[4] = {0, 0, 0, 0}, i2[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t h0 = (H[i] << 4) & 0x30303030u, h1 = (H[i] << 2) & 0x30303030u;
            const uint32_t h2 = H[i] & 0x30303030u, h3 = (H[i] >> 2) & 0x30303030u;
            const uint32_t q0 = (A[i] & 0x0F0F0F0Fu) | h0;
            const uint32_t q1 = (B[i] & 0x0F0F0F0Fu) | h1;
            const uint32_t q2 = ((A[i] >> 4) & 0x0F0F0F0Fu) | h2;
            const uint32_t q3 = ((B[i] >> 4) & 0x0F0F0F0Fu) | h3;
            i1[0] = dp4a_us(q0, xr.q1[0 + i], i1[0]);
            i2[0] = dp4a_us(q0, xr.q2[0 + i], i2[0]);
            i1[1] = dp4a_us(q1, xr.q1[4 + i], i1[1]);
            i2[1] = dp4a_us(q1, xr.q2[4 + i], i2[1]);
            i1[2] = dp4a_us(q2, xr.q1[8 + i], i1[2]);
            i2[2] = dp4a_us(q2, xr.q2[8 + i], i2[2]);
            i1[3] = dp4a_us(q3, xr.q1[12 + i], i1[3]);
            i2[3] = dp4a_us(q3, xr.q2[12 + i], i2[3]);
        }
        // scales[8hh + 2g + jj], g = 0..3: bytes jj + {0,2,4,6} of the 8 loaded
        const uint32_t sh = jj * 8;
        const int sc0 = static_cast<int8_t>((S[0] >> sh) & 0xFF);
        const int sc1 = static_cast<int8_t>((S[0] >> (sh + 16)) & 0xFF);
        const int sc2 = static_cast<int8_t>((S[1] >> sh) & 0xFF);
        const int sc3 = static_cast<int8_t>((S[1] >> (sh + 16)) & 0xFF);
        float acc;
        acc = static_cast<float>(sc0) * fmaf(xr.k[0], static_cast<float>(i1[0] * 254 + i2[0]), -xr.sx32[0]);
        acc = fmaf(static_cast<float>(sc1), fmaf(xr.k[1], static_cast<float>(i1[1] * 254 + i2[1]), -xr.sx32[1]), acc);
        acc = fmaf(static_cast<float>(sc2), fmaf(xr.k[2], static_cast<float>(i1[2] * 254 + i2[2]), -xr.sx32[2]), acc);
        acc = fmaf(static_cast<float>(sc3), fmaf(xr.k[3], static_cast<float>(i1[3] * 254 + i2[3]), -xr.sx32[3]), acc);
        return d * acc;
    }
};

}  // namespace
}  // namespace mb200
