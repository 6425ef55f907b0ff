// Q4_K policy of the streaming matvec skeleton: lane mapping, activation staging
// layout and the per-lane dot product of one super-block (shared by the plain
// matvec kernels and the fused expert kernel).
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
#pragma once
#include "stream_matvec.cuh"

namespace mb200 {
namespace {

struct Q4 {
    static constexpr int kBlockBytes = kQ4KBlock;
    static constexpr int kLanesPerBlock = 4;
    static constexpr float kByteCost = 1.0f;  // relative consumer time per weight byte (splits a shared launch)
    static constexpr int kG = 8;
    static constexpr int kSumCols = 16;
    static constexpr bool kGroup4Tail = true;  // reference src/kernels.cu:124,131
    static constexpr int kBaseAlign = 16;
    static constexpr int kTileTargetBytes = 27648;
    static constexpr int kMaxCols = 16384;
    // x staging: 16 words per lane slot, slot = 4 * block-column + g
    static constexpr int kXWords = 16;
    static constexpr int kSlotsPerBlock = 4;
    __device__ static __forceinline__ int xslot(int c0) { return c0 >> 6; }
    __device__ static __forceinline__ int xword(int c0) { return ((c0 & 31) >> 2) + ((c0 & 32) ? 8 : 0); }

    struct XRegs {
        uint32_t q1[16], q2[16];  // [0..7]: columns of the low-nibble sub-block, [8..15]: high
        float kl, kh;             // s1/254 for the low sub-block, s1/(254*16) for the high one
        float sxl, sxh;           // sum of x over each sub-block
    };

    __device__ static __forceinline__ void load_xregs(XRegs &xr, const uint8_t *smem, const stream::Layout &L,
                                                      int bpr, int col, int g, bool valid)
    {
        const int pitch = kSlotsPerBlock * bpr + 1;
        const uint32_t *q1 = reinterpret_cast<const uint32_t *>(smem + L.xq1) + col * 4 + g;
        const uint32_t *q2 = reinterpret_cast<const uint32_t *>(smem + L.xq2) + col * 4 + g;
        const float *s1 = reinterpret_cast<const float *>(smem + L.xs1) + col * 8 + g * 2;
        const float *xs = reinterpret_cast<const float *>(smem + L.xsum) + col * 16 + g * 4;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            xr.q1[i] = valid ? q1[i * pitch] : 0u;
            xr.q2[i] = valid ? q2[i * pitch] : 0u;
        }
        xr.kl = valid ? s1[0] * (1.0f / 254.0f) : 0.0f;
        xr.kh = valid ? s1[1] * (1.0f / (254.0f * 16.0f)) : 0.0f;
        xr.sxl = valid ? xs[0] + xs[1] : 0.0f;
        xr.sxh = valid ? xs[2] + xs[3] : 0.0f;
    }

    // One lane's 64 weights of one super-block of one row.
    __device__ static __forceinline__ float block_dot(const uint8_t *blk, int g, const XRegs &xr)
    {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        const uint4 c0 = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * g);
        const uint4 c1 = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * g);
        const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        int i1l = 0, i2l = 0, i1h = 0, i2h = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t lo = w[i] & 0x0F0F0F0Fu;
            const uint32_t hi = w[i] & 0xF0F0F0F0u;
            i1l = dp4a_us(lo, xr.q1[i], i1l);
            i2l = dp4a_us(lo, xr.q2[i], i2l);
            i1h = dp4a_us(hi, xr.q1[8 + i], i1h);
            i2h = dp4a_us(hi, xr.q2[8 + i], i2h);
        }
        uint32_t sc2, m2;
        q4k_scale_pair(hdr.y, hdr.z, hdr.w, g, sc2, m2);
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        const float d = dd.x, dmin = dd.y;
        const float il = static_cast<float>(i1l * 254 + i2l);
        const float ih = static_cast<float>(i1h * 254 + i2h);
        float p = static_cast<float>(sc2 & 0xFFu) * (xr.kl * il);
        p = fmaf(static_cast<float>(sc2 >> 8), xr.kh * ih, p);
        float q = static_cast<float>(m2 & 0xFFu) * xr.sxl;
        q = fmaf(static_cast<float>(m2 >> 8), xr.sxh, q);
        return fmaf(d, p, -dmin * q);
    }
};

}  // namespace
}  // namespace mb200
