// Q8_0, Q5_K and Q3_K policies of the streaming matvec skeleton (stream_matvec.cuh): the lane mapping,
// the staging layout of the int8-split activation vector and the per-lane dot product of 64 weights,
// as q4k_policy.cuh / q6k_policy.cuh do for the two main types. Bit layouts are the reference kernels'
// (src/kernels.cu:497-673), which for Q5_K's fifth bits and Q3_K's scale high bits are not GGUF's.
//
// All three use 4 lanes per 256 columns and dp4a against the two int8 levels of x
// (x ~= s (q1 + q2 / 254) per 32 columns); integer fields are decoded exactly.
#pragma once
#include "q6k_policy.cuh"  // lds16 / lds8: unaligned shared-memory loads

namespace mb200 {
namespace {

__device__ __forceinline__ int dp4a_ss(uint32_t a_s8x4, uint32_t b_s8x4, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8x4), "r"(b_s8x4), "r"(c));
    return d;
}

// ---- Q8_0: eight 34-byte blocks [d f16][32 int8] per 256 columns ("super-block" of 272 bytes) ----
// Lane `sub` owns blocks 2 sub, 2 sub + 1 = columns 64 sub .. 64 sub + 63. w = d q (src/kernels.cu:644-673).
struct Q8 {
    static constexpr int kBlockBytes = 8 * 34;
    static constexpr int kLanesPerBlock = 4;
    static constexpr float kByteCost = 1.0f;
    static constexpr int kG = 8;
    static constexpr int kSumCols = 16;
    static constexpr bool kGroup4Tail = false;
    static constexpr int kBaseAlign = 16;  // 272-byte rows of blocks; inside a block the fields sit at even offsets
    static constexpr int kTileTargetBytes = 27648;
    static constexpr int kMaxCols = 16384;
    static constexpr int kXWords = 16;
    static constexpr int kSlotsPerBlock = 4;
    __device__ static __forceinline__ int xslot(int c0) { return c0 >> 6; }
    __device__ static __forceinline__ int xword(int c0) { return (c0 & 63) >> 2; }

    struct XRegs {
        uint32_t q1[16], q2[16];  // [8 b + i]: columns 64 sub + 32 b + 4 i .. + 3
        float k[2];               // s1 / 254 of the two 32-column groups
    };
    __device__ static __forceinline__ void load_xregs(XRegs &xr, const uint8_t *smem, const stream::Layout &L,
                                                      int bpr, int col, int sub, bool valid)
    {
        const int pitch = kSlotsPerBlock * bpr + 1;
        const uint32_t *q1 = reinterpret_cast<const uint32_t *>(smem + L.xq1) + col * 4 + sub;
        const uint32_t *q2 = reinterpret_cast<const uint32_t *>(smem + L.xq2) + col * 4 + sub;
        const float *s1 = reinterpret_cast<const float *>(smem + L.xs1) + col * 8 + sub * 2;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            xr.q1[i] = valid ? q1[i * pitch] : 0u;
            xr.q2[i] = valid ? q2[i * pitch] : 0u;
        }
        xr.k[0] = valid ? s1[0] * (1.0f / 254.0f) : 0.0f;
        xr.k[1] = valid ? s1[1] * (1.0f / 254.0f) : 0.0f;
    }
    __device__ static __forceinline__ float block_dot(const uint8_t *blk, int sub, const XRegs &xr)
    {
        float acc = 0.0f;
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const uint8_t *p = blk + 68 * sub + 34 * b;
            unsigned short d_bits;
            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(d_bits) : "r"(smem_u32(p)));
            uint32_t A[4], B[4];
            lds16(p + 2, A);
            lds16(p + 18, B);
            int i1 = 0, i2 = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                i1 = dp4a_ss(A[i], xr.q1[8 * b + i], i1);
                i2 = dp4a_ss(A[i], xr.q2[8 * b + i], i2);
                i1 = dp4a_ss(B[i], xr.q1[8 * b + 4 + i], i1);
                i2 = dp4a_ss(B[i], xr.q2[8 * b + 4 + i], i2);
            }
            const float d = __half2float(__ushort_as_half(d_bits));
            acc = fmaf(d * xr.k[b], static_cast<float>(i1 * 254 + i2), acc);
        }
        return acc;
    }
};

// ---- Q5_K: 176 bytes [d][dmin][scales 12][qh 32][qs 128]; Q4_K's lane map and scale packing, plus a fifth bit ----
// Lane g owns qs[32 g .. 32 g + 31]: sub-blocks 2 g (low nibbles) and 2 g + 1 (high nibbles). In the reference's
// layout the fifth bit of weight w is bit w % 32 of the 32-bit word w / 32 of qh (src/kernels.cu:620-632).
struct Q5 {
    static constexpr int kBlockBytes = 176;
    static constexpr int kLanesPerBlock = 4;
    static constexpr float kByteCost = 1.4f;
    static constexpr int kG = 8;
    static constexpr int kSumCols = 16;
    static constexpr bool kGroup4Tail = false;
    static constexpr int kBaseAlign = 16;
    static constexpr int kTileTargetBytes = 28160;
    static constexpr int kMaxCols = 16384;
    static constexpr int kXWords = 16;
    static constexpr int kSlotsPerBlock = 4;
    __device__ static __forceinline__ int xslot(int c0) { return c0 >> 6; }
    __device__ static __forceinline__ int xword(int c0) { return ((c0 & 31) >> 2) + ((c0 & 32) ? 8 : 0); }

    struct XRegs {
        uint32_t q1[16], q2[16];
        float kl, kh, sxl, sxh;
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
        xr.kh = valid ? s1[1] * (1.0f / 254.0f) : 0.0f;
        xr.sxl = valid ? xs[0] + xs[1] : 0.0f;
        xr.sxh = valid ? xs[2] + xs[3] : 0.0f;
    }
    // four bits -> the 0x10 position of four bytes
    __device__ static __forceinline__ uint32_t spread4(uint32_t bits)
    {
        return (((bits & 0xFu) * 0x00204081u) & 0x01010101u) << 4;
    }
    __device__ static __forceinline__ float block_dot(const uint8_t *blk, int g, const XRegs &xr)
    {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        const uint2 hb = *reinterpret_cast<const uint2 *>(blk + 16 + 8 * g);  // fifth bits of the two sub-blocks
        const uint4 c0 = *reinterpret_cast<const uint4 *>(blk + 48 + 32 * g);
        const uint4 c1 = *reinterpret_cast<const uint4 *>(blk + 64 + 32 * g);
        const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        int i1l = 0, i2l = 0, i1h = 0, i2h = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t lo = (w[i] & 0x0F0F0F0Fu) | spread4(hb.x >> (4 * i));
            const uint32_t hi = ((w[i] >> 4) & 0x0F0F0F0Fu) | spread4(hb.y >> (4 * i));
            i1l = dp4a_us(lo, xr.q1[i], i1l);
            i2l = dp4a_us(lo, xr.q2[i], i2l);
            i1h = dp4a_us(hi, xr.q1[8 + i], i1h);
            i2h = dp4a_us(hi, xr.q2[8 + i], i2h);
        }
        uint32_t sc2, m2;
        q4k_scale_pair(hdr.y, hdr.z, hdr.w, g, sc2, m2);
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        const float il = static_cast<float>(i1l * 254 + i2l);
        const float ih = static_cast<float>(i1h * 254 + i2h);
        float p = static_cast<float>(sc2 & 0xFFu) * (xr.kl * il);
        p = fmaf(static_cast<float>(sc2 >> 8), xr.kh * ih, p);
        float q = static_cast<float>(m2 & 0xFFu) * xr.sxl;
        q = fmaf(static_cast<float>(m2 >> 8), xr.sxh, q);
        return fmaf(dd.x, p, -dd.y * q);
    }
};

// ---- Q3_K: 110 bytes [hmask 32][qs 64][scales 12][d]; weight 128 c + 32 p + l (c chunk, p bit plane) ----
// = ((qs[32 c + l] >> 2 p) & 3) - (hmask[l] bit (4 c + p) ? 0 : 4), scale index 8 c + 2 p + l / 16
// (src/kernels.cu:529-571). Lane (c = sub / 2, hf = sub % 2) owns l in [16 hf, 16 hf + 16) of chunk c, all four
// planes: 64 weights whose columns are 128 c + 32 p + 16 hf + (0..15) -- the column map of the Q6_K policy,
// whose activation staging it shares. The value is kept as q | h << 2 in 0..7 and the 4 comes off as 4 sum(x).
struct Q3 {
    static constexpr int kBlockBytes = 110;
    static constexpr int kLanesPerBlock = 4;
    static constexpr float kByteCost = 2.5f;
    static constexpr int kG = 8;
    static constexpr int kSumCols = 16;
    static constexpr bool kGroup4Tail = false;
    static constexpr int kBaseAlign = 2;
    static constexpr int kTileTargetBytes = 28160;
    static constexpr int kMaxCols = 16384;
    static constexpr int kXWords = 16;
    static constexpr int kSlotsPerBlock = 4;
    __device__ static __forceinline__ int xslot(int c0) { return Q6::xslot(c0); }
    __device__ static __forceinline__ int xword(int c0) { return Q6::xword(c0); }

    struct XRegs {
        uint32_t q1[16], q2[16];  // [4 p + i]: columns 128 c + 32 p + 16 hf + 4 i .. + 3
        float k[4];               // s1 / 254 per plane p (its 32-column group)
        float sx4[4];             // 4 * sum of x over the lane's 16 columns of plane p
    };
    __device__ static __forceinline__ void load_xregs(XRegs &xr, const uint8_t *smem, const stream::Layout &L,
                                                      int bpr, int col, int sub, bool valid)
    {
        const int c = sub >> 1, hf = sub & 1;
        const int c0 = col * 256 + c * 128 + hf * 16;
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
        for (int p = 0; p < 4; p++) {
            const int cc = c0 + 32 * p;
            xr.k[p] = valid ? s1[cc >> 5] * (1.0f / 254.0f) : 0.0f;
            xr.sx4[p] = valid ? 4.0f * xs[cc >> 4] : 0.0f;
        }
    }
    __device__ static __forceinline__ float block_dot(const uint8_t *blk, int sub, const XRegs &xr)
    {
        const int c = sub >> 1, hf = sub & 1;
        uint32_t Hm[4], Qs[4], S[4];
        lds16(blk + 16 * hf, Hm);
        lds16(blk + 32 + 32 * c + 16 * hf, Qs);
        lds16(blk + 94, S);  // bytes 94..109: scales at [2..13], d at [14..15]
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(S[3] >> 16)));
        // the twelve scale bytes as three words
        const uint32_t s0 = __funnelshift_r(S[0], S[1], 16), s1w = __funnelshift_r(S[1], S[2], 16),
                       s2 = __funnelshift_r(S[2], S[3], 16);
        float acc = 0.0f;
#pragma unroll
        for (int p = 0; p < 4; p++) {
            int i1 = 0, i2 = 0;
            const int bit = 4 * c + p;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t v = ((Qs[i] >> (2 * p)) & 0x03030303u) | (((Hm[i] >> bit) & 0x01010101u) << 2);
                i1 = dp4a_us(v, xr.q1[4 * p + i], i1);
                i2 = dp4a_us(v, xr.q2[4 * p + i], i2);
            }
            // scale index is = 8 c + 2 p + hf: low four bits from byte is % 8 (its low nibble for is < 8, high
            // nibble otherwise), two high bits from byte 8 + (is % 8) / 4 at bit 2 ((is % 8) % 4) + 4 (is / 8)
            const int ii = 2 * p + hf;  // is % 8
            const uint32_t lo_word = ii < 4 ? s0 : s1w;
            const uint32_t lo4 = (lo_word >> (8 * (ii & 3) + 4 * c)) & 0xFu;
            // (the reference shifts the BYTE right by up to 10: for is >= 8 and is % 4 >= 2 the two bits are zero)
            const uint32_t hi2 = (((s2 >> (8 * (ii >> 2))) & 0xFFu) >> (2 * (ii & 3) + 4 * c)) & 0x3u;
            const int sc = static_cast<int>(lo4 | (hi2 << 4)) - 32;
            acc = fmaf(static_cast<float>(sc), fmaf(xr.k[p], static_cast<float>(i1 * 254 + i2), -xr.sx4[p]), acc);
        }
        return d * acc;
    }
};

}  // namespace
}  // namespace mb200
