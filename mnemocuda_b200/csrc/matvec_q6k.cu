// Q6_K dequant-matvec for decode (V projection, expert down projection, lm_head), sm_100a.
//
// Same streaming skeleton as the Q4_K kernel: tiles of whole rows are pulled
// with 1-D bulk async copies into a shared-memory ring, the activation vector
// is split into two int8 levels once per CTA, and the 6-bit weights are
// rebuilt as bytes and multiplied with dp4a.
//
// Q6_K super-blocks are 210 bytes, so only 2-byte alignment can be assumed for
// anything inside the tensor. The bulk copy moves the enclosing 16-byte-aligned
// span (at most 15 bytes before and after the tile, always inside the same
// 16-byte granule as a valid byte, hence inside a mapped page), and lanes read
// their fields from shared memory as aligned words + funnel shift.
//
// Lane mapping: 8 lanes per super-block. Lane (hh = half 0/1, jj = 0..3) owns
// positions l = 8jj..8jj+7 of half hh: 8 bytes of ql[64hh..], 8 bytes of
// ql[64hh+32..] and 8 bytes of qh[32hh..] give its 32 weights (4 sixteen-groups
// x 8 columns): q = lo4 | hi2 << 4, weight = d * scale * (q - 32)
// (reference src/kernels.cu:455-484, tools/validate_dequant.py:286-317).
#include <cstdio>

#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kWarps = 12;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kMaxTileRows = 48;
constexpr int kMaxRounds = 16;           // 16 rounds x 4 blocks x 256 = 16384 columns
constexpr int kMaxCols = kMaxRounds * 4 * 256;
constexpr int kTileTargetBytes = 20480;

enum : int { kStore = 0, kScaledAdd = 2 };

struct Params {
    const uint8_t *w;
    float *y;
    const float *x;
    float scale;
    int n_rows, n_cols, bpr;
    int tile_rows, n_tiles, mode;
    int *err;
};

struct Smem {
    int bars, xq1, xq2, xs1, xsum, part, stages, stage_bytes, total;
};

__host__ __device__ inline Smem smem_layout(int bpr, int tile_rows)
{
    Smem s;
    const int kpad = bpr * 256;
    int o = 0;
    s.bars = o;   o += 64;
    s.xq1 = o;    o += kpad;
    s.xq2 = o;    o += kpad;
    s.xs1 = o;    o += (kpad / 32) * 4;
    s.xsum = o;   o += (kpad / 8) * 4;   // fp32 per 8 columns
    s.part = o;   o += 2 * kMaxTileRows * kMaxRounds * 4;
    o = (o + 127) & ~127;
    s.stages = o;
    s.stage_bytes = (tile_rows * bpr * kQ6KBlock + 32 + 127) & ~127;  // +32: alignment skew and word over-read
    s.total = o + kStages * s.stage_bytes;
    return s;
}

struct XRegs {
    uint32_t q1[8], q2[8];  // [2g + i]: columns 32g + 8jj + 4i .. +3 of the lane's half
    float k[4];             // s1 / 254 per sixteen-group g
    float sx32[4];          // 32 * sum of x over the lane's 8 columns of group g
};

__device__ __forceinline__ void load_xregs(XRegs &xr, const uint8_t *smem, const Smem &L, int col,
                                           int hh, int jj, bool valid)
{
    const int c0 = col * 256 + hh * 128 + jj * 8;  // first column of the lane in group 0
    const uint32_t *q1 = reinterpret_cast<const uint32_t *>(smem + L.xq1);
    const uint32_t *q2 = reinterpret_cast<const uint32_t *>(smem + L.xq2);
    const float *s1 = reinterpret_cast<const float *>(smem + L.xs1);
    const float *xs = reinterpret_cast<const float *>(smem + L.xsum);
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const int c = c0 + 32 * g;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            xr.q1[2 * g + i] = valid ? q1[(c >> 2) + i] : 0u;
            xr.q2[2 * g + i] = valid ? q2[(c >> 2) + i] : 0u;
        }
        xr.k[g] = valid ? s1[c >> 5] * (1.0f / 254.0f) : 0.0f;
        xr.sx32[g] = valid ? 32.0f * xs[c >> 3] : 0.0f;
    }
}

// 8 bytes starting at any byte address in shared memory -> two words
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

// One lane's 32 weights of one super-block of one row.
__device__ __forceinline__ float block_dot(const uint8_t *blk, int hh, int jj, const XRegs &xr)
{
    uint32_t A[2], B[2], H[2], S[2];
    lds8(blk + 64 * hh + 8 * jj, A[0], A[1]);
    lds8(blk + 64 * hh + 32 + 8 * jj, B[0], B[1]);
    lds8(blk + 128 + 32 * hh + 8 * jj, H[0], H[1]);
    lds8(blk + 192 + 8 * hh, S[0], S[1]);
    unsigned short d_bits;
    asm volatile("ld.shared.u16 %0, [%1+208];" : "=h"(d_bits) : "r"(smem_u32(blk)));
    const float d = __half2float(__ushort_as_half(d_bits));

    int i1[4] = {0, 0, 0, 0}, i2[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const uint32_t q0 = (A[i] & 0x0F0F0F0Fu) | ((H[i] << 4) & 0x30303030u);
        const uint32_t q1 = (B[i] & 0x0F0F0F0Fu) | ((H[i] << 2) & 0x30303030u);
        const uint32_t q2 = ((A[i] >> 4) & 0x0F0F0F0Fu) | (H[i] & 0x30303030u);
        const uint32_t q3 = ((B[i] >> 4) & 0x0F0F0F0Fu) | ((H[i] >> 2) & 0x30303030u);
        i1[0] = dp4a_us(q0, xr.q1[0 + i], i1[0]);
        i2[0] = dp4a_us(q0, xr.q2[0 + i], i2[0]);
        i1[1] = dp4a_us(q1, xr.q1[2 + i], i1[1]);
        i2[1] = dp4a_us(q1, xr.q2[2 + i], i2[1]);
        i1[2] = dp4a_us(q2, xr.q1[4 + i], i1[2]);
        i2[2] = dp4a_us(q2, xr.q2[4 + i], i2[2]);
        i1[3] = dp4a_us(q3, xr.q1[6 + i], i1[3]);
        i2[3] = dp4a_us(q3, xr.q2[6 + i], i2[3]);
    }
    // scales[8hh + 2g + (jj >> 1)], g = 0..3: bytes (jj>>1) + {0,2,4,6} of the 8 loaded
    const uint32_t sh = (jj >> 1) * 8;
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

// Tile -> rows and the aligned span that is copied.
__device__ __forceinline__ void tile_span(const Params &P, int tile, int &row0, int &rows,
                                          const uint8_t *&src, uint32_t &bytes, uint32_t &skew)
{
    row0 = tile * P.tile_rows;
    rows = min(P.tile_rows, P.n_rows - row0);
    const size_t row_bytes = (size_t)P.bpr * kQ6KBlock;
    const uintptr_t begin = reinterpret_cast<uintptr_t>(P.w) + (size_t)row0 * row_bytes;
    const uintptr_t end = begin + (size_t)rows * row_bytes;
    const uintptr_t a0 = begin & ~static_cast<uintptr_t>(15);
    const uintptr_t a1 = (end + 15) & ~static_cast<uintptr_t>(15);
    src = reinterpret_cast<const uint8_t *>(a0);
    bytes = static_cast<uint32_t>(a1 - a0);
    skew = static_cast<uint32_t>(begin - a0);
}

__device__ __forceinline__ void issue_tile(const Params &P, int tile, uint8_t *stage, uint64_t *bar)
{
    int row0, rows;
    const uint8_t *src;
    uint32_t bytes, skew;
    tile_span(P, tile, row0, rows, src, bytes, skew);
    mbar_expect_tx(bar, bytes);
    bulk_g2s(stage, src, bytes, bar);
}

__global__ void __launch_bounds__(kThreads, 1) q6k_stream_kernel(const Params P)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const Smem L = smem_layout(P.bpr, P.tile_rows);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.bars);
    float *part = reinterpret_cast<float *>(smem + L.part);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.bars + 48);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int my_tiles = (P.n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    if (my_tiles <= 0) return;

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kStages; s++) mbar_init(&bars[s], 1);
        mbar_fence_init();
        for (int k = 0; k < kStages && k < my_tiles; k++)
            issue_tile(P, blockIdx.x + k * gridDim.x, smem + L.stages + k * L.stage_bytes, &bars[k]);
    }
    quantize_x<kThreads, 8, false>(P.x, P.n_cols, P.bpr * 256, reinterpret_cast<int8_t *>(smem + L.xq1),
                                   reinterpret_cast<int8_t *>(smem + L.xq2),
                                   reinterpret_cast<float *>(smem + L.xs1),
                                   reinterpret_cast<float *>(smem + L.xsum));
    __syncthreads();

    const int q = lane >> 3, hh = (lane >> 2) & 1, jj = lane & 3;
    const int rounds = (P.bpr + 3) >> 2;
    const uint32_t row_bytes = P.bpr * kQ6KBlock;
    XRegs xr;
    int cur_round = -1, col = 0, roff = 0, rpp = 1, width = 32;
    bool lane_ok = false;

    for (int k = 0; k < my_tiles; k++) {
        const int tile = blockIdx.x + k * gridDim.x;
        const int st = k % kStages;
        int row0, R;
        const uint8_t *src;
        uint32_t bytes, skew;
        tile_span(P, tile, row0, R, src, bytes, skew);
        const uint8_t *stage = smem + L.stages + st * L.stage_bytes + skew;

        if (!mbar_wait(&bars[st], (k / kStages) & 1)) *abort_flag = 1;

        int total = 0;
        for (int cr = 0; cr < rounds; cr++) {
            const int v = min(4, P.bpr - 4 * cr);
            const int r_pp = (v == 1 || v == 2) ? 4 / v : 1;
            total += (R + r_pp - 1) / r_pp;
        }
        const int p_begin = (warp * total) / kWarps, p_end = ((warp + 1) * total) / kWarps;
        float *part_buf = part + (k & 1) * kMaxTileRows * kMaxRounds;

        int cr = 0, base = 0;
        for (int p = p_begin; p < p_end; p++) {
            for (;;) {
                const int v = min(4, P.bpr - 4 * cr);
                const int r_pp = (v == 1 || v == 2) ? 4 / v : 1;
                const int n = (R + r_pp - 1) / r_pp;
                if (p < base + n) break;
                base += n;
                cr++;
            }
            if (cr != cur_round) {
                cur_round = cr;
                const int v = min(4, P.bpr - 4 * cr);
                rpp = (v == 1 || v == 2) ? 4 / v : 1;
                lane_ok = q < v * rpp;
                col = 4 * cr + (q % v);
                roff = q / v;
                width = (rpp > 1) ? 8 * v : 32;
                load_xregs(xr, smem, L, lane_ok ? col : 0, hh, jj, lane_ok);
            }
            const int row = (p - base) * rpp + roff;
            const bool ok = lane_ok && row < R;
            const uint8_t *blk = stage + (size_t)(ok ? row : 0) * row_bytes + (ok ? col : 0) * kQ6KBlock;
            float acc = block_dot(blk, hh, jj, xr);
            acc = ok ? acc : 0.0f;
            acc = group_sum(acc, width);
            if ((lane & (width - 1)) == 0 && row < R) part_buf[row * kMaxRounds + cr] = acc;
        }
        __syncthreads();
        if (*abort_flag) {
            if (tid == 0) atomicExch(P.err, MB200_ERR_TIMEOUT);
            break;
        }
        if (tid == 0 && k + kStages < my_tiles)
            issue_tile(P, tile + kStages * gridDim.x, smem + L.stages + st * L.stage_bytes, &bars[st]);

        if (tid < R) {
            float s = 0.0f;
            for (int c = 0; c < rounds; c++) s += part_buf[tid * kMaxRounds + c];
            const int r = row0 + tid;
            if (P.mode == kStore)
                P.y[r] = s;
            else
                P.y[r] += P.scale * s;
        }
    }
}

int g_optin = 0;

// Rows per tile: about kTileTargetBytes, preferring a count for which the pass
// list divides evenly among the warps with round boundaries on warp boundaries
// (then a warp's share of x stays in registers for the whole kernel).
int pick_tile_rows(int bpr)
{
    const int row_bytes = bpr * kQ6KBlock;
    int target = kTileTargetBytes / row_bytes;
    target = target < 1 ? 1 : (target > kMaxTileRows ? kMaxTileRows : target);
    const int rounds = (bpr + 3) / 4;
    for (int R = target; R >= 1 && R * 2 > target; R--) {
        int total = 0;
        bool ok = true;
        for (int cr = 0; cr < rounds; cr++) {
            const int v = bpr - 4 * cr < 4 ? bpr - 4 * cr : 4;
            const int rpp = (v == 1 || v == 2) ? 4 / v : 1;
            total += (R + rpp - 1) / rpp;
        }
        if (total % kWarps != 0) continue;
        const int per = total / kWarps;
        int base = 0;
        for (int cr = 0; cr < rounds; cr++) {
            const int v = bpr - 4 * cr < 4 ? bpr - 4 * cr : 4;
            const int rpp = (v == 1 || v == 2) ? 4 / v : 1;
            if (base % per != 0) ok = false;
            base += (R + rpp - 1) / rpp;
        }
        if (ok) return R;
    }
    return target;
}

void launch(Params &P, cudaStream_t stream, const char *where)
{
    if (P.n_rows <= 0 || P.n_cols <= 0) return;
    P.bpr = (P.n_cols + 255) / 256;
    if (P.n_cols > kMaxCols) {
        fprintf(stderr, "[mnemo_b200] %s: n_cols=%d exceeds the supported %d\n", where, P.n_cols, kMaxCols);
        set_status(MB200_ERR_UNSUPPORTED, where);
        return;
    }
    if (reinterpret_cast<uintptr_t>(P.w) & 1) {
        fprintf(stderr, "[mnemo_b200] %s: Q6_K tensor is not 2-byte aligned\n", where);
        set_status(MB200_ERR_ARG, where);
        return;
    }
    P.tile_rows = pick_tile_rows(P.bpr);
    P.n_tiles = (P.n_rows + P.tile_rows - 1) / P.tile_rows;
    P.err = device_error_word();
    const Smem L = smem_layout(P.bpr, P.tile_rows);
    if (L.total > 227 * 1024) {
        set_status(MB200_ERR_UNSUPPORTED, where);
        return;
    }
    if (!g_optin) {
        cudaFuncSetAttribute(q6k_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        g_optin = 1;
    }
    const int grid = P.n_tiles < kSMs ? P.n_tiles : kSMs;
    q6k_stream_kernel<<<grid, kThreads, L.total, stream>>>(P);
    MB200_CHECK_LAUNCH(where);
}

}  // namespace

void q6k_init()
{
    cudaFuncSetAttribute(q6k_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    g_optin = 1;
}

}  // namespace mb200

using namespace mb200;

extern "C" {

void cuda_matvec_q6k(const void *weights, const float *x, float *y, int n_rows, int n_cols,
                     cudaStream_t stream)
{
    Params P{};
    P.w = static_cast<const uint8_t *>(weights);
    P.x = x;
    P.y = y;
    P.n_rows = n_rows;
    P.n_cols = n_cols;
    P.mode = kStore;
    launch(P, stream, "cuda_matvec_q6k");
}

int mb200_matvec_q6k_scaled_add(const void *weights, const float *x, float *y, int n_rows,
                                int n_cols, float scale, cudaStream_t stream)
{
    if (!weights || !x || !y || n_rows < 0 || n_cols <= 0) return MB200_ERR_ARG;
    Params P{};
    P.w = static_cast<const uint8_t *>(weights);
    P.x = x;
    P.y = y;
    P.scale = scale;
    P.n_rows = n_rows;
    P.n_cols = n_cols;
    P.mode = kScaledAdd;
    mb200_clear_status();
    launch(P, stream, "mb200_matvec_q6k_scaled_add");
    return mb200_last_status();
}

}  // extern "C"
