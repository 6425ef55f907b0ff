// Q4_K dequant-matvec family for decode (batch 1), sm_100a.
//
// One streaming kernel serves every Q4_K entry point of the reference ABI
// (plain / +residual / QKV / dual / scaled-add) plus the gate+up+SwiGLU fusion.
//
// Data path: the weight matrix is a contiguous byte stream of 144-byte
// super-blocks. It is cut into tiles of whole rows (~18 KB); CTA c takes tiles
// c, c+grid, ... and pulls each with one 1-D bulk async copy (TMA engine,
// mbarrier completion) into a 4-deep shared-memory ring, so every SM keeps
// ~72 KB of loads in flight without spending registers on them.
//
// Arithmetic: the activation vector is split once per CTA into two int8 levels
// per 32-column group, x ~= s*(q1 + q2/254) (|error| <= max|x|/64516 per group),
// and kept in registers by the lanes that need it. Nibbles are masked four at
// a time (low: w & 0x0F0F0F0F, high: w & 0xF0F0F0F0 = 16*nibble) and
// multiplied with dp4a -- exact integer dot products -- then scaled in fp32:
//   row.x = sum_sub  d*sc*(s*I/254) - dmin*m*sum(x)
// which is the reference's w = d*sc*q - dmin*m (src/kernels.cu:98-136) with the
// products re-associated. Integer fields (scales, mins, nibbles) are exact.
//
// Lane mapping: 4 lanes per super-block (lane g owns qs[32g..32g+31], i.e.
// sub-blocks 2g and 2g+1), 8 super-blocks per warp pass. A warp stays on one
// group of 8 block-columns, so its share of x never leaves its registers.
#include <cstdio>

#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kMaxTileRows = 32;
constexpr int kMaxRounds = 8;            // 8 rounds x 8 blocks x 256 = 16384 columns
constexpr int kMaxCols = kMaxRounds * 8 * 256;
constexpr int kTileTargetBytes = 18432;

enum : int { kStore = 0, kAddResidual = 1, kScaledAdd = 2, kSwiGLU = 3 };

struct Seg {
    const uint8_t *w;
    float *y;
    int rows;
    int tile0;  // index of this segment's first tile
};

struct Params {
    Seg seg[3];
    int nseg;
    int n_tiles;
    int tile_rows;  // rows per tile (SwiGLU: half from gate, half from up)
    const float *x;
    const float *residual;
    float scale;
    int n_cols;
    int bpr;
    int mode;
    int *err;
};

struct Smem {
    // offsets (bytes) inside the dynamic shared buffer
    int xq1, xq2, xs1, xsum, part, bars, stages, stage_bytes, total;
};

__host__ __device__ inline Smem smem_layout(int bpr, int tile_rows)
{
    Smem s;
    int kpad = bpr * 256;
    int o = 0;
    s.bars = o;   o += 64;
    s.xq1 = o;    o += kpad;            // int8 per column
    s.xq2 = o;    o += kpad;
    s.xs1 = o;    o += (kpad / 32) * 4; // fp32 per 32 columns
    s.xsum = o;   o += (kpad / 16) * 4; // fp32 per 16 columns
    s.part = o;   o += 2 * kMaxTileRows * kMaxRounds * 4;
    o = (o + 127) & ~127;
    s.stages = o;
    s.stage_bytes = (tile_rows * bpr * kQ4KBlock + 127) & ~127;
    s.total = o + kStages * s.stage_bytes;
    return s;
}

// A lane's share of x for one round (group of 8 block-columns).
struct XRegs {
    uint32_t q1[16], q2[16];  // [0..7]: columns of the low-nibble sub-block, [8..15]: high
    float kl, kh;             // s1/254 for the low sub-block, s1/(254*16) for the high one
    float sxl, sxh;           // sum of x over each sub-block
};

__device__ __forceinline__ void load_xregs(XRegs &xr, const uint8_t *smem, const Smem &L, int col,
                                           int g, bool valid)
{
    const uint32_t *q1 = reinterpret_cast<const uint32_t *>(smem + L.xq1) + col * 64 + g * 16;
    const uint32_t *q2 = reinterpret_cast<const uint32_t *>(smem + L.xq2) + col * 64 + g * 16;
    const float *s1 = reinterpret_cast<const float *>(smem + L.xs1) + col * 8 + g * 2;
    const float *xs = reinterpret_cast<const float *>(smem + L.xsum) + col * 16 + g * 4;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        xr.q1[i] = valid ? q1[i] : 0u;
        xr.q2[i] = valid ? q2[i] : 0u;
    }
    xr.kl = valid ? s1[0] * (1.0f / 254.0f) : 0.0f;
    xr.kh = valid ? s1[1] * (1.0f / (254.0f * 16.0f)) : 0.0f;
    xr.sxl = valid ? xs[0] + xs[1] : 0.0f;
    xr.sxh = valid ? xs[2] + xs[3] : 0.0f;
}

// One super-block share (64 weights) of one row: returns its contribution to row.x
__device__ __forceinline__ float block_dot(const uint8_t *blk, int g, const XRegs &xr)
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
    const float d = h2f_lo(hdr.x), dmin = h2f_hi(hdr.x);
    const float il = static_cast<float>(i1l * 254 + i2l);
    const float ih = static_cast<float>(i1h * 254 + i2h);
    float p = static_cast<float>(sc2 & 0xFFu) * (xr.kl * il);
    p = fmaf(static_cast<float>(sc2 >> 8), xr.kh * ih, p);
    float q = static_cast<float>(m2 & 0xFFu) * xr.sxl;
    q = fmaf(static_cast<float>(m2 >> 8), xr.sxh, q);
    return fmaf(d, p, -dmin * q);
}

// Static selects instead of P.seg[i]: dynamic indexing would force the whole
// parameter block into local memory.
__device__ __forceinline__ const uint8_t *seg_w(const Params &P, int i)
{
    return i == 0 ? P.seg[0].w : (i == 1 ? P.seg[1].w : P.seg[2].w);
}
__device__ __forceinline__ float *seg_y(const Params &P, int i)
{
    return i == 0 ? P.seg[0].y : (i == 1 ? P.seg[1].y : P.seg[2].y);
}
__device__ __forceinline__ int seg_rows(const Params &P, int i)
{
    return i == 0 ? P.seg[0].rows : (i == 1 ? P.seg[1].rows : P.seg[2].rows);
}
__device__ __forceinline__ int seg_tile0(const Params &P, int i)
{
    return i == 0 ? P.seg[0].tile0 : (i == 1 ? P.seg[1].tile0 : P.seg[2].tile0);
}

__device__ __forceinline__ void tile_info(const Params &P, int tile, int &seg, int &row0, int &rows)
{
    seg = 0;
    if (P.nseg > 1 && tile >= P.seg[1].tile0) seg = 1;
    if (P.nseg > 2 && tile >= P.seg[2].tile0) seg = 2;
    const int per = (P.mode == kSwiGLU) ? (P.tile_rows >> 1) : P.tile_rows;
    row0 = (tile - seg_tile0(P, seg)) * per;
    rows = min(per, seg_rows(P, seg) - row0);
}

__device__ __forceinline__ void issue_tile(const Params &P, int tile, uint8_t *stage, uint64_t *bar)
{
    int seg, row0, rows;
    tile_info(P, tile, seg, row0, rows);
    const uint32_t row_bytes = P.bpr * kQ4KBlock;
    const uint32_t bytes = rows * row_bytes;
    if (P.mode == kSwiGLU) {
        mbar_expect_tx(bar, 2 * bytes);
        bulk_g2s(stage, P.seg[0].w + (size_t)row0 * row_bytes, bytes, bar);
        bulk_g2s(stage + bytes, P.seg[1].w + (size_t)row0 * row_bytes, bytes, bar);
    } else {
        mbar_expect_tx(bar, bytes);
        bulk_g2s(stage, seg_w(P, seg) + (size_t)row0 * row_bytes, bytes, bar);
    }
}

__global__ void __launch_bounds__(kThreads, 1) q4k_stream_kernel(const Params P)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const Smem L = smem_layout(P.bpr, P.tile_rows);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.bars);
    float *part = reinterpret_cast<float *>(smem + L.part);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int my_tiles = (P.n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    if (my_tiles <= 0) return;

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) mbar_init(&bars[s], 1);
        mbar_fence_init();
        for (int k = 0; k < kStages && k < my_tiles; k++)
            issue_tile(P, blockIdx.x + k * gridDim.x, smem + L.stages + k * L.stage_bytes, &bars[k]);
    }
    quantize_x<kThreads, 16, true>(P.x, P.n_cols, P.bpr * 256, reinterpret_cast<int8_t *>(smem + L.xq1),
               reinterpret_cast<int8_t *>(smem + L.xq2), reinterpret_cast<float *>(smem + L.xs1),
               reinterpret_cast<float *>(smem + L.xsum));
    __syncthreads();

    const int q = lane >> 2, g = lane & 3;
    const int rounds = (P.bpr + 7) >> 3;
    const uint32_t row_bytes = P.bpr * kQ4KBlock;
    XRegs xr;
    int cur_round = -1, col = 0, roff = 0, rpp = 1, width = 32;
    bool lane_ok = false;
    // A wait that runs out does not change control flow (every thread keeps
    // taking the same barriers); it raises this flag, the results of the tile
    // are discarded, and the CTA leaves at the next barrier.
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.bars + 48);
    if (tid == 0) *abort_flag = 0;

    for (int k = 0; k < my_tiles; k++) {
        const int tile = blockIdx.x + k * gridDim.x;
        const int st = k % kStages;
        const uint8_t *stage = smem + L.stages + st * L.stage_bytes;
        int seg, row0, rows;
        tile_info(P, tile, seg, row0, rows);
        const int R = (P.mode == kSwiGLU) ? 2 * rows : rows;  // rows resident in the stage

        if (!mbar_wait(&bars[st], (k / kStages) & 1)) *abort_flag = 1;

        // pass list of this tile: round-major; warp takes a contiguous share
        int total = 0;
        for (int cr = 0; cr < rounds; cr++) {
            const int v = min(8, P.bpr - 8 * cr);
            const int r_pp = (v == 1 || v == 2 || v == 4) ? 8 / v : 1;
            total += (R + r_pp - 1) / r_pp;
        }
        const int p_begin = (warp * total) / kWarps, p_end = ((warp + 1) * total) / kWarps;
        float *part_buf = part + (k & 1) * kMaxTileRows * kMaxRounds;

        int cr = 0, base = 0;
        for (int p = p_begin; p < p_end; p++) {
            // locate the round of pass p
            for (;;) {
                const int v = min(8, P.bpr - 8 * cr);
                const int r_pp = (v == 1 || v == 2 || v == 4) ? 8 / v : 1;
                const int n = (R + r_pp - 1) / r_pp;
                if (p < base + n) break;
                base += n;
                cr++;
            }
            if (cr != cur_round) {
                cur_round = cr;
                const int v = min(8, P.bpr - 8 * cr);
                rpp = (v == 1 || v == 2 || v == 4) ? 8 / v : 1;
                lane_ok = q < v * rpp;
                col = 8 * cr + (q % v);
                roff = q / v;
                width = (rpp > 1) ? 4 * v : 32;
                load_xregs(xr, smem, L, lane_ok ? col : 0, g, lane_ok);
            }
            const int row = (p - base) * rpp + roff;
            const bool ok = lane_ok && row < R;
            const uint8_t *blk = stage + (size_t)(ok ? row : 0) * row_bytes + (ok ? col : 0) * kQ4KBlock;
            float acc = block_dot(blk, g, xr);
            acc = ok ? acc : 0.0f;
            acc = group_sum(acc, width);
            if ((lane & (width - 1)) == 0 && row < R) part_buf[row * kMaxRounds + cr] = acc;
        }
        __syncthreads();
        if (*abort_flag) {
            if (tid == 0) atomicExch(P.err, MB200_ERR_TIMEOUT);
            break;
        }

        // the stage is drained: refill it with the tile kStages ahead
        if (tid == 0 && k + kStages < my_tiles)
            issue_tile(P, tile + kStages * gridDim.x, smem + L.stages + st * L.stage_bytes, &bars[st]);

        // epilogue: one thread per output row
        const int out_rows = (P.mode == kSwiGLU) ? rows : R;
        if (tid < out_rows) {
            float s = 0.0f;
            for (int c = 0; c < rounds; c++) s += part_buf[tid * kMaxRounds + c];
            const int r = row0 + tid;
            if (P.mode == kStore) {
                seg_y(P, seg)[r] = s;
            } else if (P.mode == kAddResidual) {
                seg_y(P, seg)[r] = s + P.residual[r];
            } else if (P.mode == kScaledAdd) {
                seg_y(P, seg)[r] += P.scale * s;
            } else {
                float u = 0.0f;
                for (int c = 0; c < rounds; c++) u += part_buf[(tid + rows) * kMaxRounds + c];
                P.seg[0].y[r] = s / (1.0f + expf(-s)) * u;
            }
        }
    }
}

int g_smem_optin = 0;

void launch(Params &P, cudaStream_t stream, const char *where)
{
    if (P.n_cols <= 0) return;
    P.bpr = (P.n_cols + 255) / 256;
    const int row_bytes = P.bpr * kQ4KBlock;
    int tr = kTileTargetBytes / row_bytes;
    tr = tr < 1 ? 1 : (tr > kMaxTileRows ? kMaxTileRows : tr);
    if (P.mode == kSwiGLU) tr = tr < 2 ? 2 : (tr & ~1);
    P.tile_rows = tr;
    const int per = (P.mode == kSwiGLU) ? tr / 2 : tr;
    int tiles = 0;
    const int nseg_tiles = (P.mode == kSwiGLU) ? 1 : P.nseg;
    for (int i = 0; i < P.nseg; i++) {
        P.seg[i].tile0 = tiles;
        if (i < nseg_tiles) tiles += (P.seg[i].rows + per - 1) / per;
    }
    P.n_tiles = tiles;
    if (tiles == 0) return;
    P.err = device_error_word();
    const Smem L = smem_layout(P.bpr, P.tile_rows);
    if (P.n_cols > kMaxCols || L.total > 227 * 1024) {
        fprintf(stderr, "[mnemo_b200] %s: n_cols=%d exceeds the supported %d\n", where, P.n_cols, kMaxCols);
        set_status(MB200_ERR_UNSUPPORTED, where);
        return;
    }
    for (int i = 0; i < P.nseg; i++)
        if ((reinterpret_cast<uintptr_t>(P.seg[i].w) & 15) != 0) {
            fprintf(stderr, "[mnemo_b200] %s: Q4_K tensor %d is not 16-byte aligned\n", where, i);
            set_status(MB200_ERR_ARG, where);
            return;
        }
    if (!g_smem_optin) {
        cudaFuncSetAttribute(q4k_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        g_smem_optin = 1;
    }
    const int grid = tiles < kSMs ? tiles : kSMs;
    q4k_stream_kernel<<<grid, kThreads, L.total, stream>>>(P);
    MB200_CHECK_LAUNCH(where);
}

}  // namespace

void q4k_init()
{
    cudaFuncSetAttribute(q4k_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    g_smem_optin = 1;
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
    P.mode = kStore;
    launch(P, stream, "cuda_matvec_q4k");
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
    P.mode = kAddResidual;
    launch(P, stream, "cuda_matvec_q4k_add");
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
    P.mode = kStore;
    launch(P, stream, "cuda_matvec_q4k_qkv");
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
    P.mode = kStore;
    launch(P, stream, "cuda_matvec_q4k_dual");
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
    P.mode = kScaledAdd;
    launch(P, stream, "cuda_matvec_q4k_scaled_add");
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
    P.mode = kSwiGLU;
    mb200_clear_status();
    launch(P, stream, "mb200_matvec_q4k_dual_swiglu");
    return mb200_last_status();
}

}  // extern "C"
