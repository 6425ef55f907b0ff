// Streaming dequant-matvec skeleton shared by the Q4_K and Q6_K kernels (batch 1).
//
// A weight matrix is a contiguous stream of super-blocks. The rows of all
// segments of a call (one tensor; Q,K,V; gate,up) are split into one contiguous
// range per CTA (balanced to a row), and each range is cut into tiles of whole
// rows. Three roles per CTA:
//   * issuer (one lane of warp kConsumers): moves each tile into a ring of
//     shared-memory stages with a 1-D bulk async copy (TMA engine, completion
//     on the stage's "full" mbarrier) as soon as the stage's "empty" barrier flips;
//   * kConsumers consumer warps: wait on "full", compute their rows, publish
//     partial sums in shared memory, arrive on "empty";
//   * epilogue warp (kConsumers+1): after "empty" flips, adds the partials of
//     each row in fixed order, applies the epilogue (store, + residual, scaled
//     accumulate, SwiGLU pairing) and arrives on the stage's next "full" phase,
//     which is what lets consumers overwrite the partial-sum slot again.
// There is no block-wide barrier inside the loop, and every wait is bounded.
//
// Work split inside a tile: a warp pass covers G = 32 / lanes-per-block
// super-blocks. The block-columns of a row are split into column groups of v
// columns, v the largest power of two (<= G) dividing the blocks per row, and a
// pass covers G / v consecutive rows of its group, so no lane idles for any
// row length (rows whose block count has too small a power-of-two factor fall
// back to groups of G columns with a ragged, partly idle last group). Each
// consumer warp is bound to one column group for the whole kernel (host-made
// table in the launch parameters), so its share of the activation vector is
// loaded into registers once. A unit is RU passes issued back to back
// (independent rows: instruction-level parallelism), reduced together with one
// packed butterfly.
#pragma once

#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace mb200 {
namespace stream {

#ifndef MB200_CONSUMERS
#define MB200_CONSUMERS 12
#endif
constexpr int kConsumers = MB200_CONSUMERS;
constexpr int kThreads = (kConsumers + 2) * 32;
constexpr int kQuantThreads = kConsumers * 32;  // the consumer warps stage x; issuer/epilogue warps do not
constexpr int kMaxStages = 6;

enum : int {
    kStore = 0,
    kAddResidual = 1,
    kScaledAdd = 2,
    kSwiGLU = 3,
    // routed experts, ids and weights read on the device (reference sequence src/forward.c:1122-1142 per expert):
    kMoeGateUp = 4,  // act[e][r] = silu(gate_e[r].x) * (up_e[r].x) for the n_slots routed experts, one launch
    kMoeDown = 5     // y[r] = (residual[r] | y[r]) + sum_e w_e * (down_e[r] . act[e]), experts added in slot order
};
constexpr int kMaxSlots = 16;  // top-k limit of the router (cuda_topk_softmax: k <= 16)

struct Seg {
    const uint8_t *w;
    float *y;
    int rows;
    int start;  // first virtual row of this segment (rows of all segments are numbered consecutively)
};

struct Params {
    Seg seg[3];
    int nseg;
    int vrows;      // virtual rows to split over CTAs (SwiGLU: gate rows; each brings its up row along)
    int tile_rows;  // rows per tile and segment (SwiGLU tiles hold this many gate rows + as many up rows)
    const float *x;
    const float *residual;
    float scale;
    int n_cols, bpr, mode, stages;
    int pdl;        // launched with programmatic stream serialization: wait for the upstream grid before touching x / y
    int cta0, ncta; // this problem's CTAs are blockIdx.x in [cta0, cta0 + ncta) (two problems may share one launch)
    int per_cta, rem_cta;  // vrows / ncta and vrows % ncta: CTA c takes per_cta rows, the first rem_cta CTAs one more
    int ru;         // row unroll chosen by the host (read by the pair kernel, which holds all three bodies)
    int *err;
    // routed-expert modes
    const int *ids;          // [n_slots] expert index per slot (device); < 0 = empty slot
    const float *wts;        // [n_slots] routing weight per slot (device)
    const uint8_t *ebase;    // expert e's blob starts at ebase + e * estride
    size_t estride, off_a, off_b;  // byte offsets inside a blob: gate/up (kMoeGateUp) or down (off_a, kMoeDown)
    int n_slots, erows;      // experts per token; rows per expert tensor
    int expert_lo, expert_cnt;  // this device holds experts [expert_lo, expert_lo + expert_cnt) at ebase; other ids are skipped
    int x_stride;            // kMoeDown: floats between the activation vectors of consecutive slots
    // RMSNorm folded into the staging of x: x'[c] = x[c] * norm_w[c] / sqrt(mean(x^2) + norm_eps); every CTA
    // computes the sum of squares itself (x is read once per CTA anyway). nullptr = x is used as given.
    const float *norm_w;
    float norm_eps;
    int n_groups;   // column groups (= partial sums per row)
    // per consumer warp: group | first column << 5 | columns v << 12 | rows per pass << 16 | index in group << 20 | warps of group << 24
    uint32_t warp_cfg[kConsumers];
};

struct Layout {
    int bars, xq1, xq2, xs1, xsum, x_stride, part, stages, stage_bytes, total;
};

// bars: 2 * kMaxStages mbarriers, abort flag at +120, routed ids at +128, routing weights at +192,
// active-slot list at +256, its length at +320
template <class F>
__host__ __device__ inline Layout layout(int bpr, int tile_rows_in_stage, int n_stages, int ng, int n_x)
{
    Layout s;
    const int kpad = bpr * 256;
    int o = 0;
    s.bars = o;  o += 384;
    const int x0 = o;
    s.xq1 = o;   o += F::kXWords * (F::kSlotsPerBlock * bpr + 1) * 4;  // [word][slot], +1 pad: conflict-free both ways
    s.xq2 = o;   o += F::kXWords * (F::kSlotsPerBlock * bpr + 1) * 4;
    s.xs1 = o;   o += (kpad / 32) * 4;
    s.xsum = o;  o += (kpad / F::kSumCols) * 4;
    s.x_stride = o - x0;  // one staged activation vector; kMoeDown stages one per slot
    o += (n_x - 1) * s.x_stride;
    s.part = o;  o += n_stages * tile_rows_in_stage * ng * 4;
    o = (o + 127) & ~127;
    s.stages = o;
    s.stage_bytes = (tile_rows_in_stage * bpr * F::kBlockBytes + 32 + 127) & ~127;  // +32: alignment skew, word over-read
    s.total = o + n_stages * s.stage_bytes;
    return s;
}

// Static selects instead of P.seg[i]: dynamic indexing would push the parameter block to local memory.
__device__ __forceinline__ const uint8_t *seg_w(const Params &P, int i)
{
    return i == 0 ? P.seg[0].w : (i == 1 ? P.seg[1].w : P.seg[2].w);
}
__device__ __forceinline__ float *seg_y(const Params &P, int i)
{
    return i == 0 ? P.seg[0].y : (i == 1 ? P.seg[1].y : P.seg[2].y);
}

struct Tile {
    int seg, row0, rows;  // rows per segment (a SwiGLU tile holds 2*rows rows)
    int j;                // routed modes: position of the slot in the active list
};

// Rows [cur, end) of CTA `cta` out of P.ncta. Quotient and remainder come from the host (a division, let alone a
// 64-bit one, is a subroutine that every role of every CTA would fetch cold at the start of every launch); only the
// routed gate/up mode, whose row count depends on the slots served here, divides on the device (32-bit).
__device__ __forceinline__ void cta_rows(const Params &P, int vrows, int cta, int &cur, int &end)
{
    int per = P.per_cta, rem = P.rem_cta;
    if (vrows != P.vrows) {
        per = vrows / P.ncta;
        rem = vrows - per * P.ncta;
    }
    cur = cta * per + min(cta, rem);
    end = cur + per + (cta < rem ? 1 : 0);
}

// Walks the tiles of this CTA's row range [cur, end). Every role runs the same walk.
// t.seg is the segment (plain modes) or the expert slot (routed modes).
struct TileWalk {
    int cur, end, e, n_act;
    const int *act;  // active slots (routed modes), shared memory
    __device__ __forceinline__ void init(const Params &P, const int *act_list, int n_active)
    {
        act = act_list;
        n_act = n_active;
        const int vrows = (P.mode == kMoeGateUp) ? n_active * P.erows : P.vrows;
        const int cta = static_cast<int>(blockIdx.x) - P.cta0;
        cta_rows(P, vrows, cta, cur, end);
        if (P.mode == kMoeDown && n_active == 0) end = cur;
        e = 0;
    }
    __device__ __forceinline__ bool next(const Params &P, Tile &t)
    {
        if (cur >= end) return false;
        t.j = 0;
        if (P.mode == kMoeDown) {  // the same rows for every active slot in turn, then the next rows
            t.j = e;
            t.seg = act[e];
            t.row0 = cur;
            t.rows = min(P.tile_rows, end - cur);
            if (++e == n_act) {
                e = 0;
                cur += t.rows;
            }
            return true;
        }
        int seg = 0, s0 = 0, s1 = P.seg[0].rows;
        if (P.mode == kMoeGateUp) {
            t.j = cur / P.erows;
            seg = act[t.j];
            s0 = t.j * P.erows;
            s1 = s0 + P.erows;
        } else if (P.mode != kSwiGLU) {
            if (P.nseg > 1 && cur >= P.seg[1].start) {
                seg = 1;
                s0 = P.seg[1].start;
                s1 = s0 + P.seg[1].rows;
            }
            if (P.nseg > 2 && cur >= P.seg[2].start) {
                seg = 2;
                s0 = P.seg[2].start;
                s1 = s0 + P.seg[2].rows;
            }
        }
        const int stop = min(min(end, s1), cur + P.tile_rows);
        t.seg = seg;
        t.row0 = cur - s0;
        t.rows = stop - cur;
        cur = stop;
        return true;
    }
};

__device__ __forceinline__ bool pair_mode(int mode) { return mode == kSwiGLU || mode == kMoeGateUp; }

// First byte of the tile's rows (for pair modes: of its gate rows; `second` selects the up rows).
__device__ __forceinline__ const uint8_t *tile_src(const Params &P, const Tile &t, size_t row_bytes, const int *sid,
                                                   bool second = false)
{
    const uint8_t *w;
    if (P.mode == kMoeGateUp || P.mode == kMoeDown) {
        const int id = sid[t.seg];
        w = P.ebase + (size_t)(id < 0 ? 0 : id) * P.estride + (second ? P.off_b : P.off_a);
    } else if (P.mode == kSwiGLU) {
        w = second ? P.seg[1].w : P.seg[0].w;
    } else {
        w = seg_w(P, t.seg);
    }
    return w + (size_t)t.row0 * row_bytes;
}

template <class F>
__device__ __forceinline__ void issue_tile(const Params &P, const Tile &t, uint8_t *stage, uint64_t *bar, const int *sid)
{
    const size_t row_bytes = (size_t)P.bpr * F::kBlockBytes;
    if (pair_mode(P.mode)) {  // Q4_K only: rows are multiples of 16 bytes, spans are exact
        const uint32_t half = t.rows * (uint32_t)row_bytes;
        mbar_expect_tx(bar, 2 * half);
        bulk_g2s(stage, tile_src(P, t, row_bytes, sid, false), half, bar);
        bulk_g2s(stage + half, tile_src(P, t, row_bytes, sid, true), half, bar);
    } else {
        // The 16-byte-aligned span enclosing the rows. The few bytes read before/after them share a
        // 16-byte granule with a valid byte, hence lie inside a mapped page.
        const uintptr_t begin = reinterpret_cast<uintptr_t>(tile_src(P, t, row_bytes, sid));
        const uintptr_t stop = begin + (size_t)t.rows * row_bytes;
        const uintptr_t a0 = begin & ~static_cast<uintptr_t>(15);
        const uint32_t bytes = static_cast<uint32_t>(((stop + 15) & ~static_cast<uintptr_t>(15)) - a0);
        mbar_expect_tx(bar, bytes);
        bulk_g2s(stage, reinterpret_cast<const void *>(a0), bytes, bar);
    }
}

// Sum RU per-lane values over groups of W lanes (W = 32, 16 or 8), RU in {1,2,4}.
// On return, lane l with (l & (W/RU - 1)) == 0 holds the sum for value index
// `which` (= (l & (W-1)) / (W/RU)) of its W-lane group.
template <int RU, bool W32>
__device__ __forceinline__ float packed_sum(float (&a)[RU], int W, int lane, int &which)
{
    int off = W32 ? 16 : (W >> 1);
    float v;
    if (RU == 4) {
        const bool hi = (lane & off) != 0;
        float k0 = hi ? a[2] : a[0], k1 = hi ? a[3] : a[1];
        const float s0 = hi ? a[0] : a[2], s1 = hi ? a[1] : a[3];
        k0 += __shfl_xor_sync(0xffffffffu, s0, off);
        k1 += __shfl_xor_sync(0xffffffffu, s1, off);
        which = hi ? 2 : 0;
        off >>= 1;
        const bool hi2 = (lane & off) != 0;
        v = hi2 ? k1 : k0;
        v += __shfl_xor_sync(0xffffffffu, hi2 ? k0 : k1, off);
        which += hi2 ? 1 : 0;
        off >>= 1;
    } else if (RU == 2) {
        const bool hi = (lane & off) != 0;
        v = hi ? a[1] : a[0];
        v += __shfl_xor_sync(0xffffffffu, hi ? a[0] : a[1], off);
        which = hi ? 1 : 0;
        off >>= 1;
    } else {
        v = a[0];
        which = 0;
    }
    if (W32) {
#pragma unroll
        for (int o = 16 / RU; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    } else {
        for (; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    }
    return v;
}

#ifdef MB200_TRACE
// Developer aid (off in product builds): per-CTA clock stamps at phase boundaries.
static __device__ long long g_trace[kSMs * 2][48];  // one copy per translation unit
#define MB200_STAMP(slot)                                                     \
    do {                                                                      \
        if ((threadIdx.x & 31) == 0 && blockIdx.x < kSMs * 2) {               \
            long long t__;                                                    \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));           \
            ::mb200::stream::g_trace[blockIdx.x][slot] = t__;                                 \
        }                                                                     \
    } while (0)
#else
#define MB200_STAMP(slot) do {} while (0)
#endif

// Activation split: x[c] ~= s1[c/32] * (q1[c] + q2[c]/254) with q1, q2 int8, so
// two exact dp4a dot products recover sum(q*x) to ~1e-5 relative
// (|error| <= max|x|/64516 per 32-column group). xsum holds exact fp32 sums of
// x over F::kSumCols columns (for the terms that multiply sum(x): Q4_K's
// -dmin*m, Q6_K's -32 offset). Columns outside the matrix are stored as zero;
// F::kGroup4Tail: a group of 4 columns counts only if all four are < n_cols
// (the Q4_K kernels' tail rule, reference src/kernels.cu:124,131), else per
// column (Q6_K, :474). The int8 words are stored transposed, [word][lane slot]
// with an odd row pitch, so that the consumer lanes' register loads and these
// stores are both free of bank conflicts. All loads of a thread are issued
// before the first use: one memory round trip for K <= 3 * 4 * kQuantThreads.
// x (and everything else an upstream kernel produces: the routed ids and weights, the residual) is read
// with ld.global.cg, i.e. from L2: under programmatic dependent launch this kernel is resident before
// its producer has finished, so neither the non-coherent path (__ldg) nor lines an SM's L1 may still
// hold from an earlier use of the same buffer can be trusted.
// Called by the consumer warps only (threadIdx.x < kQuantThreads).
// With norm_w the vector is RMS-normalised on the way (needs the whole vector in one round of loads,
// n_cols <= 4 * UN * kQuantThreads, which the host checks): the consumer warps add up x^2 through `red`
// (kConsumers floats of shared memory) and hardware barrier 2.
// One quad of columns -> the two int8 levels, the group's scale and the column sums.
template <class F>
__device__ __forceinline__ void split_quad(const float (&v)[4], int c0, int lane, int pitch, uint32_t *q1, uint32_t *q2,
                                           float *s1, float *xsum)
{
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    float sum = (v[0] + v[1]) + (v[2] + v[3]);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // 8 lanes = 32 columns share a scale
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if (F::kSumCols == 16) sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const float sc = amax * (1.0f / 127.0f);
    const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
    uint32_t p1 = 0, p2 = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        // |x| <= amax, so |a| <= 127; |r| <= sc/2 (+ rounding), so |b| <= 127: clamp only guards NaN/Inf input
        const float a = rintf(v[i] * inv);
        const float r = fmaf(-a, sc, v[i]);
        const float b = fminf(fmaxf(rintf(r * inv * 254.0f), -127.0f), 127.0f);
        p1 |= (static_cast<uint32_t>(__float2int_rn(a)) & 0xFFu) << (8 * i);
        p2 |= (static_cast<uint32_t>(__float2int_rn(b)) & 0xFFu) << (8 * i);
    }
    const int idx = F::xword(c0) * pitch + F::xslot(c0);
    q1[idx] = p1;
    q2[idx] = p2;
    if ((lane & 7) == 0) s1[c0 >> 5] = sc;
    if (F::kSumCols == 16) {
        if ((lane & 3) == 0) xsum[c0 >> 4] = sum;
    } else {
        if ((lane & 1) == 0) xsum[c0 >> 3] = sum;
    }
}

template <class F>
__device__ __forceinline__ void load_quad(const float *__restrict__ x, int c0, int n_cols, bool vec_ok, float (&v)[4])
{
    if (vec_ok && c0 + 3 < n_cols) {
        const float4 t = __ldcg(reinterpret_cast<const float4 *>(x + c0));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const bool in = F::kGroup4Tail ? (c0 + 3) < n_cols : (c0 + i) < n_cols;
            v[i] = in ? __ldcg(x + c0 + i) : 0.0f;
        }
    }
}

template <class F, int UN>
__device__ __forceinline__ void quantize_x(const float *__restrict__ x, int n_cols, int bpr,
                                           uint32_t *q1, uint32_t *q2, float *s1, float *xsum,
                                           const float *__restrict__ norm_w = nullptr, float norm_eps = 0.0f,
                                           float *red = nullptr)
{
    const int kpad = bpr * 256;
    const int pitch = F::kSlotsPerBlock * bpr + 1;
    const int lane = threadIdx.x & 31;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    if (!norm_w) {
        // all loads of a round in flight, then the splits side by side (a rolled loop, one quad ahead, was
        // measured 10 % slower on the 8192 x 4096 matvec: the splits' shuffle chains need each other's company)
        for (int base = threadIdx.x * 4; base < kpad; base += kQuantThreads * 4 * UN) {
            float v[UN][4];
#pragma unroll
            for (int u = 0; u < UN; u++) load_quad<F>(x, base + u * kQuantThreads * 4, n_cols, vec_ok, v[u]);
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const int c0 = base + u * kQuantThreads * 4;
                if (c0 >= kpad) break;  // warp-uniform: a warp covers 128 columns, kpad is a multiple of 256
                split_quad<F>(v[u], c0, lane, pitch, q1, q2, s1, xsum);
            }
        }
        return;
    }
    // With the norm: every thread runs the round (also one whose columns lie beyond the vector: it loads nothing
    // and stores nothing), because all consumer threads must reach the barrier below. One round of loads (the
    // host has checked n_cols <= 4 * UN * kQuantThreads).
    const int base = threadIdx.x * 4;
    float v[UN][4];
#pragma unroll
    for (int u = 0; u < UN; u++) load_quad<F>(x, base + u * kQuantThreads * 4, n_cols, vec_ok, v[u]);
    float wv[UN][4];
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < UN; u++) {
        const int c0 = base + u * kQuantThreads * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            wv[u][i] = (c0 + i < n_cols) ? __ldg(norm_w + c0 + i) : 0.0f;
            // the sum runs over every column of x, also those a group-of-four tail rule drops below
            const float xv = (F::kGroup4Tail && c0 + i < n_cols && !(c0 + 3 < n_cols)) ? __ldcg(x + c0 + i) : v[u][i];
            ss = fmaf(xv, xv, ss);
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[threadIdx.x >> 5] = ss;
    asm volatile("bar.sync 2, %0;" ::"n"(kQuantThreads) : "memory");
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < kConsumers; w++) tot += red[w];  // fixed order: the same scale on every thread and CTA
    const float scale = 1.0f / sqrtf(tot / static_cast<float>(n_cols) + norm_eps);
#pragma unroll
    for (int u = 0; u < UN; u++) {
        const int c0 = base + u * kQuantThreads * 4;
        if (c0 >= kpad) break;  // warp-uniform
#pragma unroll
        for (int i = 0; i < 4; i++) v[u][i] = v[u][i] * scale * wv[u][i];
        split_quad<F>(v[u], c0, lane, pitch, q1, q2, s1, xsum);
    }
}

// Same split done by a single warp for one whole vector (routed down-projection:
// one activation vector per expert slot, each handled by one warp).
template <class F>
__device__ __forceinline__ void quantize_x_warp(const float *__restrict__ x, int n_cols, int bpr,
                                                uint32_t *q1, uint32_t *q2, float *s1, float *xsum)
{
    constexpr int UN = 12;  // 1536 columns (the 235B expert width) in one round of loads
    const int kpad = bpr * 256;
    const int pitch = F::kSlotsPerBlock * bpr + 1;
    const int lane = threadIdx.x & 31;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    for (int base = lane * 4; base < kpad; base += 128 * UN) {
        float v[UN][4];
#pragma unroll
        for (int u = 0; u < UN; u++) load_quad<F>(x, base + u * 128, n_cols, vec_ok, v[u]);
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int c0 = base + u * 128;
            if (c0 - lane * 4 >= kpad) break;  // warp-uniform
            split_quad<F>(v[u], c0, lane, pitch, q1, q2, s1, xsum);
        }
    }
}

__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class F, int RU>
__device__ __forceinline__ void stream_body(const Params &P, uint8_t *smem)
{
    const int S = P.stages;
    const bool pairs = pair_mode(P.mode);
    const bool routed = (P.mode == kMoeGateUp || P.mode == kMoeDown);
    const int stage_rows = pairs ? 2 * P.tile_rows : P.tile_rows;
    const int NG = P.n_groups;
    const int n_x = (P.mode == kMoeDown) ? P.n_slots : 1;
    const Layout L = layout<F>(P.bpr, stage_rows, S, NG, n_x);
    int *sid = reinterpret_cast<int *>(smem + L.bars + 128);      // routed expert per slot
    float *swt = reinterpret_cast<float *>(smem + L.bars + 192);  // routing weight per slot
    int *act_list = reinterpret_cast<int *>(smem + L.bars + 256);  // slots this device serves, in slot order
    int *n_act_p = reinterpret_cast<int *>(smem + L.bars + 320);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.bars);
    uint64_t *empty = full + kMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.bars + 120);
    float *part = reinterpret_cast<float *>(smem + L.part);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (warp == 0) MB200_STAMP(0);
    const uint32_t row_bytes = P.bpr * F::kBlockBytes;
    const int part_pitch = stage_rows * NG;

    TileWalk walk;

    if (warp == kConsumers) {
        // ---------------- issuer ----------------
        // The weights never depend on the upstream kernel, so the first stages are
        // requested before the grid-dependency wait: they stream in while the
        // upstream kernel drains and while x is staged.
        if (lane == 0) {
            *abort_flag = 0;
            for (int s = 0; s < S; s++) {
                mbar_init(&full[s], 2);  // the issuer's expect_tx arrival + the epilogue warp's "partials are free"
                mbar_init(&empty[s], kConsumers);
            }
            mbar_fence_init();
        }
        if (routed) {
            // which experts to stream is decided by the upstream kernel (the router): wait for it first. Lane e reads
            // slot e -- one round trip for all slots (one thread reading them in turn was a chain of 2 x n_slots
            // round trips before the first weight byte could be requested) -- and a ballot compacts the served slots.
            if (P.pdl) grid_dep_wait();
            int id = -1;
            float w = 0.0f;
            if (lane < P.n_slots) {
                id = __ldcg(P.ids + lane);
                if (P.wts != nullptr) w = __ldcg(P.wts + lane);  // gate/up has no routing weights
            }
            const bool here = lane < P.n_slots && id >= P.expert_lo && id - P.expert_lo < P.expert_cnt;  // empty slots have id < 0
            const unsigned served = __ballot_sync(0xffffffffu, here);
            if (lane < P.n_slots) {
                sid[lane] = here ? id - P.expert_lo : -1;
                swt[lane] = here ? w : 0.0f;
            }
            if (here) act_list[__popc(served & ((1u << lane) - 1u))] = lane;
            if (lane == 0) *n_act_p = __popc(served);
            __syncwarp();
        }
        if (lane == 0) {
            walk.init(P, act_list, routed ? *n_act_p : 0);
            Tile t;
            for (int s = 0; s < S; s++) {
                mbar_arrive(&full[s]);  // first phase: nothing to drain yet
                if (walk.next(P, t)) issue_tile<F>(P, t, smem + L.stages + s * L.stage_bytes, &full[s], sid);
            }
        }
        __syncthreads();
        if (lane == 0) {
            if (P.pdl) grid_dep_launch();
            Tile t;
            int s = 0, ph = 0;
            while (walk.next(P, t)) {
                if (!mbar_wait(&empty[s], ph)) {
                    *abort_flag = 1;
                    break;
                }
                issue_tile<F>(P, t, smem + L.stages + s * L.stage_bytes, &full[s], sid);
                if (++s == S) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
        return;
    }
    if (warp == kConsumers + 1) {
        // ---------------- epilogue warp ----------------
        __syncthreads();
        if (P.pdl) grid_dep_wait();  // y / residual may still be in use by the upstream kernel
        walk.init(P, act_list, routed ? *n_act_p : 0);
        if (P.mode == kMoeDown && walk.n_act == 0 && P.residual) {
            // no routed expert lives on this device: the block reduces to the residual
            const int cta = static_cast<int>(blockIdx.x) - P.cta0;
            int r0, r1;
            cta_rows(P, P.vrows, cta, r0, r1);
            for (int r = r0 + lane; r < r1; r += 32) P.seg[0].y[r] = __ldcg(P.residual + r);
        }
        Tile t, ahead;
        float eacc0 = 0.0f, eacc1 = 0.0f;  // kMoeDown: per-row running sums (tiles hold at most 64 rows)
        TileWalk look = walk;
        for (int i = 0; i < S; i++) look.next(P, ahead);  // `look` runs S tiles ahead: does stage s get reused?
        int s = 0, ph = 0;
        int ek = 0;
        while (walk.next(P, t)) {
            const bool reused = look.next(P, ahead);
            if (!mbar_wait(&empty[s], ph)) *abort_flag = 1;
            if (*abort_flag) break;
            if (ek < 8) MB200_STAMP(32 + ek);
            const float *pt = part + s * part_pitch;
            int it = 0;
            for (int r = lane; r < t.rows; r += 32, it++) {
                float v = 0.0f;
                for (int c = 0; c < NG; c++) v += pt[r * NG + c];
                const int row = t.row0 + r;
                if (P.mode == kStore) {
                    seg_y(P, t.seg)[row] = v;
                } else if (P.mode == kAddResidual) {
                    seg_y(P, t.seg)[row] = v + __ldcg(P.residual + row);
                } else if (P.mode == kScaledAdd) {
                    seg_y(P, t.seg)[row] = __ldcg(seg_y(P, t.seg) + row) + P.scale * v;
                } else if (P.mode == kMoeDown) {
                    // slots arrive in order 0..n_slots-1 for the same rows: keep the running sum in registers
                    float a = (t.j == 0) ? 0.0f : (it == 0 ? eacc0 : eacc1);
                    a = fmaf(swt[t.seg], v, a);
                    if (it == 0) eacc0 = a; else eacc1 = a;
                    if (t.j == walk.n_act - 1)
                        P.seg[0].y[row] = __ldcg(P.residual ? P.residual + row : P.seg[0].y + row) + a;
                } else {
                    float u = 0.0f;
                    for (int c = 0; c < NG; c++) u += pt[(r + t.rows) * NG + c];
                    const float act = v / (1.0f + expf(-v)) * u;
                    if (P.mode == kSwiGLU)
                        P.seg[0].y[row] = act;
                    else
                        P.seg[0].y[t.seg * P.erows + row] = act;
                }
            }
            __syncwarp();
            if (lane == 0 && reused) mbar_arrive(&full[s]);  // partial-sum slot s may be rewritten
            if (ek < 8) MB200_STAMP(40 + ek);
            ek++;
            if (++s == S) {
                s = 0;
                ph ^= 1;
            }
        }
        if (*abort_flag && lane == 0) atomicExch(P.err, MB200_ERR_TIMEOUT);
        MB200_STAMP(6);
        return;
    }

    // ---------------- consumer warps ----------------
    if (P.pdl) grid_dep_wait();  // x is produced by the upstream kernel
    if (n_x == 1) {
        quantize_x<F, 3>(P.x, P.n_cols, P.bpr, reinterpret_cast<uint32_t *>(smem + L.xq1),
                         reinterpret_cast<uint32_t *>(smem + L.xq2), reinterpret_cast<float *>(smem + L.xs1),
                         reinterpret_cast<float *>(smem + L.xsum), P.norm_w, P.norm_eps,
                         reinterpret_cast<float *>(smem + L.bars + 328));
    } else {
        // one activation vector per slot; warps take slots round-robin so the loads of all slots are in flight together
        for (int e = warp; e < n_x; e += kConsumers) {
            const int id = __ldcg(P.ids + e);
            if (id < P.expert_lo || id - P.expert_lo >= P.expert_cnt) continue;  // not served here: its activations do not exist
            uint8_t *xb = smem + e * L.x_stride;
            quantize_x_warp<F>(P.x + (size_t)e * P.x_stride, P.n_cols, P.bpr, reinterpret_cast<uint32_t *>(xb + L.xq1),
                               reinterpret_cast<uint32_t *>(xb + L.xq2), reinterpret_cast<float *>(xb + L.xs1),
                               reinterpret_cast<float *>(xb + L.xsum));
        }
    }
    if (warp == 0) MB200_STAMP(1);
    __syncthreads();  // the only block-wide barrier: x is staged, barriers are initialised
    if (warp == 0) MB200_STAMP(2);
    walk.init(P, act_list, routed ? *n_act_p : 0);

    // The warp's column group (host-made table).
    const uint32_t cfg = P.warp_cfg[warp];
    const int ng = cfg & 31, col0 = (cfg >> 5) & 127, v = (cfg >> 12) & 15, rpp = (cfg >> 16) & 15;
    const int idx = (cfg >> 20) & 15, cnt = (cfg >> 24) & 15;
    const int q = lane / F::kLanesPerBlock, sub = lane % F::kLanesPerBlock;
    const bool lane_ok = q < v * rpp;
    const int col = col0 + (lane_ok ? q % v : 0);
    const int roff = lane_ok ? q / v : 0;
    const int W = (rpp > 1) ? v * F::kLanesPerBlock : 32;
    typename F::XRegs xr;
    if (P.mode != kMoeDown) F::load_xregs(xr, smem, L, P.bpr, col, sub, lane_ok);  // kMoeDown loads per slot
    const int unit_rows = RU * rpp;
    const uint32_t lane_base = col * F::kBlockBytes + roff * row_bytes + idx * unit_rows * row_bytes;
    const uint32_t unit_stride = cnt * unit_rows * row_bytes;
    const uint32_t pass_stride = rpp * row_bytes;
    const bool all_lanes = (v * rpp == F::kG);  // no idle lane groups

    Tile t;
    int s = 0, ph = 0;
    int k = 0;
    int cur_slot = -1;
    while (walk.next(P, t)) {
        const int R = pairs ? 2 * t.rows : t.rows;
        uint32_t skew = 0;
        if (F::kBlockBytes % 16 != 0)
            skew = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(tile_src(P, t, row_bytes, sid)) & 15);
        if (P.mode == kMoeDown && t.seg != cur_slot) {  // next expert: its own activation vector
            cur_slot = t.seg;
            F::load_xregs(xr, smem + cur_slot * L.x_stride, L, P.bpr, col, sub, lane_ok);
        }
        const uint8_t *base = smem + L.stages + s * L.stage_bytes + skew;
        float *pt = part + s * part_pitch + ng;

        if (!mbar_wait(&full[s], ph)) *abort_flag = 1;
        if (warp == 0 && k == 0) MB200_STAMP(3);
        if (warp == 0) MB200_STAMP(4);
        if (warp == 0 && k < 8) MB200_STAMP(16 + k);
        k++;

        int r0 = idx * unit_rows;
        const uint8_t *up = base + lane_base;
        // fast path: whole units inside the tile, every lane busy -> no bounds logic
        if (all_lanes) {
            for (; r0 + unit_rows <= R; r0 += cnt * unit_rows, up += unit_stride) {
                float acc[RU];
#pragma unroll
                for (int u = 0; u < RU; u++) acc[u] = F::block_dot(up + u * pass_stride, sub, xr);
                int which;
                float sum;
                if (W == 32)
                    sum = packed_sum<RU, true>(acc, 32, lane, which);
                else
                    sum = packed_sum<RU, false>(acc, W, lane, which);
                const int wr = W / RU;  // lanes per result
                if ((lane & (wr - 1)) == 0) pt[(r0 + which * rpp + roff) * NG] = sum;
            }
        }
        // general path: ragged units, idle lane groups
        for (; r0 < R; r0 += cnt * unit_rows) {
            float acc[RU];
#pragma unroll
            for (int u = 0; u < RU; u++) {
                const int row = r0 + u * rpp + roff;
                const bool ok = lane_ok && row < R;
                const uint8_t *blk = base + (size_t)min(row, R - 1) * row_bytes + col * F::kBlockBytes;
                const float d = F::block_dot(blk, sub, xr);
                acc[u] = ok ? d : 0.0f;
            }
            int which;
            const float sum = packed_sum<RU, false>(acc, W, lane, which);
            const int wr = W / RU;
            const int row = r0 + which * rpp + roff;
            if ((lane & (wr - 1)) == 0 && row < R) pt[row * NG] = sum;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        if (*abort_flag) break;
        if (warp == 0 && k <= 8) MB200_STAMP(24 + k - 1);
        if (++s == S) {
            s = 0;
            ph ^= 1;
        }
    }
    if (warp == 0) MB200_STAMP(5);
}

template <class F, int RU>
__global__ void __launch_bounds__(kThreads, 1) stream_kernel(const __grid_constant__ Params P)
{
    extern __shared__ __align__(128) uint8_t smem[];
    stream_body<F, RU>(P, smem);
}

// Two independent problems with different block types in one launch: CTAs [0, PA.ncta) run A, the others B
// (the decode path's Q4_K Q / K projections and Q6_K V projection, which share x).
template <class F>
__device__ __forceinline__ void stream_body_any(const Params &P, uint8_t *smem)
{
    if (P.ru == 4)
        stream_body<F, 4>(P, smem);
    else if (P.ru == 2)
        stream_body<F, 2>(P, smem);
    else
        stream_body<F, 1>(P, smem);
}
template <class FA, class FB>
__global__ void __launch_bounds__(kThreads, 1) stream_pair_kernel(const __grid_constant__ Params PA,
                                                                  const __grid_constant__ Params PB)
{
    extern __shared__ __align__(128) uint8_t smem[];
    if (static_cast<int>(blockIdx.x) < PA.ncta)
        stream_body_any<FA>(PA, smem);
    else
        stream_body_any<FB>(PB, smem);
}

// 0: plain launches. 1: launches carry the programmatic-stream-serialization
// attribute, so a kernel may start while the previous kernel of the stream is
// still draining; it then prefetches weights early and waits for that kernel
// only before it reads x or writes y. Only safe when the weight tensors are
// not produced by the kernel immediately upstream in the same stream.
inline int &pdl_mode()
{
    static int mode = 0;
    return mode;
}

template <class F, int RU>
inline void launch_one(Params &P, const Layout &L, int grid, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = P.pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, stream_kernel<F, RU>, P);
}

// The shared-memory opt-in is a per-device attribute of each kernel: done once per device, with that
// device current (cuda_kernels_init() does it up front so that it never happens during a capture).
template <class F>
inline void init_attrs()
{
    static bool done[kMaxDevices] = {false};
    const int dev = current_device();
    if (done[dev]) return;
    cudaFuncSetAttribute(stream_kernel<F, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(stream_kernel<F, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(stream_kernel<F, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    done[dev] = true;
}

// Host-side geometry. Segment pointers/rows, x, mode etc. are set by the caller; fills in the rest of P, the
// shared-memory layout, the grid (at most grid_cap CTAs when that is > 0) and the row unroll (force_ru > 0 fixes it).
// Returns false when there is nothing to launch (empty problem, or an error that has been recorded).
template <class F>
inline bool prepare(Params &P, const char *where, int grid_cap, int force_ru, Layout &L_out, int &grid_out, int &ru_out)
{
    if (P.n_cols <= 0) return false;
    if (P.n_cols > F::kMaxCols) {
        fprintf(stderr, "[mnemo_b200] %s: n_cols=%d exceeds the supported %d\n", where, P.n_cols, F::kMaxCols);
        set_status(MB200_ERR_UNSUPPORTED, where);
        return false;
    }
    if (P.norm_w && (P.mode == kMoeDown || P.n_cols > 4 * 3 * kQuantThreads)) {
        fprintf(stderr, "[mnemo_b200] %s: the fused RMSNorm covers one activation vector of at most %d columns\n", where,
                4 * 3 * kQuantThreads);
        set_status(MB200_ERR_UNSUPPORTED, where);
        return false;
    }
    const bool routed = (P.mode == kMoeGateUp || P.mode == kMoeDown);
    bool misaligned = false;
    if (routed) {
        const uintptr_t b = reinterpret_cast<uintptr_t>(P.ebase);
        misaligned = ((b + P.off_a) | P.estride) & (F::kBaseAlign - 1);
        if (P.mode == kMoeGateUp) misaligned = misaligned || ((b + P.off_b) & (F::kBaseAlign - 1));
        if (P.n_slots < 1 || P.n_slots > kMaxSlots || P.erows < 1) misaligned = true;
    } else {
        for (int i = 0; i < P.nseg; i++)
            if (reinterpret_cast<uintptr_t>(P.seg[i].w) & (F::kBaseAlign - 1)) misaligned = true;
    }
    if (misaligned) {
        fprintf(stderr, "[mnemo_b200] %s: a weight tensor is not %d-byte aligned (or bad slot count)\n", where,
                F::kBaseAlign);
        set_status(MB200_ERR_ARG, where);
        return false;
    }
    P.bpr = (P.n_cols + 255) / 256;
    const int row_bytes = P.bpr * F::kBlockBytes;

    // ---- column groups and the warp table ----
    int gw = 1;
    while (gw * 2 <= F::kG && P.bpr % (gw * 2) == 0) gw *= 2;
    int NG = P.bpr / gw;
    int grp_col0[kConsumers], grp_v[kConsumers], grp_rpp[kConsumers], grp_warps[kConsumers];
    if (NG <= kConsumers) {
        for (int g = 0; g < NG; g++) {
            grp_col0[g] = g * gw;
            grp_v[g] = gw;
            grp_rpp[g] = F::kG / gw;
        }
    } else {
        NG = (P.bpr + F::kG - 1) / F::kG;
        if (NG > kConsumers) {
            fprintf(stderr, "[mnemo_b200] %s: n_cols=%d needs more column groups than consumer warps\n", where, P.n_cols);
            set_status(MB200_ERR_UNSUPPORTED, where);
            return false;
        }
        for (int g = 0; g < NG; g++) {
            const int vv = (g == NG - 1) ? P.bpr - g * F::kG : F::kG;
            grp_col0[g] = g * F::kG;
            grp_v[g] = vv;
            grp_rpp[g] = (F::kG % vv == 0) ? F::kG / vv : 1;
        }
    }
    // warps per group in proportion to passes per row (1 / rpp): every group gets one, the rest go where the load is highest
    for (int g = 0; g < NG; g++) grp_warps[g] = 1;
    for (int w = NG; w < kConsumers; w++) {
        int arg = 0;
        for (int g = 1; g < NG; g++)  // load(g) = 1 / (rpp * warps); compare by cross-multiplying
            if (grp_rpp[arg] * grp_warps[arg] > grp_rpp[g] * grp_warps[g]) arg = g;
        grp_warps[arg]++;
    }
    int sweep1 = 0;  // rows one round of the slowest-covering group handles at RU = 1 (tiles are multiples of the largest)
    {
        int w = 0;
        for (int g = 0; g < NG; g++) {
            for (int i = 0; i < grp_warps[g]; i++, w++)
                P.warp_cfg[w] = (uint32_t)g | ((uint32_t)grp_col0[g] << 5) | ((uint32_t)grp_v[g] << 12) |
                                ((uint32_t)grp_rpp[g] << 16) | ((uint32_t)i << 20) | ((uint32_t)grp_warps[g] << 24);
            const int rows = grp_warps[g] * grp_rpp[g];
            sweep1 = rows > sweep1 ? rows : sweep1;
        }
    }
    P.n_groups = NG;

    // virtual rows
    int vrows = 0;
    if (P.mode == kMoeGateUp) {
        vrows = P.n_slots * P.erows;
    } else if (P.mode == kMoeDown) {
        vrows = P.erows;
    } else if (P.mode == kSwiGLU) {
        vrows = P.seg[0].rows;
        P.seg[0].start = 0;
        P.seg[1].start = 0;
    } else {
        for (int i = 0; i < P.nseg; i++) {
            P.seg[i].start = vrows;
            vrows += P.seg[i].rows > 0 ? P.seg[i].rows : 0;
        }
    }
    if (vrows <= 0) return false;
    P.vrows = vrows;
    const int sms = grid_cap > 0 ? grid_cap : device_sms();
    const int grid = vrows < sms ? vrows : sms;
    const int per_cta = (vrows + grid - 1) / grid;  // rows of the longest range
    const int mult = (P.mode == kSwiGLU || P.mode == kMoeGateUp) ? 2 : 1;  // stage rows per virtual row
    const int n_x = (P.mode == kMoeDown) ? P.n_slots : 1;

    // RU: the fewest pass-times to cover the longest range; ties go to the larger RU (more independent work per warp)
    int ru = 1, best = 1 << 30;
    for (int cand = 1; cand <= 4; cand *= 2) {
        const int rows = mult * per_cta;
        const int cost = ((rows + sweep1 * cand - 1) / (sweep1 * cand)) * cand;
        if (cost <= best) {
            best = cost;
            ru = cand;
        }
    }
    if (force_ru > 0) ru = force_ru;
    // tile: a whole number of sweeps near the target size, never more than the range
    const int sweep = sweep1 * ru;
    int target = F::kTileTargetBytes / row_bytes;  // stage rows
    if (target < 1) target = 1;
    int stage_rows = sweep * (target / sweep > 0 ? target / sweep : 1);
    if (stage_rows > mult * per_cta) stage_rows = mult * per_cta;
    if (mult == 2 && (stage_rows & 1)) stage_rows += 1;
    P.tile_rows = stage_rows / mult;
    if (P.tile_rows < 1) P.tile_rows = 1;
    if (P.mode == kMoeDown && P.tile_rows > 64) P.tile_rows = 64;  // the epilogue keeps two running sums per lane
    stage_rows = P.tile_rows * mult;

    // no more stages than the longest range has tiles: a small matvec then takes little shared memory and can
    // be resident beside another kernel (its copies start while the upstream kernel is still running)
    int n_tiles = (per_cta + P.tile_rows - 1) / P.tile_rows;
    if (P.mode == kMoeDown) n_tiles *= P.n_slots;
    else if (P.mode != kSwiGLU && P.mode != kMoeGateUp) n_tiles += P.nseg - 1;  // a range may cross segment ends
    int S = n_tiles < 2 ? 2 : (n_tiles > kMaxStages ? kMaxStages : n_tiles);
    Layout L = layout<F>(P.bpr, stage_rows, S, NG, n_x);
    while (S > 2 && L.total > 200 * 1024) {
        S--;
        L = layout<F>(P.bpr, stage_rows, S, NG, n_x);
    }
    while (L.total > 227 * 1024 && P.tile_rows > 1) {  // very wide rows: shrink the tile
        P.tile_rows = (P.tile_rows + 1) / 2;
        stage_rows = P.tile_rows * mult;
        L = layout<F>(P.bpr, stage_rows, S, NG, n_x);
    }
    if (L.total > 227 * 1024) {
        fprintf(stderr, "[mnemo_b200] %s: shape does not fit shared memory\n", where);
        set_status(MB200_ERR_UNSUPPORTED, where);
        return false;
    }
    P.stages = S;
    P.pdl = pdl_mode();
    P.err = device_error_word();
    P.cta0 = 0;
    P.ncta = grid;
    P.per_cta = P.vrows / grid;
    P.rem_cta = P.vrows % grid;
    P.ru = ru;
    L_out = L;
    grid_out = grid;
    ru_out = ru;
    return true;
}

template <class F>
inline void launch(Params &P, cudaStream_t stream, const char *where)
{
    init_attrs<F>();
    Layout L;
    int grid, ru;
    if (!prepare<F>(P, where, 0, 0, L, grid, ru)) return;
    if (ru == 4)
        launch_one<F, 4>(P, L, grid, stream);
    else if (ru == 2)
        launch_one<F, 2>(P, L, grid, stream);
    else
        launch_one<F, 1>(P, L, grid, stream);
    MB200_CHECK_LAUNCH(where);
}

// Two problems of block types FA and FB in one launch, the SMs divided between them in proportion to their
// cost; each half runs with the row unroll it would choose alone.
// Returns false (nothing launched) when a half is empty or invalid: the caller then issues single launches.
template <class FA, class FB>
inline bool launch_pair(Params &PA, Params &PB, cudaStream_t stream, const char *where)
{
    static bool done[kMaxDevices] = {false};
    const int dev = current_device();
    if (!done[dev]) {
        cudaFuncSetAttribute(stream_pair_kernel<FA, FB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        done[dev] = true;
    }
    auto bytes = [](const Params &P, int block_bytes) {
        double b = 0.0;
        for (int i = 0; i < P.nseg; i++) b += (double)(P.seg[i].rows > 0 ? P.seg[i].rows : 0) * ((P.n_cols + 255) / 256) * block_bytes;
        return b;
    };
    // cost, not bytes: a CTA's few hundred KB arrive faster than its warps get through them, and a type's dot
    // product costs kByteCost per byte (Q6_K about twice Q4_K: measured best split of the Q / K / V launch)
    const double ba = bytes(PA, FA::kBlockBytes) * FA::kByteCost, bb = bytes(PB, FB::kBlockBytes) * FB::kByteCost;
    const int sms = device_sms();
    int gb = static_cast<int>(sms * bb / (ba + bb) + 0.5);
    gb = gb < 1 ? 1 : (gb > sms - 1 ? sms - 1 : gb);
    Layout LA, LB;
    int ga = sms - gb, rua = 0, rub = 0;
    Params A2 = PA, B2 = PB;
    const bool ok = prepare<FA>(A2, where, ga, 0, LA, ga, rua) && prepare<FB>(B2, where, gb, 0, LB, gb, rub);
    if (!ok) return false;
    PA = A2;
    PB = B2;
    PB.cta0 = ga;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ga + gb);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = LA.total > LB.total ? LA.total : LB.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = PA.pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, stream_pair_kernel<FA, FB>, PA, PB);
    MB200_CHECK_LAUNCH(where);
    return true;
}

}  // namespace stream
}  // namespace mb200
