// Routed experts of one token in ONE launch: gate/up + SwiGLU of every routed
// expert, a device-wide barrier, then the down projections with the weighted
// sum and the residual add (reference sequence per expert:
// src/forward.c:1122-1142; kernels src/kernels.cu:196-330, 455-484).
//
// Why one kernel: at batch 1 the two phases move 57 MB and 41 MB -- 9 us and
// 7 us of HBM time -- so launch gaps, prologues and pipeline ramp-up of separate
// kernels cost as much as the streaming itself. Here every CTA walks ONE
// sequence of tiles (its gate/up tiles, then its down tiles) through one ring
// of shared-memory stages fed by 1-D bulk async copies. The issuer never waits
// for the barrier, so the down-projection weights stream in while the last
// gate/up tiles are consumed and while the CTAs meet.
//
// Roles per CTA (480 threads): warps 0-11 consume tiles (int8 dp4a dot
// products, see q4k_policy.cuh / q6k_policy.cuh) and leave per-column-group
// partial sums in shared memory. Warp 12 issues the weight copies. Warp 13 (the
// courier) does every slow device-wide step so that no consumer warp waits on
// global memory: barrier arrivals, the polls, and the bulk copies that bring
// finished activation vectors into shared memory. Warp 14 (the epilogue warp)
// finishes every tile once all consumers have stored their partial sums (SwiGLU
// and the act rows, or the running weighted sum over the expert slots in slot
// order -- deterministic, no atomics).
//
// The routed slots are handled in batches of two. Gate/up tiles are dealt to
// the CTAs in batch order, and each batch has its own device-wide barrier: an
// arrival counter in global memory that only ever grows (a launch knows its
// target from the value it reads at its start). The activations of a batch
// are therefore complete, copied into every SM and split into int8 levels
// (a share per consumer warp, at tile boundaries) while later tiles are still
// being streamed; only the last batch can make the down phase wait. The launch
// is cooperative (all CTAs co-resident) and every wait gives up after a bounded
// number of polls, setting the library's device error word instead of hanging.
//
// With the routing inside (mb200_moe_block) every CTA first computes a router
// row and all of them select the experts themselves; with a communicator
// (mb200_moe_block_push, the PUSH instantiation) the epilogue warp sends the
// finished rows to the other ranks and collects theirs: the block's all-reduce
// without a second kernel.
#include <cstdio>

#include "comm.cuh"
#include "q4k_policy.cuh"
#include "q6k_policy.cuh"
#ifdef MB200_TRACE
#define MB200_TOPK_STAMP(n) do { if (threadIdx.x == 0) MB200_STAMP(44 + (n)); } while (0)
#endif
#include "topk.cuh"

#ifdef MB200_TRACE
// Developer aid: entry / exit time of CTA 0's issuer and consumer warp 0 for the last 64 launches.
static __device__ long long g_launch_times[64][4];
static __device__ unsigned g_launch_ctr;
#endif

namespace mb200 {

int pdl_enabled();

namespace {

using stream::kConsumers;
using stream::Layout;

constexpr int kFusedMaxSlots = 8;
constexpr int kFusedMaxStages = 6;
constexpr int kFusedThreads = (kConsumers + 3) * 32;  // 12 consumer warps + tile issuer + courier + epilogue
constexpr int kSrcAlign = 128;                         // down-phase copies start on a 128-byte line
constexpr int kDownPieces = 1;                         // bulk copies per down tile (more made no difference)
constexpr int kBatchSlots = 2;                         // served slots per batch
constexpr int kFusedMaxBatches = kFusedMaxSlots / kBatchSlots;
constexpr int kFusedMaxTiles = 16;  // gate/up tiles per CTA (one lane of the issuer warp lists each)
constexpr int kCtrlBytes = 656;     // mbarriers, routing tables, running sums, tile list
constexpr int kFusedMaxCStages = 4;
constexpr int kXBase = 384;  // stream::layout<> puts the first staged vector at this offset of its base pointer

struct FusedParams {
    const uint8_t *ebase;
    size_t estride, off_gate, off_up, off_down;
    const int *ids;
    const float *wts;
    // routing inside the kernel (router_w != nullptr): logits = router_w x, then the reference's top-k + softmax;
    // the ids / weights are also written to ids_out / wts_out for the caller
    const float *router_w;
    float *logits;   // [n_experts] scratch in global memory
    int *ids_out;
    float *wts_out;
    int n_experts;
    const float *x;
    const float *residual;
    float *y;
    float *act;      // [n_slots][EFF] fp32, written in phase 1 and read back (through L2) in phase 2
    unsigned long long *sync;  // arrival counters of the batch barriers (kFusedMaxBatches, monotonic)
    int *err;
    int n_slots, expert_lo, expert_cnt;
    int H, EFF, bprB, bprC;
    int ngB, wpgB, TB;             // gate/up: column groups, warps per group, pair rows per tile (= 2 * wpgB)
    int tpe;                       // gate/up tiles per expert = ceil(EFF / TB)
    int ngC, wpgC, vC, rppC, TC;   // down: column groups, warps per group, blocks per row group, rows per pass, rows per tile
    int stages, stage_bytes;
    int off_xb, off_xc, xc_stride, off_part, part_pitch, off_stages;  // shared-memory offsets (bytes; part_pitch in floats)
    int off_raw, raw_bytes;        // two buffers for the fp32 activation vectors of one batch
    int c_stages, c_stage_bytes;   // the down phase re-cuts the ring into more, smaller stages
    int off_cpart;                 // partial-sum slots of the down stages
    int pdl;
    int grid;                      // CTAs of the launch = SMs of the device (one CTA per SM, all co-resident)
    double inv_grid;               // 1 / grid
    // RMSNorm of x folded in (x' = x * norm_w / sqrt(mean(x^2) + norm_eps)): the router and the gate/up products use x'
    const float *norm_w;
    float norm_eps;
    // Expert-sharded engines (push.world > 0): the block's all-reduce inside the kernel. The warp that finishes a row
    // stores this rank's partial value ((residual +) weighted sum over the slots served here) into every rank's
    // receive cells, and once the CTA's rows are out it collects the other ranks' values for the same rows and writes
    // y = their sum in rank order (CTA b owns the same rows on every rank).
    PushDesc push;
};

struct FTile {
    int phase;  // 0: gate/up pair rows, 1: down rows
    int batch;  // gate/up: which half of the served slots the tile belongs to
    int last;   // gate/up: the CTA's last tile of that batch
    int idx;    // gate/up: position in the CTA's tile list
    int j;      // position of the slot among the slots served here
    int slot;   // expert slot (index into ids / wts / act)
    int row0, rows;
};

// Device-wide barrier state: one 64-bit arrival counter per batch that only ever grows. Every
// launch adds exactly gridDim.x arrivals to a counter it uses, so between launches its value is a
// multiple of gridDim.x; a CTA that reads c at its start (when at most gridDim.x - 1 arrivals of its
// own launch can be in) knows the launch is complete at c - c % gridDim.x + gridDim.x.
// (The remainder comes from a multiplication by 1 / gridDim.x in double precision with a correction step, exact for
// counters below 2^52: a 64-bit division is a subroutine of a hundred instructions that every CTA would fetch cold
// at its very start, with all its other warps waiting for the result.)
__device__ __forceinline__ unsigned long long barrier_target(const unsigned long long *ctr, double inv_grid)
{
    unsigned long long c;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(ctr) : "memory");
    const unsigned long long G = gridDim.x;
    unsigned long long q = static_cast<unsigned long long>(__ull2double_rz(c) * inv_grid);  // inv_grid = 1 / gridDim.x
    long long r = static_cast<long long>(c - q * G);
    if (r < 0) {
        q--;
        r += static_cast<long long>(G);
    }
    if (r >= static_cast<long long>(G)) q++;
    return (q + 1) * G;
}
// Release-arrive: every store this thread has made or observed (through the block-scope handshakes
// between the warps that finished the CTA's tiles) is visible to whoever acquires the counter.
__device__ __forceinline__ void barrier_arrive(unsigned long long *ctr)
{
    asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(ctr) : "memory");
}
// The CTA's tiles in issue order. Every role runs the same walk.
//
// Gate/up work is split in whole tiles (TB pair rows of one expert), numbered through the served
// slots in order and dealt to the CTAs round robin. The served slots form batches of kBatchSlots,
// so every CTA does its share of batch 0 first, then of batch 1, ...: the activations of the early
// batches are complete device-wide long before the down phase needs them, and the barrier that
// guards a batch (plus the copy of its activations into every SM) hides behind the remaining work.
// The issuer warp lists the CTA's gate/up tiles once (build_tiles) and leaves the list in shared
// memory; the down tiles follow by simple arithmetic.
struct FWalk {
    int bi, n_b;
    int c_cur, c_end, e, n_act;
    const int2 *tiles;
    const int *act_list;
    __device__ __forceinline__ void init(const FusedParams &P, const int2 *list, int n_list, const int *slots,
                                         int n_active)
    {
        tiles = list;
        n_b = n_list;
        bi = 0;
        act_list = slots;
        n_act = n_active;
        c_cur = static_cast<int>(static_cast<unsigned>(P.H) * blockIdx.x / gridDim.x);
        c_end = static_cast<int>(static_cast<unsigned>(P.H) * (blockIdx.x + 1) / gridDim.x);
        if (n_active == 0) c_end = c_cur;
        e = 0;
    }
    __device__ __forceinline__ bool next(const FusedParams &P, FTile &t)
    {
        if (bi < n_b) {
            t.idx = bi;
            const int2 d = tiles[bi++];
            t.phase = 0;
            t.slot = d.x & 15;
            t.j = (d.x >> 4) & 15;
            t.batch = (d.x >> 8) & 15;
            t.last = (d.x >> 12) & 1;
            t.rows = d.x >> 16;
            t.row0 = d.y;
            return true;
        }
        if (c_cur < c_end) {  // the same rows for every served slot in turn, then the next rows
            t.phase = 1;
            t.batch = e / kBatchSlots;
            t.last = 0;
            t.j = e;
            t.slot = act_list[e];
            t.row0 = c_cur;
            t.rows = min(P.TC, c_end - c_cur);
            if (++e == n_act) {
                e = 0;
                c_cur += t.rows;
            }
            return true;
        }
        return false;
    }
};

// One warp: reads the routed ids and weights (one round trip), compacts the slots served here, and
// lists this CTA's gate/up tiles. Returns the number of served slots.
// (Arguments by value: see split_share.)
__device__ __noinline__ int build_tiles(int n_slots, int expert_lo, int expert_cnt, int EFF, int TB, int tpe, const int *ids,
                                        const float *wts, int lane, int *sid, float *swt, int *act_list, int2 *tiles,
                                        int *n_tiles_p)
{
    struct { int n_slots, expert_lo, expert_cnt, EFF, TB; } P = {n_slots, expert_lo, expert_cnt, EFF, TB};
    // tpe = ceil(EFF / TB), computed on the host
    int id = -1;
    float w = 0.0f;
    if (lane < P.n_slots) {
        // shared memory (in-kernel routing) or global memory written by the upstream kernel: a volatile load
        // is right for both (it cannot be served by a stale L1 line)
        id = *static_cast<const volatile int *>(ids + lane);
        w = *static_cast<const volatile float *>(wts + lane);
    }
    const bool here = lane < P.n_slots && id >= P.expert_lo && id - P.expert_lo < P.expert_cnt;  // empty slots have id < 0
    const unsigned m = __ballot_sync(0xffffffffu, here);
    const int n = __popc(m);
    if (lane < P.n_slots) {
        sid[lane] = here ? id - P.expert_lo : -1;
        swt[lane] = here ? w : 0.0f;
    }
    if (here) act_list[__popc(m & ((1u << lane) - 1u))] = lane;
    __syncwarp();
    // Tiles are numbered through the served slots in order (tpe per slot) and dealt to the CTAs round
    // robin: CTA b takes tiles b, b + G, b + 2G, ... -- in batch order, an equal share of every batch
    // (to within one tile), and lane i lists the i-th of them.
    const int T = n * tpe, G = gridDim.x;
    const int g = blockIdx.x + lane * G;
    const int total = (T > static_cast<int>(blockIdx.x)) ? (T - static_cast<int>(blockIdx.x) + G - 1) / G : 0;
    if (lane < total && lane < kFusedMaxTiles) {
        const int j = g / tpe;
        const int row0 = (g - j * tpe) * P.TB;
        const int rows = min(P.TB, P.EFF - row0);
        const int batch = j / kBatchSlots;
        const int gn = g + G;  // this CTA's next tile, if any
        const int last = (gn >= T || (gn / tpe) / kBatchSlots != batch) ? 1 : 0;
        tiles[lane] = make_int2(act_list[j] | (j << 4) | (batch << 8) | (last << 12) | (rows << 16), row0);
    }
    if (lane == 0) *n_tiles_p = min(total, kFusedMaxTiles);
    __syncwarp();
    return n;
}

template <class FD>
__device__ __forceinline__ const uint8_t *down_src(const FusedParams &P, const FTile &t, const int *sid)
{
    return P.ebase + (size_t)sid[t.slot] * P.estride + P.off_down + (size_t)t.row0 * ((size_t)P.bprC * FD::kBlockBytes);
}

template <class FD>
__device__ __forceinline__ void issue(const FusedParams &P, const FTile &t, uint8_t *stage, uint64_t *bar, const int *sid)
{
    if (t.phase == 0) {
        const size_t row_bytes = (size_t)P.bprB * kQ4KBlock;
        const uint8_t *e = P.ebase + (size_t)sid[t.slot] * P.estride + (size_t)t.row0 * row_bytes;
        const uint32_t half = t.rows * (uint32_t)row_bytes;
        mbar_expect_tx(bar, 2 * half);
        bulk_g2s(stage, e + P.off_gate, half, bar);
        bulk_g2s(stage + (size_t)P.TB * row_bytes, e + P.off_up, half, bar);  // up rows at a fixed offset: row slot TB + r
    } else {
        // The span enclosing the rows, from the 128-byte line the first row starts in to the 16-byte granule
        // the last one ends in (Q6_K rows are only 2-byte aligned). The bytes read before / after the rows
        // share a line / granule with a valid byte, hence lie inside a mapped page.
        const uintptr_t begin = reinterpret_cast<uintptr_t>(down_src<FD>(P, t, sid));
        const uintptr_t stop = begin + (size_t)t.rows * P.bprC * FD::kBlockBytes;
        const uintptr_t a0 = begin & ~static_cast<uintptr_t>(kSrcAlign - 1);
        const uint32_t bytes = static_cast<uint32_t>(((stop + 15) & ~static_cast<uintptr_t>(15)) - a0);
        mbar_expect_tx(bar, bytes);
        // several copies in flight per tile: one bulk copy alone does not reach the SM's share of the bandwidth
        const uint32_t piece = ((bytes / kDownPieces) + 127u) & ~127u;
        for (uint32_t o = 0; o < bytes; o += piece)
            bulk_g2s(stage + o, reinterpret_cast<const void *>(a0 + o), min(piece, bytes - o), bar);
    }
}

// One quad of columns of one activation vector -> the two int8 levels, scale and sums
// (same split as stream::quantize_x; the columns are all inside the matrix here).
template <class F>
__device__ __forceinline__ void split_store(const float4 t, int c0, int lane, int pitch, uint32_t *q1, uint32_t *q2,
                                            float *s1, float *xsum)
{
    const float v[4] = {t.x, t.y, t.z, t.w};
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

// Finishes a gate/up tile: sums the column groups, SwiGLU, and leaves the act rows in the CTA's outbox
// (shared memory). The courier stores them to global memory: a consumer warp never touches global
// memory, where every access queues behind the weight stream for microseconds.
__device__ __forceinline__ void finish_gate_up(const FusedParams &P, const FTile &t, const float *pt, float *outbox,
                                               int lane)
{
    if (lane < t.rows) {
        const int NG = P.ngB;
        float g = 0.0f, u = 0.0f;
        for (int c = 0; c < NG; c++) {
            g += pt[lane * NG + c];
            u += pt[(P.TB + lane) * NG + c];
        }
        outbox[t.idx * 32 + lane] = g / (1.0f + expf(-g)) * u;
    }
}

// Finishes a down tile: adds the slot's weighted rows to the running sums (slot order), and after the
// last served slot writes y.
template <bool PUSH>
__device__ __forceinline__ void finish_down(const FusedParams &P, const FTile &t, const float *pt, float *run,
                                            float w, int n_act, int lane, uint32_t push_tag, size_t push_off)
{
    const int NG = P.ngC;
    for (int r = lane; r < t.rows; r += 32) {
        float v = 0.0f;
        for (int c = 0; c < NG; c++) v += pt[r * NG + c];
        const float a = fmaf(w, v, t.j == 0 ? 0.0f : run[r]);
        if (t.j == n_act - 1) {
            const int row = t.row0 + r;
            if (PUSH) {
                const float mine = (P.residual ? __ldcg(P.residual + row) : 0.0f) + a;
#pragma unroll 1
                for (int p = 0; p < P.push.world; p++) st_cell(P.push.peer_cells[p] + push_off + row, mine, push_tag);
            } else {
                P.y[row] = __ldcg(P.residual ? P.residual + row : P.y + row) + a;
            }
        } else {
            run[r] = a;
        }
    }
}

// Push mode, one warp, after this CTA's rows [r0, r1) have been stored to every rank: collect every rank's value of
// those rows from the local cells (bounded wait), y = sum in rank order; then the launch ticket (the last CTA of
// the launch publishes the sequence number for the next collective). `zero_mine`: this CTA had nothing to add, its
// rows go out here first ((residual +) 0).
__device__ __forceinline__ void push_collect(const FusedParams &P, unsigned long long seq, bool zero_mine, int lane)
{
    const uint32_t tag = static_cast<uint32_t>(seq);
    const size_t par_off = (size_t)(seq & 1) * P.push.world * P.push.max_floats;
    const int r0 = static_cast<int>(static_cast<unsigned>(P.H) * blockIdx.x / gridDim.x);
    const int r1 = static_cast<int>(static_cast<unsigned>(P.H) * (blockIdx.x + 1) / gridDim.x);
    if (zero_mine)
        for (int row = r0 + lane; row < r1; row += 32) {
            const float mine = P.residual ? __ldcg(P.residual + row) : 0.0f;
#pragma unroll 1
            for (int p = 0; p < P.push.world; p++)
                st_cell(P.push.peer_cells[p] + par_off + (size_t)P.push.rank * P.push.max_floats + row, mine, tag);
        }
    long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool ok = true;
    for (int row = r0 + lane; row < r1 && ok; row += 32) {
        float v[kMaxWorld];
        if (!wait_cells(P.push.self_cells + par_off + row, P.push.max_floats, P.push.world, tag, v, t0)) {
            ok = false;
            break;
        }
        float acc = v[0];
#pragma unroll
        for (int q = 1; q < kMaxWorld; q++)  // fixed order: every rank computes the same bits
            if (q < P.push.world) acc += v[q];
        P.y[row] = acc;
    }
    if (!ok) atomicExch(P.err, MB200_ERR_TIMEOUT);
    __syncwarp();
    if (lane == 0) {
        __threadfence();
        if (atomicAdd(P.push.ticket, 1u) == gridDim.x - 1) {
            *P.push.ticket = 0;
            // after a timeout the sequence still advances, so that the ranks stay in step if the caller retries
            *P.push.seq = seq;
            __threadfence();
        }
    }
}

// ---- routing inside the kernel; out of line so that this run-once code (and the stack frame of the
// top-k's serial fallback) does not weigh on the registers and code layout of the tile loops ----

// Router logits (reference src/kernels.cu:859-880): expert row b, b + G, ... per CTA, by the twelve
// consumer warps; then the CTA arrives at the routing barrier.
// NORM: the RMSNorm of x is folded in (a version of its own: the loop body is half the size without it).
template <bool NORM>
__device__ __noinline__ void route_logits(const float *router_w, const float *x, const float *norm_w, float norm_eps,
                                          float *logits, unsigned long long *route_ctr, int H, int n_experts, float *rred)
{
    struct {
        const float *router_w, *x, *norm_w;
        float norm_eps;
        float *logits;
        int H, n_experts;
    } P = {router_w, x, norm_w, norm_eps, logits, H, n_experts};
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n4 = P.H >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(P.x);
    const float4 *n4w = NORM ? reinterpret_cast<const float4 *>(P.norm_w) : nullptr;  // fused RMSNorm: logit = scale * sum Wr (x w)
    for (int row = blockIdx.x; row < P.n_experts; row += gridDim.x) {
        const float4 *w4 = reinterpret_cast<const float4 *>(P.router_w + (size_t)row * P.H);
        float acc = 0.0f, ss = 0.0f;
        for (int i0 = tid; i0 < n4; i0 += kConsumers * 32 * 4) {
            float4 a[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * kConsumers * 32;
                a[u] = i < n4 ? __ldcs(w4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * kConsumers * 32;
                if (i < n4) {
                    float4 b = __ldcg(x4 + i);
                    if (NORM) {
                        const float4 g = __ldg(n4w + i);
                        ss = fmaf(b.x, b.x, fmaf(b.y, b.y, fmaf(b.z, b.z, fmaf(b.w, b.w, ss))));
                        b.x *= g.x; b.y *= g.y; b.z *= g.z; b.w *= g.w;
                    }
                    acc = fmaf(a[u].x, b.x, acc);
                    acc = fmaf(a[u].y, b.y, acc);
                    acc = fmaf(a[u].z, b.z, acc);
                    acc = fmaf(a[u].w, b.w, acc);
                }
            }
        }
        acc = warp_sum(acc);
        if (NORM) ss = warp_sum(ss);
        if (lane == 0) {
            rred[warp] = acc;
            rred[kConsumers + warp] = ss;
        }
        asm volatile("bar.sync 3, %0;" ::"n"(kConsumers * 32) : "memory");
        if (tid == 0) {
            float v = 0.0f, t = 0.0f;
            for (int w = 0; w < kConsumers; w++) v += rred[w];  // fixed order
            if (NORM) {
                for (int w = 0; w < kConsumers; w++) t += rred[kConsumers + w];
                v *= 1.0f / sqrtf(t / static_cast<float>(P.H) + P.norm_eps);
            }
            P.logits[row] = v;
        }
        asm volatile("bar.sync 3, %0;" ::"n"(kConsumers * 32) : "memory");
    }
    if (tid == 0) barrier_arrive(route_ctr);  // release: this thread stored the CTA's logits
    if (warp == 0) MB200_STAMP(3);
}

// Every CTA selects the experts itself, from the logits all CTAs have stored: warps 0-3. Returns
// false (on thread 0) if the routing barrier did not complete within the poll budget.
// The group top-k as a function of its own (one copy of the code: the warm-up pass below runs the very
// instructions the routing warps will run).
__device__ __noinline__ void route_topk(const float *scores, int *ids, float *wts, int n_experts, int k, TopkShared *sh,
                                        int n_warps, int bar_id, int warp0)
{
    // the small forms of the selection (see topk_softmax_group): this code is fetched cold at every launch
    if (k <= 8)  // (the shapes are checked on the host: n_experts <= 32 k, k <= 16)
        topk_softmax_group<false, 8, 2>(scores, ids, wts, n_experts, k, *sh, n_warps, bar_id, warp0);
    else
        topk_softmax_group<false, 16, 2>(scores, ids, wts, n_experts, k, *sh, n_warps, bar_id, warp0);
}

// Instruction-cache warm-up. The selection is a few thousand instructions of run-once code; fetched cold it
// takes 5-7 us during which nothing streams. The three service warps have nothing to do until the routing is
// done, so at kernel entry they run the same code on made-up scores (distinct values, hence the tie-free path
// the real logits take) with outputs in an idle part of the ring; when the routing warps get there, the
// instructions are in the SM's instruction cache.
__device__ __forceinline__ void route_warmup(const FusedParams &P, uint8_t *ring)
{
    const int lane = threadIdx.x & 31;
    uint8_t *base = ring + 64 * 1024;  // the routing warps use the first bytes of the ring
    float *scores = reinterpret_cast<float *>(base);
    int *ids = reinterpret_cast<int *>(base + 2048);
    float *wts = reinterpret_cast<float *>(base + 2048 + 64);
    TopkShared *sh = reinterpret_cast<TopkShared *>(base + 4096);
    const int warp = static_cast<int>(threadIdx.x >> 5) - kConsumers;
    for (int i = warp * 32 + lane; i < P.n_experts; i += 96)
        scores[i] = static_cast<float>((i * 37) % 509) * 0.01f - 2.0f;  // distinct for i < 509
    asm volatile("bar.sync 5, 96;" ::: "memory");
    route_topk(scores, ids, wts, P.n_experts, P.n_slots, sh, 3, 5, kConsumers);
    if (warp == 0) {  // the issuer's tile list from the made-up selection: same idea, its code is run-once too
        __syncwarp();
        int *scratch = reinterpret_cast<int *>(base + 3072);
        build_tiles(P.n_slots, P.expert_lo, P.expert_cnt, P.EFF, P.TB, P.tpe, ids, wts, lane, scratch,
                    reinterpret_cast<float *>(scratch + 16), scratch + 32, reinterpret_cast<int2 *>(scratch + 64), scratch + 48);
    }
}

__device__ __noinline__ bool route_select(const unsigned long long *route_ctr, const float *logits, int n_experts,
                                          int n_slots, int *ids_out, float *wts_out, unsigned long long tgt_route,
                                          int *rid, float *rwt, uint8_t *ring)
{
    struct {
        const float *logits;
        int n_experts, n_slots;
        int *ids_out;
        float *wts_out;
    } P = {logits, n_experts, n_slots, ids_out, wts_out};
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    bool ok = true;
    if (tid == 0) {
        ok = false;
        for (uint32_t i = 0; i < (1u << 19); i++) {
            unsigned long long c;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(route_ctr) : "memory");
            if (c >= tgt_route) {
                ok = true;
                break;
            }
            __nanosleep(40);
        }
    }
    topk_group_sync(2, 128);
    if (warp == 0) MB200_STAMP(4);
    TopkShared &tsh = *reinterpret_cast<TopkShared *>(ring);  // the ring is idle until the first tile is requested
    route_topk(P.logits, rid, rwt, P.n_experts, P.n_slots, &tsh,
               4, 2, 0);
    if (warp == 0) {
        MB200_STAMP(6);
        __syncwarp();
        if (blockIdx.x == 0 && lane < P.n_slots) {  // for the caller
            P.ids_out[lane] = rid[lane];
            P.wts_out[lane] = rwt[lane];
        }
    }
    return ok;
}

// A consumer warp's share of the activation staging of batch `batch` (whose fp32 vectors have landed in the raw
// buffer): columns [128 w, 128 w + 128) of each vector of the batch -> the int8 levels of the down phase.
// Everything it needs comes by value. A reference to the kernel's parameter block or to a struct of the caller
// would be read with ordinary loads (parameter space / local memory through a generic address), and any load that
// misses L1 queues behind the weight stream for microseconds.
template <class FD>
__device__ __noinline__ void split_share(const float *raw, uint8_t *xc0, int xc_stride, int EFF, int bprC, int batch,
                                         int n_act, uint64_t *rawempty_u, uint64_t *xready_b)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const Layout LC = stream::layout<FD>(bprC, 0, 0, 1, 1);
    const int pitch = FD::kSlotsPerBlock * bprC + 1;
    const int j0 = batch * kBatchSlots, jn = min(kBatchSlots, n_act - j0);
    for (int c0 = warp * 128 + lane * 4; c0 < EFF; c0 += kConsumers * 128) {
#pragma unroll
        for (int j = 0; j < kBatchSlots; j++) {  // unrolled: the two vectors' shuffle chains overlap
            if (j < jn) {
                const float4 v = *reinterpret_cast<const float4 *>(raw + (size_t)j * EFF + c0);
                uint8_t *xc = xc0 + (j0 + j) * xc_stride;
                split_store<FD>(v, c0, lane, pitch, reinterpret_cast<uint32_t *>(xc + LC.xq1),
                                reinterpret_cast<uint32_t *>(xc + LC.xq2), reinterpret_cast<float *>(xc + LC.xs1),
                                reinterpret_cast<float *>(xc + LC.xsum));
            }
        }
    }
    __syncwarp();
    if (lane == 0) {
        mbar_arrive(xready_b);    // release: this warp's share of the levels is visible to whoever waits
        mbar_arrive(rawempty_u);  // and it no longer reads the raw buffer
    }
}

template <class FD, bool PUSH>
__global__ void __launch_bounds__(kFusedThreads, 1) moe_fused_kernel(const __grid_constant__ FusedParams P)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kFusedMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 120);
    int *sid = reinterpret_cast<int *>(smem + 128);        // expert (relative to expert_lo) per slot, -1 = not served
    float *swt = reinterpret_cast<float *>(smem + 160);    // routing weight per slot
    int *act_list = reinterpret_cast<int *>(smem + 192);   // slots served here, in slot order
    int *n_act_p = reinterpret_cast<int *>(smem + 224);
    int *n_tiles_p = reinterpret_cast<int *>(smem + 228);
    int2 *tiles = reinterpret_cast<int2 *>(smem + 456);
    uint64_t *cfull = reinterpret_cast<uint64_t *>(smem + 592);    // [4] down-phase stages (re-cut ring)
    uint64_t *cempty = reinterpret_cast<uint64_t *>(smem + 624);   // [4]
    float *cpart = reinterpret_cast<float *>(smem + P.off_cpart);
    // routing inside the kernel: results and reduction scratch sit in the partial-sum region (idle until tiles flow)
    int *rid = reinterpret_cast<int *>(smem + P.off_part);
    float *rwt = reinterpret_cast<float *>(smem + P.off_part + 64);
    float *rred = reinterpret_cast<float *>(smem + P.off_part + 128);
    const int CS = P.c_stages;   // [kFusedMaxTiles] this CTA's gate/up tiles
    uint64_t *rawfull = reinterpret_cast<uint64_t *>(smem + 232);   // [2] a batch's fp32 activation vectors have landed
    uint64_t *rawempty = reinterpret_cast<uint64_t *>(smem + 248);  // [2] ... and every consumer warp has split its share
    uint64_t *bdone = reinterpret_cast<uint64_t *>(smem + 264);     // [4] this CTA has stored its act rows of batch k
    uint64_t *xready = reinterpret_cast<uint64_t *>(smem + 296);    // [4] the int8 levels of batch k are staged (all shares)
    float *run = reinterpret_cast<float *>(smem + 328);    // down: running sums of the tile's rows over the slots (<= 32)
    float *part = reinterpret_cast<float *>(smem + P.off_part);
    // act rows of the CTA's gate/up tiles (32 floats per tile) on their way to global memory. Lives where x was
    // staged: every consumer warp has its x in registers before the first tile can be finished.
    float *outbox = reinterpret_cast<float *>(smem + P.off_xb);
    uint8_t *stages = smem + P.off_stages;
    const int S = P.stages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (warp == 0) MB200_STAMP(0);
    if (P.router_w && warp >= kConsumers) route_warmup(P, stages);
#ifdef MB200_TRACE
    unsigned launch_no = 0;
    if (blockIdx.x == 0 && tid == 0) {
        launch_no = atomicAdd(&g_launch_ctr, 1u);
        long long t__;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));
        g_launch_times[launch_no & 63][0] = t__;
    }
#endif

    FWalk walk;

    if (warp == kConsumers) {
        // ---------------- issuer ----------------
        if (lane == 0) {
            *abort_flag = 0;
            for (int s = 0; s < S; s++) {
                mbar_init(&full[s], 2);  // the issuer's expect_tx arrival + "the stage's partial sums are free"
                mbar_init(&empty[s], kConsumers);
            }
            for (int u = 0; u < 2; u++) {
                mbar_init(&rawfull[u], 1);
                mbar_init(&rawempty[u], kConsumers);
            }
            for (int k = 0; k < kFusedMaxBatches; k++) {
                mbar_init(&bdone[k], 1);
                mbar_init(&xready[k], kConsumers);
            }
            for (int c = 0; c < kFusedMaxCStages; c++) {
                mbar_init(&cfull[c], 2);
                mbar_init(&cempty[c], kConsumers);
            }
            mbar_fence_init();
        }
        int n = 0;
        if (!P.router_w) {
            if (P.pdl) stream::grid_dep_wait();  // the routed ids come from the upstream kernel
            n = build_tiles(P.n_slots, P.expert_lo, P.expert_cnt, P.EFF, P.TB, P.tpe, P.ids, P.wts, lane, sid, swt, act_list, tiles, n_tiles_p);
            if (lane == 0) *n_act_p = n;
        }
        __syncthreads();
        if (P.router_w) {  // the consumer warps have routed: ids and weights are in shared memory
            n = build_tiles(P.n_slots, P.expert_lo, P.expert_cnt, P.EFF, P.TB, P.tpe, rid, rwt, lane, sid, swt, act_list, tiles, n_tiles_p);
            if (lane == 0) *n_act_p = n;
            __syncthreads();
        }
        if (*abort_flag) return;
        if (lane == 0) {
            if (P.pdl) stream::grid_dep_launch();
            const int n_b = *n_tiles_p;
            walk.init(P, tiles, n_b, act_list, n);
            for (int s = 0; s < S; s++) mbar_arrive(&full[s]);     // first use: no partial sums to drain yet
            for (int c = 0; c < CS; c++) mbar_arrive(&cfull[c]);
            // Gate/up tile i lives in stage i % S of the ring. The down phase cuts the same memory into CS
            // smaller stages (more copies in flight when the tiles are smaller): down tile m lives in down
            // stage m % CS, and the first tile of a down stage may only be requested once the gate/up stages
            // it overlaps have been read for the last time.
            FTile t;
            int ib = 0, ic = 0;
            int ist = 0, iuse = 0, ics = 0, icuse = 0;  // stage and number of earlier uses of it, both rings
            bool ok = true;
            MB200_STAMP(47);  // tile list ready, first copy about to be requested
            while (ok && walk.next(P, t)) {
                if (t.phase == 0) {
                    // (stage and use counters are kept by increments: a division by a run-time S is a subroutine)
                    const int st = ist;
                    if (ib >= S) ok = mbar_wait(&empty[st], (iuse - 1) & 1);
                    if (ok && !*abort_flag) issue<FD>(P, t, stages + (size_t)st * P.stage_bytes, &full[st], sid);
                    ib++;
                    if (++ist == S) {
                        ist = 0;
                        iuse++;
                    }
                } else {
                    const int c = ics;
                    if (ic < CS) {
                        const int lo = (c * P.c_stage_bytes) / P.stage_bytes;
                        const int hi = ((c + 1) * P.c_stage_bytes - 1) / P.stage_bytes;
                        for (int s2 = lo; s2 <= hi && ok; s2++) {
                            const int uses = n_b > s2 ? (n_b - s2 + S - 1) / S : 0;  // gate/up tiles that lived in stage s2
                            if (uses > 0) ok = mbar_wait(&empty[s2], (uses - 1) & 1);
                        }
                    } else {
                        ok = mbar_wait(&cempty[c], (icuse - 1) & 1);
                    }
                    if (ok && !*abort_flag) issue<FD>(P, t, stages + (size_t)c * P.c_stage_bytes, &cfull[c], sid);
                    if (ic < 4) MB200_STAMP(40 + ic);  // issue time of the first down tiles
                    ic++;
                    if (++ics == CS) {
                        ics = 0;
                        icuse++;
                    }
                }
                if (*abort_flag) break;
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(P.err, MB200_ERR_TIMEOUT);
            }
        }
        return;
    }

    if (warp == kConsumers + 1) {
        // ---------------- courier ----------------
        // One thread that does every slow device-wide step, so that no consumer warp ever waits on one:
        // it arrives at a batch's barrier once this CTA's rows of the batch are stored (the release
        // waits for those stores to be visible, which takes microseconds while weights stream in), and
        // once every CTA has arrived it pulls the batch's fp32 activation vectors into shared memory.
        unsigned long long tgt[kFusedMaxBatches];
#pragma unroll
        for (int b = 0; b < kFusedMaxBatches; b++) tgt[b] = barrier_target(P.sync + b, P.inv_grid);  // before this CTA can have arrived
        __syncthreads();
        if (P.router_w) __syncthreads();
        if (PUSH && *n_act_p == 0 && !*abort_flag) {
            // No routed expert lives on this rank: its share of the all-reduce is (residual +) 0. `out` may be the very
            // vector the CTAs have just read as x, so the rows are only written once every CTA is past its reads: the
            // first batch barrier (otherwise unused in such a launch) counts them.
            bool met = true;
            if (lane == 0) {
                barrier_arrive(P.sync + 0);
                met = false;
                for (uint32_t i = 0; i < (1u << 18); i++) {
                    unsigned long long c;
                    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(P.sync + 0) : "memory");
                    if (c >= tgt[0]) {
                        met = true;
                        break;
                    }
                    __nanosleep(200);
                }
                if (!met) atomicExch(P.err, MB200_ERR_TIMEOUT);
            }
            met = __shfl_sync(0xffffffffu, met, 0);
            if (P.pdl) stream::grid_dep_wait();  // the previous collective on this communicator has published its number
            if (met) push_collect(P, __ldcg(P.push.seq) + 1, true, lane);
            return;
        }
        if (lane != 0 || *abort_flag) return;
        const int n_act = *n_act_p;
        const int nb = (n_act + kBatchSlots - 1) / kBatchSlots;
        const uint32_t vec_bytes = static_cast<uint32_t>(P.EFF) * 4u;
        unsigned present = 0;  // batches this CTA has tiles in (the others it arrives at right away)
        {
            const int nt = *n_tiles_p;
            for (int i = 0; i < nt; i++) present |= 1u << ((tiles[i].x >> 8) & 15);
        }
        // Pull batch kc's activation vectors into shared memory once every CTA has arrived at its barrier.
        auto fetch = [&](int kc) -> bool {
            const int u = kc & 1;
            if (kc >= 2 && !mbar_wait(&rawempty[u], ((kc >> 1) - 1) & 1)) return false;  // consumers still split batch kc-2
            const unsigned long long target = kc == 0 ? tgt[0] : kc == 1 ? tgt[1] : kc == 2 ? tgt[2] : tgt[3];
            bool met = false;
            for (uint32_t i = 0; i < (1u << 18) && !*abort_flag; i++) {
                unsigned long long c;
                asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(P.sync + kc) : "memory");
                if (c >= target) {
                    met = true;
                    break;
                }
                __nanosleep(200);
            }
            if (!met) return false;
            MB200_STAMP(11 + kc);  // 11..14
            // the rows were stored through the generic proxy (by other SMs); the bulk copy reads through the async proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
            const int j0 = kc * kBatchSlots, jn = min(kBatchSlots, n_act - j0);
            uint8_t *dst = smem + P.off_raw + u * P.raw_bytes;
            mbar_expect_tx(&rawfull[u], jn * vec_bytes);
            for (int j = 0; j < jn; j++)
                bulk_g2s(dst + (size_t)j * vec_bytes, P.act + (size_t)act_list[j0 + j] * P.EFF, vec_bytes, &rawfull[u]);
            return true;
        };
        // Batch k: wait (on a shared-memory barrier, no spinning) until this CTA's rows are in the outbox,
        // store them, arrive; then fetch batch k-1, whose barrier every CTA has passed by now.
        bool ok = true;
        for (int k = 0; k < nb && ok; k++) {
            if (present & (1u << k)) {
                ok = mbar_wait(&bdone[k], 0);
                if (!ok) break;
                const int nt = *n_tiles_p;
                for (int i = 0; i < nt; i++) {  // this CTA's act rows of the batch: outbox -> global
                    const int2 d = tiles[i];
                    if (((d.x >> 8) & 15) != k) continue;
                    float *dst = P.act + (size_t)(d.x & 15) * P.EFF + d.y;
                    const int rows = d.x >> 16;
                    for (int r = 0; r < rows; r++) dst[r] = outbox[i * 32 + r];
                }
            }
            barrier_arrive(P.sync + k);
            MB200_STAMP(7 + k);  // 7..10
            if (k > 0) ok = fetch(k - 1);
        }
        if (ok && nb > 0) ok = fetch(nb - 1);
        if (!ok) {
            *abort_flag = 1;
            atomicExch(P.err, MB200_ERR_TIMEOUT);
        }
        return;
    }

    if (warp == kConsumers + 2) {
        // ---------------- epilogue warp ----------------
        // Finishes every tile once all twelve consumer warps have stored their partial sums. A warp of its
        // own, so that its latency (a serial chain of shared-memory reads, expf, a division) never delays a
        // consumer: when consumers took turns at this, each finisher came late to its next tile and the
        // delay was handed from tile to tile.
        __syncthreads();
        if (P.router_w) __syncthreads();
        if (*abort_flag) return;
        const int n_act = *n_act_p;
        if (n_act == 0) return;  // (push mode: the courier warp sends and collects this CTA's rows)
        unsigned long long pseq = 0;
        if (PUSH) {
            if (P.pdl) stream::grid_dep_wait();  // the previous collective on this communicator has published its number
            pseq = __ldcg(P.push.seq) + 1;       // the same on every CTA: written only by the last CTA of a launch
        }
        const size_t push_off = ((size_t)(pseq & 1) * P.push.world + P.push.rank) * P.push.max_floats;
        walk.init(P, tiles, *n_tiles_p, act_list, n_act);
        FTile t;
        int ib = 0, ic = 0;
        int est = 0, euse = 0, ecs = 0, ecuse = 0;  // stage and number of earlier uses of it, both rings
        while (walk.next(P, t)) {
            if (t.phase == 0) {
                const int st = est;
                if (!mbar_wait(&empty[st], euse & 1)) *abort_flag = 1;
                if (*abort_flag) break;
                finish_gate_up(P, t, part + st * P.part_pitch, outbox, lane);
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full[st]);  // the stage's partial sums may be rewritten
                    // every act row this CTA owes to the batch is in the outbox: tell the courier
                    if (t.last) mbar_arrive(&bdone[t.batch]);
                }
                ib++;
                if (++est == S) {
                    est = 0;
                    euse++;
                }
            } else {
                const int c = ecs;
                if (!mbar_wait(&cempty[c], ecuse & 1)) *abort_flag = 1;
                if (*abort_flag) break;
                if (ic < 8) MB200_STAMP(16 + ic);  // all consumers done with down tile ic
                finish_down<PUSH>(P, t, cpart + c * P.part_pitch, run, swt[t.slot], n_act, lane, static_cast<uint32_t>(pseq), push_off);
                __syncwarp();
                if (lane == 0) mbar_arrive(&cfull[c]);
                ic++;
                if (++ecs == CS) {
                    ecs = 0;
                    ecuse++;
                }
            }
        }
        if (*abort_flag && lane == 0) atomicExch(P.err, MB200_ERR_TIMEOUT);
        if (PUSH && !*abort_flag) push_collect(P, pseq, false, lane);
        return;
    }

    // ---------------- consumer warps ----------------
    unsigned long long tgt_route = 0;
    if (P.router_w && tid == 0) tgt_route = barrier_target(P.sync + kFusedMaxBatches, P.inv_grid);  // before this CTA arrives
    if (P.pdl) stream::grid_dep_wait();  // x is produced upstream; act / y may still be in use there
    if (P.router_w) {
        if (P.norm_w)
            route_logits<true>(P.router_w, P.x, P.norm_w, P.norm_eps, P.logits, P.sync + kFusedMaxBatches, P.H, P.n_experts, rred);
        else
            route_logits<false>(P.router_w, P.x, P.norm_w, P.norm_eps, P.logits, P.sync + kFusedMaxBatches, P.H, P.n_experts, rred);
    }
    const Layout LB = stream::layout<Q4>(P.bprB, 0, 0, 1, 1);
    const Layout LC = stream::layout<FD>(P.bprC, 0, 0, 1, 1);
    {
        uint8_t *xb = smem + P.off_xb - kXBase;
        stream::quantize_x<Q4, 3>(P.x, P.H, P.bprB, reinterpret_cast<uint32_t *>(xb + LB.xq1),
                                  reinterpret_cast<uint32_t *>(xb + LB.xq2), reinterpret_cast<float *>(xb + LB.xs1),
                                  reinterpret_cast<float *>(xb + LB.xsum), P.norm_w, P.norm_eps, rred + 2 * kConsumers);
    }
    if (warp == 0) MB200_STAMP(1);
    bool routed_ok = true;
    if (P.router_w && warp < 4) routed_ok = route_select(P.sync + kFusedMaxBatches, P.logits, P.n_experts, P.n_slots, P.ids_out, P.wts_out,
                                                              tgt_route, rid, rwt, stages);
    __syncthreads();  // x is staged, barriers are initialised, the served slots are known (or the routing is done)
    if (P.router_w) {
        if (tid == 0 && !routed_ok) {
            *abort_flag = 1;
            atomicExch(P.err, MB200_ERR_TIMEOUT);
        }
        __syncthreads();  // the issuer warp has listed the tiles
    }
    if (*abort_flag) return;
    const int n_act = *n_act_p;
    if (n_act == 0) {
        // no routed expert is served here: the block reduces to the residual (if this call carries one)
        if (PUSH) {
            // (the courier warp sends and collects this CTA's rows, once every CTA has read x: out may be x)
        } else if (warp == 0 && P.residual) {
            const int r0 = static_cast<int>(static_cast<unsigned>(P.H) * blockIdx.x / gridDim.x);
            const int r1 = static_cast<int>(static_cast<unsigned>(P.H) * (blockIdx.x + 1) / gridDim.x);
            for (int r = r0 + lane; r < r1; r += 32) P.y[r] = __ldcg(P.residual + r);
        }
        return;
    }
    walk.init(P, tiles, *n_tiles_p, act_list, n_act);
    const int nb = (n_act + kBatchSlots - 1) / kBatchSlots;  // one device-wide barrier and one staging step each

    const int q = lane >> 2, sub = lane & 3;
    FTile t, nt;
    int s = 0, ph = 0;
    bool have = walk.next(P, t);

    // Activation staging, spread over the consumer warps and over time: whenever a batch's fp32 vectors
    // have landed in shared memory (courier), a warp that passes a tile boundary splits its share of
    // them -- columns [128 w, 128 w + 128) of each vector -- into the int8 levels of the down phase.
    // By the time the batch's first down tile comes up all twelve shares are normally long done.
    int n_q = 0;  // batches this warp has done its share of
    // The test is inline (one mbarrier probe per tile); the split itself is a call, so that the two hot loops
    // below stay small (instruction fetch is what they stall on most).
    auto stage_share = [&](bool blocking) {
        while (n_q < nb) {
            const int u = n_q & 1, par = (n_q >> 1) & 1;
            if (blocking) {
                if (!mbar_wait(&rawfull[u], par)) {
                    *abort_flag = 1;
                    return;
                }
            } else if (!mbar_test_wait(&rawfull[u], par)) {
                return;
            }
            split_share<FD>(reinterpret_cast<const float *>(smem + P.off_raw + u * P.raw_bytes), smem + P.off_xc - kXBase,
                            P.xc_stride, P.EFF, P.bprC, n_q, n_act, &rawempty[u], &xready[n_q]);
            n_q++;
            if (blocking) return;
        }
    };

    // ---- gate/up: warp i of column group g takes gate rows 2i, 2i+1 and up rows 2i, 2i+1 of every tile ----
    {
        const int gB = warp / P.wpgB, iB = warp % P.wpgB;
        const int colB = gB * 8 + q;
        Q4::XRegs xr;
        Q4::load_xregs(xr, smem + P.off_xb - kXBase, LB, P.bprB, colB, sub, true);
        // x lives in registers from here on; its staging area is reused (outbox, down-phase partial sums)
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");
        const uint32_t row_bytes = P.bprB * kQ4KBlock;
        const uint32_t lane_off = colB * kQ4KBlock;
        const uint32_t off_g = 2 * iB * row_bytes + lane_off, off_u = (P.TB + 2 * iB) * row_bytes + lane_off;
        int k = 0;
        while (have && t.phase == 0) {
            stage_share(false);
            const bool hn = walk.next(P, nt);
            if (!mbar_wait(&full[s], ph)) *abort_flag = 1;
            if (warp == 0 && k == 0) MB200_STAMP(15);  // first gate/up tile has landed
            k++;
            const uint8_t *st = stages + (size_t)s * P.stage_bytes;
            float acc[4];
            // rows beyond t.rows hold stale bytes: their sums are computed and never read
            acc[0] = Q4::block_dot(st + off_g, sub, xr);
            acc[1] = Q4::block_dot(st + off_g + row_bytes, sub, xr);
            acc[2] = Q4::block_dot(st + off_u, sub, xr);
            acc[3] = Q4::block_dot(st + off_u + row_bytes, sub, xr);
            int which;
            const float sum = stream::packed_sum<4, true>(acc, 32, lane, which);
            float *pt = part + s * P.part_pitch;
            if ((lane & 7) == 0) pt[((which & 2 ? P.TB : 0) + 2 * iB + (which & 1)) * P.ngB + gB] = sum;
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);  // partial sums stored, the stage's weights no longer read
            if (*abort_flag) break;
            if (++s == S) {
                s = 0;
                ph ^= 1;
            }
            have = hn;
            t = nt;
        }
    }
    if (warp == 0) MB200_STAMP(2);

    int n_staged = 0;

    // ---- down: warp i of column group g takes rows (2i + u) * rpp + roff, u = 0, 1 ----
    {
        const int gC = warp / P.wpgC, iC = warp % P.wpgC;
        const int v = P.vC, rpp = P.rppC;
        const int colC = gC * v + (q % v), roff = q / v;
        const int W = 4 * v;  // lanes that share a row
        const uint32_t row_bytes = P.bprC * FD::kBlockBytes;
        const int ra = (2 * iC) * rpp + roff, rb = (2 * iC + 1) * rpp + roff;
        typename FD::XRegs xr;
        int cur_j = -1;
        int k = 0;
        int cs = 0, cph = 0;  // down-phase stage and parity (the ring re-cut into CS stages)
        while (have) {
            stage_share(false);
            if (n_staged < nb && t.j == n_staged * kBatchSlots) {  // first down tile of a batch: are its levels staged?
                if (warp == 0) MB200_STAMP(32 + 2 * n_staged);
                while (n_q <= n_staged && !*abort_flag) stage_share(true);  // this warp's own share first
                if (!*abort_flag && !mbar_wait(&xready[n_staged], 0)) *abort_flag = 1;
                if (warp == 0) MB200_STAMP(33 + 2 * n_staged);
                n_staged++;
            }
            if (*abort_flag) break;
            if (t.j != cur_j) {
                cur_j = t.j;
                FD::load_xregs(xr, smem + P.off_xc + cur_j * P.xc_stride - kXBase, LC, P.bprC, colC, sub, true);
            }
            uint32_t skew = 0;
            if (FD::kBlockBytes % kSrcAlign != 0)
                skew = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(down_src<FD>(P, t, sid)) & (kSrcAlign - 1));
            const bool hn = walk.next(P, nt);
            if (!mbar_wait(&cfull[cs], cph)) *abort_flag = 1;
            if (warp == 0 && k < 8) MB200_STAMP(24 + k);
            k++;
            const uint8_t *base = stages + (size_t)cs * P.c_stage_bytes + skew + colC * FD::kBlockBytes;
            float acc[2];
            acc[0] = FD::block_dot(base + min(ra, t.rows - 1) * row_bytes, sub, xr);
            acc[1] = FD::block_dot(base + min(rb, t.rows - 1) * row_bytes, sub, xr);
            int which;
            float sum;
            if (W == 32)
                sum = stream::packed_sum<2, true>(acc, 32, lane, which);
            else
                sum = stream::packed_sum<2, false>(acc, W, lane, which);
            const int row = which ? rb : ra;
            float *pt = cpart + cs * P.part_pitch;
            if ((lane & (W / 2 - 1)) == 0 && row < t.rows) pt[row * P.ngC + gC] = sum;
            __syncwarp();
            if (lane == 0) mbar_arrive(&cempty[cs]);
            if (*abort_flag) break;
            if (++cs == CS) {
                cs = 0;
                cph ^= 1;
            }
            have = hn;
            t = nt;
        }
    }
    if (*abort_flag && lane == 0) atomicExch(P.err, MB200_ERR_TIMEOUT);
    if (warp == 0) MB200_STAMP(5);
#ifdef MB200_TRACE
    if (blockIdx.x == 0 && tid == 0) {
        long long t__;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));
        g_launch_times[launch_no & 63][1] = t__;
    }
#endif
}

int g_fused_mode = 2;          // see mb200_set_fused
int g_fused_pdl_ok = 1;        // cleared if the driver refuses cooperative + programmatic serialization together

// Shared-memory opt-in of the kernel, once per device (a per-device attribute).
template <class FD, bool PUSH>
bool fused_attr()
{
    static bool done[kMaxDevices] = {false};
    const int dev = current_device();
    if (done[dev]) return true;
    if (cudaFuncSetAttribute(moe_fused_kernel<FD, PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
        cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    done[dev] = true;
    return true;
}

// PUSH: the instantiation with the all-reduce over the ranks in its epilogue (a kernel of its own, so that the
// single-device kernel's instruction layout is what it was without it).
template <class FD, bool PUSH>
int launch_fused_as(FusedParams &P, int smem_bytes, cudaStream_t stream)
{
    if (!fused_attr<FD, PUSH>()) return MB200_ERR_LAUNCH;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(P.grid);
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;  // the CTAs meet at a device-wide barrier: all must be resident
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    P.pdl = (pdl_enabled() && g_fused_pdl_ok) ? 1 : 0;
    cfg.numAttrs = P.pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, moe_fused_kernel<FD, PUSH>, P);
    if (e != cudaSuccess && P.pdl) {
        cudaGetLastError();
        g_fused_pdl_ok = 0;
        P.pdl = 0;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, moe_fused_kernel<FD, PUSH>, P);
    }
    if (e != cudaSuccess) {
        fprintf(stderr, "[mnemo_b200] fused expert kernel launch failed: %s\n", cudaGetErrorString(e));
        cudaGetLastError();
        return MB200_ERR_LAUNCH;
    }
    return MB200_OK;
}
template <class FD>
int launch_fused(FusedParams &P, int smem_bytes, cudaStream_t stream)
{
    return P.push.world > 0 ? launch_fused_as<FD, true>(P, smem_bytes, stream) : launch_fused_as<FD, false>(P, smem_bytes, stream);
}

}  // namespace

// Geometry of the fused kernel for a shape; returns false when the shape is outside what it covers
// (the caller then uses the separate gate/up and down kernels).
static bool fused_plan(FusedParams &P, int &smem_bytes)
{
    const int H = P.H, EFF = P.EFF;
    if (H % 256 || EFF % 256 || P.n_slots < 1 || P.n_slots > kFusedMaxSlots) return false;
    if (static_cast<unsigned long long>(H) * (P.grid + 1) >= (1ull << 32)) return false;  // row ranges in 32-bit arithmetic
    P.bprB = H / 256;
    P.bprC = EFF / 256;
    if (P.bprB % 8) return false;
    P.ngB = P.bprB / 8;
    if (P.ngB > kConsumers || kConsumers % P.ngB) return false;
    P.wpgB = kConsumers / P.ngB;
    P.TB = 2 * P.wpgB;
    P.tpe = (EFF + P.TB - 1) / P.TB;
    {   // the issuer warp lists the CTA's gate/up tiles with one lane per tile
        const int tpe = P.tpe;
        if ((P.n_slots * tpe + P.grid - 1) / P.grid + kFusedMaxBatches > kFusedMaxTiles) return false;
    }
    int v = 1;
    while (v * 2 <= 8 && P.bprC % (v * 2) == 0) v *= 2;
    // one column per lane group (three blocks per down row: the 30B expert shape) works but does not pay: with
    // experts that small the block is faster as router kernel + two stream kernels (3.37 vs 3.50 ms per token)
    if (v < 2) return false;
    P.vC = v;
    P.rppC = 8 / v;
    P.ngC = P.bprC / v;
    if (P.ngC > kConsumers || kConsumers % P.ngC) return false;
    P.wpgC = kConsumers / P.ngC;
    P.TC = P.wpgC * P.rppC * 2;
    if (P.TC > 32) P.TC = 32;  // one running sum per lane of the finishing warp
    return true;
}

template <class FD>
static bool fused_layout(FusedParams &P, int &smem_bytes)
{
    const int per_cta = (P.H + P.grid - 1) / P.grid;
    const int c_rows = per_cta < P.TC ? per_cta : P.TC;
    const int tileB = 2 * P.TB * P.bprB * kQ4KBlock;
    const int tileC = c_rows * P.bprC * FD::kBlockBytes + kSrcAlign + 32;  // + alignment skew, word over-read
    P.stage_bytes = ((tileB > tileC ? tileB : tileC) + 127) & ~127;
    const Layout LB = stream::layout<Q4>(P.bprB, 0, 0, 1, 1);
    const Layout LC = stream::layout<FD>(P.bprC, 0, 0, 1, 1);
    int o = kCtrlBytes;
    P.off_xb = o;
    o += LB.x_stride;
    P.off_xc = o;
    P.xc_stride = LC.x_stride;
    o += P.n_slots * LC.x_stride;
    const int pB = 2 * P.TB * P.ngB, pC = P.TC * P.ngC;
    P.part_pitch = pB > pC ? pB : pC;
    P.off_part = o;
    P.raw_bytes = kBatchSlots * P.EFF * 4;
    // x's staging area is reused once x is in registers: outbox (kFusedMaxTiles x 32 floats), then the
    // partial-sum slots of the down stages
    P.off_cpart = P.off_xb + kFusedMaxTiles * 32 * 4;
    if (kFusedMaxTiles * 32 * 4 + kFusedMaxCStages * P.part_pitch * 4 > LB.x_stride) return false;
    P.c_stage_bytes = (tileC + 127) & ~127;
    for (int S = kFusedMaxStages; S >= 3; S--) {
        int t = o + S * P.part_pitch * 4;
        t = (t + 127) & ~127;
        if (t + S * P.stage_bytes + 2 * P.raw_bytes <= 227 * 1024) {
            P.stages = S;
            P.off_stages = t;
            P.off_raw = t + S * P.stage_bytes;
            smem_bytes = P.off_raw + 2 * P.raw_bytes;
            P.c_stages = (S * P.stage_bytes) / P.c_stage_bytes;
            if (P.c_stages > kFusedMaxCStages) P.c_stages = kFusedMaxCStages;
            return true;
        }
    }
    return false;
}

void moe_fused_init()
{
    fused_attr<Q6, false>();
    fused_attr<Q4, false>();
    fused_attr<Q6, true>();
    fused_attr<Q4, true>();
}
void moe_fused_set_mode(int mode) { g_fused_mode = mode; }
int moe_fused_mode() { return g_fused_mode; }

// Returns MB200_OK after a launch, MB200_ERR_UNSUPPORTED when the shape is not covered (nothing launched).
// With router_w != nullptr the kernel routes itself (logits into `logits`, ids / weights also to ids_out /
// wts_out); otherwise it reads the routed ids / weights from `ids` / `wts`.
int moe_fused(const void *experts, size_t stride, size_t gate_off, size_t up_off, size_t down_off, int down_type,
              const int *ids, const float *wts, int n_slots, int expert_lo, int expert_cnt, const float *x, float *act,
              const float *residual, float *y, int H, int EFF, unsigned long long *sync, cudaStream_t stream,
              const float *router_w, int n_experts, float *logits, int *ids_out, float *wts_out, const float *norm_w,
              float norm_eps, const PushDesc *push)
{
    FusedParams P{};
    if (push) {  // the all-reduce over the ranks inside the kernel: only with the routing inside as well
        if (!router_w || push->world < 1 || push->world > kMaxWorld || static_cast<unsigned long long>(H) > push->max_floats)
            return MB200_ERR_UNSUPPORTED;
        P.push = *push;
    }
    if (norm_w && (H > 4 * 3 * stream::kQuantThreads || (reinterpret_cast<uintptr_t>(norm_w) & 15))) return MB200_ERR_UNSUPPORTED;
    P.norm_w = norm_w;
    P.norm_eps = norm_eps;
    if (router_w) {
        // the group top-k covers n_experts <= 32 * k and <= 512; 16-byte loads of the router rows
        if (n_experts < 1 || n_experts > 512 || n_experts > 32 * n_slots || n_slots > 16 || !logits || !ids_out || !wts_out)
            return MB200_ERR_UNSUPPORTED;
        if ((reinterpret_cast<uintptr_t>(router_w) & 15) || (H & 3)) return MB200_ERR_UNSUPPORTED;
        P.router_w = router_w;
        P.n_experts = n_experts;
        P.logits = logits;
        P.ids_out = ids_out;
        P.wts_out = wts_out;
    }
    P.ebase = static_cast<const uint8_t *>(experts);
    P.estride = stride;
    P.off_gate = gate_off;
    P.off_up = up_off;
    P.off_down = down_off;
    P.ids = ids;
    P.wts = wts;
    P.x = x;
    P.residual = residual;
    P.y = y;
    P.act = act;
    P.sync = sync;
    P.err = device_error_word();
    P.n_slots = n_slots;
    P.expert_lo = expert_lo;
    P.expert_cnt = expert_cnt;
    P.H = H;
    P.EFF = EFF;
    P.grid = device_sms();
    P.inv_grid = 1.0 / static_cast<double>(P.grid);
    int smem_bytes = 0;
    if (!fused_plan(P, smem_bytes)) return MB200_ERR_UNSUPPORTED;
    const uintptr_t b = reinterpret_cast<uintptr_t>(experts);
    if (((b + gate_off) | (b + up_off) | stride) & 15) return MB200_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(act)) & 15) return MB200_ERR_UNSUPPORTED;
    if (down_type == 14) {
        if ((b + down_off) & 1) return MB200_ERR_UNSUPPORTED;
        if (!fused_layout<Q6>(P, smem_bytes)) return MB200_ERR_UNSUPPORTED;
        return launch_fused<Q6>(P, smem_bytes, stream);
    }
    if (down_type == 12) {
        if ((b + down_off) & 15) return MB200_ERR_UNSUPPORTED;
        if (!fused_layout<Q4>(P, smem_bytes)) return MB200_ERR_UNSUPPORTED;
        return launch_fused<Q4>(P, smem_bytes, stream);
    }
    return MB200_ERR_UNSUPPORTED;
}

}  // namespace mb200

#ifdef MB200_TRACE
extern "C" void mb200_trace_read_launches(void *dst)
{
    cudaMemcpyFromSymbol(dst, g_launch_times, sizeof(long long) * 64 * 4, 0, cudaMemcpyDeviceToDevice);
}
extern "C" void mb200_trace_read_fused(void *dst)
{
    cudaMemcpyFromSymbol(dst, mb200::stream::g_trace, sizeof(long long) * mb200::kSMs * 2 * 48, 0,
                         cudaMemcpyDeviceToDevice);
}
#endif
