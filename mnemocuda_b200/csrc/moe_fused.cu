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
// Roles per CTA (416 threads): warps 0-11 consume tiles (int8 dp4a dot
// products, see q4k_policy.cuh / q6k_policy.cuh) and leave per-column-group
// partial sums in shared memory; the warp that stores the last partial sum of
// a tile finishes it (SwiGLU and the act store, or the running weighted sum
// over the expert slots in slot order -- deterministic, no atomics). Warp 12
// issues the copies. The warp that finishes the CTA's last gate/up tile
// arrives at the device-wide barrier.
//
// The device-wide barrier: an arrival counter and a generation word in global
// memory (zero before the first use, left ready for the next launch). The last
// CTA to arrive clears the counter and bumps the generation; consumer warps
// poll the generation with a bounded loop. The launch is cooperative (all
// CTAs co-resident) and every wait gives up after a bounded number of polls,
// setting the library's device error word instead of hanging.
#include <cstdio>

#include "q4k_policy.cuh"
#include "q6k_policy.cuh"

namespace mb200 {

int pdl_enabled();

namespace {

using stream::kConsumers;
using stream::Layout;

constexpr int kFusedMaxSlots = 8;
constexpr int kFusedMaxStages = 6;
constexpr int kFusedThreads = (kConsumers + 1) * 32;  // 12 consumer warps + the issuer warp
constexpr int kXBase = 384;  // stream::layout<> puts the first staged vector at this offset of its base pointer

struct FusedParams {
    const uint8_t *ebase;
    size_t estride, off_gate, off_up, off_down;
    const int *ids;
    const float *wts;
    const float *x;
    const float *residual;
    float *y;
    float *act;      // [n_slots][EFF] fp32, written in phase 1 and read back (through L2) in phase 2
    unsigned long long *sync;  // arrival counters of the two batch barriers (monotonic)
    int *err;
    int n_slots, expert_lo, expert_cnt;
    int H, EFF, bprB, bprC;
    int ngB, wpgB, TB;             // gate/up: column groups, warps per group, pair rows per tile (= 2 * wpgB)
    int ngC, wpgC, vC, rppC, TC;   // down: column groups, warps per group, blocks per row group, rows per pass, rows per tile
    int stages, stage_bytes;
    int off_xb, off_xc, xc_stride, off_part, part_pitch, off_stages;  // shared-memory offsets (bytes; part_pitch in floats)
    int pdl;
};

struct FTile {
    int phase;  // 0: gate/up pair rows, 1: down rows
    int batch;  // gate/up: which half of the served slots the tile belongs to
    int last;   // gate/up: the CTA's last tile of that batch
    int j;      // position of the slot among the slots served here
    int slot;   // expert slot (index into ids / wts / act)
    int row0, rows;
};

// The CTA's tiles in issue order. Every role runs the same walk.
//
// Gate/up work is split in whole tiles (TB pair rows of one expert). The served slots form two
// batches (first half, second half); every CTA does its share of batch 0 first, then its share of
// batch 1, so that the activations of batch 0 are complete device-wide half way through the phase
// and the barrier that guards them costs nothing. With T0 tiles in batch 0 and T in total, CTA b
// takes batch-0 tiles [T0*b/G, T0*(b+1)/G) and batch-1 tiles [F(b), F(b+1)), F(b) = T*b/G - T0*b/G,
// which gives every CTA T/G tiles (rounded) in total.
struct FWalk {
    int g0, g0_end, g1, g1_end, tpe;
    int c_cur, c_end, e, n_act, n0;
    const int *act_list;
    __device__ __forceinline__ void init(const FusedParams &P, const int *list, int n_active)
    {
        act_list = list;
        n_act = n_active;
        n0 = (n_active + 1) >> 1;
        tpe = (P.EFF + P.TB - 1) / P.TB;
        const long long T0 = (long long)n0 * tpe, T = (long long)n_active * tpe;
        const long long b = blockIdx.x, G = gridDim.x;
        g0 = static_cast<int>(T0 * b / G);
        g0_end = static_cast<int>(T0 * (b + 1) / G);
        g1 = static_cast<int>(T0 + T * b / G - T0 * b / G);
        g1_end = static_cast<int>(T0 + T * (b + 1) / G - T0 * (b + 1) / G);
        c_cur = static_cast<int>((long long)P.H * b / G);
        c_end = static_cast<int>((long long)P.H * (b + 1) / G);
        if (n_active == 0) c_end = c_cur;
        e = 0;
    }
    __device__ __forceinline__ bool has_batch(int b) const { return b == 0 ? g0 < g0_end : g1 < g1_end; }
    __device__ __forceinline__ bool next(const FusedParams &P, FTile &t)
    {
        int g = -1;
        if (g0 < g0_end) {
            g = g0++;
            t.batch = 0;
            t.last = (g0 == g0_end);
        } else if (g1 < g1_end) {
            g = g1++;
            t.batch = 1;
            t.last = (g1 == g1_end);
        }
        if (g >= 0) {
            const int j = g / tpe;
            t.phase = 0;
            t.j = j;
            t.slot = act_list[j];
            t.row0 = (g - j * tpe) * P.TB;
            t.rows = min(P.TB, P.EFF - t.row0);
            return true;
        }
        if (c_cur < c_end) {  // the same rows for every served slot in turn, then the next rows
            t.phase = 1;
            t.batch = 0;
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
        // the 16-byte-aligned span enclosing the rows (Q6_K rows are only 2-byte aligned); the bytes read
        // before / after them share a 16-byte granule with a valid byte, hence lie inside a mapped page
        const uintptr_t begin = reinterpret_cast<uintptr_t>(down_src<FD>(P, t, sid));
        const uintptr_t stop = begin + (size_t)t.rows * P.bprC * FD::kBlockBytes;
        const uintptr_t a0 = begin & ~static_cast<uintptr_t>(15);
        const uint32_t bytes = static_cast<uint32_t>(((stop + 15) & ~static_cast<uintptr_t>(15)) - a0);
        mbar_expect_tx(bar, bytes);
        bulk_g2s(stage, reinterpret_cast<const void *>(a0), bytes, bar);
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

// Device-wide barrier state: one 64-bit arrival counter per batch that only ever grows. Every
// launch adds exactly gridDim.x arrivals to a counter it uses, so between launches its value is a
// multiple of gridDim.x; a CTA that reads c at its start (when at most gridDim.x - 1 arrivals of its
// own launch can be in) knows the launch is complete at c - c % gridDim.x + gridDim.x.
__device__ __forceinline__ unsigned long long barrier_target(const unsigned long long *ctr)
{
    unsigned long long c;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(ctr) : "memory");
    return c - c % gridDim.x + gridDim.x;
}
// Release-arrive: every store this thread has made or observed (through the block-scope handshakes
// between the warps that finished the CTA's tiles) is visible to whoever acquires the counter.
__device__ __forceinline__ void barrier_arrive(unsigned long long *ctr)
{
    asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(ctr) : "memory");
}
// Lane 0 polls until the counter reaches `target`; the result is broadcast. Bounded.
__device__ __forceinline__ bool barrier_wait(const unsigned long long *ctr, unsigned long long target,
                                             volatile int *abort_flag, int lane)
{
    int ok = 0;
    if (lane == 0) {
        for (uint32_t i = 0; i < (1u << 20); i++) {
            unsigned long long c;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(ctr) : "memory");
            if (c >= target) {
                ok = 1;
                break;
            }
            if (*abort_flag) break;
            __nanosleep(40);
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void consumers_sync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");
}

// Before the first down tile of a batch: wait until every CTA has stored its act rows of the batch,
// then split the batch's activation vectors (all loads in flight before the first use). Every
// consumer warp calls this at the same points of the walk; the named barrier inside is matched by
// the catch-up loop at the end of the kernel when a warp gave up early. Kept out of line so that
// its registers do not weigh on the tile loops.
template <class FD>
__device__ __noinline__ void stage_batch(const FusedParams &P, uint8_t *smem, const int *act_list, int j0, int jn,
                                         const unsigned long long *ctr, unsigned long long target,
                                         volatile int *abort_flag, int stamp)
{
    const int tid = threadIdx.x, lane = tid & 31;
    const bool met = !*abort_flag && barrier_wait(ctr, target, abort_flag, lane);
    if (!met) *abort_flag = 1;
    if (tid == 0) MB200_STAMP(stamp);
    if (met) {
        const Layout LC = stream::layout<FD>(P.bprC, 0, 0, 1, 1);
        const int pitch = FD::kSlotsPerBlock * P.bprC + 1;
        for (int c0 = tid * 4; c0 < P.EFF; c0 += kConsumers * 32 * 4) {
            float4 v[kFusedMaxSlots / 2];
#pragma unroll
            for (int j = 0; j < kFusedMaxSlots / 2; j++)
                if (j < jn) v[j] = __ldcg(reinterpret_cast<const float4 *>(P.act + (size_t)act_list[j0 + j] * P.EFF + c0));
#pragma unroll
            for (int j = 0; j < kFusedMaxSlots / 2; j++) {
                if (j < jn) {
                    uint8_t *xc = smem + P.off_xc + (j0 + j) * P.xc_stride - kXBase;
                    split_store<FD>(v[j], c0, lane, pitch, reinterpret_cast<uint32_t *>(xc + LC.xq1),
                                    reinterpret_cast<uint32_t *>(xc + LC.xq2), reinterpret_cast<float *>(xc + LC.xs1),
                                    reinterpret_cast<float *>(xc + LC.xsum));
                }
            }
        }
    }
    consumers_sync();
    if (tid == 0) MB200_STAMP(stamp + 1);
}

// Finishes a gate/up tile: sums the column groups, SwiGLU, stores the act rows.
__device__ __forceinline__ void finish_gate_up(const FusedParams &P, const FTile &t, const float *pt, int lane)
{
    if (lane < t.rows) {
        const int NG = P.ngB;
        float g = 0.0f, u = 0.0f;
        for (int c = 0; c < NG; c++) {
            g += pt[lane * NG + c];
            u += pt[(P.TB + lane) * NG + c];
        }
        P.act[(size_t)t.slot * P.EFF + t.row0 + lane] = g / (1.0f + expf(-g)) * u;
    }
}

// Finishes a down tile: adds the slot's weighted rows to the running sums (slot order), and after the
// last served slot writes y.
__device__ __forceinline__ void finish_down(const FusedParams &P, const FTile &t, const float *pt, float *run,
                                            float w, int n_act, int lane)
{
    const int NG = P.ngC;
    for (int r = lane; r < t.rows; r += 32) {
        float v = 0.0f;
        for (int c = 0; c < NG; c++) v += pt[r * NG + c];
        const float a = fmaf(w, v, t.j == 0 ? 0.0f : run[r]);
        if (t.j == n_act - 1) {
            const int row = t.row0 + r;
            P.y[row] = (P.residual ? P.residual[row] : P.y[row]) + a;
        } else {
            run[r] = a;
        }
    }
}

template <class FD>
__global__ void __launch_bounds__(kFusedThreads, 1) moe_fused_kernel(const __grid_constant__ FusedParams P)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kFusedMaxStages;
    int *cnt = reinterpret_cast<int *>(smem + 96);         // per stage: consumer warps that stored their partial sums
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 120);
    int *sid = reinterpret_cast<int *>(smem + 128);        // expert (relative to expert_lo) per slot, -1 = not served
    float *swt = reinterpret_cast<float *>(smem + 160);    // routing weight per slot
    int *act_list = reinterpret_cast<int *>(smem + 192);   // slots served here, in slot order
    int *n_act_p = reinterpret_cast<int *>(smem + 224);
    float *run = reinterpret_cast<float *>(smem + 256);    // down: running sums of the tile's rows over the slots (<= 64)
    float *part = reinterpret_cast<float *>(smem + P.off_part);
    uint8_t *stages = smem + P.off_stages;
    const int S = P.stages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (warp == 0) MB200_STAMP(0);

    FWalk walk;

    if (warp == kConsumers) {
        // ---------------- issuer ----------------
        if (lane == 0) {
            *abort_flag = 0;
            for (int s = 0; s < S; s++) {
                mbar_init(&full[s], 2);  // the issuer's expect_tx arrival + "the stage's partial sums are free"
                mbar_init(&empty[s], kConsumers);
                cnt[s] = 0;
            }
            mbar_fence_init();
            if (P.pdl) stream::grid_dep_wait();  // the routed ids come from the upstream kernel
            int n = 0;
            for (int e = 0; e < P.n_slots; e++) {
                const int id = P.ids[e];
                const bool here = id >= P.expert_lo && id - P.expert_lo < P.expert_cnt;  // empty slots have id < 0
                sid[e] = here ? id - P.expert_lo : -1;
                swt[e] = here ? P.wts[e] : 0.0f;
                if (here) act_list[n++] = e;
            }
            *n_act_p = n;
            walk.init(P, act_list, n);
            FTile t;
            for (int s = 0; s < S; s++) {
                mbar_arrive(&full[s]);  // first phase: no partial sums to drain yet
                if (walk.next(P, t)) issue<FD>(P, t, stages + (size_t)s * P.stage_bytes, &full[s], sid);
            }
        }
        __syncthreads();
        if (lane == 0) {
            if (P.pdl) stream::grid_dep_launch();
            FTile t;
            int s = 0, ph = 0;
            while (walk.next(P, t)) {
                if (!mbar_wait(&empty[s], ph)) {
                    *abort_flag = 1;
                    atomicExch(P.err, MB200_ERR_TIMEOUT);
                    break;
                }
                if (*abort_flag) break;
                issue<FD>(P, t, stages + (size_t)s * P.stage_bytes, &full[s], sid);
                if (++s == S) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    unsigned long long tgt0 = 0, tgt1 = 0;  // read before this CTA can have arrived
    if (lane == 0) {
        tgt0 = barrier_target(P.sync);
        tgt1 = barrier_target(P.sync + 1);
    }
    tgt0 = __shfl_sync(0xffffffffu, tgt0, 0);
    tgt1 = __shfl_sync(0xffffffffu, tgt1, 0);
    if (P.pdl) stream::grid_dep_wait();  // x is produced upstream; act / y may still be in use there
    const Layout LB = stream::layout<Q4>(P.bprB, 0, 0, 1, 1);
    const Layout LC = stream::layout<FD>(P.bprC, 0, 0, 1, 1);
    {
        uint8_t *xb = smem + P.off_xb - kXBase;
        stream::quantize_x<Q4, 3>(P.x, P.H, P.bprB, reinterpret_cast<uint32_t *>(xb + LB.xq1),
                                  reinterpret_cast<uint32_t *>(xb + LB.xq2), reinterpret_cast<float *>(xb + LB.xs1),
                                  reinterpret_cast<float *>(xb + LB.xsum));
    }
    if (warp == 0) MB200_STAMP(1);
    __syncthreads();  // x is staged, barriers are initialised, the served slots are known
    const int n_act = *n_act_p;
    if (n_act == 0) {
        // no routed expert is served here: the block reduces to the residual (if this call carries one)
        if (warp == 0 && P.residual) {
            const int r0 = static_cast<int>((long long)P.H * blockIdx.x / gridDim.x);
            const int r1 = static_cast<int>((long long)P.H * (blockIdx.x + 1) / gridDim.x);
            for (int r = r0 + lane; r < r1; r += 32) P.y[r] = P.residual[r];
        }
        return;
    }
    walk.init(P, act_list, n_act);
    const int n0 = walk.n0;
    const int n_sync = n_act > n0 ? 2 : 1;  // batches whose activations get staged (one named barrier each)
    if (tid == 0) {  // a CTA without tiles in a batch still has to arrive at that batch's barrier
        if (!walk.has_batch(0)) barrier_arrive(P.sync);
        if (n_act > n0 && !walk.has_batch(1)) barrier_arrive(P.sync + 1);
    }

    const int q = lane >> 2, sub = lane & 3;
    FTile t, nt;
    int s = 0, ph = 0;
    bool have = walk.next(P, t);

    // After a warp has stored its partial sums of stage s: count it; the warp that completes the
    // count finishes the tile (the other warps move on to the next tile at once).
    auto stored_last = [&](int stage) -> bool {
        int old = 0;
        __syncwarp();
        if (lane == 0) {
            __threadfence_block();
            old = atomicAdd(&cnt[stage], 1);
            mbar_arrive(&empty[stage]);  // this warp no longer reads the stage's weights
            if (old == kConsumers - 1) {
                cnt[stage] = 0;
                __threadfence_block();
            }
        }
        return __shfl_sync(0xffffffffu, old, 0) == kConsumers - 1;
    };

    // ---- gate/up: warp i of column group g takes gate rows 2i, 2i+1 and up rows 2i, 2i+1 of every tile ----
    {
        const int gB = warp / P.wpgB, iB = warp % P.wpgB;
        const int colB = gB * 8 + q;
        Q4::XRegs xr;
        Q4::load_xregs(xr, smem + P.off_xb - kXBase, LB, P.bprB, colB, sub, true);
        const uint32_t row_bytes = P.bprB * kQ4KBlock;
        const uint32_t lane_off = colB * kQ4KBlock;
        const uint32_t off_g = 2 * iB * row_bytes + lane_off, off_u = (P.TB + 2 * iB) * row_bytes + lane_off;
        int k = 0;
        while (have && t.phase == 0) {
            const bool hn = walk.next(P, nt);
            if (!mbar_wait(&full[s], ph)) *abort_flag = 1;
            if (warp == 0 && k < 8) MB200_STAMP(16 + k);
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
            if (stored_last(s)) {
                __syncwarp();  // lane 0's acquire covers the whole warp
                finish_gate_up(P, t, pt, lane);
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full[s]);  // the stage's partial sums may be rewritten
                    if (t.last) {
                        // Every act row this CTA owes to the batch is stored: arrive at the batch's barrier.
                        // The finishing warps of a CTA are ordered one after the other through the stage
                        // counters (block-scope fences), so the release also covers the rows they stored.
                        barrier_arrive(P.sync + t.batch);
                        MB200_STAMP(7 + t.batch);
                    }
                }
            }
            if (*abort_flag) break;  // no early return: every consumer warp must reach the named barrier below
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
        while (have) {
            if (n_staged == 0 && t.j == 0) {
                stage_batch<FD>(P, smem, act_list, 0, n0, P.sync, tgt0, abort_flag, 9);
                n_staged = 1;
            }
            if (n_staged == 1 && n_sync == 2 && t.j == n0) {
                stage_batch<FD>(P, smem, act_list, n0, n_act - n0, P.sync + 1, tgt1, abort_flag, 11);
                n_staged = 2;
            }
            if (*abort_flag) break;
            if (t.j != cur_j) {
                cur_j = t.j;
                FD::load_xregs(xr, smem + P.off_xc + cur_j * P.xc_stride - kXBase, LC, P.bprC, colC, sub, true);
            }
            uint32_t skew = 0;
            if (FD::kBlockBytes % 16 != 0)
                skew = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(down_src<FD>(P, t, sid)) & 15);
            const bool hn = walk.next(P, nt);
            if (!mbar_wait(&full[s], ph)) *abort_flag = 1;
            if (warp == 0 && k < 8) MB200_STAMP(24 + k);
            k++;
            const uint8_t *base = stages + (size_t)s * P.stage_bytes + skew + colC * FD::kBlockBytes;
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
            float *pt = part + s * P.part_pitch;
            if ((lane & (W / 2 - 1)) == 0 && row < t.rows) pt[row * P.ngC + gC] = sum;
            if (stored_last(s)) {
                __syncwarp();
                finish_down(P, t, pt, run, swt[t.slot], n_act, lane);
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
            }
            if (*abort_flag) break;
            if (++s == S) {
                s = 0;
                ph ^= 1;
            }
            have = hn;
            t = nt;
        }
    }
    while (n_staged < n_sync) {  // a warp that gave up early still owes the other warps its barrier arrivals
        consumers_sync();
        n_staged++;
    }
    if (*abort_flag && lane == 0) atomicExch(P.err, MB200_ERR_TIMEOUT);
    if (warp == 0) MB200_STAMP(5);
}

int g_fused_mode = 1;          // 0: never use the fused kernel
int g_fused_pdl_ok = 1;        // cleared if the driver refuses cooperative + programmatic serialization together

template <class FD>
int launch_fused(FusedParams &P, int smem_bytes, cudaStream_t stream)
{
    static bool attr_done = false;
    if (!attr_done) {
        if (cudaFuncSetAttribute(moe_fused_kernel<FD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess)
            return MB200_ERR_LAUNCH;
        attr_done = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kSMs);
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, moe_fused_kernel<FD>, P);
    if (e != cudaSuccess && P.pdl) {
        cudaGetLastError();
        g_fused_pdl_ok = 0;
        P.pdl = 0;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, moe_fused_kernel<FD>, P);
    }
    if (e != cudaSuccess) {
        fprintf(stderr, "[mnemo_b200] fused expert kernel launch failed: %s\n", cudaGetErrorString(e));
        cudaGetLastError();
        return MB200_ERR_LAUNCH;
    }
    return MB200_OK;
}

}  // namespace

// Geometry of the fused kernel for a shape; returns false when the shape is outside what it covers
// (the caller then uses the separate gate/up and down kernels).
static bool fused_plan(FusedParams &P, int &smem_bytes)
{
    const int H = P.H, EFF = P.EFF;
    if (H % 256 || EFF % 256 || P.n_slots < 1 || P.n_slots > kFusedMaxSlots) return false;
    P.bprB = H / 256;
    P.bprC = EFF / 256;
    if (P.bprB % 8) return false;
    P.ngB = P.bprB / 8;
    if (P.ngB > kConsumers || kConsumers % P.ngB) return false;
    P.wpgB = kConsumers / P.ngB;
    P.TB = 2 * P.wpgB;
    int v = 1;
    while (v * 2 <= 8 && P.bprC % (v * 2) == 0) v *= 2;
    if (v < 2) return false;
    P.vC = v;
    P.rppC = 8 / v;
    P.ngC = P.bprC / v;
    if (P.ngC > kConsumers || kConsumers % P.ngC) return false;
    P.wpgC = kConsumers / P.ngC;
    P.TC = P.wpgC * P.rppC * 2;
    if (P.TC > 64) P.TC = 64;  // the epilogue keeps two running sums per lane
    return true;
}

template <class FD>
static bool fused_layout(FusedParams &P, int &smem_bytes)
{
    const int per_cta = (P.H + kSMs - 1) / kSMs;
    const int c_rows = per_cta < P.TC ? per_cta : P.TC;
    const int tileB = 2 * P.TB * P.bprB * kQ4KBlock;
    const int tileC = c_rows * P.bprC * FD::kBlockBytes + 32;  // + alignment skew, word over-read
    P.stage_bytes = ((tileB > tileC ? tileB : tileC) + 127) & ~127;
    const Layout LB = stream::layout<Q4>(P.bprB, 0, 0, 1, 1);
    const Layout LC = stream::layout<FD>(P.bprC, 0, 0, 1, 1);
    int o = 512;
    P.off_xb = o;
    o += LB.x_stride;
    P.off_xc = o;
    P.xc_stride = LC.x_stride;
    o += P.n_slots * LC.x_stride;
    const int pB = 2 * P.TB * P.ngB, pC = P.TC * P.ngC;
    P.part_pitch = pB > pC ? pB : pC;
    P.off_part = o;
    for (int S = kFusedMaxStages; S >= 3; S--) {
        int t = o + S * P.part_pitch * 4;
        t = (t + 127) & ~127;
        if (t + S * P.stage_bytes <= 227 * 1024) {
            P.stages = S;
            P.off_stages = t;
            smem_bytes = t + S * P.stage_bytes;
            return true;
        }
    }
    return false;
}

void moe_fused_set_mode(int mode) { g_fused_mode = mode; }
int moe_fused_mode() { return g_fused_mode; }

// Returns MB200_OK after a launch, MB200_ERR_UNSUPPORTED when the shape is not covered (nothing launched).
int moe_fused(const void *experts, size_t stride, size_t gate_off, size_t up_off, size_t down_off, int down_type,
              const int *ids, const float *wts, int n_slots, int expert_lo, int expert_cnt, const float *x, float *act,
              const float *residual, float *y, int H, int EFF, unsigned long long *sync, cudaStream_t stream)
{
    FusedParams P{};
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
extern "C" void mb200_trace_read_fused(void *dst)
{
    cudaMemcpyFromSymbol(dst, mb200::stream::g_trace, sizeof(long long) * mb200::kSMs * 2 * 48, 0,
                         cudaMemcpyDeviceToDevice);
}
#endif
