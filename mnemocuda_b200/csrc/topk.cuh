// Router selection shared by cuda_topk_softmax and the fused router kernel.
#pragma once
#ifndef MB200_TOPK_STAMP
#define MB200_TOPK_STAMP(n) do {} while (0)
#endif

#include "common.cuh"

namespace mb200 {

// ---- top-k + softmax (reference src/kernels.cu:993-1057) ----------------------
// Same two-stage selection as the reference so that the kept set AND the order
// of the output slots are identical: (1) each of 32 lanes keeps a local top-k
// of scores lane, lane+32, ... by "replace the first minimum when strictly
// greater"; (2) the 32 x 16 candidate table is scanned in (lane, slot) order by
// the same rule. Stage 2 keeps its k slots in registers and tracks the running
// minimum, so a rejected candidate costs one compare.
// The k live slots kept sorted by (value, slot) in registers, so the reference's "first index
// of the minimum" is always entry 0. Replacing the minimum = evict entry 0 and insert the
// newcomer, which inherits the evicted slot. The insert is branch-free and shallow: all
// compares are independent, then an add tree, then independent selects. KW = 8 or 16 wide.
template <int KW>
struct SortedSlots {
    float v[KW];
    int slot[KW];
    int id[KW];
    __device__ __forceinline__ void reset(int k)
    {
#pragma unroll
        for (int i = 0; i < KW; i++) {
            v[i] = i < k ? -1e30f : 3.0e38f;  // entries >= k: +huge sentinels that never move
            slot[i] = i;
            id[i] = -1;
        }
    }
    __device__ __forceinline__ void replace_min(float val, int ident)
    {
        const int s = slot[0];
        int before[KW];
#pragma unroll
        for (int i = 1; i < KW; i++) before[i] = (v[i] < val || (v[i] == val && slot[i] < s)) ? 1 : 0;
        before[0] = 0;
        int pos = 0;  // entries 1..KW-1 ordered before the newcomer
#pragma unroll
        for (int i = 1; i < KW; i++) pos += before[i];
        // entries 1..pos move down one place, the newcomer lands at pos; sorted order makes
        // "i < pos" the same as before[i+1]
#pragma unroll
        for (int i = 0; i < KW - 1; i++) {
            const bool shift = before[i + 1] != 0;
            const bool here = (i == pos);
            v[i] = shift ? v[i + 1] : (here ? val : v[i]);
            slot[i] = shift ? slot[i + 1] : (here ? s : slot[i]);
            id[i] = shift ? id[i + 1] : (here ? ident : id[i]);
        }
        if (pos == KW - 1) {
            v[KW - 1] = val;
            slot[KW - 1] = s;
            id[KW - 1] = ident;
        }
    }
};

// One warp. Stage 1: each lane keeps the local top-k of scores lane, lane+32, ... and writes it
// to the 32 x 16 candidate table by slot. Stage 2: every lane runs the same walk over the table
// in (lane, slot) order (broadcast reads, uniform branches); a source lane whose best candidate
// cannot enter is skipped with one compare.
template <int KW>
__device__ __noinline__ void topk_softmax_warp_seq_kw(const float *scores, int *indices, float *weights,
                                                     int n_experts, int k, float *s_vals, int *s_ids)
{
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    SortedSlots<KW> loc;
    loc.reset(k);
    int cnt = 0;  // live entries of this lane (slots 0..cnt-1: stage 1 fills them in order before it ever replaces)
    float lmax = -1e30f;
    for (int j0 = lane; j0 < n_experts; j0 += 32 * 8) {
        float sv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) sv[u] = (j0 + 32 * u < n_experts) ? scores[j0 + 32 * u] : -1e30f;  // loads in flight together
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (sv[u] > loc.v[0]) {
                loc.replace_min(sv[u], j0 + 32 * u);
                lmax = fmaxf(lmax, sv[u]);
                if (cnt < k) cnt++;
            }
    }
#pragma unroll
    for (int i = 0; i < 16; i++) s_vals[lane * 16 + i] = -1e30f;
#pragma unroll
    for (int i = 0; i < KW; i++)
        if (i < k && loc.id[i] >= 0) {
            s_vals[lane * 16 + loc.slot[i]] = loc.v[i];
            s_ids[lane * 16 + loc.slot[i]] = loc.id[i];
        }
    const int cmax = __reduce_max_sync(full, cnt);
    __syncwarp();

    SortedSlots<KW> top;
    top.reset(k);
    for (int l = 0; l < 32; l++) {
        const float best = __shfl_sync(full, lmax, l);
        if (!(best > top.v[0])) continue;  // uniform: nothing of this source lane can enter
        float cv[KW];
#pragma unroll
        for (int i = 0; i < KW; i++) cv[i] = i < cmax ? s_vals[l * 16 + i] : -1e30f;
#pragma unroll
        for (int i = 0; i < KW; i++) {
            if (i >= cmax) break;
            if (__any_sync(full, cv[i] > top.v[0]))  // uniform by construction; sentinels (-1e30) never pass
                top.replace_min(cv[i], s_ids[l * 16 + i]);
        }
    }
    // back to slot order through the (now free) table, then softmax summed in slot order like the reference
    __syncwarp();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < KW; i++)
            if (i < k) {
                s_vals[top.slot[i]] = top.v[i];
                s_ids[top.slot[i]] = top.id[i];
            }
        float mx = s_vals[0];
        for (int i = 1; i < k; i++) mx = fmaxf(mx, s_vals[i]);
        float sum = 0.0f;
        for (int i = 0; i < k; i++) {
            const float e = expf(s_vals[i] - mx);
            s_vals[i] = e;
            sum += e;
        }
        for (int i = 0; i < k; i++) {
            weights[i] = s_vals[i] / sum;
            indices[i] = s_ids[i];
        }
    }
}

// ---- parallel form -------------------------------------------------------------
// The replace-the-minimum walk of stage 2 has a closed form when no two ACCEPTED
// candidates are equal. With candidates p = 0..M-1 in the reference's (lane, slot) order:
//   accept(p)  <=>  #{q < p : v_q >= v_p} < k            (v_p beats the k-th largest so far)
//   t(p) = number of accepted candidates before p        (arrival index)
//   r(p) = number of accepted candidates smaller than p  (the j-th eviction removes rank j,
//                                                         because evicted values never decrease)
//   slot(p) = t(p) if t(p) < k, else slot(the accepted candidate of rank t(p) - k)
// and the survivors are the k accepted candidates of highest rank. All counts are data-parallel;
// only the slot chain is a short pointer walk. Equal accepted values fall back to the serial form.
struct __align__(16) TopkShared {
    float val[512];   // candidates in sequence order
    int cid[512];
    float aval[512];  // accepted candidates in arrival order
    int aid[512];
    int byrank[512];
    float outv[16];
    int outid[16];
    unsigned bal[16];  // block form: accept flags of each row of 32 candidates
    int n_cand;        // block form: number of candidates
};

// Second half of the parallel form, one warp: `m` accepted candidates (values sh.aval, ids sh.aid, in
// arrival order) -> ranks, tie check, slot chains, softmax. Returns false on a tie among the accepted.
// kSmall: loops kept rolled (for code that is fetched cold at every launch).
template <bool kSmall = false>
__device__ __forceinline__ bool topk_finish_warp(int m, int *indices, float *weights, int k, TopkShared &sh)
{
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int mpad = (m + 3) & ~3;
    __syncwarp();
    if (lane < mpad - m) sh.aval[m + lane] = __int_as_float(0x7FC00000);
    __syncwarp();

    // ---- ranks among the accepted, and the tie check ----
    bool tie = false;
    for (int t0 = 0; t0 < m; t0 += 32) {
        const int t = t0 + lane;
        const float av = t < m ? sh.aval[t] : __int_as_float(0x7FC00000);
        int r = 0, eq = 0;
#pragma unroll(kSmall ? 1 : 4)
        for (int u = 0; u < mpad; u += 4) {
            const float4 w = *reinterpret_cast<const float4 *>(&sh.aval[u]);
            r += (w.x < av) + (w.y < av) + (w.z < av) + (w.w < av);
            eq += (w.x == av) + (w.y == av) + (w.z == av) + (w.w == av);
        }
        if (t < m) {
            if (eq > 1) tie = true;
            sh.byrank[r] = t;
            sh.cid[t] = r;  // cid is free now: rank by arrival index
        }
    }
    if (__any_sync(full, tie)) return false;
    __syncwarp();

    // ---- survivors walk their slot chain ----
    for (int t0 = 0; t0 < m; t0 += 32) {
        const int t = t0 + lane;
        if (t < m && sh.cid[t] >= m - k) {
            int cur = t;
            while (cur >= k) cur = sh.byrank[cur - k];
            sh.outv[cur] = sh.aval[t];
            sh.outid[cur] = sh.aid[t];
        }
    }
    __syncwarp();
    // ---- softmax over the k kept logits, summed in slot order like the reference ----
    // Lane i holds slot i; the sum runs over the slots in order (every lane repeats it), so the result
    // is the reference's, without a serial pass over an array by one lane.
    {
        const float v = lane < k ? sh.outv[lane] : -3.0e38f;
        float mx = v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(full, mx, o));
        const float e = lane < k ? expf(v - mx) : 0.0f;
        float sum = 0.0f;
#pragma unroll(kSmall ? 1 : 4)
        for (int i = 0; i < k; i++) sum += __shfl_sync(full, e, i);
        if (lane < k) {
            weights[lane] = e / sum;
            indices[lane] = sh.outid[lane];
        }
    }
    return true;
}

template <int KW>
__device__ __forceinline__ bool topk_softmax_warp_par(const float *scores, int *indices, float *weights,
                                                      int n_experts, int k, TopkShared &sh)
{
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    // ---- stage 1: the lane's candidates, in slot order ----
    float lv[KW];
    int li[KW];
    int cnt = 0;
#pragma unroll
    for (int i = 0; i < KW; i++) {
        lv[i] = -1e30f;
        li[i] = -1;
    }
    if (n_experts <= 32 * k) {
        // at most k scores per lane: nothing is ever replaced, slots fill in arrival order
        float sv[KW];
#pragma unroll
        for (int u = 0; u < KW; u++) sv[u] = (u < k && lane + 32 * u < n_experts) ? scores[lane + 32 * u] : -1e30f;
#pragma unroll
        for (int u = 0; u < KW; u++)
            if (sv[u] > -1e30f) {
#pragma unroll
                for (int i = 0; i < KW; i++)
                    if (i == cnt) {
                        lv[i] = sv[u];
                        li[i] = lane + 32 * u;
                    }
                cnt++;
            }
    } else {
        SortedSlots<KW> loc;
        loc.reset(k);
        for (int j0 = lane; j0 < n_experts; j0 += 32 * 8) {
            float sv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) sv[u] = (j0 + 32 * u < n_experts) ? scores[j0 + 32 * u] : -1e30f;
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (sv[u] > loc.v[0]) {
                    loc.replace_min(sv[u], j0 + 32 * u);
                    if (cnt < k) cnt++;
                }
        }
#pragma unroll
        for (int i = 0; i < KW; i++)
            if (i < k && loc.id[i] >= 0) {
#pragma unroll
                for (int j = 0; j < KW; j++)
                    if (loc.slot[i] == j) {
                        lv[j] = loc.v[i];
                        li[j] = loc.id[i];
                    }
            }
    }
    // dense sequence index: exclusive scan of cnt over lanes
    int base = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(full, base, o);
        if (lane >= o) base += t;
    }
    const int M = __shfl_sync(full, base, 31);
    base -= cnt;
#pragma unroll
    for (int i = 0; i < KW; i++)
        if (i < cnt) {
            sh.val[base + i] = lv[i];
            sh.cid[base + i] = li[i];
        }
    const int Mpad = (M + 3) & ~3;
    if (lane < Mpad - M) sh.val[M + lane] = __int_as_float(0x7FC00000);  // NaN padding: compares false
    if (lane < 16) {
        sh.outv[lane] = -1e30f;
        sh.outid[lane] = -1;
    }
    __syncwarp();

    // ---- accept flags and arrival indices, four rows of 32 candidates at a time ----
    int m = 0;
    for (int row0 = 0; row0 * 32 < M; row0 += 4) {
        float v[4];
        int c[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int p = (row0 + i) * 32 + lane;
            v[i] = p < M ? sh.val[p] : __int_as_float(0x7FC00000);
            c[i] = 0;
        }
        // rows before row0: every q is earlier than every p of this chunk
        const int q_full = row0 * 32;
        for (int q = 0; q < q_full; q += 4) {
            const float4 w = *reinterpret_cast<const float4 *>(&sh.val[q]);
#pragma unroll
            for (int i = 0; i < 4; i++)
                c[i] += (w.x >= v[i]) + (w.y >= v[i]) + (w.z >= v[i]) + (w.w >= v[i]);
        }
        // the chunk's own rows: q counts only if q < p
        const int q_end = min(Mpad, (row0 + 4) * 32);
        for (int q = q_full; q < q_end; q += 4) {
            const float4 w = *reinterpret_cast<const float4 *>(&sh.val[q]);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int p = (row0 + i) * 32 + lane;
                c[i] += (q + 0 < p && w.x >= v[i]) + (q + 1 < p && w.y >= v[i]) + (q + 2 < p && w.z >= v[i]) +
                        (q + 3 < p && w.w >= v[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int p = (row0 + i) * 32 + lane;
            const bool acc = p < M && c[i] < k;
            const unsigned bal = __ballot_sync(full, acc);
            if (acc) {
                const int t = m + __popc(bal & ((1u << lane) - 1u));
                sh.aval[t] = v[i];
                sh.aid[t] = sh.cid[p];
            }
            m += __popc(bal);
        }
    }
    return topk_finish_warp(m, indices, weights, k, sh);
}

// One warp. `sh` is shared memory. Results are identical to the reference's kernel
// (src/kernels.cu:993-1057): same kept set, same output slot order.
__device__ __forceinline__ void topk_softmax_warp(const float *scores, int *indices, float *weights, int n_experts,
                                                  int k, TopkShared &sh)
{
    bool done;
    if (k <= 8)
        done = topk_softmax_warp_par<8>(scores, indices, weights, n_experts, k, sh);
    else
        done = topk_softmax_warp_par<16>(scores, indices, weights, n_experts, k, sh);
    if (done) return;
    __syncwarp();
    // equal accepted values: the serial walk decides
    if (k <= 8)
        topk_softmax_warp_seq_kw<8>(scores, indices, weights, n_experts, k, sh.val, sh.cid);
    else
        topk_softmax_warp_seq_kw<16>(scores, indices, weights, n_experts, k, sh.val, sh.cid);
}

// The same selection by a group of warps -- the first n_warps warps of the CTA, all of whose threads
// call it; they meet on hardware barrier `bar_id`: warp 0 lists the candidates, the rows of 32
// candidates are then counted by all warps side by side, and warp 0 finishes. Only for
// n_experts <= 32 * k (no score is dropped before the merge), which covers the routers of the
// supported models; other shapes use the one-warp form on warp 0.
__device__ __forceinline__ void topk_group_sync(int bar_id, int n_threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(n_threads) : "memory");
}
// kBigShapes = false leaves out the one-warp general form for n_experts > 32 k or > 512 (a third of a megabyte of
// code): for a caller that has checked the shape on the host.
// The group is warps [warp0, warp0 + n_warps) of the CTA.
// KW: scores per lane the candidate listing is unrolled for (k <= KW). UNR: unrolling of the counting loops -- 8 where
// the code stays resident (a kernel of its own that is launched back to back), 2 where it is fetched cold at every
// launch and its size is what its first run costs (inside the one-launch MoE kernel).
template <bool kBigShapes = true, int KW = 16, int UNR = 8>
__device__ __forceinline__ void topk_softmax_group(const float *scores, int *indices, float *weights, int n_experts,
                                                   int k, TopkShared &sh, int n_warps, int bar_id, int warp0 = 0)
{
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31, warp = static_cast<int>(threadIdx.x >> 5) - warp0;
    if (n_experts > 32 * k || k > KW || n_experts > 512) {  // block-uniform
        if (kBigShapes && warp == 0) topk_softmax_warp(scores, indices, weights, n_experts, k, sh);
        return;
    }
    // ---- candidates in the reference's (lane, slot) order: lane l holds scores l, l + 32, ... ----
    if (warp == 0) {
        float sv[KW];
        int cnt = 0;
#pragma unroll
        for (int u = 0; u < KW; u++) sv[u] = (u < k && lane + 32 * u < n_experts) ? scores[lane + 32 * u] : -1e30f;
#pragma unroll
        for (int u = 0; u < KW; u++) cnt += (sv[u] > -1e30f) ? 1 : 0;
        int base = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(full, base, o);
            if (lane >= o) base += t;
        }
        const int M = __shfl_sync(full, base, 31);
        base -= cnt;
        int w = 0;
#pragma unroll
        for (int u = 0; u < KW; u++)
            if (sv[u] > -1e30f) {
                sh.val[base + w] = sv[u];
                sh.cid[base + w] = lane + 32 * u;
                w++;
            }
        const int Mpad = (M + 3) & ~3;
        if (lane < Mpad - M) sh.val[M + lane] = __int_as_float(0x7FC00000);  // NaN padding: compares false
        if (lane < 16) {
            sh.outv[lane] = -1e30f;
            sh.outid[lane] = -1;
        }
        if (lane == 0) sh.n_cand = M;
    }
    topk_group_sync(bar_id, n_warps * 32);
    MB200_TOPK_STAMP(0);
    const int M = sh.n_cand;
    const int Mpad = (M + 3) & ~3;
    const int n_rows = (M + 31) >> 5;
    // ---- accept(p) <=> #{q < p : v_q >= v_p} < k, one row of 32 candidates per warp at a time ----
    for (int row = warp; row < n_rows; row += n_warps) {
        const int p = row * 32 + lane;
        const float v = p < M ? sh.val[p] : __int_as_float(0x7FC00000);
        int c = 0;
#pragma unroll UNR
        for (int q = 0; q < row * 32; q += 4) {  // earlier rows: every q < p
            const float4 w = *reinterpret_cast<const float4 *>(&sh.val[q]);
            c += (w.x >= v) + (w.y >= v) + (w.z >= v) + (w.w >= v);
        }
        const int q_end = min(Mpad, (row + 1) * 32);
#pragma unroll UNR
        for (int q = row * 32; q < q_end; q += 4) {  // own row: q counts only if q < p
            const float4 w = *reinterpret_cast<const float4 *>(&sh.val[q]);
            c += (q + 0 < p && w.x >= v) + (q + 1 < p && w.y >= v) + (q + 2 < p && w.z >= v) + (q + 3 < p && w.w >= v);
        }
        const unsigned bal = __ballot_sync(full, p < M && c < k);
        if (lane == 0) sh.bal[row] = bal;
    }
    topk_group_sync(bar_id, n_warps * 32);
    MB200_TOPK_STAMP(1);
    // ---- arrival order: compact the accepted ----
    int m = 0;
#pragma unroll(UNR < 8 ? 1 : 4)
    for (int row = 0; row < n_rows; row++) {
        const unsigned bal = sh.bal[row];
        if ((row % n_warps) == warp && (bal & (1u << lane))) {
            const int p = row * 32 + lane;
            const int t = m + __popc(bal & ((1u << lane) - 1u));
            sh.aval[t] = sh.val[p];
            sh.aid[t] = sh.cid[p];
        }
        m += __popc(bal);
    }
    topk_group_sync(bar_id, n_warps * 32);
    MB200_TOPK_STAMP(2);
    if (warp != 0) return;
    if (topk_finish_warp<(UNR < 8)>(m, indices, weights, k, sh)) return;
    __syncwarp();
    // equal accepted values: the serial walk decides
    if (k <= 8)
        topk_softmax_warp_seq_kw<8>(scores, indices, weights, n_experts, k, sh.val, sh.cid);
    else
        topk_softmax_warp_seq_kw<16>(scores, indices, weights, n_experts, k, sh.val, sh.cid);
}


// Whole CTA (blockDim.x a multiple of 32, every thread calls it).
__device__ __forceinline__ void topk_softmax_block(const float *scores, int *indices, float *weights, int n_experts,
                                                   int k, TopkShared &sh)
{
    topk_softmax_group(scores, indices, weights, n_experts, k, sh, blockDim.x >> 5, 0);
}

}  // namespace mb200
