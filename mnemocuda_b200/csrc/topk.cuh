// Router selection shared by cuda_topk_softmax and the fused router kernel.
#pragma once

#include "common.cuh"

namespace mb200 {

// ---- top-k + softmax (reference src/kernels.cu:993-1057) ----------------------
// Same two-stage selection as the reference so that the kept set AND the order
// of the output slots are identical: (1) each of 32 lanes keeps a local top-k
// of scores lane, lane+32, ... by "replace the first minimum when strictly
// greater"; (2) the 32 x 16 candidate table is scanned in (lane, slot) order by
// the same rule. Stage 2 keeps its k slots in registers and tracks the running
// minimum, so a rejected candidate costs one compare.
struct TopK {
    float v[16];
    int id[16];
    float cur_min;
    int cur_mi;
    __device__ void reset(int k)
    {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            v[i] = -1e30f;
            id[i] = -1;
        }
        cur_min = -1e30f;
        cur_mi = 0;
        (void)k;
    }
    __device__ void offer(float val, int ident, int k)
    {
        if (!(val > cur_min)) return;
#pragma unroll
        for (int i = 0; i < 16; i++)
            if (i == cur_mi) {
                v[i] = val;
                id[i] = ident;
            }
        // first index of the minimum over the k live slots
        float m = v[0];
        int mi = 0;
#pragma unroll
        for (int i = 1; i < 16; i++)
            if (i < k && v[i] < m) {
                m = v[i];
                mi = i;
            }
        cur_min = m;
        cur_mi = mi;
    }
};

// Order-preserving map float -> int (for redux.sync min/max); -0.0 is folded onto +0.0 so that
// keys compare exactly like the floats do.
__device__ __forceinline__ int float_key(float f)
{
    int b = __float_as_int(f);
    if (b == static_cast<int>(0x80000000u)) b = 0;
    return b ^ ((b >> 31) & 0x7FFFFFFF);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7FFFFFFF)); }

// One warp. Stage 1 runs in parallel (one local top-k per lane, registers). Stage 2 walks the
// candidates in the reference's (lane, slot) order with the k result slots spread over lanes
// 0..k-1: a rejected candidate costs a shuffle and a compare, an accepted one a warp-wide
// integer min (redux.sync) plus a ballot to find the first slot that holds the new minimum.
// s_vals / s_ids are unused scratch kept for interface stability.
__device__ __forceinline__ void topk_softmax_warp(const float *scores, int *indices, float *weights, int n_experts,
                                                  int k, float *s_vals, int *s_ids)
{
    (void)s_vals;
    (void)s_ids;
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    TopK loc;
    loc.reset(k);
    int cnt = 0;  // live entries of this lane: stage 1 fills slots 0,1,.. in order before it ever replaces
    for (int j = lane; j < n_experts; j += 32) {
        const float val = scores[j];
        if (val > loc.cur_min) {
            loc.offer(val, j, k);
            if (cnt < k) cnt++;
        }
    }
    const int cmax = __reduce_max_sync(full, cnt);

    float sv = -1e30f;  // lane i < k holds result slot i
    int sid = -1;
    float cur_min = -1e30f;
    int cur_mi = 0;
    for (int l = 0; l < 32; l++) {
        const int cl = __shfl_sync(full, cnt, l);
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (i >= cmax) break;
            const float val = __shfl_sync(full, loc.v[i], l);
            if (i >= cl || !(val > cur_min)) continue;  // warp-uniform
            const int cid = __shfl_sync(full, loc.id[i], l);
            if (lane == cur_mi) {
                sv = val;
                sid = cid;
            }
            const int key = lane < k ? float_key(sv) : 0x7FFFFFFF;
            const int mkey = __reduce_min_sync(full, key);
            cur_mi = __ffs(__ballot_sync(full, key == mkey)) - 1;
            cur_min = key_float(mkey);
        }
    }
    // softmax over the k kept logits, summed in slot order like the reference
    const int xkey = __reduce_max_sync(full, lane < k ? float_key(sv) : static_cast<int>(0x80000000u));
    const float mx = key_float(xkey);
    const float ex = lane < k ? expf(sv - mx) : 0.0f;
    float sum = 0.0f;
    for (int i = 0; i < k; i++) sum += __shfl_sync(full, ex, i);
    if (lane < k) {
        weights[lane] = ex / sum;
        indices[lane] = sid;
    }
}

}  // namespace mb200
