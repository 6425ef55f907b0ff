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

__device__ __forceinline__ void topk_softmax_warp(const float *scores, int *indices, float *weights, int n_experts, int k,
                                  float *s_vals, int *s_ids)
{
    const int tid = threadIdx.x & 31;
    TopK loc;
    loc.reset(k);
    for (int j = tid; j < n_experts; j += 32) loc.offer(scores[j], j, k);
#pragma unroll
    for (int i = 0; i < 16; i++) {
        s_vals[tid * 16 + i] = i < k ? loc.v[i] : -1e30f;
        s_ids[tid * 16 + i] = i < k ? loc.id[i] : -1;
    }
    __syncwarp();
    if (tid == 0) {
        TopK top;
        top.reset(k);
        for (int l = 0; l < 32; l++) {
#pragma unroll 4
            for (int i = 0; i < k; i++) {
                const float val = s_vals[l * 16 + i];
                if (val <= -1e30f) continue;
                top.offer(val, s_ids[l * 16 + i], k);
            }
        }
        float mx = top.v[0];
#pragma unroll
        for (int i = 1; i < 16; i++)
            if (i < k && top.v[i] > mx) mx = top.v[i];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++)
            if (i < k) {
                top.v[i] = expf(top.v[i] - mx);
                sum += top.v[i];
            }
#pragma unroll
        for (int i = 0; i < 16; i++)
            if (i < k) {
                weights[i] = top.v[i] / sum;
                indices[i] = top.id[i];
            }
    }
}

}  // namespace mb200
