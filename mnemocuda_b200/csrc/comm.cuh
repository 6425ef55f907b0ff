// Device-side pieces of the push collectives (comm.cu) that other kernels use to exchange their own results:
// the 8-byte cell {fp32 value, 32-bit sequence tag}, stored to a peer with ONE store and polled locally.
#pragma once
#include "common.cuh"

namespace mb200 {

constexpr int kMaxWorld = 8;
constexpr long long kSpinBudgetNs = 2000000000ll;  // 2 s of wall clock, then MB200_ERR_TIMEOUT

// What a kernel needs of a communicator (mb200_comm_create): the receive cells of every rank, this rank's
// sequence word and launch ticket. Cell (parity, source rank q, element i) of a rank's buffer is
// cells[(parity * world + q) * max_floats + i].
struct PushDesc {
    uint2 *peer_cells[kMaxWorld];
    uint2 *self_cells;
    unsigned long long *seq;  // sequence number of the last completed collective on this communicator
    unsigned int *ticket;     // CTAs of the running launch that have finished
    int rank, world;          // world == 0: no exchange
    unsigned long long max_floats;
};

// Fills `d` from a communicator handle; false if the handle is null.
bool comm_describe(void *comm, PushDesc *d);

__device__ __forceinline__ void st_cell(uint2 *p, float v, uint32_t tag)
{
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_cell(const uint2 *p)
{
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// Spins until the cell carries `tag`; false once the time budget is spent.
__device__ __forceinline__ bool wait_cell(const uint2 *p, uint32_t tag, float &v, long long t0)
{
    for (unsigned it = 0;; it++) {
        const uint2 c = ld_cell(p);
        if (c.y == tag) {
            v = __uint_as_float(c.x);
            return true;
        }
        if ((it & 255) == 255) {
            long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > kSpinBudgetNs) return false;
        }
    }
}

// The cells of one element from every source rank (rank q's cell at p + q * stride): all of them are requested at
// once -- the pieces arrive at about the same time, and polling them one after the other would cost a memory round
// trip per rank -- and only a cell that does not carry `tag` yet is waited for. v[q] receives rank q's value.
__device__ __forceinline__ bool wait_cells(const uint2 *p, size_t stride, int world, uint32_t tag, float (&v)[kMaxWorld],
                                           long long t0)
{
    uint2 c[kMaxWorld];
#pragma unroll
    for (int q = 0; q < kMaxWorld; q++)
        if (q < world) c[q] = ld_cell(p + (size_t)q * stride);
#pragma unroll
    for (int q = 0; q < kMaxWorld; q++) {
        if (q >= world) break;
        if (c[q].y == tag) {
            v[q] = __uint_as_float(c[q].x);
        } else if (!wait_cell(p + (size_t)q * stride, tag, v[q], t0)) {
            return false;
        }
    }
    return true;
}

}  // namespace mb200
