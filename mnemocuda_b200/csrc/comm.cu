// Push collectives over NVLink peer memory for the tiny vectors of a sharded decode step.
//
// The reference's only multi-GPU traffic is one hidden vector copied from GPU to GPU at each layer-range
// boundary (cudaMemcpyPeerAsync, src/forward.c:1555-1581). Sharding the work itself (rows of a matvec,
// experts of a MoE block) needs an all-gather / all-reduce of 16-32 KB several times per layer: far too
// small for a bandwidth-oriented collective, so the cost is latency. Here every rank STORES its piece
// straight into every peer's receive buffer (plain 16-byte peer stores through NVSwitch; no bulk / TMA
// copy and no multicast touches peer memory), then raises a per-source arrival counter on the peer with
// a system-scope release; the receiver spins on its own local counters (bounded), then sums the pieces
// in rank order -- deterministic, identical on every rank -- or just concatenates them (all-gather).
//
// One process per GPU. Buffers are cudaMalloc'ed here and shared through CUDA IPC handles that the host
// side exchanges (torch.distributed, or anything else); the library itself never talks to other ranks.
// Receive slots are double-buffered by the parity of a sequence number kept in device memory (so a CUDA
// graph that contains the call can be replayed), counters only grow, and a wait that runs out of its
// budget raises the device error word (MB200_ERR_TIMEOUT) and returns instead of hanging.
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace mb200 {
int pdl_enabled();

namespace {

constexpr int kMaxWorld = 8;
constexpr int kPushCtas = 4;        // CTAs of a collective launch; each raises every peer's counter once
constexpr int kPushThreads = 256;
constexpr long long kSpinBudgetNs = 2000000000ll;  // 2 s of wall clock, then MB200_ERR_TIMEOUT

// Receive area of one rank: [2 parities][world sources][max_floats] payload, then the arrival counters
// [2][world] (64-bit, only ever incremented), then the sequence word and a launch ticket.
struct CommBuf {
    float *slots;
    unsigned long long *arrived;
    unsigned long long *seq;     // sequence number of the last completed collective (local use)
    unsigned int *ticket;        // CTAs of the running launch that have finished (local use)
};

struct Comm {
    int rank, world;
    size_t max_floats;
    void *local_base;
    bool ipc = true;             // peers were opened from IPC handles (and are closed on destroy)
    void *peer_base[kMaxWorld];  // peer_base[rank] == local_base
    CommBuf buf[kMaxWorld];
};

size_t slots_bytes(int world, size_t max_floats) { return 2 * (size_t)world * max_floats * sizeof(float); }
size_t comm_bytes(int world, size_t max_floats)
{
    return slots_bytes(world, max_floats) + 2 * (size_t)world * 8 + 64;
}
CommBuf carve(void *base, int world, size_t max_floats)
{
    CommBuf b;
    uint8_t *p = static_cast<uint8_t *>(base);
    b.slots = reinterpret_cast<float *>(p);
    b.arrived = reinterpret_cast<unsigned long long *>(p + slots_bytes(world, max_floats));
    b.seq = b.arrived + 2 * world;
    b.ticket = reinterpret_cast<unsigned int *>(b.seq + 1);
    return b;
}

struct PushParams {
    CommBuf self;
    float *peer_slots[kMaxWorld];
    unsigned long long *peer_arrived[kMaxWorld];
    int rank, world;
    size_t max_floats;
    const float *in;   // this rank's piece
    float *out;        // all-reduce: [n]; all-gather: [world * n] (piece of rank q at q * n)
    int n;             // floats per piece (multiple of 4)
    int reduce;        // 1: sum of the pieces in rank order; 0: concatenation
    int *err;
};

__device__ __forceinline__ void st_release_sys_add(unsigned long long *p)
{
    asm volatile("red.release.sys.global.add.u64 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kPushThreads) push_collective_kernel(const PushParams P)
{
    // the successor may launch at once (it waits for this kernel's completion itself); this kernel waits for
    // the producer of `in`
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ int ok_flag;
    const int tid = threadIdx.x;
    const unsigned long long seq = __ldcg(P.self.seq) + 1;  // the same on every CTA: written only by the last CTA of a launch
    const int par = static_cast<int>(seq & 1);
    const int n4 = P.n >> 2;
    // ---- push: this CTA's share of the piece into every rank's slot for (parity, source = this rank) ----
    const int per = (n4 + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(n4, lo + per);
    const float4 *src = reinterpret_cast<const float4 *>(P.in);
    for (int p = 0; p < P.world; p++) {
        float4 *dst = reinterpret_cast<float4 *>(P.peer_slots[p] + ((size_t)par * P.world + P.rank) * P.max_floats);
        for (int i = lo + tid; i < hi; i += kPushThreads) dst[i] = __ldcg(src + i);
    }
    __threadfence_system();  // the stores above are performed system-wide before the counters move
    __syncthreads();
    if (tid < P.world) st_release_sys_add(P.peer_arrived[tid] + (size_t)par * P.world + P.rank);
    // ---- wait until every source's gridDim.x CTAs have arrived for this sequence number (bounded) ----
    // sequence numbers of one parity are seq, seq - 2, ...: the counter of (parity, source) must reach
    // gridDim.x * ceil(seq / 2)
    if (tid == 0) ok_flag = 1;
    __syncthreads();
    if (tid < P.world) {
        const unsigned long long target = static_cast<unsigned long long>(gridDim.x) * ((seq + 1) >> 1);
        const unsigned long long *ctr = P.self.arrived + (size_t)par * P.world + tid;
        long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        bool ok = false;
        for (unsigned it = 0;; it++) {
            if (ld_acquire_sys(ctr) >= target) {
                ok = true;
                break;
            }
            if ((it & 63) == 63) {
                long long t1;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                if (t1 - t0 > kSpinBudgetNs) break;
            }
        }
        if (!ok) {
            ok_flag = 0;
            atomicExch(P.err, MB200_ERR_TIMEOUT);
        }
    }
    __syncthreads();
    if (ok_flag) {
        const float *slots = P.self.slots + (size_t)par * P.world * P.max_floats;
        if (P.reduce) {
            float4 *out = reinterpret_cast<float4 *>(P.out);
            for (int i = lo + tid; i < hi; i += kPushThreads) {
                float4 a = __ldcg(reinterpret_cast<const float4 *>(slots) + i);
                for (int q = 1; q < P.world; q++) {  // fixed order: every rank computes the same bits
                    const float4 b = __ldcg(reinterpret_cast<const float4 *>(slots + (size_t)q * P.max_floats) + i);
                    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                }
                out[i] = a;
            }
        } else {
            for (int q = 0; q < P.world; q++) {
                float4 *out = reinterpret_cast<float4 *>(P.out + (size_t)q * P.n);
                for (int i = lo + tid; i < hi; i += kPushThreads)
                    out[i] = __ldcg(reinterpret_cast<const float4 *>(slots + (size_t)q * P.max_floats) + i);
            }
        }
    }
    // ---- the last CTA to finish publishes the sequence number for the next launch ----
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(P.self.ticket, 1u) == gridDim.x - 1) {
            *P.self.ticket = 0;
            // after a timeout the sequence still advances, so that the ranks stay in step if the caller retries
            *P.self.seq = seq;
            __threadfence();
        }
    }
}

int launch_push(Comm *c, const float *in, float *out, int n, int reduce, cudaStream_t stream)
{
    if (!c || !in || !out || n < 4 || (n & 3) || static_cast<size_t>(n) > c->max_floats) return MB200_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) return MB200_ERR_ARG;
    PushParams P{};
    P.self = c->buf[c->rank];
    for (int p = 0; p < c->world; p++) {
        P.peer_slots[p] = c->buf[p].slots;
        P.peer_arrived[p] = c->buf[p].arrived;
    }
    P.rank = c->rank;
    P.world = c->world;
    P.max_floats = c->max_floats;
    P.in = in;
    P.out = out;
    P.n = n;
    P.reduce = reduce;
    P.err = device_error_word();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kPushCtas);
    cfg.blockDim = dim3(kPushThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, push_collective_kernel, P) != cudaSuccess) {
        cudaGetLastError();
        return MB200_ERR_LAUNCH;
    }
    return MB200_OK;
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" {

size_t mb200_comm_buffer_bytes(int world, size_t max_floats)
{
    if (world < 1 || world > kMaxWorld || max_floats < 4) return 0;
    return comm_bytes(world, (max_floats + 3) & ~static_cast<size_t>(3));
}

int mb200_comm_alloc(int world, size_t max_floats, void **dev_ptr, void *ipc_handle_64)
{
    const size_t bytes = mb200_comm_buffer_bytes(world, max_floats);
    if (!bytes || !dev_ptr || !ipc_handle_64) return MB200_ERR_ARG;
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return MB200_ERR_LAUNCH;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(p);
        return MB200_ERR_LAUNCH;
    }
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaGetLastError();
        memset(&h, 0, sizeof h);  // single-process use (world 1) does not need the handle
        if (world > 1) {
            cudaFree(p);
            return MB200_ERR_LAUNCH;
        }
    }
    memcpy(ipc_handle_64, &h, sizeof h);
    *dev_ptr = p;
    return MB200_OK;
}

int mb200_comm_create(int rank, int world, size_t max_floats, void *local_ptr, const void *ipc_handles_64,
                      void **comm_out)
{
    if (rank < 0 || world < 1 || world > kMaxWorld || rank >= world || !local_ptr || !comm_out || max_floats < 4)
        return MB200_ERR_ARG;
    if (world > 1 && !ipc_handles_64) return MB200_ERR_ARG;
    Comm *c = new Comm();
    c->rank = rank;
    c->world = world;
    c->max_floats = (max_floats + 3) & ~static_cast<size_t>(3);
    c->local_base = local_ptr;
    for (int p = 0; p < world; p++) {
        void *base = local_ptr;
        if (p != rank) {
            cudaIpcMemHandle_t h;
            memcpy(&h, static_cast<const uint8_t *>(ipc_handles_64) + 64 * (size_t)p, sizeof h);
            if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                fprintf(stderr, "[mnemo_b200] mb200_comm_create: cannot open the buffer of rank %d: %s\n", p,
                        cudaGetErrorString(cudaGetLastError()));
                for (int q = 0; q < p; q++)
                    if (q != rank) cudaIpcCloseMemHandle(c->peer_base[q]);
                delete c;
                return MB200_ERR_LAUNCH;
            }
        }
        c->peer_base[p] = base;
        c->buf[p] = carve(base, world, c->max_floats);
    }
    *comm_out = c;
    return MB200_OK;
}

int mb200_comm_create_ptrs(int rank, int world, size_t max_floats, void *const *bases, void **comm_out)
{
    if (rank < 0 || world < 1 || world > kMaxWorld || rank >= world || !bases || !comm_out || max_floats < 4)
        return MB200_ERR_ARG;
    for (int p = 0; p < world; p++)
        if (!bases[p] || (reinterpret_cast<uintptr_t>(bases[p]) & 15)) return MB200_ERR_ARG;
    Comm *c = new Comm();
    c->rank = rank;
    c->world = world;
    c->max_floats = (max_floats + 3) & ~static_cast<size_t>(3);
    c->local_base = bases[rank];
    c->ipc = false;
    for (int p = 0; p < world; p++) {
        c->peer_base[p] = bases[p];
        c->buf[p] = carve(bases[p], world, c->max_floats);
    }
    *comm_out = c;
    return MB200_OK;
}

void mb200_comm_destroy(void *comm, int free_local)
{
    Comm *c = static_cast<Comm *>(comm);
    if (!c) return;
    for (int p = 0; p < c->world; p++)
        if (c->ipc && p != c->rank) cudaIpcCloseMemHandle(c->peer_base[p]);
    if (free_local) cudaFree(c->local_base);
    delete c;
}

int mb200_push_allreduce(void *comm, const float *in, float *out, int n, cudaStream_t stream)
{
    return launch_push(static_cast<Comm *>(comm), in, out, n, 1, stream);
}

int mb200_push_allgather(void *comm, const float *in, float *out, int n_per_rank, cudaStream_t stream)
{
    return launch_push(static_cast<Comm *>(comm), in, out, n_per_rank, 0, stream);
}

}  // extern "C"
