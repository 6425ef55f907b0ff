// Push collectives over NVLink peer memory for the tiny vectors of a sharded decode step.
//
// The reference's only multi-GPU traffic is one hidden vector copied from GPU to GPU at each layer-range
// boundary (cudaMemcpyPeerAsync, src/forward.c:1555-1581). Sharding the work itself (rows of a matvec,
// experts of a MoE block) needs an all-gather / all-reduce of 16-32 KB several times per layer: far too
// small for a bandwidth-oriented collective, so the cost is latency. Here every rank STORES its piece
// straight into every peer's receive buffer (plain 8-byte peer stores through NVSwitch; no bulk / TMA
// copy and no multicast touches peer memory). Every float travels with the collective's sequence number
// in the same 8-byte store, so the receiver needs no fence and no separate flag: it spins on its own
// local cells (bounded) until they carry the number, then sums the pieces in rank order -- deterministic,
// identical on every rank -- or just concatenates them (all-gather). One one-way NVLink trip per piece.
//
// One process per GPU. Buffers are cudaMalloc'ed here and shared through CUDA IPC handles that the host
// side exchanges (torch.distributed, or anything else); the library itself never talks to other ranks.
// Receive cells are double-buffered by the parity of the sequence number, which is kept in device memory
// (so a CUDA graph that contains the call can be replayed); a rank can be at most one collective ahead of
// the slowest one, so a cell is never overwritten before it has been read. A wait that runs out of its
// budget raises the device error word (MB200_ERR_TIMEOUT) and returns instead of hanging.
#include <cstdio>
#include <cstring>

#include "comm.cuh"

namespace mb200 {
int pdl_enabled();

namespace {

constexpr int kPushCtas = 8;
constexpr int kPushThreads = 256;

// Receive area of one rank: [2 parities][world sources][max_floats] cells of 8 bytes -- a float and the
// 32-bit sequence number of the collective that wrote it, stored together with ONE 8-byte store (single-copy
// atomic, also across NVLink), so a cell whose number matches is valid: no fence, no separate flag, one
// one-way trip per piece. Then the sequence word and a launch ticket (local use).
struct CommBuf {
    uint2 *cells;
    unsigned long long *seq;     // sequence number of the last completed collective
    unsigned int *ticket;        // CTAs of the running launch that have finished
};

struct Comm {
    int rank, world;
    size_t max_floats;
    void *local_base;
    bool ipc = true;             // peers were opened from IPC handles (and are closed on destroy)
    void *peer_base[kMaxWorld];  // peer_base[rank] == local_base
    CommBuf buf[kMaxWorld];
};

size_t cells_bytes(int world, size_t max_floats) { return 2 * (size_t)world * max_floats * sizeof(uint2); }
size_t comm_bytes(int world, size_t max_floats) { return cells_bytes(world, max_floats) + 64; }
CommBuf carve(void *base, int world, size_t max_floats)
{
    CommBuf b;
    uint8_t *p = static_cast<uint8_t *>(base);
    b.cells = reinterpret_cast<uint2 *>(p);
    b.seq = reinterpret_cast<unsigned long long *>(p + cells_bytes(world, max_floats));
    b.ticket = reinterpret_cast<unsigned int *>(b.seq + 1);
    return b;
}

struct PushParams {
    CommBuf self;
    uint2 *peer_cells[kMaxWorld];
    int rank, world;
    size_t max_floats;
    const float *in;   // this rank's piece
    float *out;        // all-reduce: [n]; all-gather: [world * n] (piece of rank q at q * n)
    int n;             // floats per piece
    int reduce;        // 1: sum of the pieces in rank order; 0: concatenation
    int *err;
};

__global__ void __launch_bounds__(kPushThreads) push_collective_kernel(const PushParams P)
{
    // the successor may launch at once (it waits for this kernel's completion itself); this kernel waits for
    // the producer of `in`
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int tid = blockIdx.x * kPushThreads + threadIdx.x, nthr = gridDim.x * kPushThreads;
    const unsigned long long seq = __ldcg(P.self.seq) + 1;  // the same on every CTA: written only by the last CTA of a launch
    const uint32_t tag = static_cast<uint32_t>(seq);        // never 0 in the first 2^32 collectives; the buffers start zeroed
    const size_t par_off = (size_t)(seq & 1) * P.world * P.max_floats;
    // ---- push: element i of this rank's piece into cell (parity, source = this rank, i) of every rank ----
    for (int i = tid; i < P.n; i += nthr) {
        const float v = __ldcg(P.in + i);
#pragma unroll 1
        for (int p = 0; p < P.world; p++) st_cell(P.peer_cells[p] + par_off + (size_t)P.rank * P.max_floats + i, v, tag);
    }
    // ---- receive: the same elements from every source, as they land ----
    long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool ok = true;
    const uint2 *mine = P.self.cells + par_off;
    for (int i = tid; i < P.n && ok; i += nthr) {
        float v[kMaxWorld];
        if (!wait_cells(mine + i, P.max_floats, P.world, tag, v, t0)) {
            ok = false;
            break;
        }
        if (P.reduce) {
            float acc = v[0];
#pragma unroll
            for (int q = 1; q < kMaxWorld; q++)  // fixed order: every rank computes the same bits
                if (q < P.world) acc += v[q];
            P.out[i] = acc;
        } else {
#pragma unroll
            for (int q = 0; q < kMaxWorld; q++)
                if (q < P.world) P.out[(size_t)q * P.n + i] = v[q];
        }
    }
    if (!ok) atomicExch(P.err, MB200_ERR_TIMEOUT);
    // ---- the last CTA to finish publishes the sequence number for the next launch ----
    __syncthreads();
    if (threadIdx.x == 0) {
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
    if (!c || !in || !out || n < 1 || static_cast<size_t>(n) > c->max_floats) return MB200_ERR_ARG;
    PushParams P{};
    P.self = c->buf[c->rank];
    for (int p = 0; p < c->world; p++) P.peer_cells[p] = c->buf[p].cells;
    P.rank = c->rank;
    P.world = c->world;
    P.max_floats = c->max_floats;
    P.in = in;
    P.out = out;
    P.n = n;
    P.reduce = reduce;
    P.err = device_error_word();
    cudaLaunchConfig_t cfg = {};
    int ctas = (n + kPushThreads * 2 - 1) / (kPushThreads * 2);  // two elements per thread
    ctas = ctas < 1 ? 1 : (ctas > kPushCtas ? kPushCtas : ctas);
    cfg.gridDim = dim3(ctas);
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

bool comm_describe(void *comm, PushDesc *d)
{
    const Comm *c = static_cast<const Comm *>(comm);
    if (!c || !d) return false;
    for (int p = 0; p < kMaxWorld; p++) d->peer_cells[p] = p < c->world ? c->buf[p].cells : nullptr;
    d->self_cells = c->buf[c->rank].cells;
    d->seq = c->buf[c->rank].seq;
    d->ticket = c->buf[c->rank].ticket;
    d->rank = c->rank;
    d->world = c->world;
    d->max_floats = c->max_floats;
    return true;
}

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
