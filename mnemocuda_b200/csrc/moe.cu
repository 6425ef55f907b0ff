// Decode-time MoE block with the routed expert ids kept on the device.
//
// The reference selects experts on the GPU, copies the k ids and weights to
// the host, synchronises, and then issues 3-4 launches per expert
// (src/forward.c:818-882, 1122-1142). With every expert resident in HBM the
// ids never need to leave the device: three launches do the whole block --
//   1. router logits (fp32 matvec) + top-k + softmax in one kernel,
//   2. gate/up + SwiGLU of all routed experts (stream kernel, mode kMoeGateUp),
//   3. down projections of all routed experts, weighted sum and residual add
//      (stream kernel, mode kMoeDown),
// and the sequence can be captured in a CUDA graph.
#include <cstdio>
#include <cstring>

#include "comm.cuh"
#include "topk.cuh"

namespace mb200 {

void moe_gate_up_q4k(const void *experts, size_t stride, size_t gate_off, size_t up_off, const int *ids, int n_slots,
                     int expert_lo, int expert_cnt, const float *x, float *act, int EFF, int H, cudaStream_t stream,
                     const char *where);
void moe_down_q4k(const void *experts, size_t stride, size_t down_off, const int *ids, const float *wts, int n_slots,
                  int expert_lo, int expert_cnt, const float *act, const float *residual, float *y, int H, int EFF,
                  cudaStream_t stream, const char *where);
void moe_down_q6k(const void *experts, size_t stride, size_t down_off, const int *ids, const float *wts, int n_slots,
                  int expert_lo, int expert_cnt, const float *act, const float *residual, float *y, int H, int EFF,
                  cudaStream_t stream, const char *where);
int pdl_enabled();
int moe_fused(const void *experts, size_t stride, size_t gate_off, size_t up_off, size_t down_off, int down_type,
              const int *ids, const float *wts, int n_slots, int expert_lo, int expert_cnt, const float *x, float *act,
              const float *residual, float *y, int H, int EFF, unsigned long long *sync, cudaStream_t stream,
              const float *router_w, int n_experts, float *logits, int *ids_out, float *wts_out, const float *norm_w,
              float norm_eps, const PushDesc *push = nullptr);
void launch_rms_norm(const float *in, const float *w, float *out, float *res_out, int n, float eps, cudaStream_t stream);
void moe_fused_set_mode(int mode);
int moe_fused_mode();

namespace {

constexpr int kRouterThreads = 128;

// One CTA per expert row computes its logit; the CTA that finishes last (device-wide
// ticket in scratch[0]) runs the reference's top-k + softmax over all logits.
// scratch: int ticket (zero before the first use; the kernel leaves it zero) followed by
// n_experts floats of logits starting at scratch + 8 words.
template <bool PDL>
__global__ void __launch_bounds__(kRouterThreads) router_topk_kernel(const float *__restrict__ w,
                                                                      const float *__restrict__ x, int *scratch,
                                                                      int *__restrict__ indices,
                                                                      float *__restrict__ weights, int n_experts,
                                                                      int n_cols, int k, int vec_ok)
{
    __shared__ float red[kRouterThreads / 32];
    __shared__ int is_last;
    __shared__ TopkShared topk_sh;
    float *logits = reinterpret_cast<float *>(scratch + 8);
    const int row = blockIdx.x;
    const float *wr = w + (size_t)row * n_cols;
    float acc = 0.0f;
    if (vec_ok) {
        // the router weights do not depend on the upstream kernel: fetch them before waiting for it
        const float4 *w4 = reinterpret_cast<const float4 *>(wr);
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        const int n4 = n_cols >> 2;
        bool waited = false;
        for (int i0 = threadIdx.x; i0 < n4; i0 += kRouterThreads * 8) {
            float4 a[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * kRouterThreads;
                a[u] = i < n4 ? __ldcs(w4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (PDL && !waited) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * kRouterThreads;
                if (i < n4) {
                    const float4 b = __ldcg(x4 + i);  // produced upstream: from L2, never the non-coherent path
                    acc = fmaf(a[u].x, b.x, acc);
                    acc = fmaf(a[u].y, b.y, acc);
                    acc = fmaf(a[u].z, b.z, acc);
                    acc = fmaf(a[u].w, b.w, acc);
                }
            }
        }
        if (PDL && !waited) asm volatile("griddepcontrol.wait;" ::: "memory");
    } else {
        if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int c = threadIdx.x; c < n_cols; c += kRouterThreads) acc = fmaf(wr[c], __ldcg(x + c), acc);
    }
    if (PDL) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        logits[row] = (red[0] + red[1]) + (red[2] + red[3]);
        __threadfence();
        const int ticket = atomicAdd(scratch, 1);
        is_last = (ticket == n_experts - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // the whole CTA: the candidate rows are counted by its four warps side by side
    topk_softmax_block(const_cast<const float *>(static_cast<volatile float *>(logits)), indices, weights, n_experts, k,
                       topk_sh);
    if (threadIdx.x == 0) scratch[0] = 0;  // ready for the next call
}

}  // namespace

int launch_router(const float *router_w, const float *x, void *scratch, int *ids, float *wts, int n_experts, int H,
                  int k, cudaStream_t stream)
{
    const int vec_ok = (H % 4 == 0) && ((reinterpret_cast<uintptr_t>(router_w) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_experts);
    cfg.blockDim = dim3(kRouterThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    const int pdl = pdl_enabled();
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e;
    if (pdl)
        e = cudaLaunchKernelEx(&cfg, router_topk_kernel<true>, router_w, x, static_cast<int *>(scratch), ids, wts,
                               n_experts, H, k, vec_ok);
    else
        e = cudaLaunchKernelEx(&cfg, router_topk_kernel<false>, router_w, x, static_cast<int *>(scratch), ids, wts,
                               n_experts, H, k, vec_ok);
    return e == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

// ---- scratch that lives in the library image (for mb200_router_topk_static) ----
// Ticket word + logits, same layout as the caller-provided scratch of mb200_router_topk.
// One copy exists on every device that loads the library, for the life of the process.
constexpr int kStaticRouterMaxExperts = 1024;
static __device__ __align__(256) int g_router_scratch[8 + kStaticRouterMaxExperts];
static int *g_router_scratch_ptr[kMaxDevices] = {nullptr};  // device address of the array, per device ordinal

// The array's name is only a host-side handle; kernels need its device address, which the
// runtime hands out per device. Looked up once per device, with that device current.
static int *static_router_scratch()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!g_router_scratch_ptr[dev]) {
        int *ptr = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_router_scratch) != cudaSuccess) return nullptr;
        g_router_scratch_ptr[dev] = ptr;
    }
    return g_router_scratch_ptr[dev];
}

// cuda_kernels_init() resolves the array on the current device, so that an engine that initialises
// each device at load never pays the lookup (and the module load behind it) on a hot call.
void router_static_init() { (void)static_router_scratch(); }

}  // namespace mb200

namespace mb200 {
namespace {
// x and the residual from mapped host memory into device memory: volatile loads (the host rewrites the buffer
// between calls; nothing of it may be served from a cache), one 16-byte load per thread and round.
__global__ void __launch_bounds__(1024) host_stage_in_kernel(const float4 *src, float4 *dst, int n4)
{
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        float4 v;
        asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                     : "l"(src + i));
        dst[i] = v;
    }
}

// Last node of a host call: the kernels before it have completed (stream order), so the result rows are on their
// way to host memory ahead of this store; the host spins on the word instead of asking the driver to wait.
__global__ void host_signal_kernel(unsigned int *dev_counter, volatile unsigned int *host_flag)
{
    const unsigned int v = *dev_counter + 1;
    *dev_counter = v;
    __threadfence_system();
    *host_flag = v;
}

// Per device: the completion word (mapped host memory) and its device-side counter; and the instantiated graphs
// of recent host calls. A host call is a fixed little sequence of launches whose arguments repeat from token to
// token (same layer, same buffers): replaying an instantiated graph costs one driver call instead of three
// launches. Keyed by every argument; least recently used entry replaced.
struct HostKey {
    const void *router_w, *experts, *d_in, *d_out, *dev_io, *ids, *wts, *act, *scratch;
    size_t stride, gate_sz, up_sz;
    int down_type, n_experts, expert_lo, cnt, k, H, EFF, fused, pdl;
    cudaStream_t stream;
    bool operator==(const HostKey &o) const { return memcmp(this, &o, sizeof(HostKey)) == 0; }
};
struct HostEntry {
    HostKey key;
    cudaGraphExec_t exec;
    unsigned long long used;
};
constexpr int kHostEntries = 64;
struct HostState {
    volatile unsigned int *flag = nullptr;  // mapped host word
    unsigned int *flag_dev = nullptr;       // its device alias
    unsigned int *counter = nullptr;        // device counter
    unsigned int expected = 0;
    unsigned long long tick = 0;
    int n = 0;
    HostEntry e[kHostEntries];
};
HostState g_host[kMaxDevices];

bool host_state_ready(HostState &st)
{
    if (st.flag) return true;
    void *h = nullptr, *d = nullptr, *c = nullptr;
    if (cudaHostAlloc(&h, 64, cudaHostAllocMapped) != cudaSuccess) return false;
    memset(h, 0, 64);
    if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess || cudaMalloc(&c, 64) != cudaSuccess || cudaMemset(c, 0, 64) != cudaSuccess) {
        cudaFreeHost(h);
        (void)cudaGetLastError();
        return false;
    }
    st.flag = static_cast<volatile unsigned int *>(h);
    st.flag_dev = static_cast<unsigned int *>(d);
    st.counter = static_cast<unsigned int *>(c);
    return true;
}
}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" {

// ticket + padding (8 words), the logits, then (16-byte aligned) the 64 bytes of barrier counters that
// mb200_moe_block hands to the fused expert kernel
static size_t router_part_bytes(int n_experts)
{
    return (sizeof(int) * 8 + sizeof(float) * (size_t)(n_experts > 0 ? n_experts : 0) + 15) & ~static_cast<size_t>(15);
}
size_t mb200_router_scratch_bytes(int n_experts) { return router_part_bytes(n_experts) + 64; }

int mb200_router_topk(const float *router_w, const float *x, void *scratch, int *indices, float *weights,
                      int n_experts, int n_cols, int k, cudaStream_t stream)
{
    if (!router_w || !x || !scratch || !indices || !weights || n_experts < 1 || n_cols < 1 || k < 1 || k > 16)
        return MB200_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(scratch) & 15) return MB200_ERR_ARG;
    return launch_router(router_w, x, scratch, indices, weights, n_experts, n_cols, k, stream);
}

int mb200_router_topk_static(const float *router_w, const float *x, int *indices, float *weights, int n_experts,
                             int n_cols, int k, cudaStream_t stream)
{
    if (!router_w || !x || !indices || !weights || n_experts < 1 || n_cols < 1 || k < 1 || k > 16) return MB200_ERR_ARG;
    if (n_experts > kStaticRouterMaxExperts) {
        fprintf(stderr, "[mnemo_b200] mb200_router_topk_static: n_experts=%d exceeds the built-in scratch (max %d); "
                        "use mb200_router_topk with caller-provided scratch\n", n_experts, kStaticRouterMaxExperts);
        return MB200_ERR_UNSUPPORTED;
    }
    int *scratch = static_router_scratch();
    if (!scratch) {
        fprintf(stderr, "[mnemo_b200] mb200_router_topk_static: could not resolve the built-in scratch on this device\n");
        return MB200_ERR_LAUNCH;
    }
    // The array keeps whatever the previous call left; the ticket must start at zero.
    if (cudaMemsetAsync(scratch, 0, sizeof(int), stream) != cudaSuccess) return MB200_ERR_LAUNCH;
    return launch_router(router_w, x, scratch, indices, weights, n_experts, n_cols, k, stream);
}

int mb200_moe_gate_up_local(const void *experts, size_t expert_stride, size_t gate_off, size_t up_off, const int *ids,
                            int n_slots, int expert_lo, int expert_cnt, const float *x, float *act, int EFF, int H,
                            cudaStream_t stream)
{
    if (!experts || !ids || !x || !act || n_slots < 1 || n_slots > 16 || EFF < 1 || H < 1 || expert_lo < 0 ||
        expert_cnt < 0)
        return MB200_ERR_ARG;
    mb200_clear_status();
    moe_gate_up_q4k(experts, expert_stride, gate_off, up_off, ids, n_slots, expert_lo, expert_cnt, x, act, EFF, H,
                    stream, "mb200_moe_gate_up");
    return mb200_last_status();
}

int mb200_moe_gate_up(const void *experts, size_t expert_stride, size_t gate_off, size_t up_off, const int *ids,
                      int n_slots, const float *x, float *act, int EFF, int H, cudaStream_t stream)
{
    return mb200_moe_gate_up_local(experts, expert_stride, gate_off, up_off, ids, n_slots, 0, 0x7fffffff, x, act, EFF,
                                   H, stream);
}

int mb200_moe_down_local(const void *experts, size_t expert_stride, size_t down_off, int down_type, const int *ids,
                         const float *wts, int n_slots, int expert_lo, int expert_cnt, const float *act,
                         const float *residual, float *y, int H, int EFF, cudaStream_t stream)
{
    if (!experts || !ids || !wts || !act || !y || n_slots < 1 || n_slots > 16 || EFF < 1 || H < 1 || expert_lo < 0 ||
        expert_cnt < 0)
        return MB200_ERR_ARG;
    if (down_type != 12 && down_type != 14) return MB200_ERR_UNSUPPORTED;
    mb200_clear_status();
    if (down_type == 14)
        moe_down_q6k(experts, expert_stride, down_off, ids, wts, n_slots, expert_lo, expert_cnt, act, residual, y, H,
                     EFF, stream, "mb200_moe_down");
    else
        moe_down_q4k(experts, expert_stride, down_off, ids, wts, n_slots, expert_lo, expert_cnt, act, residual, y, H,
                     EFF, stream, "mb200_moe_down");
    return mb200_last_status();
}

int mb200_moe_down(const void *experts, size_t expert_stride, size_t down_off, int down_type, const int *ids,
                   const float *wts, int n_slots, const float *act, const float *residual, float *y, int H, int EFF,
                   cudaStream_t stream)
{
    return mb200_moe_down_local(experts, expert_stride, down_off, down_type, ids, wts, n_slots, 0, 0x7fffffff, act,
                                residual, y, H, EFF, stream);
}

void mb200_set_fused(int mode) { moe_fused_set_mode(mode < 0 ? 0 : (mode > 2 ? 2 : mode)); }

int mb200_moe_experts_fused(const void *experts, size_t expert_stride, size_t gate_off, size_t up_off, size_t down_off,
                            int down_type, const int *ids, const float *wts, int n_slots, int expert_lo, int expert_cnt,
                            const float *x, float *act, const float *residual, float *y, int H, int EFF, void *sync,
                            cudaStream_t stream)
{
    if (!experts || !ids || !wts || !x || !act || !y || !sync || n_slots < 1 || EFF < 1 || H < 1 || expert_lo < 0 ||
        expert_cnt < 0)
        return MB200_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(sync) & 7) return MB200_ERR_ARG;
    return moe_fused(experts, expert_stride, gate_off, up_off, down_off, down_type, ids, wts, n_slots, expert_lo,
                     expert_cnt, x, act, residual, y, H, EFF, static_cast<unsigned long long *>(sync), stream, nullptr, 0,
                     nullptr, nullptr, nullptr, nullptr, 0.0f);
}

int mb200_moe_block_local(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz,
                          size_t up_sz, int down_type, int n_experts, int expert_lo, int expert_cnt, int k, int H,
                          int EFF, const float *x, const float *residual, float *out, int *ids, float *wts, float *act,
                          void *scratch, cudaStream_t stream)
{
    return mb200_moe_block_norm(router_w, experts, expert_stride, gate_sz, up_sz, down_type, n_experts, expert_lo, expert_cnt,
                                k, H, EFF, x, nullptr, 0.0f, nullptr, residual, out, ids, wts, act, scratch, stream);
}

int mb200_moe_block_push(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz, size_t up_sz,
                         int down_type, int n_experts, int expert_lo, int expert_cnt, int k, int H, int EFF,
                         const float *x, const float *norm_w, float norm_eps, const float *residual, float *out, int *ids,
                         float *wts, float *act, void *scratch, void *comm, cudaStream_t stream)
{
    if (!router_w || !x || !scratch || !ids || !wts || !act || !out || !comm || n_experts < 1 || H < 1 || k < 1 || k > 16 ||
        expert_lo < 0 || expert_cnt < 0)
        return MB200_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(scratch) & 15) return MB200_ERR_ARG;
    if (moe_fused_mode() != 2) return MB200_ERR_UNSUPPORTED;
    PushDesc d;
    if (!comm_describe(comm, &d)) return MB200_ERR_ARG;
    unsigned long long *sync =
        reinterpret_cast<unsigned long long *>(static_cast<char *>(scratch) + router_part_bytes(n_experts));
    float *logits = reinterpret_cast<float *>(static_cast<int *>(scratch) + 8);
    return moe_fused(experts, expert_stride, 0, gate_sz, gate_sz + up_sz, down_type, nullptr, nullptr, k, expert_lo,
                     expert_cnt, x, act, residual, out, H, EFF, sync, stream, router_w, n_experts, logits, ids, wts, norm_w,
                     norm_eps, &d);
}

int mb200_moe_block_norm(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz, size_t up_sz,
                         int down_type, int n_experts, int expert_lo, int expert_cnt, int k, int H, int EFF,
                         const float *x, const float *norm_w, float norm_eps, float *normed_scratch,
                         const float *residual, float *out, int *ids, float *wts, float *act, void *scratch,
                         cudaStream_t stream)
{
    if (!router_w || !x || !scratch || !ids || !wts || n_experts < 1 || H < 1 || k < 1 || k > 16 || expert_lo < 0 ||
        expert_cnt < 0)
        return MB200_ERR_ARG;
    if (norm_w && !normed_scratch) return MB200_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(scratch) & 15) return MB200_ERR_ARG;
    // the last 64 bytes of the scratch are the fused kernel's barrier counters
    unsigned long long *sync =
        reinterpret_cast<unsigned long long *>(static_cast<char *>(scratch) + router_part_bytes(n_experts));
    float *logits = reinterpret_cast<float *>(static_cast<int *>(scratch) + 8);
    int rc;
    if (moe_fused_mode() == 2 && act) {
        // one launch: routing, gate/up, down
        rc = moe_fused(experts, expert_stride, 0, gate_sz, gate_sz + up_sz, down_type, nullptr, nullptr, k, expert_lo,
                       expert_cnt, x, act, residual, out, H, EFF, sync, stream, router_w, n_experts, logits, ids, wts,
                       norm_w, norm_eps);
        // not covered, or the device refused the cooperative launch (fewer SMs available than the grid
        // needs): nothing ran, the separate kernels below do the block
        if (rc != MB200_ERR_UNSUPPORTED && rc != MB200_ERR_LAUNCH) return rc;
    }
    if (norm_w) {  // the other forms take the normalised vector from memory: one small kernel more
        launch_rms_norm(x, norm_w, normed_scratch, nullptr, H, norm_eps, stream);
        x = normed_scratch;
    }
    rc = mb200_router_topk(router_w, x, scratch, ids, wts, n_experts, H, k, stream);
    if (rc != MB200_OK) return rc;
    if (moe_fused_mode() && act) {
        rc = moe_fused(experts, expert_stride, 0, gate_sz, gate_sz + up_sz, down_type, ids, wts, k, expert_lo, expert_cnt,
                       x, act, residual, out, H, EFF, sync, stream, nullptr, 0, nullptr, nullptr, nullptr, nullptr, 0.0f);
        if (rc != MB200_ERR_UNSUPPORTED && rc != MB200_ERR_LAUNCH) return rc;
    }
    rc = mb200_moe_gate_up_local(experts, expert_stride, 0, gate_sz, ids, k, expert_lo, expert_cnt, x, act, EFF, H,
                                 stream);
    if (rc != MB200_OK) return rc;
    return mb200_moe_down_local(experts, expert_stride, gate_sz + up_sz, down_type, ids, wts, k, expert_lo, expert_cnt,
                                act, residual, out, H, EFF, stream);
}

int mb200_moe_block_host(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz,
                         size_t up_sz, int down_type, int n_experts, int expert_lo, int expert_cnt, int k, int H,
                         int EFF, const float *host_x_res, float *host_out, float *dev_io, int *ids, float *wts,
                         float *act, void *scratch, cudaStream_t stream)
{
    if (!host_x_res || !host_out || !dev_io || H < 1) return MB200_ERR_ARG;
    const int cnt = expert_cnt > 0 ? expert_cnt : 0x7fffffff;
    // Pinned (page-locked, mapped) host buffers are reachable from the device: a one-CTA kernel pulls x and the
    // residual across PCIe into dev_io (one round trip instead of a copy-engine launch), the block writes its
    // result rows straight into the host buffer (each row is written once), and a last one-thread kernel raises a
    // word in host memory that this call spins on. The launches of a call are kept as an instantiated graph per
    // argument set, so a repeated call (the same layer and buffers, token after token) is one graph launch.
    void *d_in = nullptr, *d_out = nullptr;
    const bool mapped = (H % 4 == 0) && cudaHostGetDevicePointer(&d_in, const_cast<float *>(host_x_res), 0) == cudaSuccess &&
                        cudaHostGetDevicePointer(&d_out, host_out, 0) == cudaSuccess;
    if (mapped) {
        HostState &st = g_host[current_device()];
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        const bool plain = !host_state_ready(st) || cudaStreamIsCapturing(stream, &cap) != cudaSuccess ||
                           cap != cudaStreamCaptureStatusNone;
        auto enqueue = [&](bool signal) -> int {
            host_stage_in_kernel<<<1, 1024, 0, stream>>>(static_cast<const float4 *>(d_in), reinterpret_cast<float4 *>(dev_io),
                                                         2 * H / 4);
            const int rc = mb200_moe_block_local(router_w, experts, expert_stride, gate_sz, up_sz, down_type, n_experts,
                                                 expert_lo, cnt, k, H, EFF, dev_io, dev_io + H, static_cast<float *>(d_out),
                                                 ids, wts, act, scratch, stream);
            if (rc == MB200_OK && signal) host_signal_kernel<<<1, 1, 0, stream>>>(st.counter, st.flag_dev);
            return rc;
        };
        if (plain) {  // no completion word, or the caller is capturing this stream itself
            const int rc = enqueue(false);
            if (rc != MB200_OK) return rc;
            return cudaStreamSynchronize(stream) == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
        }
        HostKey key;
        memset(&key, 0, sizeof(key));
        key.router_w = router_w; key.experts = experts; key.d_in = d_in; key.d_out = d_out; key.dev_io = dev_io;
        key.ids = ids; key.wts = wts; key.act = act; key.scratch = scratch;
        key.stride = expert_stride; key.gate_sz = gate_sz; key.up_sz = up_sz;
        key.down_type = down_type; key.n_experts = n_experts; key.expert_lo = expert_lo; key.cnt = cnt; key.k = k;
        key.H = H; key.EFF = EFF; key.fused = moe_fused_mode(); key.pdl = pdl_enabled(); key.stream = stream;
        HostEntry *hit = nullptr;
        for (int i = 0; i < st.n; i++)
            if (st.e[i].key == key) hit = &st.e[i];
        bool direct = false;
        if (!hit && cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            (void)cudaGetLastError();  // the legacy default stream cannot be captured: plain launches, same completion word
            direct = true;
        }
        if (direct) {
            const int rc = enqueue(true);
            if (rc != MB200_OK) return rc;
        } else if (!hit) {
            const int rc = enqueue(true);
            cudaGraph_t graph = nullptr;
            const cudaError_t ce = cudaStreamEndCapture(stream, &graph);
            if (rc != MB200_OK || ce != cudaSuccess || !graph) {
                if (graph) cudaGraphDestroy(graph);
                (void)cudaGetLastError();
                return rc != MB200_OK ? rc : MB200_ERR_LAUNCH;
            }
            cudaGraphExec_t exec = nullptr;
            const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (ie != cudaSuccess) return MB200_ERR_LAUNCH;
            int slot = st.n;
            if (st.n < kHostEntries) {
                st.n++;
            } else {  // replace the least recently used
                slot = 0;
                for (int i = 1; i < kHostEntries; i++)
                    if (st.e[i].used < st.e[slot].used) slot = i;
                cudaGraphExecDestroy(st.e[slot].exec);
            }
            st.e[slot].key = key;
            st.e[slot].exec = exec;
            hit = &st.e[slot];
        }
        if (!direct) {
            hit->used = ++st.tick;
            if (cudaGraphLaunch(hit->exec, stream) != cudaSuccess) return MB200_ERR_LAUNCH;
        }
        const unsigned int want = ++st.expected;
        // spin on the completion word (bounded: two seconds, then ask the driver)
        for (unsigned long long spins = 0;; spins++) {
            if (*st.flag == want) return MB200_OK;
            if ((spins & 0xFFFFF) == 0xFFFFF) {
                if (cudaStreamQuery(stream) != cudaErrorNotReady) break;  // finished (or failed) without the word matching
                if (spins > (1ull << 33)) break;
            }
        }
        const cudaError_t se = cudaStreamSynchronize(stream);
        st.expected = *st.flag;  // re-align with the device counter
        return se == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
    }
    (void)cudaGetLastError();  // pageable buffers: the query above failed, which is not an error of this call
    // one copy in (x and the residual are adjacent), the block, one copy out, one wait
    if (cudaMemcpyAsync(dev_io, host_x_res, sizeof(float) * 2 * (size_t)H, cudaMemcpyHostToDevice, stream) != cudaSuccess)
        return MB200_ERR_LAUNCH;
    const int rc = mb200_moe_block_local(router_w, experts, expert_stride, gate_sz, up_sz, down_type, n_experts, expert_lo,
                                         cnt, k, H, EFF, dev_io, dev_io + H, dev_io + 2 * (size_t)H, ids, wts, act, scratch,
                                         stream);
    if (rc != MB200_OK) return rc;
    if (cudaMemcpyAsync(host_out, dev_io + 2 * (size_t)H, sizeof(float) * (size_t)H, cudaMemcpyDeviceToHost, stream) !=
        cudaSuccess)
        return MB200_ERR_LAUNCH;
    return cudaStreamSynchronize(stream) == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

int mb200_moe_block(const float *router_w, const void *experts, size_t expert_stride, size_t gate_sz, size_t up_sz,
                    int down_type, int n_experts, int k, int H, int EFF, const float *x, const float *residual,
                    float *out, int *ids, float *wts, float *act, void *scratch, cudaStream_t stream)
{
    return mb200_moe_block_local(router_w, experts, expert_stride, gate_sz, up_sz, down_type, n_experts, 0, 0x7fffffff, k,
                                 H, EFF, x, residual, out, ids, wts, act, scratch, stream);
}

}  // extern "C"
