// Library-wide state: status of the last failure, the per-device error word that
// kernels raise when a bounded wait runs out, and one-time initialisation.
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace mb200 {

void q4k_init();
void q6k_init();
void pair_init();
void other_types_init();
void gemm_init();
void moe_fused_init();
void router_static_init();
void support_init();

namespace {
int g_status = MB200_OK;
char g_where[96] = "";
__device__ int g_device_error;  // one copy per device that loads the library
int *g_err_ptr[kMaxDevices] = {nullptr};
int g_sms[kMaxDevices] = {0};
}  // namespace

int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    return dev;
}

int device_sms()
{
    const int dev = current_device();
    if (!g_sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = kSMs;
        g_sms[dev] = n;
    }
    return g_sms[dev];
}

void set_status(int code, const char *where)
{
    if (g_status == MB200_OK) {
        g_status = code;
        snprintf(g_where, sizeof g_where, "%s", where ? where : "");
    }
}

// Address of the current device's error word. The first call on a device asks
// the runtime for the symbol's address; cuda_kernels_init() makes that call so
// it never happens during stream capture.
int *device_error_word()
{
    const int dev = current_device();
    if (!g_err_ptr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_error) != cudaSuccess) {
            set_status(MB200_ERR_LAUNCH, "cudaGetSymbolAddress(g_device_error)");
            return nullptr;
        }
        g_err_ptr[dev] = static_cast<int *>(p);
    }
    return g_err_ptr[dev];
}

}  // namespace mb200

using namespace mb200;

extern "C" {

void cuda_kernels_init(void)
{
    // Everything here is per device: call once per device the engine drives, with that device current.
    q4k_init();
    q6k_init();
    pair_init();
    other_types_init();
    gemm_init();
    moe_fused_init();
    support_init();
    router_static_init();
    (void)device_sms();
    (void)device_error_word();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "[mnemo_b200] cuda_kernels_init: %s\n", cudaGetErrorString(e));
        set_status(MB200_ERR_LAUNCH, "cuda_kernels_init");
    }
}

int mb200_init(void)
{
    mb200_clear_status();
    cuda_kernels_init();
    return g_status;
}

int mb200_last_status(void) { return g_status; }
const char *mb200_last_status_where(void) { return g_where; }
void mb200_clear_status(void)
{
    g_status = MB200_OK;
    g_where[0] = 0;
}

int mb200_clear_device_error(cudaStream_t stream)
{
    int *p = device_error_word();
    if (!p) return MB200_ERR_LAUNCH;
    return cudaMemsetAsync(p, 0, sizeof(int), stream) == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

int mb200_device_error(void)
{
    int *p = device_error_word();
    if (!p) return MB200_ERR_LAUNCH;
    int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return MB200_ERR_LAUNCH;
    if (cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return MB200_ERR_LAUNCH;
    return v;
}

}  // extern "C"
