// Seeded synthetic GGUF blocks and activations written directly in device
// memory (a 150 GB model cannot be staged through the host). Same counter-based
// stream as mnemocuda_b200/synth.py: word i of stream s = mix(mix(s) + i). The
// integer fields are bit-identical to the host generator; d/dmin use fp32
// Box-Muller here and fp64 there, so they follow the same distribution but may
// differ in the last fp16 bit.
#include <cstdio>

#include "common.cuh"

namespace mb200 {
namespace {

__host__ __device__ inline uint64_t mix(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ inline float normal_from(uint64_t w)
{
    const float u1 = (static_cast<float>(static_cast<uint32_t>(w >> 32)) + 1.0f) * (1.0f / 4294967296.0f);
    const float u2 = static_cast<float>(static_cast<uint32_t>(w)) * (1.0f / 4294967296.0f);
    return sqrtf(-2.0f * logf(fminf(u1, 1.0f))) * cospif(2.0f * u2);
}

// one thread per 64-bit word; blocks are 18 (Q4_K) or 27 (Q6_K, last 6 bytes dropped) words
__global__ void fill_q4k_kernel(uint8_t *dst, size_t n_blocks, uint64_t base, uint64_t nbase)
{
    const size_t n_words = n_blocks * 18;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_words;
         i += (size_t)gridDim.x * blockDim.x) {
        uint64_t w = mix(base + i);
        const size_t blk = i / 18, j = i % 18;
        if (j == 0) {
            const float d = fabsf(normal_from(mix(nbase + 2 * blk))) * 2e-3f;
            const float m = fabsf(normal_from(mix(nbase + 2 * blk + 1))) * 2e-3f;
            const uint32_t dd = __half_as_ushort(__float2half_rn(d)) |
                                (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(m))) << 16);
            w = (w & 0xFFFFFFFF00000000ull) | dd;
        }
        *reinterpret_cast<uint64_t *>(dst + i * 8) = w;  // 144 = 18 * 8: always 8-byte aligned
    }
}

__global__ void fill_q6k_kernel(uint8_t *dst, size_t n_blocks, uint64_t base, uint64_t nbase)
{
    const size_t n_words = n_blocks * 27;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_words;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint64_t w = mix(base + i);
        const size_t blk = i / 27, j = i % 27;
        uint8_t *b = dst + blk * kQ6KBlock;
        uint32_t d_bits = 0;
        if (j == 26) {
            const float d = fabsf(normal_from(mix(nbase + blk))) * 1e-3f;
            d_bits = __half_as_ushort(__float2half_rn(d));
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int off = static_cast<int>(j) * 8 + k;
            if (off >= kQ6KBlock) continue;  // bytes 210..215 of the last word do not exist
            uint8_t v = static_cast<uint8_t>(w >> (8 * k));
            if (off >= 208)
                v = static_cast<uint8_t>(d_bits >> (8 * (off - 208)));
            else if (off >= 192)
                v = static_cast<uint8_t>(static_cast<int8_t>((v & 63) - 32));
            b[off] = v;
        }
    }
}

__global__ void fill_normal_f32_kernel(float *dst, size_t n, uint64_t nbase, float scale)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = normal_from(mix(nbase + i)) * scale;
}

__global__ void fill_normal_f16_kernel(__half *dst, size_t n, uint64_t nbase, float scale)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __float2half_rn(normal_from(mix(nbase + i)) * scale);
}

inline int grid_for(size_t n)
{
    size_t g = (n + 255) / 256;
    const size_t cap = (size_t)kSMs * 16;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" {

int mb200_fill_q4k(void *dst, size_t n_blocks, uint64_t seed, cudaStream_t stream)
{
    if (!dst || (reinterpret_cast<uintptr_t>(dst) & 7)) return MB200_ERR_ARG;
    if (n_blocks == 0) return MB200_OK;
    fill_q4k_kernel<<<grid_for(n_blocks * 18), 256, 0, stream>>>(
        static_cast<uint8_t *>(dst), n_blocks, mix(seed), mix((seed ^ 0xD0D0ull) ^ 0x5EEDFACEull));
    return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

// Blocks [first_block, first_block + n_blocks) of the same stream: a row range of a tensor gets the bytes it has
// inside the whole tensor (a rank that holds only its shard of a sharded model).
int mb200_fill_q4k_at(void *dst, size_t first_block, size_t n_blocks, uint64_t seed, cudaStream_t stream)
{
    if (!dst || (reinterpret_cast<uintptr_t>(dst) & 7)) return MB200_ERR_ARG;
    if (n_blocks == 0) return MB200_OK;
    fill_q4k_kernel<<<grid_for(n_blocks * 18), 256, 0, stream>>>(
        static_cast<uint8_t *>(dst), n_blocks, mix(seed) + first_block * 18,
        mix((seed ^ 0xD0D0ull) ^ 0x5EEDFACEull) + 2 * first_block);
    return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

int mb200_fill_q6k_at(void *dst, size_t first_block, size_t n_blocks, uint64_t seed, cudaStream_t stream)
{
    if (!dst) return MB200_ERR_ARG;
    if (n_blocks == 0) return MB200_OK;
    fill_q6k_kernel<<<grid_for(n_blocks * 27), 256, 0, stream>>>(
        static_cast<uint8_t *>(dst), n_blocks, mix(seed) + first_block * 27,
        mix((seed ^ 0xD0D0ull) ^ 0x5EEDFACEull) + first_block);
    return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

int mb200_fill_q6k(void *dst, size_t n_blocks, uint64_t seed, cudaStream_t stream)
{
    if (!dst) return MB200_ERR_ARG;
    if (n_blocks == 0) return MB200_OK;
    fill_q6k_kernel<<<grid_for(n_blocks * 27), 256, 0, stream>>>(
        static_cast<uint8_t *>(dst), n_blocks, mix(seed), mix((seed ^ 0xD0D0ull) ^ 0x5EEDFACEull));
    return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

int mb200_fill_normal_f32(float *dst, size_t n, uint64_t seed, float scale, cudaStream_t stream)
{
    if (!dst) return MB200_ERR_ARG;
    if (n == 0) return MB200_OK;
    fill_normal_f32_kernel<<<grid_for(n), 256, 0, stream>>>(dst, n, mix(seed ^ 0x5EEDFACEull), scale);
    return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

int mb200_fill_normal_f16(void *dst, size_t n, uint64_t seed, float scale, cudaStream_t stream)
{
    if (!dst) return MB200_ERR_ARG;
    if (n == 0) return MB200_OK;
    fill_normal_f16_kernel<<<grid_for(n), 256, 0, stream>>>(static_cast<__half *>(dst), n,
                                                           mix(seed ^ 0x5EEDFACEull), scale);
    return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

}  // extern "C"
