// The remaining cases of the reference's matvec() type switch (src/forward.c:160-173) and its INT8
// KV-cache variant, under the reference's own names and signatures:
//
//   cuda_matvec_q8_0 (src/kernels.cu:644-673, 1159-1168)   34-byte blocks of 32 weights
//   cuda_matvec_q5k  (src/kernels.cu:578-640, 1137-1146)  176-byte blocks of 256 weights
//   cuda_matvec_q3k  (src/kernels.cu:497-575, 1148-1157)  110-byte blocks of 256 weights
//   cuda_embedding_lookup_q3k (src/kernels.cu:1955-2030)
//   cuda_f32_to_int8_kv, cuda_f32_to_int8_kv_dual (src/kernels.cu:1339-1376, 1484-1534)
//   cuda_attention_int8kv (src/kernels.cu:1382-1480, 1536-1546)
//
// The bit layouts are the reference's, which for Q5_K (fifth bits taken in weight order from qh) and
// Q3_K (the two high bits of scale i taken from byte 8 + i/4) are not the ones of the GGUF
// specification; a drop-in has to give the answers of the code it replaces.
//
// Matvec: whole 256-column blocks at the type's alignment run on the streaming skeleton (matvec_other.cu,
// other_policies.cuh: bulk-copied tiles, dp4a against the int8 split of x). Anything else: one warp per row, grid-stride. The warp copies the row's bytes into its slice of shared
// memory with 16-byte loads (2-byte loads at a ragged head or tail), then each lane decodes whole
// 32-weight groups (scale decode once per group) against x, which the CTA holds in shared memory
// padded by one float per 32 so that lanes on different groups hit different banks.
#include <stdio.h>

#include "common.cuh"
#include "support.cuh"

namespace mb200 {
int pdl_enabled();
// the streaming forms (matvec_other.cu); false = shape or alignment they do not take
bool stream_matvec_q8_0(const void *w, const float *x, float *y, int n_rows, int n_cols, cudaStream_t s);
bool stream_matvec_q5k(const void *w, const float *x, float *y, int n_rows, int n_cols, cudaStream_t s);
bool stream_matvec_q3k(const void *w, const float *x, float *y, int n_rows, int n_cols, cudaStream_t s);

namespace {

__device__ __forceinline__ void pdl_enter()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr int kWarps = 8;

__device__ __forceinline__ float f16_bits(unsigned v) { return __half2float(__ushort_as_half((unsigned short)v)); }
__device__ __forceinline__ unsigned ld16(const uint8_t *p) { return *reinterpret_cast<const unsigned short *>(p); }

// ---- per-type decode of one 32-weight group `g` of a row held in shared memory ----
struct Q8_0 {
    static constexpr int kBlockBytes = 34, kBlockWeights = 32;
    // sum over the group's 32 weights of w * x (x is zero past n_cols)
    static __device__ __forceinline__ float group(const uint8_t *row, int g, const float *xs)
    {
        const uint8_t *blk = row + (size_t)g * 34;
        const float d = f16_bits(ld16(blk));
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            const unsigned two = ld16(blk + 2 + j);
            const float w0 = (float)(int)(signed char)(two & 0xFF), w1 = (float)(int)(signed char)(two >> 8);
            s = fmaf(w0, xs[j], s);
            s = fmaf(w1, xs[j + 1], s);
        }
        return d * s;
    }
};

__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, int &sc, int &m)
{
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

struct Q5K {
    static constexpr int kBlockBytes = 176, kBlockWeights = 256;
    static __device__ __forceinline__ float group(const uint8_t *row, int g, const float *xs)
    {
        const uint8_t *blk = row + (size_t)(g >> 3) * 176;
        const int u = g & 7;  // 32-weight group inside the block: weights 32u .. 32u+31
        const float d = f16_bits(ld16(blk)), dmin = f16_bits(ld16(blk + 2));
        int sc, m;
        scale_min_k4(u, blk + 4, sc, m);
        // fifth bits in weight order: weight 32u + l is bit l of the u-th 32-bit word of qh
        const unsigned hb = ld16(blk + 16 + 4 * u) | (ld16(blk + 18 + 4 * u) << 16);
        const uint8_t *q = blk + 48 + 32 * (u >> 1);
        const int sh = (u & 1) * 4;
        float s = 0.0f, sx = 0.0f;
#pragma unroll
        for (int l = 0; l < 32; l += 2) {
            const unsigned two = ld16(q + l);
            const int q0 = ((two >> sh) & 0xF) | (((hb >> l) & 1) << 4);
            const int q1 = ((two >> (8 + sh)) & 0xF) | (((hb >> (l + 1)) & 1) << 4);
            const float x0 = xs[l], x1 = xs[l + 1];
            s = fmaf((float)q0, x0, s);
            s = fmaf((float)q1, x1, s);
            sx += x0 + x1;
        }
        return d * (float)sc * s - dmin * (float)m * sx;
    }
};

struct Q3K {
    static constexpr int kBlockBytes = 110, kBlockWeights = 256;
    static __device__ __forceinline__ int scale6(const uint8_t *sc, int i)  // i in 0..15
    {
        const int ii = i & 7, hi = i >> 3;
        const int lo4 = hi ? (sc[ii] >> 4) : (sc[ii] & 0xF);
        const int hi2 = (sc[8 + (ii >> 2)] >> (2 * (ii & 3) + 4 * hi)) & 3;
        return (int)(signed char)(lo4 | (hi2 << 4)) - 32;
    }
    static __device__ __forceinline__ float group(const uint8_t *row, int g, const float *xs)
    {
        const uint8_t *blk = row + (size_t)(g >> 3) * 110;
        const int u = g & 7;  // chunk = u >> 2, 2-bit plane = u & 3; weights 32u .. 32u+31
        const float d = f16_bits(ld16(blk + 108));
        const uint8_t *hm = blk, *q = blk + 32 + 32 * (u >> 2), *sc = blk + 96;
        const int shift = 2 * (u & 3);
        const float d0 = d * (float)scale6(sc, 2 * u), d1 = d * (float)scale6(sc, 2 * u + 1);
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int l = 0; l < 32; l += 2) {
            const unsigned two = ld16(q + l), hh = ld16(hm + l);
            const int v0 = (int)((two >> shift) & 3) - (((hh >> u) & 1) ? 0 : 4);
            const int v1 = (int)((two >> (8 + shift)) & 3) - (((hh >> (8 + u)) & 1) ? 0 : 4);
            const float t = fmaf((float)v1, xs[l + 1], (float)v0 * xs[l]);
            if (l < 16) s0 += t;
            else s1 += t;
        }
        return d0 * s0 + d1 * s1;
    }
};

// Warp copy of `bytes` (even) from a 2-byte-aligned global address into shared memory at the same
// offset modulo 16, so that the body moves as 16-byte words.
__device__ __forceinline__ void stage_row(const uint8_t *src, int bytes, uint8_t *dst, int lane)
{
    const int head = min(bytes, (int)((16 - (reinterpret_cast<uintptr_t>(src) & 15)) & 15));
    const int body = (bytes - head) & ~15;
    for (int i = 2 * lane; i < head; i += 64)
        *reinterpret_cast<unsigned short *>(dst + i) = __ldg(reinterpret_cast<const unsigned short *>(src + i));
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src + head);
    uint4 *d4 = reinterpret_cast<uint4 *>(dst + head);
    for (int i = lane; i < body / 16; i += 32) d4[i] = __ldcs(s4 + i);
    for (int i = head + body + 2 * lane; i < bytes; i += 64)
        *reinterpret_cast<unsigned short *>(dst + i) = __ldg(reinterpret_cast<const unsigned short *>(src + i));
}

template <class T>
__global__ void __launch_bounds__(kWarps * 32) typed_matvec_kernel(const uint8_t *__restrict__ w, const float *x, float *y,
                                                                  int n_rows, int n_cols, int row_slot)
{
    pdl_enter();
    extern __shared__ __align__(16) uint8_t tsm[];
    const int groups = (n_cols + 31) / 32;
    float *xs = reinterpret_cast<float *>(tsm);            // groups * 33 floats (one pad per 32)
    uint8_t *rows = tsm + (((size_t)groups * 33 * 4 + 15) & ~(size_t)15);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < groups * 32; i += blockDim.x) xs[i + (i >> 5)] = i < n_cols ? __ldcg(x + i) : 0.0f;
    __syncthreads();
    const int bpr = (n_cols + T::kBlockWeights - 1) / T::kBlockWeights;
    const int row_bytes = bpr * T::kBlockBytes;
    uint8_t *mine = rows + (size_t)warp * row_slot;
    for (int r = blockIdx.x * kWarps + warp; r < n_rows; r += gridDim.x * kWarps) {
        const uint8_t *src = w + (size_t)r * row_bytes;
        uint8_t *dst = mine + (reinterpret_cast<uintptr_t>(src) & 15);
        stage_row(src, row_bytes, dst, lane);
        __syncwarp();
        float s = 0.0f;
        for (int g = lane; g < groups; g += 32) s += T::group(dst, g, xs + g * 33);
        s = warp_sum(s);
        if (lane == 0) y[r] = s;
        __syncwarp();
    }
}

template <class T>
int typed_matvec(const void *w, const float *x, float *y, int n_rows, int n_cols, cudaStream_t stream, const char *who)
{
    if (n_rows <= 0 || n_cols <= 0) return MB200_OK;
    const int groups = (n_cols + 31) / 32;
    const int bpr = (n_cols + T::kBlockWeights - 1) / T::kBlockWeights;
    const int row_slot = (bpr * T::kBlockBytes + 16 + 15) & ~15;
    const size_t smem = (((size_t)groups * 33 * 4 + 15) & ~(size_t)15) + (size_t)kWarps * row_slot;
    if (smem > 224 * 1024 || (reinterpret_cast<uintptr_t>(w) & 1)) {
        fprintf(stderr, "[mnemo_b200] %s: n_cols %d too wide or weights not 2-byte aligned\n", who, n_cols);
        set_status(MB200_ERR_UNSUPPORTED, who);
        return MB200_ERR_UNSUPPORTED;
    }
    static bool done[kMaxDevices] = {};
    const int dev = current_device();
    if (!done[dev]) {
        if (cudaFuncSetAttribute(typed_matvec_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) !=
            cudaSuccess) {
            set_status(MB200_ERR_LAUNCH, who);
            return MB200_ERR_LAUNCH;
        }
        done[dev] = true;
    }
    const int per_sm = (int)min((size_t)4, (size_t)(226 * 1024) / (smem + 1024));
    int ctas = device_sms() * (per_sm < 1 ? 1 : per_sm);
    const int need = (n_rows + kWarps - 1) / kWarps;
    if (ctas > need) ctas = need;
    launch_k(typed_matvec_kernel<T>, dim3(ctas), dim3(kWarps * 32), smem, stream, static_cast<const uint8_t *>(w), x, y,
             n_rows, n_cols, row_slot);
    if (cudaGetLastError() != cudaSuccess) {
        set_status(MB200_ERR_LAUNCH, who);
        return MB200_ERR_LAUNCH;
    }
    return MB200_OK;
}

// ---- Q3_K embedding row ----
__global__ void __launch_bounds__(256) embed_q3k_kernel(const uint8_t *__restrict__ table, float *__restrict__ out,
                                                        const int *token_ptr, int token_imm, int hidden, int row_bytes)
{
    pdl_enter();
    const int token = token_ptr ? __ldcg(token_ptr) : token_imm;
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= hidden) return;
    const uint8_t *blk = table + (size_t)token * row_bytes + (size_t)blockIdx.x * 110;
    const int j = threadIdx.x, u = j >> 5, l = j & 31;
    const float d = f16_bits(ld16(blk + 108));
    const int sc = Q3K::scale6(blk + 96, j >> 4);
    const int q2 = (blk[32 + 32 * (u >> 2) + l] >> (2 * (u & 3))) & 3;
    const int v = q2 - (((blk[l] >> u) & 1) ? 0 : 4);
    out[c] = __fmul_rn(__fmul_rn(d, (float)sc), (float)v);
}

// ---- INT8 KV store: one warp per head, per-head absmax / 127 ----
__global__ void __launch_bounds__(128) int8_kv_kernel(const float *in_a, const float *in_b, int8_t *out_a, int8_t *out_b,
                                                      float *sc_a, float *sc_b, int head_dim, int n_kv_heads, int n_total)
{
    pdl_enter();
    const int h = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= n_total) return;
    const bool is_b = h >= n_kv_heads;
    const int head = is_b ? h - n_kv_heads : h;
    const float *in = (is_b ? in_b : in_a) + (size_t)head * head_dim;
    int8_t *out = (is_b ? out_b : out_a) + (size_t)head * head_dim;
    float mx = 0.0f;
    for (int d = lane; d < head_dim; d += 32) mx = fmaxf(mx, fabsf(__ldcg(in + d)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float inv = mx > 0.0f ? __fdiv_rn(127.0f, mx) : 0.0f;
    if (lane == 0) (is_b ? sc_b : sc_a)[head] = mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 0.0f;
    for (int d = lane; d < head_dim; d += 32) {
        int iv = __float2int_rn(__fmul_rn(__ldcg(in + d), inv));
        iv = iv > 127 ? 127 : (iv < -127 ? -127 : iv);
        out[d] = (int8_t)iv;
    }
}

// ---- attention over the INT8 cache ----
// One CTA per (group of HPB query heads that share a KV head, chunk of positions): the group's heads
// share every K / V byte read.
// Each warp walks positions of the chunk with an online softmax per query head, lanes over head
// dimensions (4 consecutive int8 per lane per 128 dims); the warps' and chunks' partial (m, l, acc)
// are merged by the last CTA of the KV head to arrive (ticket in the workspace).
constexpr int kI8Warps = 8;
constexpr int kI8MaxGqa = 8;    // query heads per CTA (registers: q and the running sums of each)
constexpr int kI8Groups = 64;   // head groups per launch
constexpr int kI8Slots = 512;   // (group, chunk) pairs per launch

struct I8Work {  // library-resident workspace: 512 slots x 8 query heads x (128 + 2) floats (2.1 MB per device)
    float part[kI8Slots * kI8MaxGqa * 128];
    float ml[kI8Slots * kI8MaxGqa * 2];
    int tickets[kI8Groups];
};
__device__ I8Work g_i8;

template <int GQA>
__global__ void __launch_bounds__(kI8Warps * 32) attn_int8_kernel(const float *q, const int8_t *__restrict__ kv_k,
                                                                  const int8_t *__restrict__ kv_v, const float *k_scales,
                                                                  const float *v_scales, float *out, int n_kv_heads,
                                                                  int seq_len, float scale, int chunks, int gqa_ratio)
{
    pdl_enter();
    __shared__ float s_acc[kI8Warps][GQA][128];
    __shared__ float s_ml[kI8Warps][GQA][2];
    __shared__ int s_last;
    // group blockIdx.x = query heads [GQA * blockIdx.x, GQA * (blockIdx.x + 1)), all on KV head kvh
    const int grp = blockIdx.x, kvh = grp * GQA / gqa_ratio, chunk = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t stride = (size_t)n_kv_heads * 128;
    float qv[GQA][4], acc[GQA][4], m[GQA], l[GQA];
#pragma unroll
    for (int h = 0; h < GQA; h++) {
        const float4 t = __ldcg(reinterpret_cast<const float4 *>(q + ((size_t)grp * GQA + h) * 128) + lane);
        qv[h][0] = t.x * scale; qv[h][1] = t.y * scale; qv[h][2] = t.z * scale; qv[h][3] = t.w * scale;
        acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.0f;
        m[h] = -INFINITY;
        l[h] = 0.0f;
    }
    const int per = (seq_len + chunks - 1) / chunks;
    const int p0 = chunk * per, p1 = min(seq_len, p0 + per);
    for (int p = p0 + warp; p < p1; p += kI8Warps) {
        const unsigned kb = __ldcg(reinterpret_cast<const unsigned *>(kv_k + (size_t)p * stride + (size_t)kvh * 128) + lane);
        const unsigned vb = __ldcg(reinterpret_cast<const unsigned *>(kv_v + (size_t)p * stride + (size_t)kvh * 128) + lane);
        const float ks = __ldcg(k_scales + (size_t)p * n_kv_heads + kvh), vs = __ldcg(v_scales + (size_t)p * n_kv_heads + kvh);
        float kf[4], vf[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            kf[i] = (float)(int)(signed char)((kb >> (8 * i)) & 0xFF) * ks;
            vf[i] = (float)(int)(signed char)((vb >> (8 * i)) & 0xFF) * vs;
        }
#pragma unroll
        for (int h = 0; h < GQA; h++) {
            float s = qv[h][0] * kf[0] + qv[h][1] * kf[1] + qv[h][2] * kf[2] + qv[h][3] * kf[3];
            s = warp_sum(s);
            const float mn = fmaxf(m[h], s), r = __expf(m[h] - mn), pw = __expf(s - mn);
#pragma unroll
            for (int i = 0; i < 4; i++) acc[h][i] = acc[h][i] * r + pw * vf[i];
            l[h] = l[h] * r + pw;
            m[h] = mn;
        }
    }
#pragma unroll
    for (int h = 0; h < GQA; h++) {
#pragma unroll
        for (int i = 0; i < 4; i++) s_acc[warp][h][4 * lane + i] = acc[h][i];
        if (lane == 0) {
            s_ml[warp][h][0] = m[h];
            s_ml[warp][h][1] = l[h];
        }
    }
    __syncthreads();
    // the CTA's partial for this chunk
    float *part = g_i8.part + ((size_t)(grp * chunks + chunk) * kI8MaxGqa) * 128;
    float *ml = g_i8.ml + ((size_t)(grp * chunks + chunk) * kI8MaxGqa) * 2;
    for (int i = threadIdx.x; i < GQA * 128; i += blockDim.x) {
        const int h = i >> 7, d = i & 127;
        float M = -INFINITY;
        for (int w2 = 0; w2 < kI8Warps; w2++) M = fmaxf(M, s_ml[w2][h][0]);
        float o = 0.0f, L = 0.0f;
        for (int w2 = 0; w2 < kI8Warps; w2++) {
            const float f = s_ml[w2][h][0] == -INFINITY ? 0.0f : __expf(s_ml[w2][h][0] - M);
            o += s_acc[w2][h][d] * f;
            L += s_ml[w2][h][1] * f;
        }
        part[i] = o;
        if (d == 0) {
            ml[2 * h] = M;
            ml[2 * h + 1] = L;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&g_i8.tickets[grp], 1) == chunks - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < GQA * 128; i += blockDim.x) {
        const int h = i >> 7;
        // eight chunks' loads in flight at a time (one chunk after the other would be a chain of L2 round trips)
        float M = -INFINITY;
        for (int c0 = 0; c0 < chunks; c0 += 8) {
            float mv[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                mv[u] = c0 + u < chunks ? __ldcg(g_i8.ml + ((size_t)(grp * chunks + c0 + u) * kI8MaxGqa + h) * 2) : -INFINITY;
#pragma unroll
            for (int u = 0; u < 8; u++) M = fmaxf(M, mv[u]);
        }
        float o = 0.0f, L = 0.0f;
        for (int c0 = 0; c0 < chunks; c0 += 8) {
            float mv[8], lv[8], pv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const size_t b = (size_t)(grp * chunks + min(c0 + u, chunks - 1)) * kI8MaxGqa;
                mv[u] = __ldcg(g_i8.ml + (b + h) * 2);
                lv[u] = __ldcg(g_i8.ml + (b + h) * 2 + 1);
                pv[u] = __ldcg(g_i8.part + b * 128 + i);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const float f = (c0 + u >= chunks || mv[u] == -INFINITY) ? 0.0f : __expf(mv[u] - M);
                o += pv[u] * f;
                L += lv[u] * f;
            }
        }
        out[((size_t)grp * GQA) * 128 + i] = L > 0.0f ? o / L : 0.0f;
    }
    if (threadIdx.x == 0) g_i8.tickets[grp] = 0;  // ready for the next launch
}

// Any head_dim / ratio: one CTA per query head, a warp per position (reference's shape of work).
__global__ void __launch_bounds__(256) attn_int8_generic_kernel(const float *q, const int8_t *__restrict__ kv_k,
                                                               const int8_t *__restrict__ kv_v, const float *k_scales,
                                                               const float *v_scales, float *out, int head_dim,
                                                               int n_kv_heads, int seq_len, int gqa_ratio, float scale)
{
    pdl_enter();
    extern __shared__ float gsm[];  // [8 warps][head_dim] + [8] m + [8] l
    const int head = blockIdx.x, kvh = head / gqa_ratio, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t stride = (size_t)n_kv_heads * head_dim;
    const int per = (head_dim + 31) / 32;  // <= 32
    float qv[32], acc[32];
    for (int i = 0; i < per; i++) {
        const int d = lane + 32 * i;
        qv[i] = d < head_dim ? __ldcg(q + (size_t)head * head_dim + d) * scale : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int p = warp; p < seq_len; p += 8) {
        const int8_t *kp = kv_k + (size_t)p * stride + (size_t)kvh * head_dim;
        const int8_t *vp = kv_v + (size_t)p * stride + (size_t)kvh * head_dim;
        const float ks = __ldcg(k_scales + (size_t)p * n_kv_heads + kvh), vs = __ldcg(v_scales + (size_t)p * n_kv_heads + kvh);
        float s = 0.0f;
        for (int i = 0; i < per; i++) {
            const int d = lane + 32 * i;
            if (d < head_dim) s = fmaf(qv[i], (float)__ldcg(kp + d), s);
        }
        s = warp_sum(s) * ks;
        const float mn = fmaxf(m, s), r = expf(m - mn), pw = expf(s - mn);
        for (int i = 0; i < per; i++) {
            const int d = lane + 32 * i;
            acc[i] = acc[i] * r + (d < head_dim ? pw * vs * (float)__ldcg(vp + d) : 0.0f);
        }
        l = l * r + pw;
        m = mn;
    }
    float *ow = gsm + warp * head_dim, *ms = gsm + 8 * head_dim, *ls = ms + 8;
    for (int i = 0; i < per; i++) {
        const int d = lane + 32 * i;
        if (d < head_dim) ow[d] = acc[i];
    }
    if (lane == 0) {
        ms[warp] = m;
        ls[warp] = l;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int w2 = 0; w2 < 8; w2++) M = fmaxf(M, ms[w2]);
    float L = 0.0f;
    for (int w2 = 0; w2 < 8; w2++) L += ms[w2] == -INFINITY ? 0.0f : ls[w2] * expf(ms[w2] - M);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float o = 0.0f;
        for (int w2 = 0; w2 < 8; w2++) o += ms[w2] == -INFINITY ? 0.0f : gsm[w2 * head_dim + d] * expf(ms[w2] - M);
        out[(size_t)head * head_dim + d] = L > 0.0f ? o / L : 0.0f;
    }
}

template <int GQA>
void launch_attn_int8(const float *q, const void *kv_k, const void *kv_v, const float *ks, const float *vs, float *out,
                      int n_heads_q, int n_kv_heads, int gqa_ratio, int seq_len, float scale, cudaStream_t stream)
{
    const int groups = n_heads_q / GQA;
    int chunks = 2 * device_sms() / groups;  // two CTAs per SM
    if (chunks > kI8Slots / groups) chunks = kI8Slots / groups;
    if (chunks < 1) chunks = 1;
    if (chunks > (seq_len + kI8Warps - 1) / kI8Warps) chunks = (seq_len + kI8Warps - 1) / kI8Warps;
    launch_k(attn_int8_kernel<GQA>, dim3(groups, chunks), dim3(kI8Warps * 32), 0, stream, q,
             static_cast<const int8_t *>(kv_k), static_cast<const int8_t *>(kv_v), ks, vs, out, n_kv_heads, seq_len, scale,
             chunks, gqa_ratio);
}

}  // namespace

void launch_embed_q3k(const void *table, float *out, const int *token_ptr, int token, int hidden, int row_bytes,
                      cudaStream_t stream)
{
    launch_k(embed_q3k_kernel, dim3((hidden + 255) / 256), dim3(256), 0, stream, static_cast<const uint8_t *>(table), out,
             token_ptr, token, hidden, row_bytes);
}

}  // namespace mb200

using namespace mb200;

extern "C" {

void cuda_matvec_q8_0(const void *weights, const float *x, float *y, int n_rows, int n_cols, cudaStream_t stream)
{
    if (n_rows > 0 && stream_matvec_q8_0(weights, x, y, n_rows, n_cols, stream)) return;
    typed_matvec<Q8_0>(weights, x, y, n_rows, n_cols, stream, "cuda_matvec_q8_0");
}

void cuda_matvec_q5k(const void *weights, const float *x, float *y, int n_rows, int n_cols, cudaStream_t stream)
{
    if (n_rows > 0 && stream_matvec_q5k(weights, x, y, n_rows, n_cols, stream)) return;
    typed_matvec<Q5K>(weights, x, y, n_rows, n_cols, stream, "cuda_matvec_q5k");
}

void cuda_matvec_q3k(const void *weights, const float *x, float *y, int n_rows, int n_cols, cudaStream_t stream)
{
    if (n_rows > 0 && stream_matvec_q3k(weights, x, y, n_rows, n_cols, stream)) return;
    typed_matvec<Q3K>(weights, x, y, n_rows, n_cols, stream, "cuda_matvec_q3k");
}

void cuda_embedding_lookup_q3k(const void *embd_table, float *output, int token_id, int hidden_size, int row_bytes,
                               cudaStream_t stream)
{
    if (hidden_size <= 0) return;
    launch_embed_q3k(embd_table, output, nullptr, token_id, hidden_size, row_bytes, stream);
    MB200_CHECK_LAUNCH("cuda_embedding_lookup_q3k");
}

void cuda_f32_to_int8_kv(const float *in, void *out, float *scales, int head_dim, int n_kv_heads, cudaStream_t stream)
{
    if (head_dim <= 0 || n_kv_heads <= 0) return;
    launch_k(int8_kv_kernel, dim3((n_kv_heads + 3) / 4), dim3(128), 0, stream, in, in, static_cast<int8_t *>(out),
             static_cast<int8_t *>(out), scales, scales, head_dim, n_kv_heads, n_kv_heads);
    MB200_CHECK_LAUNCH("cuda_f32_to_int8_kv");
}

void cuda_f32_to_int8_kv_dual(const float *k, const float *v, void *out_k, void *out_v, float *k_scales, float *v_scales,
                              int head_dim, int n_kv_heads, cudaStream_t stream)
{
    if (head_dim <= 0 || n_kv_heads <= 0) return;
    launch_k(int8_kv_kernel, dim3((2 * n_kv_heads + 3) / 4), dim3(128), 0, stream, k, v, static_cast<int8_t *>(out_k),
             static_cast<int8_t *>(out_v), k_scales, v_scales, head_dim, n_kv_heads, 2 * n_kv_heads);
    MB200_CHECK_LAUNCH("cuda_f32_to_int8_kv_dual");
}

void cuda_attention_int8kv(const float *q, const void *kv_k, const void *kv_v, const float *k_scales,
                           const float *v_scales, float *out, int n_heads_q, int head_dim, int n_kv_heads, int seq_len,
                           int gqa_ratio, float scale, cudaStream_t stream)
{
    if (n_heads_q <= 0 || seq_len <= 0) return;
    if (head_dim > 1024) {
        set_status(MB200_ERR_UNSUPPORTED, "cuda_attention_int8kv");
        return;
    }
    const bool fast = head_dim == 128 && n_heads_q == n_kv_heads * gqa_ratio;
    if (fast && gqa_ratio % 8 == 0 && n_heads_q / 8 <= kI8Groups) {
        launch_attn_int8<8>(q, kv_k, kv_v, k_scales, v_scales, out, n_heads_q, n_kv_heads, gqa_ratio, seq_len, scale, stream);
    } else if (fast && gqa_ratio % 4 == 0 && n_heads_q / 4 <= kI8Groups) {
        launch_attn_int8<4>(q, kv_k, kv_v, k_scales, v_scales, out, n_heads_q, n_kv_heads, gqa_ratio, seq_len, scale, stream);
    } else {
        const size_t smem = ((size_t)8 * head_dim + 16) * sizeof(float);
        launch_k(attn_int8_generic_kernel, dim3(n_heads_q), dim3(256), smem, stream, q, static_cast<const int8_t *>(kv_k),
                 static_cast<const int8_t *>(kv_v), k_scales, v_scales, out, head_dim, n_kv_heads, seq_len, gqa_ratio,
                 scale);
    }
    MB200_CHECK_LAUNCH("cuda_attention_int8kv");
}

}  // extern "C"
