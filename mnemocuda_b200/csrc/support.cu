// Support kernels of a decode step around the quantized matvecs: RMSNorm (plain, with
// residual save, per head), RoPE, fp16 KV store, decode attention over an fp16 KV cache,
// residual add, Q4_K embedding row, greedy sampling. They replace the reference's
// src/kernels.cu:692-852, 1196-1219, 1309-1333, 1550-1671, 1901-1951, 2026-2071 behind the
// same extern "C" names, and come in fused forms for the whole-token decode path
// (decode.cu) that read the position / token from device memory, so that one CUDA graph
// can be replayed token after token without patching any node.
//
// Decode attention is the only heavy one: the KV cache of a layer is read once per token
// (16.8 MB at context 8192 with 4 KV heads), so it is HBM-bound like the matvecs. One CTA
// handles one KV head and one contiguous chunk of positions for ALL query heads that
// share the KV head (grouped-query attention: 16 per KV head at the 235B shape), so K and
// V are read from HBM once, not once per query head as in the reference (one CTA per
// query head, src/kernels.cu:1550-1660). The 16 query heads are the M dimension of
// mma.sync.m16n8k16 tiles (Q K^T and P V; fp16 operands with q carried as hi + lo halves,
// fp32 accumulation), the position chunks are combined flash-decoding style: every CTA
// leaves (max, sum, weighted V) in a workspace and the last CTA of a KV head to finish
// (device-wide ticket) merges them.
#include <cstdio>

#include "common.cuh"
#include "support.cuh"

namespace mb200 {
int pdl_enabled();

namespace {

// Programmatic dependent launch (mb200_set_pdl): every kernel here lets its successor launch at once
// (the successor's own wait still orders it after this kernel's completion) and waits for its
// predecessor before it touches memory. In a decode chain this lets the next matvec stream its first
// weight tiles into shared memory while these small kernels run. Both instructions do nothing in a
// launch without the attribute.
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

// ---------------------------------------------------------------- RMSNorm ----
// out[i] = in[i] * w[i] / sqrt(mean(in^2) + eps); optionally copies `in` to res_out
// (reference src/kernels.cu:692-749). One CTA; in-place (out == in) is fine.
constexpr int kNormThreads = 1024;

__device__ __forceinline__ float block_sum(float v, float *red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(const float *__restrict__ in,
                                                                const float *__restrict__ w, float *out,
                                                                float *res_out, int n, float eps)
{
    pdl_enter();
    __shared__ float red[33];
    float ss = 0.0f;
    // inputs an upstream kernel wrote are read from L2 (ld.global.cg) in every kernel of this file: under
    // programmatic dependent launch the kernel is resident before its producer has finished
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = __ldcg(in + i);
        ss = fmaf(v, v, ss);
        if (res_out) res_out[i] = v;
    }
    const float tot = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(tot / static_cast<float>(n) + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = __ldcg(in + i) * scale * w[i];
}

// One warp per head: head h of `a` (n_a heads, weight wa) or of `b` (n_b heads, weight wb),
// each normalised over head_dim (reference src/kernels.cu:754-780, 1196-1219).
__global__ void __launch_bounds__(128) rms_norm_heads_kernel(const float *a_in, float *a_out, const float *__restrict__ wa,
                                                             int n_a, const float *b_in, float *b_out,
                                                             const float *__restrict__ wb, int n_b, int head_dim,
                                                             float eps)
{
    pdl_enter();
    const int head = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= n_a + n_b) return;
    const bool is_a = head < n_a;
    const float *in = is_a ? a_in + (size_t)head * head_dim : b_in + (size_t)(head - n_a) * head_dim;
    float *out = is_a ? a_out + (size_t)head * head_dim : b_out + (size_t)(head - n_a) * head_dim;
    const float *w = is_a ? wa : wb;
    float ss = 0.0f;
    for (int i = lane; i < head_dim; i += 32) ss = fmaf(__ldcg(in + i), __ldcg(in + i), ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(head_dim) + eps);
    for (int i = lane; i < head_dim; i += 32) out[i] = __ldcg(in + i) * scale * w[i];
}

// ------------------------------------------------------------------- RoPE ----
// Half-split ("NeoX") rotation of every head of q and k at position pos (reference
// src/kernels.cu:818-852). The angle pos / theta^(2j/head_dim) and its sine / cosine are
// evaluated in double precision, as the reference's own validator does
// (tools/validate_rope_norm.py:168-197); the reference kernel's fast-math __sincosf is
// less accurate at large positions. The parameter order is the reference kernel's: its
// graph builder patches `pos` (parameter 3) per token (src/forward.c:636-662).
__global__ void rope_kernel(float *q, float *k, int head_dim, int pos, float theta, int n_heads_q, int n_heads_k)
{
    pdl_enter();
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    const int half = head_dim / 2;
    if (tid >= (n_heads_q + n_heads_k) * half) return;
    const int head = tid / half, j = tid % half;
    float *vec = head < n_heads_q ? q + (size_t)head * head_dim : k + (size_t)(head - n_heads_q) * head_dim;
    const double freq = 1.0 / pow(static_cast<double>(theta), (2.0 * j) / head_dim);
    double s, c;
    sincos(static_cast<double>(pos) * freq, &s, &c);
    const float cf = static_cast<float>(c), sf = static_cast<float>(s);
    const float v0 = __ldcg(vec + j), v1 = __ldcg(vec + j + half);
    vec[j] = v0 * cf - v1 * sf;
    vec[j + half] = v0 * sf + v1 * cf;
}

// cos / sin of the rotation angles of one position, [half] floats each: computed once per
// token (in double) and shared by all layers of the decode path.
__global__ void rope_table_kernel(float *cos_out, float *sin_out, int head_dim, const int *pos_ptr, int pos_imm,
                                  float theta)
{
    pdl_enter();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= head_dim / 2) return;
    const int pos = pos_ptr ? __ldcg(pos_ptr) : pos_imm;
    const double freq = 1.0 / pow(static_cast<double>(theta), (2.0 * j) / head_dim);
    double s, c;
    sincos(static_cast<double>(pos) * freq, &s, &c);
    cos_out[j] = static_cast<float>(c);
    sin_out[j] = static_cast<float>(s);
}

// ---------------------------------------------------------- fp32 -> fp16 ----
__global__ void f32_to_f16_kernel(const float *__restrict__ in, __half *__restrict__ out, int n)
{
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(__ldcg(in + i));
}

// Parameter order of the reference kernel: its graph builder patches the two destination
// pointers (parameters 2 and 3) per token (src/forward.c:636-662).
__global__ void f32_to_f16_dual_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                       __half *__restrict__ oa, __half *__restrict__ ob, int n)
{
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        oa[i] = __float2half_rn(__ldcg(a + i));
        ob[i] = __float2half_rn(__ldcg(b + i));
    }
}

// ------------------------- fused: q/k norm + RoPE + KV store (decode path) ----
// One warp per head. Query heads: RMSNorm over the head, RoPE, written back in place.
// KV heads: K likewise, then K and V rounded to fp16 into the cache row of the position.
// Replaces the reference's cuda_rms_norm_qk + cuda_rope + cuda_f32_to_f16_dual
// (src/forward.c:722-768) with one launch. cos/sin: the per-token table; the position comes
// from device memory when pos_ptr is given.
__global__ void __launch_bounds__(128) qk_norm_rope_store_kernel(float *q, const float *__restrict__ k,
                                                                 const float *__restrict__ v,
                                                                 const float *__restrict__ wq,
                                                                 const float *__restrict__ wk,
                                                                 const float *__restrict__ cos_t,
                                                                 const float *__restrict__ sin_t, __half *kv_k,
                                                                 __half *kv_v, int n_q, int n_k, int head_dim,
                                                                 float eps, const int *pos_ptr, int pos_imm)
{
    pdl_enter();
    const int head = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= n_q + n_k) return;
    const bool is_q = head < n_q;
    const int hk = head - n_q;
    const float *in = is_q ? q + (size_t)head * head_dim : k + (size_t)hk * head_dim;
    const float *w = is_q ? wq : wk;
    const int half = head_dim / 2;
    float ss = 0.0f;
    for (int i = lane; i < head_dim; i += 32) ss = fmaf(__ldcg(in + i), __ldcg(in + i), ss);
    ss = warp_sum(ss);
    const float scale = w ? 1.0f / sqrtf(ss / static_cast<float>(head_dim) + eps) : 1.0f;
    const int pos = pos_ptr ? __ldcg(pos_ptr) : pos_imm;
    const size_t row = ((size_t)pos * n_k + (is_q ? 0 : hk)) * head_dim;
    for (int j = lane; j < half; j += 32) {
        const float v0 = __ldcg(in + j) * scale * (w ? w[j] : 1.0f);
        const float v1 = __ldcg(in + j + half) * scale * (w ? w[j + half] : 1.0f);
        const float c = __ldcg(cos_t + j), s = __ldcg(sin_t + j);
        const float r0 = v0 * c - v1 * s, r1 = v0 * s + v1 * c;
        if (is_q) {
            q[(size_t)head * head_dim + j] = r0;
            q[(size_t)head * head_dim + j + half] = r1;
        } else {
            kv_k[row + j] = __float2half_rn(r0);
            kv_k[row + j + half] = __float2half_rn(r1);
        }
    }
    if (!is_q)
        for (int i = lane; i < head_dim; i += 32) kv_v[row + i] = __float2half_rn(__ldcg(v + (size_t)hk * head_dim + i));
}

// ------------------------------------------------------------ attention ----
constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kHD = 128;      // head dimension of the tensor-core kernel
constexpr int kTile = 16;     // positions per warp step
constexpr int kOPitch = 132;  // floats between heads in the warps' shared-memory results (4 x 33, see the stores)
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
{
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// Grid (kv head x query-head block of 16, chunk). Fragment indices (g = lane / 4, t = lane % 4):
//  Q K^T:  A = Q   rows = query heads g, g + 8; the 16 k of step j are dims 32 (j / 2) + 8 t + 4 (j % 2) + {0,1 | 2,3}
//          B = K^T column = position g of the 8-position tile, same dims: each thread reads 64 contiguous bytes
//              of a K row as four 16-byte loads (the dot product does not care about the order of the dims)
//  P V:    A = P   taken from the Q K^T accumulators in place (k = position within the 16-position tile)
//          B = V   rows = positions 2t, 2t+1, 2t+8, 2t+9, column g of output tile u = dim 16 g + u: each thread
//              reads 32 contiguous bytes of four V rows and pairs the halves of two rows with byte permutes
//          C       rows = query heads g, g + 8; columns 2t, 2t + 1 of tile u = dims 16 (2t) + u, 16 (2t + 1) + u
//
// The first nine parameters are the reference kernel's, in its order (src/kernels.cu:1550-1554): the
// reference's graph builder finds this kernel's node by its address and patches seq_len (parameter 6)
// before every replay (src/forward.c:656-661), so the chunking is derived from seq_len inside the kernel
// and the grid does not depend on it.
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_decode_kernel(const float *__restrict__ q, const __half *__restrict__ kv_k, const __half *__restrict__ kv_v,
                   float *out, int head_dim_unused, int n_kv_heads, int seq_len_arg, int gqa, float scale,
                   float *part, float *ml, int *tickets, const int *pos_ptr)
{
    (void)head_dim_unused;  // always kHD here
    pdl_enter();
    AttnParams P;
    P.q = q; P.kv_k = kv_k; P.kv_v = kv_v; P.out = out; P.n_kv_heads = n_kv_heads; P.gqa = gqa;
    P.seq_len = seq_len_arg; P.pos_ptr = pos_ptr; P.scale = scale; P.part = part; P.ml = ml; P.tickets = tickets;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint32_t *afrag = reinterpret_cast<uint32_t *>(smem_raw);                  // [2 hi/lo][8 steps][4 regs][32 lanes]
    float *osm = reinterpret_cast<float *>(smem_raw + 8192);                    // [8 warps][16 heads][kOPitch]
    float *msm = osm + kAttnWarps * 16 * kOPitch;                               // [8][16]
    float *lsm = msm + kAttnWarps * 16;                                         // [8][16]
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int qb = (P.gqa + 15) / 16;            // query-head blocks per KV head
    const int kvh = blockIdx.x / qb, blk = blockIdx.x % qb;
    const int h0 = kvh * P.gqa + blk * 16;       // first query head of this CTA
    const int nh = min(16, P.gqa - blk * 16);    // query heads handled here
    const int S = gridDim.y, chunk = blockIdx.y;
    const int seq_len = P.pos_ptr ? __ldcg(P.pos_ptr) + 1 : P.seq_len;
    const int tiles_total = (seq_len + kTile - 1) / kTile;
    const int tpc = (tiles_total + S - 1) / S;
    const int p_begin = min(seq_len, chunk * tpc * kTile), p_end = min(seq_len, (chunk + 1) * tpc * kTile);
    const size_t row_stride = (size_t)P.n_kv_heads * kHD;  // halves between consecutive positions
    const __half *kbase = P.kv_k + (size_t)kvh * kHD;
    const __half *vbase = P.kv_v + (size_t)kvh * kHD;

    // ---- Q fragments (hi + lo halves of q * scale * log2 e) into shared memory: warp j builds step j ----
    {
        const int j = warp, d0 = (j >> 1) * 32 + t * 8 + (j & 1) * 4;
        const float sc = P.scale * kLog2e;
        float4 r0 = make_float4(0.f, 0.f, 0.f, 0.f), r1 = r0;
        if (g < nh) r0 = __ldcg(reinterpret_cast<const float4 *>(P.q + (size_t)(h0 + g) * kHD + d0));
        if (g + 8 < nh) r1 = __ldcg(reinterpret_cast<const float4 *>(P.q + (size_t)(h0 + g + 8) * kHD + d0));
        const float v[8] = {r0.x * sc, r0.y * sc, r0.z * sc, r0.w * sc, r1.x * sc, r1.y * sc, r1.z * sc, r1.w * sc};
        float hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            hi[i] = __half2float(__float2half_rn(v[i]));
            lo[i] = v[i] - hi[i];
        }
        uint32_t *ah = afrag + (0 * 8 + j) * 128 + lane, *al = afrag + (1 * 8 + j) * 128 + lane;
        ah[0] = pack_half2(hi[0], hi[1]);   // a0: row g,     k 2t, 2t+1
        ah[32] = pack_half2(hi[4], hi[5]);  // a1: row g + 8
        ah[64] = pack_half2(hi[2], hi[3]);  // a2: row g,     k 2t+8, 2t+9
        ah[96] = pack_half2(hi[6], hi[7]);  // a3: row g + 8
        al[0] = pack_half2(lo[0], lo[1]);
        al[32] = pack_half2(lo[4], lo[5]);
        al[64] = pack_half2(lo[2], lo[3]);
        al[96] = pack_half2(lo[6], lo[7]);
    }
    __syncthreads();

    float O[16][4];
#pragma unroll
    for (int u = 0; u < 16; u++) O[u][0] = O[u][1] = O[u][2] = O[u][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;  // rows g and g + 8 (l: this thread's share)

    const int n_tiles = (p_end - p_begin + kTile - 1) / kTile;
    const int last_row = max(p_end - 1, 0);
    uint4 kq[2][4];
    auto load_k = [&](int tile, uint4 (&dst)[2][4]) {
        const int base = p_begin + tile * kTile;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            const int p = min(base + nt * 8 + g, last_row);
            const uint4 *src = reinterpret_cast<const uint4 *>(kbase + (size_t)p * row_stride) + t;
#pragma unroll
            for (int i = 0; i < 4; i++) dst[nt][i] = __ldcg(src + i * 4);  // bytes 64 i + 16 t of the row
        }
    };
    if (warp < n_tiles) load_k(warp, kq);
    for (int tile = warp; tile < n_tiles; tile += kAttnWarps) {
        const int base = p_begin + tile * kTile;
        // V rows of this tile and K rows of the warp's next tile: in flight during the Q K^T products
        uint4 vr[4][2];
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int p = min(base + 2 * t + (r & 1) + (r >> 1) * 8, last_row);
            const uint4 *src = reinterpret_cast<const uint4 *>(vbase + (size_t)p * row_stride) + g * 2;
            vr[r][0] = __ldcg(src);
            vr[r][1] = __ldcg(src + 1);
        }
        uint4 kn[2][4];
        const bool more = tile + kAttnWarps < n_tiles;
        if (more) load_k(tile + kAttnWarps, kn);

        float Sx[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            Sx[nt][0] = Sx[nt][1] = Sx[nt][2] = Sx[nt][3] = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint4 kk = kq[nt][j >> 1];
                const uint32_t b0 = (j & 1) ? kk.z : kk.x, b1 = (j & 1) ? kk.w : kk.y;
                const uint32_t *ah = afrag + (0 * 8 + j) * 128 + lane, *al = afrag + (1 * 8 + j) * 128 + lane;
                mma16816(Sx[nt], ah[0], ah[32], ah[64], ah[96], b0, b1);
                mma16816(Sx[nt], al[0], al[32], al[64], al[96], b0, b1);
            }
        }
        // mask positions beyond the chunk, running max / sum in the log2 domain
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            const int p = base + nt * 8 + 2 * t;
            if (p >= p_end) Sx[nt][0] = Sx[nt][2] = -INFINITY;
            if (p + 1 >= p_end) Sx[nt][1] = Sx[nt][3] = -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(Sx[nt][0], Sx[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(Sx[nt][2], Sx[nt][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);  // finite: a tile holds at least one position
        const float r0 = exp2f(m0 - n0), r1 = exp2f(m1 - n1);  // exp2f(-inf) = 0 on the first tile
        m0 = n0;
        m1 = n1;
        l0 *= r0;
        l1 *= r1;
#pragma unroll
        for (int u = 0; u < 16; u++) {
            O[u][0] *= r0;
            O[u][1] *= r0;
            O[u][2] *= r1;
            O[u][3] *= r1;
        }
        uint32_t pa[4];
        {
            float p[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                p[nt][0] = exp2f(Sx[nt][0] - n0);
                p[nt][1] = exp2f(Sx[nt][1] - n0);
                p[nt][2] = exp2f(Sx[nt][2] - n1);
                p[nt][3] = exp2f(Sx[nt][3] - n1);
                l0 += p[nt][0] + p[nt][1];
                l1 += p[nt][2] + p[nt][3];
            }
            pa[0] = pack_half2(p[0][0], p[0][1]);  // row g,     positions 2t, 2t+1
            pa[1] = pack_half2(p[0][2], p[0][3]);  // row g + 8
            pa[2] = pack_half2(p[1][0], p[1][1]);  // row g,     positions 8+2t, 8+2t+1
            pa[3] = pack_half2(p[1][2], p[1][3]);
        }
        const uint32_t *v0 = reinterpret_cast<const uint32_t *>(&vr[0][0]);  // 8 words = 16 halves of row 2t
        const uint32_t *v1 = reinterpret_cast<const uint32_t *>(&vr[1][0]);
        const uint32_t *v2 = reinterpret_cast<const uint32_t *>(&vr[2][0]);
        const uint32_t *v3 = reinterpret_cast<const uint32_t *>(&vr[3][0]);
#pragma unroll
        for (int u = 0; u < 16; u++) {
            const uint32_t sel = (u & 1) ? 0x7632u : 0x5410u;
            const uint32_t b0 = __byte_perm(v0[u >> 1], v1[u >> 1], sel);
            const uint32_t b1 = __byte_perm(v2[u >> 1], v3[u >> 1], sel);
            mma16816(O[u], pa[0], pa[1], pa[2], pa[3], b0, b1);
        }
        if (more) {
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) kq[nt][i] = kn[nt][i];
        }
    }
    // ---- this warp's share to shared memory ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (t == 0) {
        msm[warp * 16 + g] = m0;
        msm[warp * 16 + g + 8] = m1;
        lsm[warp * 16 + g] = l0;
        lsm[warp * 16 + g + 8] = l1;
    }
    {
        // dim d of a head sits at (d / 32) * 33 + d % 32, heads 132 floats apart: the 32 lanes of a store
        // (bank 4 g + t + const) hit 32 different banks
        float *ow = osm + warp * 16 * kOPitch;
#pragma unroll
        for (int u = 0; u < 16; u++) {
            ow[g * kOPitch + 33 * t + u] = O[u][0];            // dim 16 (2t) + u
            ow[g * kOPitch + 33 * t + 16 + u] = O[u][1];       // dim 16 (2t + 1) + u
            ow[(g + 8) * kOPitch + 33 * t + u] = O[u][2];
            ow[(g + 8) * kOPitch + 33 * t + 16 + u] = O[u][3];
        }
    }
    __syncthreads();
    // ---- the CTA's partial result: thread -> head tid / 16, dims 8 (tid % 16) .. + 7 ----
    const int head = tid >> 4, d0 = (tid & 15) * 8;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; w++) M = fmaxf(M, msm[w * 16 + head]);
    float L = 0.0f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < kAttnWarps; w++) {
        const float mw = msm[w * 16 + head];
        const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
        L = fmaf(lsm[w * 16 + head], f, L);
        const float *ow = osm + (w * 16 + head) * kOPitch + (d0 >> 5) * 33 + (d0 & 31);
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = fmaf(ow[i], f, acc[i]);
    }
    const size_t slot = (size_t)blockIdx.x * S + chunk;
    float *pdst = P.part + (slot * 16 + head) * kHD + d0;
    *reinterpret_cast<float4 *>(pdst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4 *>(pdst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if ((tid & 15) == 0) {
        P.ml[(slot * 2 + 0) * 16 + head] = M;
        P.ml[(slot * 2 + 1) * 16 + head] = L;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int ticket = atomicAdd(P.tickets + blockIdx.x, 1);
        is_last = (ticket == S - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // ---- last CTA of this KV head: merge the chunks ----
    // The sixteen threads of a head (half a warp) first fetch the chunks' (max, sum) pairs side by side -- chunk
    // c by lane c mod 16 -- and reduce them with shuffles; then every thread adds up its eight dims over the chunks,
    // eight chunks' loads in flight at a time. (A loop that loads and uses one chunk after the other is a chain of S
    // L2 round trips: with 37 chunks it was most of this kernel's time.)
    if (head < nh) {
        const int sub = tid & 15;
        const unsigned half_mask = 0xFFFFu << (tid & 16);
        float *fsm = osm;  // [S][16] weights of the chunks (the warps' results above have been consumed)
        constexpr int kMaxPer = 10;  // chunks per lane: S <= 160
        float mc[kMaxPer], lc[kMaxPer];
#pragma unroll
        for (int i = 0; i < kMaxPer; i++) {
            const int c = sub + 16 * i;
            const size_t sl = (size_t)blockIdx.x * S + (c < S ? c : 0);
            mc[i] = c < S ? __ldcg(P.ml + (sl * 2 + 0) * 16 + head) : -INFINITY;
            lc[i] = c < S ? __ldcg(P.ml + (sl * 2 + 1) * 16 + head) : 0.0f;
        }
        float Mt = -INFINITY;
#pragma unroll
        for (int i = 0; i < kMaxPer; i++) Mt = fmaxf(Mt, mc[i]);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) Mt = fmaxf(Mt, __shfl_xor_sync(half_mask, Mt, o));
        float Lt = 0.0f;
#pragma unroll
        for (int i = 0; i < kMaxPer; i++) {
            const int c = sub + 16 * i;
            const float f = (mc[i] == -INFINITY) ? 0.0f : exp2f(mc[i] - Mt);
            Lt = fmaf(lc[i], f, Lt);
            if (c < S) fsm[c * 16 + head] = f;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) Lt += __shfl_xor_sync(half_mask, Lt, o);
        __syncwarp(half_mask);
        float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int c0 = 0; c0 < S; c0 += 8) {
            float4 a[8], b[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int c = min(c0 + u, S - 1);
                const size_t sl = (size_t)blockIdx.x * S + c;
                a[u] = __ldcg(reinterpret_cast<const float4 *>(P.part + (sl * 16 + head) * kHD + d0));
                b[u] = __ldcg(reinterpret_cast<const float4 *>(P.part + (sl * 16 + head) * kHD + d0 + 4));
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const float f = (c0 + u < S) ? fsm[(c0 + u) * 16 + head] : 0.0f;  // in chunk order, as before
                o[0] = fmaf(a[u].x, f, o[0]); o[1] = fmaf(a[u].y, f, o[1]); o[2] = fmaf(a[u].z, f, o[2]); o[3] = fmaf(a[u].w, f, o[3]);
                o[4] = fmaf(b[u].x, f, o[4]); o[5] = fmaf(b[u].y, f, o[5]); o[6] = fmaf(b[u].z, f, o[6]); o[7] = fmaf(b[u].w, f, o[7]);
            }
        }
        const float inv = Lt > 0.0f ? 1.0f / Lt : 0.0f;
        float *dst = P.out + (size_t)(h0 + head) * kHD + d0;
        *reinterpret_cast<float4 *>(dst) = make_float4(o[0] * inv, o[1] * inv, o[2] * inv, o[3] * inv);
        *reinterpret_cast<float4 *>(dst + 4) = make_float4(o[4] * inv, o[5] * inv, o[6] * inv, o[7] * inv);
    }
    if (tid == 0) P.tickets[blockIdx.x] = 0;  // ready for the next launch
}

constexpr int kAttnSmem = 8192 + (kAttnWarps * 16 * kOPitch + 2 * kAttnWarps * 16) * 4;

// Any head dimension (<= 1024): one CTA per query head, online softmax per warp over a
// strided share of the positions, warps merged through shared memory. Correct, not fast.
__global__ void __launch_bounds__(256) attn_generic_kernel(const float *__restrict__ q, const __half *__restrict__ kv_k,
                                                           const __half *__restrict__ kv_v, float *out, int head_dim,
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
        const __half *kp = kv_k + (size_t)p * stride + (size_t)kvh * head_dim;
        float s = 0.0f;
        for (int i = 0; i < per; i++) {
            const int d = lane + 32 * i;
            if (d < head_dim) s = fmaf(qv[i], __half2float(__ldcg(kp + d)), s);
        }
        s = warp_sum(s);
        const float mn = fmaxf(m, s), r = expf(m - mn), pw = expf(s - mn);
        const __half *vp = kv_v + (size_t)p * stride + (size_t)kvh * head_dim;
        for (int i = 0; i < per; i++) {
            const int d = lane + 32 * i;
            acc[i] = acc[i] * r + (d < head_dim ? pw * __half2float(__ldcg(vp + d)) : 0.0f);
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
    for (int w = 0; w < 8; w++) M = fmaxf(M, ms[w]);
    float L = 0.0f;
    for (int w = 0; w < 8; w++) L += ms[w] == -INFINITY ? 0.0f : ls[w] * expf(ms[w] - M);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float o = 0.0f;
        for (int w = 0; w < 8; w++) o += ms[w] == -INFINITY ? 0.0f : gsm[w * head_dim + d] * expf(ms[w] - M);
        out[(size_t)head * head_dim + d] = L > 0.0f ? o / L : 0.0f;
    }
}

// --------------------------------------------------------- residual add ----
__global__ void residual_add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *out, int n)
{
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __ldcg(a + i) + __ldcg(b + i);
}

// ----------------------------------------------------- Q4_K embedding row ----
// out[c] = d * sc * q - dmin * m for row `token` of a Q4_K table (reference
// src/kernels.cu:1901-1951): products and the difference rounded separately (no fused
// multiply-add), which is the arithmetic of the reference's validator
// (tools/validate_dequant.py:68-115), so the row is bit-exact against it.
__global__ void __launch_bounds__(256) embed_q4k_kernel(const uint8_t *__restrict__ table, float *__restrict__ out,
                                                        const int *token_ptr, int token_imm, int hidden, int row_bytes)
{
    pdl_enter();
    const int token = token_ptr ? __ldcg(token_ptr) : token_imm;
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= hidden) return;
    const uint8_t *blk = table + (size_t)token * row_bytes + (size_t)blockIdx.x * kQ4KBlock;
    const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blk)));
    const float dmin = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blk + 2)));
    const uint8_t *sc12 = blk + 4;
    const int j = threadIdx.x, is = j >> 5;
    int sc, m;
    if (is < 4) {
        sc = sc12[is] & 63;
        m = sc12[is + 4] & 63;
    } else {
        sc = (sc12[is + 4] & 0xF) | ((sc12[is - 4] >> 6) << 4);
        m = (sc12[is + 4] >> 4) | ((sc12[is] >> 6) << 4);
    }
    const uint8_t byte = blk[16 + (j >> 6) * 32 + (j & 31)];
    const int qv = (j & 32) ? (byte >> 4) : (byte & 0xF);
    const float d1 = __fmul_rn(d, static_cast<float>(sc));
    const float m1 = __fmul_rn(dmin, static_cast<float>(m));
    out[c] = __fsub_rn(__fmul_rn(d1, static_cast<float>(qv)), m1);
}

// --------------------------------------------------------------- argmax ----
// Greedy sampling (reference src/kernels.cu:2048-2071): the index of the largest logit.
// Ties resolve as in the reference's 256-thread strided scan + shared-memory tree: thread
// t = index % 256 keeps its first maximum, and of two tied threads the tree keeps the one
// whose lowest differing bit of t is 0 -- i.e. the smaller bit-reversed t wins.
__device__ __forceinline__ bool argmax_better(float v, int i, float bv, int bi)
{
    if (v > bv) return true;
    if (v < bv || !(v == bv)) return false;
    const unsigned a = __brev(static_cast<unsigned>(i & 255)), b = __brev(static_cast<unsigned>(bi & 255));
    return a < b || (a == b && i < bi);
}

// Candidates of the CTAs of one launch: a slot per CTA plus a ticket. It lives in the library image (the
// reference's cuda_sample_token has no workspace argument); launches that overlap on a device would race on it.
constexpr int kArgmaxCtas = 128;
__device__ float g_argmax_val[kArgmaxCtas];
__device__ int g_argmax_idx[kArgmaxCtas];
__device__ int g_argmax_ticket;

__device__ __forceinline__ void argmax_warp(float &bv, int &bi)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (argmax_better(ov, oi, bv, bi)) {
            bv = ov;
            bi = oi;
        }
    }
}

// Every CTA scans a strided share of the logits; the last one to finish (ticket) picks among the CTAs'
// candidates. The preference order is total, so the result does not depend on how the scan is split.
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ logits, int n, int *result, int *pos_ptr,
                                                     float *pair_out, int index_offset)
{
    pdl_enter();
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ int is_last;
    float bv = -1e30f;
    int bi = 0;
    // candidates are compared by their index in the whole vocabulary (index_offset + i), so that a row shard
    // orders ties as the whole vector would; bi stays shard-local until the end
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = __ldcg(logits + i);
        if (argmax_better(v, i + index_offset, bv, bi + index_offset)) {
            bv = v;
            bi = i;
        }
    }
    bi += index_offset;
    argmax_warp(bv, bi);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        sv[warp] = bv;
        si[warp] = bi;
    }
    __syncthreads();
    if (warp != 0) return;
    bv = lane < 8 ? sv[lane] : -1e30f;
    bi = lane < 8 ? si[lane] : index_offset;
    argmax_warp(bv, bi);
    if (lane == 0) {
        g_argmax_val[blockIdx.x] = bv;
        g_argmax_idx[blockIdx.x] = bi;
        __threadfence();
        is_last = (atomicAdd(&g_argmax_ticket, 1) == static_cast<int>(gridDim.x) - 1);
    }
    __syncwarp();
    if (!is_last) return;
    __threadfence();
    bv = -1e30f;
    bi = index_offset;
    for (int c = lane; c < static_cast<int>(gridDim.x); c += 32) {
        const float v = __ldcg(&g_argmax_val[c]);
        const int i = __ldcg(&g_argmax_idx[c]);
        if (argmax_better(v, i, bv, bi)) {
            bv = v;
            bi = i;
        }
    }
    argmax_warp(bv, bi);
    if (lane == 0) {
        if (pair_out) {  // a row shard of the logits: (value, index in the whole vocabulary) for the merge over the shards
            pair_out[0] = bv;
            pair_out[1] = __int_as_float(bi);
        } else {
            *result = bi;
            if (pos_ptr) *pos_ptr = __ldcg(pos_ptr) + 1;  // decode path: the next replay of the graph handles the next position
        }
        g_argmax_ticket = 0;
    }
}

// ------------------------------------------------- temperature + top-p ----
// The reference samples in one 256-thread block (src/kernels.cu:2073-2174): p_i = exp((l_i - max) / T), every
// thread keeps the eight largest p of its residue class i mod 256, thread 0 picks the 2048 candidates largest
// first until their sum reaches top_p * sum(p), draws once from xoroshiro128+ and walks the nucleus. Here:
// the maximum comes from the argmax scan above; 32 CTAs scan eight residue classes each (so that a warp's loads
// are whole 32-byte sectors), merge the classes' candidates, and the last CTA to finish (ticket) sorts the 2048
// candidates and walks them with the reference's arithmetic (float sums in descending order). Among equal
// probabilities the smaller token id is preferred; the sum of all p is added in another order than the
// reference's, so a cut that falls within rounding of top_p * sum can come out one candidate apart.
constexpr int kSampleClasses = 256, kSampleKeep = 8, kSampleCands = kSampleClasses * kSampleKeep;
constexpr int kSampleCtas = kSampleClasses / 8;
__device__ float g_sample_pair[2];
__device__ float g_sample_p[kSampleCands];
__device__ int g_sample_id[kSampleCands];
__device__ float g_sample_sum[kSampleCtas];
__device__ int g_sample_ticket;

__device__ __forceinline__ bool cand_better(float p, int id, float bp, int bid)
{
    return p > bp || (p == bp && id >= 0 && (bid < 0 || id < bid));
}

__global__ void __launch_bounds__(256) sample_top_p_kernel(const float *__restrict__ logits, int n, float temperature,
                                                           float top_p, unsigned long long seed, int *result)
{
    pdl_enter();
    __shared__ float sp[256 * kSampleKeep];
    __shared__ int si[256 * kSampleKeep];
    __shared__ float ssum[8];
    __shared__ int is_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float mx = __ldcg(&g_sample_pair[0]);
    const float inv_t = 1.0f / temperature;
    // ---- scan: thread (jj = tid / 8, k = tid % 8) takes i = 256 (jj + 32 m) + 8 blockIdx.x + k ----
    const int k = tid & 7, jj = tid >> 3;
    float vp[kSampleKeep];
    int vi[kSampleKeep];
#pragma unroll
    for (int q = 0; q < kSampleKeep; q++) {
        vp[q] = -1.0f;
        vi[q] = -1;
    }
    float sum = 0.0f;
    for (int i = 256 * jj + 8 * blockIdx.x + k; i < n; i += 256 * 32) {
        const float p = expf((__ldcg(logits + i) - mx) * inv_t);
        sum += p;
        int mi = 0;
#pragma unroll
        for (int q = 1; q < kSampleKeep; q++)
            if (vp[q] < vp[mi]) mi = q;
#pragma unroll
        for (int q = 0; q < kSampleKeep; q++)
            if (q == mi && p > vp[q]) {
                vp[q] = p;
                vi[q] = i;
            }
    }
    // lists to shared memory, class-major: class k holds 32 threads x 8 = 256 candidates
#pragma unroll
    for (int q = 0; q < kSampleKeep; q++) {
        sp[(k * 32 + jj) * kSampleKeep + q] = vp[q];
        si[(k * 32 + jj) * kSampleKeep + q] = vi[q];
    }
    sum = warp_sum(sum);
    if (lane == 0) ssum[warp] = sum;
    __syncthreads();
    // ---- warp w keeps the eight best of class w: eight rounds of a warp-wide maximum ----
    {
        float cp[kSampleKeep];
        int ci[kSampleKeep];
#pragma unroll
        for (int q = 0; q < kSampleKeep; q++) {
            cp[q] = sp[(warp * 32 + lane) * kSampleKeep + q];
            ci[q] = si[(warp * 32 + lane) * kSampleKeep + q];
        }
        for (int round = 0; round < kSampleKeep; round++) {
            float bp = -1.0f;
            int bi = -1;
#pragma unroll
            for (int q = 0; q < kSampleKeep; q++)
                if (cand_better(cp[q], ci[q], bp, bi)) {
                    bp = cp[q];
                    bi = ci[q];
                }
            float wp = bp;
            int wi = bi;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float op = __shfl_xor_sync(0xffffffffu, wp, o);
                const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
                if (cand_better(op, oi, wp, wi)) {
                    wp = op;
                    wi = oi;
                }
            }
            if (wi >= 0 && wi == bi) {  // the winner's owner retires it
#pragma unroll
                for (int q = 0; q < kSampleKeep; q++)
                    if (ci[q] == wi) {
                        cp[q] = -1.0f;
                        ci[q] = -1;
                    }
            }
            if (lane == 0) {
                const int c = (8 * blockIdx.x + warp) * kSampleKeep + round;
                g_sample_p[c] = wi >= 0 ? wp : -1.0f;
                g_sample_id[c] = wi;
            }
        }
    }
    if (tid == 0) {
        float s = 0.0f;
        for (int w = 0; w < 8; w++) s += ssum[w];
        g_sample_sum[blockIdx.x] = s;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = (atomicAdd(&g_sample_ticket, 1) == static_cast<int>(gridDim.x) - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // ---- last CTA: sort the candidates (probability descending, token id ascending), walk them ----
    for (int c = tid; c < kSampleCands; c += 256) {
        sp[c] = __ldcg(&g_sample_p[c]);
        si[c] = __ldcg(&g_sample_id[c]);
    }
    __syncthreads();
    for (int size = 2; size <= kSampleCands; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < kSampleCands / 2; t += 256) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool desc = ((lo & size) == 0);
                const bool hi_first = cand_better(sp[hi], si[hi], sp[lo], si[lo]);
                if (hi_first == desc) {
                    const float tp = sp[lo];
                    const int ti = si[lo];
                    sp[lo] = sp[hi];
                    si[lo] = si[hi];
                    sp[hi] = tp;
                    si[hi] = ti;
                }
            }
            __syncthreads();
        }
    }
    if (tid == 0) {
        float total = 0.0f;
        for (int c = 0; c < static_cast<int>(gridDim.x); c++) total += __ldcg(&g_sample_sum[c]);
        unsigned long long rs0 = seed, rs1 = seed ^ 0xDEADBEEFCAFEBABEULL;
        for (int w = 0; w < 4; w++) {  // three warm-up rounds and the draw
            const unsigned long long t = rs0 ^ (rs0 << 23);
            rs0 = rs1;
            rs1 = t ^ rs1 ^ (t >> 17) ^ (rs1 >> 26);
        }
        const float r = static_cast<float>((rs0 + rs1) >> 11) * (1.0f / 9007199254740992.0f);
        const float mass = top_p * total;
        float cumul = 0.0f;
        int nucleus = 0;
        for (int c = 0; c < kSampleCands; c++) {
            if (sp[c] <= 0.0f) break;
            cumul += sp[c];
            nucleus = c + 1;
            if (cumul >= mass) break;
        }
        float nsum = 0.0f;
        for (int c = 0; c < nucleus; c++) nsum += sp[c];
        const float target = r * nsum;
        float acc = 0.0f;
        int sampled = si[0];
        for (int c = 0; c < nucleus; c++) {
            acc += sp[c];
            if (acc >= target) {
                sampled = si[c];
                break;
            }
        }
        *result = sampled;
        g_sample_ticket = 0;
    }
}

// The best of the shards' (value, index) pairs, by the same order as above; writes the token and advances the position.
__global__ void argmax_merge_kernel(const float *__restrict__ pairs, int n, int *result, int *pos_ptr)
{
    pdl_enter();
    if (threadIdx.x != 0) return;
    float bv = -1e30f;
    int bi = 0;
    for (int q = 0; q < n; q++) {
        const float v = __ldcg(pairs + 2 * q);
        const int i = __float_as_int(__ldcg(pairs + 2 * q + 1));
        if (q == 0 || argmax_better(v, i, bv, bi)) {
            bv = v;
            bi = i;
        }
    }
    *result = bi;
    if (pos_ptr) *pos_ptr = __ldcg(pos_ptr) + 1;
}

// ---- attention workspace that lives in the library image (for the reference-named entry
// point, whose signature has no workspace argument): partial results of up to
// kStaticAttnSlots (query-head block, chunk) pairs. One copy per device that loads the library.
constexpr int kStaticAttnSlots = 256;
constexpr int kStaticAttnBlocks = 64;
__device__ __align__(256) float g_attn_part[kStaticAttnSlots * 16 * kHD];
__device__ __align__(16) float g_attn_ml[kStaticAttnSlots * 2 * 16];
__device__ int g_attn_tickets[kStaticAttnBlocks];
struct StaticAttn {
    float *part, *ml;
    int *tickets;
};
StaticAttn g_static_attn[kMaxDevices] = {};
bool g_attn_attr[kMaxDevices] = {false};

const StaticAttn *static_attn()
{
    const int dev = current_device();
    StaticAttn &s = g_static_attn[dev];
    if (!s.part) {
        void *a = nullptr, *b = nullptr, *c = nullptr;
        if (cudaGetSymbolAddress(&a, g_attn_part) != cudaSuccess || cudaGetSymbolAddress(&b, g_attn_ml) != cudaSuccess ||
            cudaGetSymbolAddress(&c, g_attn_tickets) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        s.ml = static_cast<float *>(b);
        s.tickets = static_cast<int *>(c);
        s.part = static_cast<float *>(a);
    }
    return &s;
}

bool attn_attr()
{
    const int dev = current_device();
    if (g_attn_attr[dev]) return true;
    if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    cudaFuncSetAttribute(attn_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    g_attn_attr[dev] = true;
    return true;
}

}  // namespace

// Device address of the sampling kernels' (max, index) pair, looked up once per device (cuda_kernels_init does it,
// so that no symbol is resolved inside a stream capture).
float *sample_pair_addr()
{
    static float *addr[kMaxDevices] = {};
    const int dev = current_device();
    if (!addr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_sample_pair) != cudaSuccess) return nullptr;
        addr[dev] = static_cast<float *>(p);
    }
    return addr[dev];
}

void support_init()
{
    attn_attr();
    (void)static_attn();
    (void)sample_pair_addr();
}

int attn_chunks_for(int n_kv_heads, int gqa, int max_slots)
{
    const int blocks = n_kv_heads * ((gqa + 15) / 16);
    int S = device_sms() / (blocks > 0 ? blocks : 1);
    if (S < 1) S = 1;
    if (max_slots > 0 && blocks * S > max_slots) S = max_slots / blocks;
    return S < 1 ? 1 : S;
}

size_t attn_workspace_bytes(int n_kv_heads, int gqa)
{
    const int blocks = n_kv_heads * ((gqa + 15) / 16);
    const size_t slots = (size_t)blocks * attn_chunks_for(n_kv_heads, gqa, 0);
    return slots * 16 * kHD * 4 + slots * 2 * 16 * 4 + (size_t)blocks * 4 + 64;
}

// Decode attention with a caller-provided workspace (zeroed once; the tickets are left zero).
int launch_attn_decode(const float *q, const void *kv_k, const void *kv_v, float *out, int n_heads_q, int n_kv_heads,
                       int seq_len, const int *pos_ptr, float scale, void *workspace, cudaStream_t stream)
{
    if (!attn_attr()) return MB200_ERR_LAUNCH;
    const int gqa = n_heads_q / n_kv_heads;
    const int blocks = n_kv_heads * ((gqa + 15) / 16);
    const int S = attn_chunks_for(n_kv_heads, gqa, 0);
    const size_t slots = (size_t)blocks * S;
    AttnParams P{};
    P.q = q;
    P.kv_k = static_cast<const __half *>(kv_k);
    P.kv_v = static_cast<const __half *>(kv_v);
    P.out = out;
    P.n_kv_heads = n_kv_heads;
    P.gqa = gqa;
    P.seq_len = seq_len;
    P.pos_ptr = pos_ptr;
    P.scale = scale;
    P.part = static_cast<float *>(workspace);
    P.ml = P.part + slots * 16 * kHD;
    P.tickets = reinterpret_cast<int *>(P.ml + slots * 2 * 16);
    launch_k(attn_decode_kernel, dim3(blocks, S), dim3(kAttnThreads), kAttnSmem, stream, P.q, P.kv_k, P.kv_v, P.out, kHD,
             P.n_kv_heads, P.seq_len, P.gqa, P.scale, P.part, P.ml, P.tickets, P.pos_ptr);
    return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ERR_LAUNCH;
}

void launch_rms_norm(const float *in, const float *w, float *out, float *res_out, int n, float eps, cudaStream_t stream)
{
    launch_k(rms_norm_kernel, dim3(1), dim3(kNormThreads), 0, stream, in, w, out, res_out, n, eps);
}

void launch_rope_table(float *cos_out, float *sin_out, int head_dim, const int *pos_ptr, int pos, float theta,
                       cudaStream_t stream)
{
    launch_k(rope_table_kernel, dim3((head_dim / 2 + 63) / 64), dim3(64), 0, stream, cos_out, sin_out, head_dim, pos_ptr, pos,
             theta);
}

void launch_qk_norm_rope_store(float *q, const float *k, const float *v, const float *wq, const float *wk,
                               const float *cos_t, const float *sin_t, void *kv_k, void *kv_v, int n_q, int n_k,
                               int head_dim, float eps, const int *pos_ptr, int pos, cudaStream_t stream)
{
    launch_k(qk_norm_rope_store_kernel, dim3((n_q + n_k + 3) / 4), dim3(128), 0, stream, q, k, v, wq, wk, cos_t, sin_t,
             static_cast<__half *>(kv_k), static_cast<__half *>(kv_v), n_q, n_k, head_dim, eps, pos_ptr, pos);
}

void launch_embed_q4k(const void *table, float *out, const int *token_ptr, int token, int hidden, int row_bytes,
                      cudaStream_t stream)
{
    launch_k(embed_q4k_kernel, dim3((hidden + 255) / 256), dim3(256), 0, stream, static_cast<const uint8_t *>(table), out,
             token_ptr, token, hidden, row_bytes);
}

void launch_argmax(const float *logits, int n, int *result, int *pos_ptr, cudaStream_t stream)
{
    int ctas = (n + 2047) / 2048;  // eight logits per thread
    ctas = ctas < 1 ? 1 : (ctas > kArgmaxCtas ? kArgmaxCtas : ctas);
    launch_k(argmax_kernel, dim3(ctas), dim3(256), 0, stream, logits, n, result, pos_ptr, static_cast<float *>(nullptr), 0);
}

void launch_argmax_pair(const float *logits, int n, int index_offset, float *pair_out, cudaStream_t stream)
{
    int ctas = (n + 2047) / 2048;
    ctas = ctas < 1 ? 1 : (ctas > kArgmaxCtas ? kArgmaxCtas : ctas);
    launch_k(argmax_kernel, dim3(ctas), dim3(256), 0, stream, logits, n, static_cast<int *>(nullptr),
             static_cast<int *>(nullptr), pair_out, index_offset);
}

void launch_argmax_merge(const float *pairs, int n, int *result, int *pos_ptr, cudaStream_t stream)
{
    launch_k(argmax_merge_kernel, dim3(1), dim3(32), 0, stream, pairs, n, result, pos_ptr);
}

}  // namespace mb200

using namespace mb200;

extern "C" {

void cuda_rms_norm(const float *input, const float *weight, float *output, int n, float eps, cudaStream_t stream)
{
    if (n <= 0) return;
    launch_rms_norm(input, weight, output, nullptr, n, eps, stream);
    MB200_CHECK_LAUNCH("cuda_rms_norm");
}

void cuda_rms_norm_residual(const float *input, const float *weight, float *normed_output, float *residual_output,
                            int n, float eps, cudaStream_t stream)
{
    if (n <= 0) return;
    launch_rms_norm(input, weight, normed_output, residual_output, n, eps, stream);
    MB200_CHECK_LAUNCH("cuda_rms_norm_residual");
}

void cuda_rms_norm_batched(const float *input, const float *weight, float *output, int head_dim, int n_heads,
                           float eps, cudaStream_t stream)
{
    if (n_heads <= 0 || head_dim <= 0) return;
    launch_k(rms_norm_heads_kernel, dim3((n_heads + 3) / 4), dim3(128), 0, stream, input, output, weight, n_heads,
             static_cast<const float *>(nullptr), static_cast<float *>(nullptr), static_cast<const float *>(nullptr), 0,
             head_dim, eps);
    MB200_CHECK_LAUNCH("cuda_rms_norm_batched");
}

void cuda_rms_norm_qk(float *q, float *k, const float *q_weight, const float *k_weight, int head_dim, int n_q,
                      int n_k, float eps, cudaStream_t stream)
{
    if (n_q + n_k <= 0 || head_dim <= 0) return;
    launch_k(rms_norm_heads_kernel, dim3((n_q + n_k + 3) / 4), dim3(128), 0, stream, q, q, q_weight, n_q, k, k, k_weight,
             n_k, head_dim, eps);
    MB200_CHECK_LAUNCH("cuda_rms_norm_qk");
}

void cuda_rope(float *q, float *k, int head_dim, int pos, float theta, int n_heads_q, int n_heads_k,
               cudaStream_t stream)
{
    const int total = (n_heads_q + n_heads_k) * (head_dim / 2);
    if (total <= 0) return;
    launch_k(rope_kernel, dim3((total + 127) / 128), dim3(128), 0, stream, q, k, head_dim, pos, theta, n_heads_q, n_heads_k);
    MB200_CHECK_LAUNCH("cuda_rope");
}

void cuda_f32_to_f16(const float *in, void *out, int n, cudaStream_t stream)
{
    if (n <= 0) return;
    launch_k(f32_to_f16_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, in, static_cast<__half *>(out), n);
    MB200_CHECK_LAUNCH("cuda_f32_to_f16");
}

void cuda_f32_to_f16_dual(const float *a, const float *b, void *oa, void *ob, int n, cudaStream_t stream)
{
    if (n <= 0) return;
    launch_k(f32_to_f16_dual_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, a, b, static_cast<__half *>(oa),
             static_cast<__half *>(ob), n);
    MB200_CHECK_LAUNCH("cuda_f32_to_f16_dual");
}

void cuda_attention_f16kv(const void *q, const void *kv_k, const void *kv_v, float *out, int n_heads_q, int head_dim,
                          int n_kv_heads, int seq_len, int gqa_ratio, float scale, cudaStream_t stream)
{
    if (n_heads_q <= 0 || seq_len <= 0 || head_dim <= 0 || n_kv_heads <= 0 || gqa_ratio <= 0) return;
    const int blocks = n_kv_heads * ((gqa_ratio + 15) / 16);
    const StaticAttn *ws = static_attn();
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv_k) |
                           reinterpret_cast<uintptr_t>(kv_v) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (head_dim == kHD && n_heads_q == n_kv_heads * gqa_ratio && blocks <= kStaticAttnBlocks && ws && aligned &&
        attn_attr()) {
        AttnParams P{};
        P.q = static_cast<const float *>(q);
        P.kv_k = static_cast<const __half *>(kv_k);
        P.kv_v = static_cast<const __half *>(kv_v);
        P.out = out;
        P.n_kv_heads = n_kv_heads;
        P.gqa = gqa_ratio;
        P.seq_len = seq_len;
        P.scale = scale;
        P.part = ws->part;
        P.ml = ws->ml;
        P.tickets = ws->tickets;
        const int S = attn_chunks_for(n_kv_heads, gqa_ratio, kStaticAttnSlots);
        launch_k(attn_decode_kernel, dim3(blocks, S), dim3(kAttnThreads), kAttnSmem, stream, P.q, P.kv_k, P.kv_v, P.out, kHD,
                 P.n_kv_heads, P.seq_len, P.gqa, P.scale, P.part, P.ml, P.tickets, static_cast<const int *>(nullptr));
    } else {
        if (head_dim > 1024 || !attn_attr()) {
            fprintf(stderr, "[mnemo_b200] cuda_attention_f16kv: head_dim=%d not supported\n", head_dim);
            set_status(MB200_ERR_UNSUPPORTED, "cuda_attention_f16kv");
            return;
        }
        const size_t smem = (8 * (size_t)head_dim + 16) * sizeof(float);
        launch_k(attn_generic_kernel, dim3(n_heads_q), dim3(256), smem, stream, static_cast<const float *>(q),
                 static_cast<const __half *>(kv_k), static_cast<const __half *>(kv_v), out, head_dim, n_kv_heads, seq_len,
                 gqa_ratio, scale);
    }
    MB200_CHECK_LAUNCH("cuda_attention_f16kv");
}

// Kernel addresses for a caller that captures these launches in a CUDA graph and patches their
// parameters per token by index (the reference does: src/forward.c:1295-1297, 1399-1408, 636-661).
// The three kernels keep the reference kernels' parameter order for that reason.
void *cuda_get_rope_kernel_ptr(void) { return reinterpret_cast<void *>(rope_kernel); }
void *cuda_get_f16dual_kernel_ptr(void) { return reinterpret_cast<void *>(f32_to_f16_dual_kernel); }
void *cuda_get_attn_f16kv_kernel_ptr(void) { return reinterpret_cast<void *>(attn_decode_kernel); }

void cuda_residual_add(const float *a, const float *b, float *out, int n, cudaStream_t stream)
{
    if (n <= 0) return;
    launch_k(residual_add_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, a, b, out, n);
    MB200_CHECK_LAUNCH("cuda_residual_add");
}

void cuda_embedding_lookup_q4k(const void *embd_table, float *output, int token_id, int hidden_size, int row_bytes,
                               cudaStream_t stream)
{
    if (hidden_size <= 0) return;
    launch_embed_q4k(embd_table, output, nullptr, token_id, hidden_size, row_bytes, stream);
    MB200_CHECK_LAUNCH("cuda_embedding_lookup_q4k");
}

void cuda_sample_token(const float *logits, int vocab_size, float temperature, float top_p,
                       unsigned long long rng_state, int *d_result, cudaStream_t stream)
{
    if (vocab_size <= 0) return;
    if (temperature > 0.0f) {
        float *pair = sample_pair_addr();
        if (!pair) {
            set_status(MB200_ERR_LAUNCH, "cuda_sample_token");
            return;
        }
        launch_argmax_pair(logits, vocab_size, 0, pair, stream);  // the maximum, for exp(l - max)
        launch_k(sample_top_p_kernel, dim3(kSampleCtas), dim3(256), 0, stream, logits, vocab_size, temperature, top_p,
                 rng_state, d_result);
        MB200_CHECK_LAUNCH("cuda_sample_token");
        return;
    }
    launch_argmax(logits, vocab_size, d_result, nullptr, stream);
    MB200_CHECK_LAUNCH("cuda_sample_token");
}

}  // extern "C"
