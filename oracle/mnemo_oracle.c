/*
 * mnemo_oracle.c -- CPU restatement of the reference's Q4_K / Q6_K hot path.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA library and the timed CPU
 * baseline. The product path never calls into this file.
 *
 * Build with -ffp-contract=off: the dequant expressions must round exactly as
 * the numpy float32 statements of tools/validate_dequant.py do (product first,
 * then subtraction), which is also what gguf.quants.dequantize produces.
 *
 * Parity pin: no golden vectors exist in the reference for this path; see the
 * header of mnemo_oracle.h for how the restatement is pinned.
 */
#include "mnemo_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* helpers                                                                   */
/* ------------------------------------------------------------------------ */

/* kernels.cu:41-43 (__half2float): exact, subnormals included
 * (forward.c:1197-1202 spells the subnormal branch out on the host). */
float mo_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t mo_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ex = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (ex == 255) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
    int e = (int)ex - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - e; /* 14..24 */
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
    return (uint16_t)(sign | half);
}

/* kernels.cu:45-53 == validate_dequant.py:53-61 */
void mo_get_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m)
{
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

static uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ------------------------------------------------------------------------ */
/* integer unpack                                                            */
/* ------------------------------------------------------------------------ */

/* kernels.cu:20-25 layout; validate_dequant.py:92-113 weight order:
 * qs chunk c (32 bytes): low nibbles -> weights 64c..64c+31 with (sc,m)[2c],
 * high nibbles -> 64c+32..64c+63 with (sc,m)[2c+1]. */
void mo_unpack_q4k_block(const uint8_t *blk, uint16_t *d_bits, uint16_t *dmin_bits,
                         uint8_t sc[8], uint8_t m[8], uint8_t q[256])
{
    *d_bits = rd16(blk);
    *dmin_bits = rd16(blk + 2);
    for (int j = 0; j < 8; j++) mo_get_scale_min_k4(j, blk + 4, &sc[j], &m[j]);
    const uint8_t *qs = blk + 16;
    for (int c = 0; c < 4; c++)
        for (int l = 0; l < 32; l++) {
            q[64 * c + l] = qs[32 * c + l] & 0xF;
            q[64 * c + 32 + l] = qs[32 * c + l] >> 4;
        }
}

/* kernels.cu:27-32 layout; validate_dequant.py:286-317 order. */
void mo_unpack_q6k_block(const uint8_t *blk, uint16_t *d_bits, int8_t scales[16], int8_t q[256])
{
    const uint8_t *ql = blk, *qh = blk + 128;
    for (int i = 0; i < 16; i++) scales[i] = (int8_t)blk[192 + i];
    *d_bits = rd16(blk + 208);
    for (int h = 0; h < 2; h++)
        for (int g = 0; g < 4; g++)
            for (int l = 0; l < 32; l++) {
                uint8_t lo4 = (uint8_t)((ql[64 * h + 32 * (g & 1) + l] >> (4 * (g >> 1))) & 0xF);
                uint8_t hi2 = (uint8_t)((qh[32 * h + l] >> (2 * g)) & 3);
                q[128 * h + 32 * g + l] = (int8_t)((int)((hi2 << 4) | lo4) - 32);
            }
}

/* ------------------------------------------------------------------------ */
/* dequant                                                                   */
/* ------------------------------------------------------------------------ */

static void dequant_q4k_block(const uint8_t *blk, float out[256])
{
    uint16_t db, mb;
    uint8_t sc[8], m[8], q[256];
    mo_unpack_q4k_block(blk, &db, &mb, sc, m, q);
    float d = mo_f16_to_f32(db), dmin = mo_f16_to_f32(mb);
    for (int s = 0; s < 8; s++) {
        float ds = d * (float)sc[s];    /* validate_dequant.py:94,97 */
        float ms = dmin * (float)m[s];  /* validate_dequant.py:95,98 */
        for (int l = 0; l < 32; l++) out[32 * s + l] = ds * (float)q[32 * s + l] - ms;
    }
}

static void dequant_q6k_block(const uint8_t *blk, float out[256])
{
    uint16_t db;
    int8_t sc[16], q[256];
    mo_unpack_q6k_block(blk, &db, sc, q);
    float d = mo_f16_to_f32(db);
    for (int g = 0; g < 16; g++) {
        float s = d * (float)sc[g]; /* validate_dequant.py:309 */
        for (int l = 0; l < 16; l++) out[16 * g + l] = s * (float)q[16 * g + l];
    }
}

static inline int bpr_of(int n_cols) { return (n_cols + 255) / 256; }

void mo_dequant_q4k(const uint8_t *w, int n_rows, int n_cols, float *out)
{
    int bpr = bpr_of(n_cols);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        float tmp[256];
        for (int b = 0; b < bpr; b++) {
            dequant_q4k_block(w + ((size_t)r * bpr + b) * MO_Q4K_BLOCK_BYTES, tmp);
            int n = n_cols - b * 256 < 256 ? n_cols - b * 256 : 256;
            memcpy(out + (size_t)r * n_cols + b * 256, tmp, (size_t)n * sizeof(float));
        }
    }
}

void mo_dequant_q6k(const uint8_t *w, int n_rows, int n_cols, float *out)
{
    int bpr = bpr_of(n_cols);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        float tmp[256];
        for (int b = 0; b < bpr; b++) {
            dequant_q6k_block(w + ((size_t)r * bpr + b) * MO_Q6K_BLOCK_BYTES, tmp);
            int n = n_cols - b * 256 < 256 ? n_cols - b * 256 : 256;
            memcpy(out + (size_t)r * n_cols + b * 256, tmp, (size_t)n * sizeof(float));
        }
    }
}

/* ------------------------------------------------------------------------ */
/* matvecs                                                                   */
/* ------------------------------------------------------------------------ */

/* One Q4_K row dot. Tail rule of the kernels (kernels.cu:124,131): a group of
 * four consecutive columns contributes only if all four are < n_cols. */
static void row_dot_q4k(const uint8_t *row, const float *x, int n_cols, float *s32, double *s64,
                        double *sabs)
{
    int bpr = bpr_of(n_cols);
    float acc = 0.0f;
    double acc64 = 0.0, a = 0.0;
    float tmp[256];
    for (int b = 0; b < bpr; b++) {
        dequant_q4k_block(row + (size_t)b * MO_Q4K_BLOCK_BYTES, tmp);
        int base = b * 256;
        for (int c = 0; c < 256; c += 4) {
            if (base + c + 3 >= n_cols) continue;
            for (int i = 0; i < 4; i++) {
                float w = tmp[c + i], xv = x[base + c + i];
                acc += w * xv;
                acc64 += (double)w * (double)xv;
                a += fabs((double)w * (double)xv);
            }
        }
    }
    *s32 = acc;
    *s64 = acc64;
    *sabs = a;
}

/* Q6_K row dot. Tail rule: per element (kernels.cu:474). */
static void row_dot_q6k(const uint8_t *row, const float *x, int n_cols, float *s32, double *s64,
                        double *sabs)
{
    int bpr = bpr_of(n_cols);
    float acc = 0.0f;
    double acc64 = 0.0, a = 0.0;
    float tmp[256];
    for (int b = 0; b < bpr; b++) {
        dequant_q6k_block(row + (size_t)b * MO_Q6K_BLOCK_BYTES, tmp);
        int base = b * 256;
        for (int c = 0; c < 256 && base + c < n_cols; c++) {
            float w = tmp[c], xv = x[base + c];
            acc += w * xv;
            acc64 += (double)w * (double)xv;
            a += fabs((double)w * (double)xv);
        }
    }
    *s32 = acc;
    *s64 = acc64;
    *sabs = a;
}

void mo_matvec_q4k(const uint8_t *w, const float *x, float *y, double *y64, double *abs_dot,
                   int n_rows, int n_cols)
{
    size_t rb = (size_t)bpr_of(n_cols) * MO_Q4K_BLOCK_BYTES;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        float s;
        double s64, a;
        row_dot_q4k(w + (size_t)r * rb, x, n_cols, &s, &s64, &a);
        y[r] = s;
        if (y64) y64[r] = s64;
        if (abs_dot) abs_dot[r] = a;
    }
}

void mo_matvec_q4k_add(const uint8_t *w, const float *x, const float *residual, float *y,
                       double *y64, int n_rows, int n_cols)
{
    size_t rb = (size_t)bpr_of(n_cols) * MO_Q4K_BLOCK_BYTES;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        float s;
        double s64, a;
        row_dot_q4k(w + (size_t)r * rb, x, n_cols, &s, &s64, &a);
        y[r] = s + residual[r]; /* kernels.cu:197 */
        if (y64) y64[r] = s64 + (double)residual[r];
    }
}

void mo_matvec_q4k_qkv(const uint8_t *wq, const uint8_t *wk, const uint8_t *wv, const float *x,
                       float *q, float *k, float *v, int q_rows, int kv_rows, int n_cols)
{
    mo_matvec_q4k(wq, x, q, NULL, NULL, q_rows, n_cols);
    mo_matvec_q4k(wk, x, k, NULL, NULL, kv_rows, n_cols);
    mo_matvec_q4k(wv, x, v, NULL, NULL, kv_rows, n_cols);
}

void mo_matvec_q4k_dual(const uint8_t *wa, const uint8_t *wb, const float *x, float *ya, float *yb,
                        int n_rows, int n_cols)
{
    mo_matvec_q4k(wa, x, ya, NULL, NULL, n_rows, n_cols);
    mo_matvec_q4k(wb, x, yb, NULL, NULL, n_rows, n_cols);
}

void mo_matvec_q4k_scaled_add(const uint8_t *w, const float *x, float *y, int n_rows, int n_cols,
                              float scale)
{
    size_t rb = (size_t)bpr_of(n_cols) * MO_Q4K_BLOCK_BYTES;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        float s;
        double s64, a;
        row_dot_q4k(w + (size_t)r * rb, x, n_cols, &s, &s64, &a);
        y[r] += scale * s; /* kernels.cu:413 */
    }
}

void mo_matvec_q6k(const uint8_t *w, const float *x, float *y, double *y64, double *abs_dot,
                   int n_rows, int n_cols)
{
    size_t rb = (size_t)bpr_of(n_cols) * MO_Q6K_BLOCK_BYTES;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        float s;
        double s64, a;
        row_dot_q6k(w + (size_t)r * rb, x, n_cols, &s, &s64, &a);
        y[r] = s;
        if (y64) y64[r] = s64;
        if (abs_dot) abs_dot[r] = a;
    }
}

/* kernels.cu:859-880: lane l accumulates columns l, l+32, ... with a fused
 * multiply-add (nvcc's default contraction), then the shfl_down tree
 * (offsets 16,8,4,2,1; an out-of-range source returns the lane's own value). */
void mo_matvec_f32(const float *w, const float *x, float *y, int n_rows, int n_cols)
{
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        const float *row = w + (size_t)r * n_cols;
        float p[32], t[32];
        for (int l = 0; l < 32; l++) {
            float s = 0.0f;
            for (int c = l; c < n_cols; c += 32) s = fmaf(row[c], x[c], s);
            p[l] = s;
        }
        for (int off = 16; off > 0; off >>= 1) {
            for (int l = 0; l < 32; l++) t[l] = p[l] + (l + off < 32 ? p[l + off] : p[l]);
            memcpy(p, t, sizeof p);
        }
        y[r] = p[0];
    }
}

void mo_matvec_f32_f64(const float *w, const float *x, double *y, int n_rows, int n_cols)
{
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        const float *row = w + (size_t)r * n_cols;
        double s = 0.0;
        for (int c = 0; c < n_cols; c++) s += (double)row[c] * (double)x[c];
        y[r] = s;
    }
}

/* ------------------------------------------------------------------------ */
/* elementwise                                                               */
/* ------------------------------------------------------------------------ */

/* kernels.cu:677-688 */
void mo_swiglu(const float *gate, const float *up, float *out, int n)
{
    for (int i = 0; i < n; i++) {
        float g = gate[i];
        float silu = g / (1.0f + expf(-g));
        out[i] = silu * up[i];
    }
}

/* kernels.cu:980-988 */
void mo_scaled_add(float *out, const float *x, float scale, int n)
{
    for (int i = 0; i < n; i++) out[i] += scale * x[i];
}

/* ------------------------------------------------------------------------ */
/* router select                                                             */
/* ------------------------------------------------------------------------ */

/* kernels.cu:993-1057. 32 lanes each keep a local top-k of their strided
 * slice with "replace the first minimum if strictly greater"; the 32x16
 * candidate table is then scanned in (lane, slot) order by the same rule;
 * weights = softmax over the k kept logits, emitted in slot order. */
void mo_topk_softmax(const float *scores, int *indices, float *weights, int n_experts, int k)
{
    float s_vals[32 * 16];
    int s_ids[32 * 16];
    for (int tid = 0; tid < 32; tid++) {
        float v[16];
        int id[16];
        for (int i = 0; i < k; i++) {
            v[i] = -1e30f;
            id[i] = -1;
        }
        for (int j = tid; j < n_experts; j += 32) {
            float val = scores[j];
            int mi = 0;
            for (int i = 1; i < k; i++)
                if (v[i] < v[mi]) mi = i;
            if (val > v[mi]) {
                v[mi] = val;
                id[mi] = j;
            }
        }
        for (int i = 0; i < 16; i++) {
            s_vals[tid * 16 + i] = i < k ? v[i] : -1e30f;
            s_ids[tid * 16 + i] = i < k ? id[i] : -1;
        }
    }
    float tv[16];
    int ti[16];
    for (int i = 0; i < k; i++) {
        tv[i] = -1e30f;
        ti[i] = -1;
    }
    for (int j = 0; j < 32 * 16; j++) {
        float val = s_vals[j];
        if (val <= -1e30f) continue;
        int mi = 0;
        for (int i = 1; i < k; i++)
            if (tv[i] < tv[mi]) mi = i;
        if (val > tv[mi]) {
            tv[mi] = val;
            ti[mi] = s_ids[j];
        }
    }
    float mx = tv[0];
    for (int i = 1; i < k; i++)
        if (tv[i] > mx) mx = tv[i];
    float sum = 0.0f;
    for (int i = 0; i < k; i++) {
        tv[i] = expf(tv[i] - mx);
        sum += tv[i];
    }
    for (int i = 0; i < k; i++) {
        weights[i] = tv[i] / sum;
        indices[i] = ti[i];
    }
}

/* ------------------------------------------------------------------------ */
/* expert / MoE block                                                        */
/* ------------------------------------------------------------------------ */

/* forward.c:1122-1142 */
void mo_expert_fwd(const uint8_t *expert, size_t gate_sz, size_t up_sz, int H, int EFF,
                   int down_type, float weight, const float *x, float *moe_out)
{
    float *g = (float *)malloc(sizeof(float) * (size_t)EFF * 3);
    float *u = g + EFF, *act = u + EFF;
    mo_matvec_q4k_dual(expert, expert + gate_sz, x, g, u, EFF, H);
    mo_swiglu(g, u, act, EFF);
    const uint8_t *down = expert + gate_sz + up_sz;
    if (down_type == 12) {
        mo_matvec_q4k_scaled_add(down, act, moe_out, H, EFF, weight);
    } else {
        float *o = (float *)malloc(sizeof(float) * (size_t)H);
        mo_matvec_q6k(down, act, o, NULL, NULL, H, EFF);
        mo_scaled_add(moe_out, o, weight, H);
        free(o);
    }
    free(g);
}

/* forward.c:818-823 (router + select), :875 (zero), expert loop, :1114 (residual add) */
void mo_moe_block(const float *router_w, const uint8_t *experts, size_t expert_stride,
                  size_t gate_sz, size_t up_sz, int down_type, int NE, int K, int H, int EFF,
                  const float *x, const float *residual, float *out, int *indices, float *weights)
{
    float *logits = (float *)malloc(sizeof(float) * (size_t)NE);
    float *moe = (float *)calloc((size_t)H, sizeof(float));
    mo_matvec_f32(router_w, x, logits, NE, H);
    mo_topk_softmax(logits, indices, weights, NE, K);
    for (int i = 0; i < K; i++) {
        if (indices[i] < 0) continue;
        mo_expert_fwd(experts + (size_t)indices[i] * expert_stride, gate_sz, up_sz, H, EFF,
                      down_type, weights[i], x, moe);
    }
    for (int i = 0; i < H; i++) out[i] = moe[i] + residual[i];
    free(logits);
    free(moe);
}

/* ------------------------------------------------------------------------ */
/* GEMM oracle                                                               */
/* ------------------------------------------------------------------------ */

static void gemm_f16(const uint8_t *w, int q6, const uint16_t *x_f16, float *out, int M, int N,
                     int K)
{
    int bpr = bpr_of(K);
    size_t rb = (size_t)bpr * (q6 ? MO_Q6K_BLOCK_BYTES : MO_Q4K_BLOCK_BYTES);
    float *xf = (float *)malloc(sizeof(float) * (size_t)M * K);
    for (size_t i = 0; i < (size_t)M * K; i++) xf[i] = mo_f16_to_f32(x_f16[i]);
#pragma omp parallel
    {
        float *wrow = (float *)malloc(sizeof(float) * (size_t)bpr * 256);
#pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            for (int b = 0; b < bpr; b++) {
                const uint8_t *blk = w + (size_t)n * rb + (size_t)b * (q6 ? 210 : 144);
                if (q6)
                    dequant_q6k_block(blk, wrow + b * 256);
                else
                    dequant_q4k_block(blk, wrow + b * 256);
            }
            for (int t = 0; t < M; t++) {
                const float *xr = xf + (size_t)t * K;
                double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
                int c = 0;
                for (; c + 3 < K; c += 4) {
                    s0 += (double)wrow[c] * xr[c];
                    s1 += (double)wrow[c + 1] * xr[c + 1];
                    s2 += (double)wrow[c + 2] * xr[c + 2];
                    s3 += (double)wrow[c + 3] * xr[c + 3];
                }
                for (; c < K; c++) s0 += (double)wrow[c] * xr[c];
                out[(size_t)t * N + n] = (float)((s0 + s1) + (s2 + s3));
            }
        }
        free(wrow);
    }
    free(xf);
}

void mo_gemm_q4k_f16(const uint8_t *w, const uint16_t *x_f16, float *out, int M, int N, int K)
{
    gemm_f16(w, 0, x_f16, out, M, N, K);
}

void mo_gemm_q6k_f16(const uint8_t *w, const uint16_t *x_f16, float *out, int M, int N, int K)
{
    gemm_f16(w, 1, x_f16, out, M, N, K);
}

/* ======================================================================== */
/* Support operators of a decode step (not the hot path; they surround it). */
/* Each is computed in double and rounded to fp32 once.                     */
/* ======================================================================== */

/* kernels.cu:692-722 / 725-749; tools/validate_rope_norm.py:47-59 (kernel_rms_norm):
 * scale = 1 / sqrt(sum(x^2) / n + eps); out = x * scale * w. */
void mo_rms_norm(const float *x, const float *w, float *out, int n, float eps)
{
    double ss = 0.0;
    for (int i = 0; i < n; i++) ss += (double)x[i] * (double)x[i];
    const double scale = 1.0 / sqrt(ss / (double)n + (double)eps);
    for (int i = 0; i < n; i++) out[i] = (float)((double)x[i] * scale * (double)w[i]);
}

/* kernels.cu:754-780, 1196-1219: the same norm per head, one weight vector for all heads. */
void mo_rms_norm_heads(const float *x, const float *w, float *out, int head_dim, int n_heads, float eps)
{
    for (int h = 0; h < n_heads; h++) mo_rms_norm(x + (size_t)h * head_dim, w, out + (size_t)h * head_dim, head_dim, eps);
}

/* kernels.cu:818-852 as restated by tools/validate_rope_norm.py:168-197 (kernel_rope): half-split
 * pairs (j, j + head_dim/2), freq = 1 / theta^(2j/head_dim), angle = pos * freq, all in double. */
void mo_rope(float *vec, int n_heads, int head_dim, int pos, float theta)
{
    const int half = head_dim / 2;
    for (int h = 0; h < n_heads; h++)
        for (int j = 0; j < half; j++) {
            const double freq = 1.0 / pow((double)theta, (2.0 * j) / (double)head_dim);
            const double a = (double)pos * freq, c = cos(a), s = sin(a);
            float *v = vec + (size_t)h * head_dim;
            const double v0 = v[j], v1 = v[j + half];
            v[j] = (float)(v0 * c - v1 * s);
            v[j + half] = (float)(v0 * s + v1 * c);
        }
}

/* kernels.cu:1309-1326: fp32 -> fp16 round-to-nearest-even. */
void mo_f32_to_f16_array(const float *in, uint16_t *out, int n)
{
    for (int i = 0; i < n; i++) out[i] = mo_f32_to_f16(in[i]);
}

/* kernels.cu:1550-1660 (attention over an fp16 KV cache, [position][kv head][head_dim]):
 * out[h] = sum_p softmax_p(scale * q[h].K[p][h / gqa]) * V[p][h / gqa], in double. */
void mo_attention_f16kv(const float *q, const uint16_t *kv_k, const uint16_t *kv_v, float *out, int n_heads_q,
                        int head_dim, int n_kv_heads, int seq_len, int gqa_ratio, float scale)
{
    const size_t stride = (size_t)n_kv_heads * head_dim;
#pragma omp parallel for schedule(dynamic)
    for (int h = 0; h < n_heads_q; h++) {
        const int kvh = h / gqa_ratio;
        double *sc = (double *)malloc(sizeof(double) * (size_t)seq_len);
        double *acc = (double *)calloc((size_t)head_dim, sizeof(double));
        double mx = -1e300;
        for (int p = 0; p < seq_len; p++) {
            const uint16_t *kp = kv_k + (size_t)p * stride + (size_t)kvh * head_dim;
            double s = 0.0;
            for (int d = 0; d < head_dim; d++) s += (double)q[(size_t)h * head_dim + d] * (double)mo_f16_to_f32(kp[d]);
            sc[p] = s * (double)scale;
            if (sc[p] > mx) mx = sc[p];
        }
        double sum = 0.0;
        for (int p = 0; p < seq_len; p++) {
            const double e = exp(sc[p] - mx);
            sum += e;
            const uint16_t *vp = kv_v + (size_t)p * stride + (size_t)kvh * head_dim;
            for (int d = 0; d < head_dim; d++) acc[d] += e * (double)mo_f16_to_f32(vp[d]);
        }
        for (int d = 0; d < head_dim; d++) out[(size_t)h * head_dim + d] = (float)(sum > 0.0 ? acc[d] / sum : 0.0);
        free(sc);
        free(acc);
    }
}

/* kernels.cu:784-793 */
void mo_residual_add(const float *a, const float *b, float *out, int n)
{
    for (int i = 0; i < n; i++) out[i] = a[i] + b[i];
}

/* Row `token` of a Q4_K table, dequantised (forward.c:1189-1229, the reference's CPU embedding;
 * same arithmetic as tools/validate_dequant.py:68-115). */
void mo_embedding_q4k(const uint8_t *table, int token, int hidden, float *out)
{
    const int bpr = bpr_of(hidden);
    float tmp[256];
    for (int b = 0; b < bpr; b++) {
        dequant_q4k_block(table + ((size_t)token * bpr + b) * MO_Q4K_BLOCK_BYTES, tmp);
        for (int j = 0; j < 256 && b * 256 + j < hidden; j++) out[b * 256 + j] = tmp[j];
    }
}

/* kernels.cu:2048-2071 (greedy branch of sample_token_kernel): thread t of 256 scans i = t, t + 256, ...
 * keeping the first strict maximum; the tree keeps the lower thread on ties. */
int mo_argmax(const float *logits, int n)
{
    float bv[256];
    int bi[256];
    for (int t = 0; t < 256; t++) {
        bv[t] = -1e30f;
        bi[t] = 0;
        for (int i = t; i < n; i += 256)
            if (logits[i] > bv[t]) {
                bv[t] = logits[i];
                bi[t] = i;
            }
    }
    for (int s = 128; s > 0; s >>= 1)
        for (int t = 0; t < s; t++)
            if (bv[t + s] > bv[t]) {
                bv[t] = bv[t + s];
                bi[t] = bi[t + s];
            }
    return bi[0];
}

/* ======================================================================== */
/* Other GGUF types on the reference's matvec() switch (forward.c:160-173).  */
/* ======================================================================== */

/* Q8_0: 34-byte blocks of 32 weights, w = d * q (kernels.cu:34-37, 644-673; validate_dequant.py:326-356). */
static void dequant_q8_0_block(const uint8_t *blk, float out[32])
{
    const float d = mo_f16_to_f32(rd16(blk));
    for (int j = 0; j < 32; j++) out[j] = d * (float)(int8_t)blk[2 + j];
}

/* Q5_K: 176-byte blocks [d][dmin][scales 12][qh 32][qs 128]; w = d*sc*(lo4 | hi << 4) - dmin*m
 * (kernels.cu:578-640; validate_dequant.py:122-183). */
static void dequant_q5k_block(const uint8_t *blk, float out[256])
{
    const float d = mo_f16_to_f32(rd16(blk)), dmin = mo_f16_to_f32(rd16(blk + 2));
    const uint8_t *scales = blk + 4, *qh = blk + 16, *q = blk + 48;
    int is = 0;
    for (int j = 0; j < 256; j += 64) {
        uint8_t sc1, m1, sc2, m2;
        mo_get_scale_min_k4(is, scales, &sc1, &m1);
        mo_get_scale_min_k4(is + 1, scales, &sc2, &m2);
        const float d1 = d * sc1, m1f = dmin * m1, d2 = d * sc2, m2f = dmin * m2;
        for (int l = 0; l < 32; l++) {
            const int lo = q[l] & 0xF, hi = (qh[(j + l) / 8] >> ((j + l) % 8)) & 1;
            out[j + l] = d1 * (float)(lo | (hi << 4)) - m1f;
        }
        for (int l = 0; l < 32; l++) {
            const int lo = q[l] >> 4, hi = (qh[(j + 32 + l) / 8] >> ((j + 32 + l) % 8)) & 1;
            out[j + 32 + l] = d2 * (float)(lo | (hi << 4)) - m2f;
        }
        q += 32;
        is += 2;
    }
}

/* Q3_K: 110-byte blocks [hmask 32][qs 64][scales 12][d]; w = d * (sc - 32) * (q2 - (hbit ? 0 : 4))
 * (kernels.cu:497-575). */
static void dequant_q3k_block(const uint8_t *blk, float out[256])
{
    const uint8_t *hmask = blk, *q = blk + 32, *scales = blk + 96;
    const float d_all = mo_f16_to_f32(rd16(blk + 108));
    int sc16[16];
    for (int i = 0; i < 8; i++) {
        sc16[i] = (int8_t)((scales[i] & 0xF) | (((scales[8 + (i >> 2)] >> (2 * (i & 3))) & 3) << 4)) - 32;
        sc16[i + 8] = (int8_t)((scales[i] >> 4) | (((scales[8 + (i >> 2)] >> (2 * (i & 3) + 4)) & 3) << 4)) - 32;
    }
    int is = 0, val = 0;
    uint8_t m = 1;
    for (int chunk = 0; chunk < 2; chunk++) {
        int shift = 0;
        for (int grp = 0; grp < 4; grp++) {
            const float dl = d_all * (float)sc16[is++];
            for (int l = 0; l < 16; l++) {
                const int q2 = (q[l] >> shift) & 3;
                out[val++] = dl * (float)(q2 - ((hmask[l] & m) ? 0 : 4));
            }
            const float dl2 = d_all * (float)sc16[is++];
            for (int l = 0; l < 16; l++) {
                const int q2 = (q[l + 16] >> shift) & 3;
                out[val++] = dl2 * (float)(q2 - ((hmask[l + 16] & m) ? 0 : 4));
            }
            shift += 2;
            m = (uint8_t)(m << 1);
        }
        q += 32;
    }
}

/* type ids as in forward.c:160-173: 8 = Q8_0, 11 = Q3_K, 13 = Q5_K (12 = Q4_K, 14 = Q6_K) */
static int block_weights(int type) { return type == 8 ? 32 : 256; }
static int block_bytes(int type)
{
    switch (type) {
        case 8: return 34;
        case 11: return 110;
        case 12: return 144;
        case 13: return 176;
        case 14: return 210;
        default: return 0;
    }
}
static void dequant_block(int type, const uint8_t *blk, float *out)
{
    switch (type) {
        case 8: dequant_q8_0_block(blk, out); break;
        case 11: dequant_q3k_block(blk, out); break;
        case 12: dequant_q4k_block(blk, out); break;
        case 13: dequant_q5k_block(blk, out); break;
        default: dequant_q6k_block(blk, out); break;
    }
}

int mo_dequant_type(int type, const uint8_t *w, int n_rows, int n_cols, float *out)
{
    const int bw = block_weights(type), bb = block_bytes(type);
    if (!bb) return -1;
    const int bpr = (n_cols + bw - 1) / bw;
    for (int r = 0; r < n_rows; r++)
        for (int b = 0; b < bpr; b++) {
            float tmp[256];
            dequant_block(type, w + ((size_t)r * bpr + b) * bb, tmp);
            for (int j = 0; j < bw && b * bw + j < n_cols; j++) out[(size_t)r * n_cols + b * bw + j] = tmp[j];
        }
    return 0;
}

/* y = dequant(W) x for any of the types above; fp32 result, optional fp64 result and sum |w x| per row. */
int mo_matvec_type(int type, const uint8_t *w, const float *x, float *y, double *y64, double *abs_dot, int n_rows,
                   int n_cols)
{
    const int bw = block_weights(type), bb = block_bytes(type);
    if (!bb) return -1;
    const int bpr = (n_cols + bw - 1) / bw;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_rows; r++) {
        float s32 = 0.0f;
        double s64 = 0.0, ad = 0.0;
        for (int b = 0; b < bpr; b++) {
            float tmp[256];
            dequant_block(type, w + ((size_t)r * bpr + b) * bb, tmp);
            for (int j = 0; j < bw && b * bw + j < n_cols; j++) {
                const float xv = x[b * bw + j];
                s32 += tmp[j] * xv;
                s64 += (double)tmp[j] * (double)xv;
                ad += fabs((double)tmp[j] * (double)xv);
            }
        }
        y[r] = s32;
        if (y64) y64[r] = s64;
        if (abs_dot) abs_dot[r] = ad;
    }
    return 0;
}

/* INT8 KV cache: per-head absmax quantisation (kernels.cu:1339-1376): scale = absmax / 127,
 * q = clamp(rint(v * 127 / absmax), -127, 127). */
void mo_f32_to_int8_kv(const float *in, int8_t *out, float *scales, int head_dim, int n_kv_heads)
{
    for (int h = 0; h < n_kv_heads; h++) {
        float absmax = 0.0f;
        for (int d = 0; d < head_dim; d++) absmax = fmaxf(absmax, fabsf(in[h * head_dim + d]));
        const float inv = absmax > 0.0f ? 127.0f / absmax : 0.0f;
        scales[h] = absmax > 0.0f ? absmax / 127.0f : 0.0f;
        for (int d = 0; d < head_dim; d++) {
            int iv = (int)rintf(in[h * head_dim + d] * inv);
            iv = iv > 127 ? 127 : (iv < -127 ? -127 : iv);
            out[h * head_dim + d] = (int8_t)iv;
        }
    }
}

/* Attention over an INT8 KV cache with per-position per-head scales (kernels.cu:1382-1480), in double. */
void mo_attention_int8kv(const float *q, const int8_t *kv_k, const int8_t *kv_v, const float *k_scales,
                         const float *v_scales, float *out, int n_heads_q, int head_dim, int n_kv_heads, int seq_len,
                         int gqa_ratio, float scale)
{
    const size_t stride = (size_t)n_kv_heads * head_dim;
#pragma omp parallel for schedule(dynamic)
    for (int h = 0; h < n_heads_q; h++) {
        const int kvh = h / gqa_ratio;
        double *sc = (double *)malloc(sizeof(double) * (size_t)seq_len);
        double *acc = (double *)calloc((size_t)head_dim, sizeof(double));
        double mx = -1e300;
        for (int p = 0; p < seq_len; p++) {
            const int8_t *kp = kv_k + (size_t)p * stride + (size_t)kvh * head_dim;
            double s = 0.0;
            for (int d = 0; d < head_dim; d++) s += (double)q[(size_t)h * head_dim + d] * (double)kp[d];
            sc[p] = s * (double)k_scales[(size_t)p * n_kv_heads + kvh] * (double)scale;
            if (sc[p] > mx) mx = sc[p];
        }
        double sum = 0.0;
        for (int p = 0; p < seq_len; p++) {
            const double e = exp(sc[p] - mx);
            sum += e;
            const int8_t *vp = kv_v + (size_t)p * stride + (size_t)kvh * head_dim;
            const double vs = (double)v_scales[(size_t)p * n_kv_heads + kvh];
            for (int d = 0; d < head_dim; d++) acc[d] += e * vs * (double)vp[d];
        }
        for (int d = 0; d < head_dim; d++) out[(size_t)h * head_dim + d] = (float)(sum > 0.0 ? acc[d] / sum : 0.0);
        free(sc);
        free(acc);
    }
}

/* Temperature + top-p sampling of one token (kernels.cu:2073-2174), the reference's own order of
 * operations restated serially: p_i = exp((l_i - max) / T); total = sum p; per residue class i mod 256
 * the eight largest p (first minimum replaced, a later equal value does not enter); the 2048
 * candidates picked largest first (first maximum) until their running sum reaches top_p * total;
 * a xoroshiro128+ draw (seed, seed ^ 0xDEADBEEFCAFEBABE, three warm-up rounds) scaled by the nucleus
 * sum; the first candidate at which the running sum reaches it. The sums are taken in double here
 * (the reference adds floats in a thread-strided / tree order this restatement does not reproduce):
 * tests use logits whose cut and draw are not within rounding of a boundary. */
int mo_sample_top_p(const float *logits, int n, float temperature, float top_p, unsigned long long seed)
{
    float mx = -1e30f;
    for (int i = 0; i < n; i++) mx = fmaxf(mx, logits[i]);
    double total = 0.0;
    static float cand_p[2048];
    static int cand_id[2048];
    for (int c = 0; c < 2048; c++) { cand_p[c] = -1.0f; cand_id[c] = -1; }
    for (int i = 0; i < n; i++) {
        const float p = expf((logits[i] - mx) / temperature);
        total += p;
        float *v = cand_p + (i % 256) * 8;
        int *id = cand_id + (i % 256) * 8;
        int mi = 0;
        for (int k = 1; k < 8; k++) if (v[k] < v[mi]) mi = k;
        if (p > v[mi]) { v[mi] = p; id[mi] = i; }
    }
    unsigned long long rs0 = seed, rs1 = seed ^ 0xDEADBEEFCAFEBABEULL, t;
    for (int w = 0; w < 4; w++) {
        t = rs0 ^ (rs0 << 23);
        rs0 = rs1;
        rs1 = t ^ rs1 ^ (t >> 17) ^ (rs1 >> 26);
    }
    const float r = (float)((rs0 + rs1) >> 11) * (1.0f / 9007199254740992.0f);
    const double mass = (double)top_p * total;
    double cumul = 0.0;
    int nucleus = 0;
    for (int pick = 0; pick < 2048; pick++) {
        int best = pick;
        for (int j = pick + 1; j < 2048; j++) if (cand_p[j] > cand_p[best]) best = j;
        if (cand_p[best] <= 0.0f) break;
        const float tp = cand_p[pick]; const int ti = cand_id[pick];
        cand_p[pick] = cand_p[best]; cand_id[pick] = cand_id[best];
        cand_p[best] = tp; cand_id[best] = ti;
        cumul += cand_p[pick];
        nucleus = pick + 1;
        if (cumul >= mass) break;
    }
    double nsum = 0.0;
    for (int i = 0; i < nucleus; i++) nsum += cand_p[i];
    const double target = (double)r * nsum;
    double acc = 0.0;
    int sampled = cand_id[0];
    for (int i = 0; i < nucleus; i++) {
        acc += cand_p[i];
        if (acc >= target) { sampled = cand_id[i]; break; }
    }
    return sampled;
}

int mo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void mo_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
