/* oracle.c — CPU restatement of the genie-ai-runtime quantized-transformer hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library in
 * genie-ai-runtime_b200/csrc: it is linked or called only by tests/, by the
 * smoke check and by the CPU-baseline leg of bench.py.  Nothing in the shipped
 * library includes, links or calls it, and the shipped library has no CPU path.
 *
 * Every function restates one piece of the reference's arithmetic and cites the
 * reference file:line it follows (paths are relative to the reference project).
 * Parity status: the float dequant+dot, the q8_1 int8 epilogue models and the
 * INT8-KV quantiser are pinned against vectors produced by the reference's own
 * host code (tests/golden); the decode dp4a GEMV, the INT8-KV decode attention,
 * QK-norm/RoPE and the whole-decoder greedy stream have no stored vectors in the
 * reference and are derived from its kernel source ("parity unpinned" by the
 * reference's own tests for those rows; the same-box run of the reference's
 * kernels is the tie-breaker there).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -fPIC -shared (see oracle/Makefile).
 * -ffp-contract=off matters: the restatement must not fuse a*b+c.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK_K 256
#define Q4K_BYTES 144
#define Q5K_BYTES 176
#define Q6K_BYTES 210

/* ── fp16 <-> fp32 (IEEE binary16, round-to-nearest-even) ─────────────────
 * Follows raw_fp16_to_float, src/kernels/gemv_q4.cu:166-183, and the
 * __float2half (rn) conversions used throughout the reference. */
float orc_h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) & 1u, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
    float r;
    if (exp == 0)       r = ldexpf((float)mant, -24);
    else if (exp == 31) r = mant ? NAN : INFINITY;
    else                r = ldexpf((float)(mant + 1024), (int)exp - 25);
    return sign ? -r : r;
}

uint16_t orc_f2h(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7FFFFFFFu;
    if (x > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);           /* NaN */
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);          /* >= 65520 -> inf */
    if (x < 0x38800000u) {                                            /* below 2^-14: subnormal half */
        float a; memcpy(&a, &x, 4);
        uint32_t m = (uint32_t)lrintf(a * 16777216.0f);              /* RNE in the default mode */
        return (uint16_t)(sign | m);
    }
    uint32_t mant = x & 0x7FFFFFu, e = (x >> 23) - 112u;
    uint32_t h = (e << 10) | (mant >> 13), rem = mant & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ── Q4_K / Q5_K 6-bit scale+min unpack — src/kernels/gemv_q4.cu:185-195 ── */
static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else {
        *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}
void orc_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) { scale_min_k4(j, q, d, m); }

static inline int type_block_bytes(int t) { return t == 12 ? Q4K_BYTES : t == 13 ? Q5K_BYTES : t == 14 ? Q6K_BYTES : 0; }
int orc_block_bytes(int ggml_type) { return type_block_bytes(ggml_type); }

/* 6-bit quant value q6 (0..63) of element i (0..255) of a Q6_K block, and its
 * scale index i/16 — layout per src/kernels/gemv_q4.cu:378-393, :559-561. */
static inline int q6_value(const uint8_t* blk, int i) {
    int n = i >> 7, r = i & 127, quarter = r >> 5, l = r & 31;
    const uint8_t* ql = blk + 64 * n; const uint8_t* qh = blk + 128 + 32 * n;
    int lo = (quarter & 1) ? ql[l + 32] : ql[l];
    lo = (quarter & 2) ? (lo >> 4) : (lo & 0xF);
    return lo | (((qh[l] >> (2 * quarter)) & 3) << 4);
}
static inline int q4_value(const uint8_t* blk, int i) {              /* :2543-2559 */
    int il = i >> 6, r = i & 63; uint8_t b = blk[16 + 32 * il + (r & 31)];
    return (r < 32) ? (b & 0xF) : (b >> 4);
}

/* ── One dequantised row → fp32 (no rounding to half).  Expression shapes
 * follow gemv_quant_cpu, src/kernels/gemv_q4.cu:2533-2624. ─────────────── */
void orc_dequant_row(const uint8_t* row, int ggml_type, int n_blocks, float* out) {
    for (int b = 0; b < n_blocks; b++) {
        if (ggml_type == 12 || ggml_type == 13) {
            const uint8_t* blk = row + (size_t)b * (ggml_type == 12 ? Q4K_BYTES : Q5K_BYTES);
            float dall = orc_h2f(rd16(blk)), dmin = orc_h2f(rd16(blk + 2));
            const uint8_t* sc = blk + 4;
            const uint8_t* qh = blk + 16;                              /* Q5_K only */
            const uint8_t* qs = blk + (ggml_type == 12 ? 16 : 48);
            for (int il = 0; il < 4; il++) {
                uint8_t s1, m1, s2, m2;
                scale_min_k4(2 * il, sc, &s1, &m1); scale_min_k4(2 * il + 1, sc, &s2, &m2);
                float d1 = dall * s1, dm1 = dmin * m1, d2 = dall * s2, dm2 = dmin * m2;
                for (int l = 0; l < 32; l++) {
                    int lo = qs[32 * il + l] & 0xF, hi = qs[32 * il + l] >> 4;
                    if (ggml_type == 13) {                              /* :2583-2588 */
                        lo += (qh[l] & (1 << (2 * il))) ? 16 : 0;
                        hi += (qh[l] & (2 << (2 * il))) ? 16 : 0;
                    }
                    out[b * QK_K + 64 * il + l]      = d1 * lo - dm1;
                    out[b * QK_K + 64 * il + 32 + l] = d2 * hi - dm2;
                }
            }
        } else {                                                        /* Q6_K :2598-2623 */
            const uint8_t* blk = row + (size_t)b * Q6K_BYTES;
            float d = orc_h2f(rd16(blk + 208));
            const int8_t* sc = (const int8_t*)(blk + 192);
            for (int i = 0; i < QK_K; i++)
                out[b * QK_K + i] = d * (float)sc[i >> 4] * (float)(q6_value(blk, i) - 32);
        }
    }
}

/* ── Float golden GEMV: y_f32[M] = W·x with fp16 x, fp32 accumulate, in the
 * sequential element order of gemv_quant_cpu, src/kernels/gemv_q4.cu:2519-2631.
 * (acc += (d*q - dm) * x  for Q4_K/Q5_K;  acc += d*sc*q*x for Q6_K in the
 * l-major order of :2607-2619.) ───────────────────────────────────────── */
void orc_gemv_float(const uint8_t* W, int ggml_type, const uint16_t* x, int M, int K, float* y) {
    const int nb = K / QK_K, bb = type_block_bytes(ggml_type);
    float* xf = (float*)malloc(sizeof(float) * (size_t)K);
    for (int k = 0; k < K; k++) xf[k] = orc_h2f(x[k]);
    #pragma omp parallel for schedule(static)
    for (int row = 0; row < M; row++) {
        const uint8_t* rb = W + (size_t)row * nb * bb;
        float acc = 0.0f;
        if (ggml_type == 12 || ggml_type == 13) {
            for (int b = 0; b < nb; b++) {
                const uint8_t* blk = rb + (size_t)b * bb;
                float dall = orc_h2f(rd16(blk)), dmin = orc_h2f(rd16(blk + 2));
                const uint8_t* sc = blk + 4; const uint8_t* qh = blk + 16;
                const uint8_t* q = blk + (ggml_type == 12 ? 16 : 48);
                int k = b * QK_K; uint8_t u1 = 1, u2 = 2;
                for (int il = 0; il < 4; il++) {
                    uint8_t s1, m1, s2, m2;
                    scale_min_k4(2 * il, sc, &s1, &m1); scale_min_k4(2 * il + 1, sc, &s2, &m2);
                    float d1 = dall * s1, dm1 = dmin * m1, d2 = dall * s2, dm2 = dmin * m2;
                    for (int l = 0; l < 32; l++) {
                        int v = q[l] & 0xF; if (ggml_type == 13 && (qh[l] & u1)) v += 16;
                        acc += (d1 * v - dm1) * xf[k + l];
                    }
                    for (int l = 0; l < 32; l++) {
                        int v = q[l] >> 4; if (ggml_type == 13 && (qh[l] & u2)) v += 16;
                        acc += (d2 * v - dm2) * xf[k + 32 + l];
                    }
                    q += 32; k += 64; u1 <<= 2; u2 <<= 2;
                }
            }
        } else {
            for (int b = 0; b < nb; b++) {
                const uint8_t* blk = rb + (size_t)b * bb;
                float d = orc_h2f(rd16(blk + 208));
                const uint8_t* ql = blk; const uint8_t* qh = blk + 128; const int8_t* sc = (const int8_t*)(blk + 192);
                int kb = b * QK_K;
                for (int n = 0; n < QK_K; n += 128) {
                    for (int l = 0; l < 32; l++) {
                        int is = l / 16;
                        int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                        int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                        int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        int k = kb + n + l;
                        acc += d * (float)sc[is + 0] * (float)q1 * xf[k];
                        acc += d * (float)sc[is + 2] * (float)q2 * xf[k + 32];
                        acc += d * (float)sc[is + 4] * (float)q3 * xf[k + 64];
                        acc += d * (float)sc[is + 6] * (float)q4 * xf[k + 96];
                    }
                    ql += 64; qh += 32; sc += 8;
                }
            }
        }
        y[row] = acc;
    }
    free(xf);
}

/* ── q8_1 activation quantiser (decode) — quantize_q8_1_kernel,
 * src/kernels/gemv_q4.cu:445-466: d = amax/127 (fp32), id = 1/d, q =
 * clamp(rn(x*id), ±127), stored d = half(d), s = half(d_fp32 * sum q).
 * IEEE division here; the reference GPU build uses approximate division,
 * so its codes may differ by one on exact ties.
 * orc_set_q8_override: the reference's kernel, as nvcc 12.9 compiles its
 * packed 36-byte block struct for sm_100a, was observed on a B200 to store
 * corrupted block scales (d with its low byte zero, s with a wrong low byte;
 * the codes are right).  The source says full fp16, and that is what this
 * oracle models.  To compare with records of the reference's GPU run all
 * the same, a test can hand over the q8_1 blocks the reference itself
 * produced for an activation vector: while an override of matching length is
 * set, the quantiser returns those blocks instead of quantising — which pins
 * integer dots, scale unpacking and epilogue to the reference's GPU
 * execution without adopting its corrupted scales. ─────────────────── */
static const int8_t* g_ovr_qs = 0; static const uint16_t* g_ovr_d = 0; static const uint16_t* g_ovr_s = 0; static int g_ovr_K = 0;
void orc_set_q8_override(const int8_t* qs, const uint16_t* d, const uint16_t* s, int K) { g_ovr_qs = qs; g_ovr_d = d; g_ovr_s = s; g_ovr_K = K; }
void orc_quantize_q8_1(const uint16_t* x, int K, int8_t* qs, uint16_t* d_out, uint16_t* s_out) {
    if (g_ovr_qs && g_ovr_K == K) {
        memcpy(qs, g_ovr_qs, (size_t)K); memcpy(d_out, g_ovr_d, sizeof(uint16_t) * (size_t)(K / 32)); memcpy(s_out, g_ovr_s, sizeof(uint16_t) * (size_t)(K / 32));
        return;
    }
    for (int b = 0; b < K / 32; b++) {
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(orc_h2f(x[b * 32 + i])));
        float d = amax / 127.0f, id = d > 0.0f ? 1.0f / d : 0.0f;
        int sum = 0;
        for (int i = 0; i < 32; i++) {
            int q = (int)lrintf(orc_h2f(x[b * 32 + i]) * id);
            q = q > 127 ? 127 : (q < -127 ? -127 : q);
            qs[b * 32 + i] = (int8_t)q; sum += q;
        }
        d_out[b] = orc_f2h(d);
        s_out[b] = orc_f2h(d * (float)sum);
    }
}

/* Integer accumulators of the dp4a path: dots[row][sub] = Σ_{32} q4·q8 for
 * Q4_K (dot_q4k_row_q8_1, gemv_q4.cu:487-494) and dots[row][g] = Σ_{16}
 * (q6-32)·q8 per 16-element scale group for Q6_K (the sum of the four
 * 4-element dp4a results of :609-614 that share one scale). */
void orc_q8_int_dots(const uint8_t* W, int ggml_type, int M, int K, const int8_t* qs, int32_t* dots) {
    const int nb = K / QK_K;
    #pragma omp parallel for schedule(static)
    for (int row = 0; row < M; row++) {
        if (ggml_type == 12) {
            for (int s = 0; s < nb * 8; s++) {
                const uint8_t* blk = W + ((size_t)row * nb + (s >> 3)) * Q4K_BYTES;
                int dot = 0;
                for (int i = 0; i < 32; i++) dot += q4_value(blk, (s & 7) * 32 + i) * (int)qs[s * 32 + i];
                dots[(size_t)row * nb * 8 + s] = dot;
            }
        } else {
            for (int g = 0; g < nb * 16; g++) {
                const uint8_t* blk = W + ((size_t)row * nb + (g >> 4)) * Q6K_BYTES;
                int dot = 0;
                for (int i = 0; i < 16; i++) dot += (q6_value(blk, (g & 15) * 16 + i) - 32) * (int)qs[g * 16 + i];
                dots[(size_t)row * nb * 16 + g] = dot;
            }
        }
    }
}

/* ── dp4a GEMV golden: quantise x to q8_1, integer dots, fp32 epilogue in
 * the reference's lane-strided order followed by the xor-shuffle tree
 * (gemv_q4.cu:474-502 Q4_K, :581-618 Q6_K, :423-428 reduction).
 * Q4_K term: acc += dall*sc*(d8*dot) - dmin*m*s8.  Q6_K term per 4 elements:
 * acc += d*sc*(d8*(float)dp4a). ──────────────────────────────────────── */
static float lane_tree(float* lane_acc) {
    for (int off = 16; off > 0; off >>= 1) {
        float t[32];
        for (int l = 0; l < 32; l++) t[l] = lane_acc[l] + lane_acc[l ^ off];
        memcpy(lane_acc, t, sizeof t);
    }
    return lane_acc[0];
}

void orc_gemv_q8(const uint8_t* W, int ggml_type, const uint16_t* x, int M, int K, float* y) {
    const int nb = K / QK_K;
    int8_t* qs = (int8_t*)malloc((size_t)K);
    uint16_t* dh = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(K / 32));
    uint16_t* sh = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(K / 32));
    orc_quantize_q8_1(x, K, qs, dh, sh);
    #pragma omp parallel for schedule(static)
    for (int row = 0; row < M; row++) {
        float lane_acc[32];
        for (int lane = 0; lane < 32; lane++) {
            float acc = 0.0f;
            if (ggml_type == 12) {
                for (int s = lane; s < nb * 8; s += 32) {
                    const uint8_t* blk = W + ((size_t)row * nb + (s >> 3)) * Q4K_BYTES;
                    uint8_t sc, m; scale_min_k4(s & 7, blk + 4, &sc, &m);
                    int dot = 0;
                    for (int i = 0; i < 32; i++) dot += q4_value(blk, (s & 7) * 32 + i) * (int)qs[s * 32 + i];
                    float dall = orc_h2f(rd16(blk)), dmin = orc_h2f(rd16(blk + 2));
                    float d8 = orc_h2f(dh[s]), s8 = orc_h2f(sh[s]);
                    acc += dall * sc * (d8 * dot) - dmin * m * s8;
                }
            } else {
                for (int sb = 0; sb < nb; sb++) {
                    const uint8_t* blk = W + ((size_t)row * nb + sb) * Q6K_BYTES;
                    float d = orc_h2f(rd16(blk + 208));
                    const int8_t* scv = (const int8_t*)(blk + 192);
                    for (int gi = lane; gi < 64; gi += 32) {
                        int p = 4 * gi, dot = 0;
                        for (int i = 0; i < 4; i++) dot += (q6_value(blk, p + i) - 32) * (int)qs[sb * 256 + p + i];
                        float d8 = orc_h2f(dh[sb * 8 + (p >> 5)]);
                        int sc = scv[p >> 4];
                        acc += d * sc * (d8 * (float)dot);
                    }
                }
            }
            lane_acc[lane] = acc;
        }
        y[row] = lane_tree(lane_acc);
    }
    free(qs); free(dh); free(sh);
}

/* ── Public entry-point models.  Which arithmetic each entry point uses:
 * gemv_quant: Q4_K and Q6_K → q8_1/dp4a, Q5_K → float (gemv_q4.cu:1263-1293);
 * gemv_quant_f32: Q4_K → dp4a, Q5_K/Q6_K → float (:1334-1356);
 * gemv_quant_add: always float, y = half(half(acc) + residual) (:996-999);
 * pair: dp4a only for Q4_K+Q4_K (:1391); triple: dp4a for the four listed
 * type combinations (:1474-1489), float otherwise. ───────────────────── */
void orc_entry_gemv_quant(const uint8_t* W, int t, const uint16_t* x, int M, int K, uint16_t* y) {
    float* yf = (float*)malloc(sizeof(float) * (size_t)M);
    if (t == 13) orc_gemv_float(W, t, x, M, K, yf); else orc_gemv_q8(W, t, x, M, K, yf);
    for (int i = 0; i < M; i++) y[i] = orc_f2h(yf[i]);
    free(yf);
}
void orc_entry_gemv_quant_f32(const uint8_t* W, int t, const uint16_t* x, int M, int K, float* y) {
    if (t == 12) orc_gemv_q8(W, t, x, M, K, y); else orc_gemv_float(W, t, x, M, K, y);
}
void orc_entry_gemv_quant_add(const uint8_t* W, int t, const uint16_t* x, const uint16_t* res, int M, int K, uint16_t* y) {
    float* yf = (float*)malloc(sizeof(float) * (size_t)M);
    orc_gemv_float(W, t, x, M, K, yf);
    for (int i = 0; i < M; i++) y[i] = orc_f2h(orc_h2f(orc_f2h(yf[i])) + orc_h2f(res[i]));
    free(yf);
}
static int triple_is_dp4a(int a, int b, int c) {
    return (a == 12 && b == 12 && c == 14) || (a == 12 && b == 12 && c == 12) ||
           (a == 14 && b == 14 && c == 14) || (a == 14 && b == 12 && c == 12);
}
void orc_entry_gemv_multi(int n, const uint8_t* const* W, const int* t, const int* M, const uint16_t* x, int K, uint16_t* const* y) {
    int dp4a = (n == 2) ? (t[0] == 12 && t[1] == 12) : (n == 3 ? triple_is_dp4a(t[0], t[1], t[2]) : 0);
    for (int i = 0; i < n; i++) {
        float* yf = (float*)malloc(sizeof(float) * (size_t)M[i]);
        if (dp4a) orc_gemv_q8(W[i], t[i], x, M[i], K, yf); else orc_gemv_float(W[i], t[i], x, M[i], K, yf);
        for (int r = 0; r < M[i]; r++) y[i][r] = orc_f2h(yf[r]);
        free(yf);
    }
}

/* ── Own-q8_1 int8 MMA models used by the reference's MMQ tests:
 * float model host_reference (tests/test_mmq_q4k_int8.cu:340-371,
 * tests/test_mmq_q6k_int8.cu:202-222) and int8 model host_int8_reference
 * (tests/test_mmq_q4k_int8.cu:373-432, tests/test_mmq_q6k_int8.cu:224-255):
 * acc += d*d8*(float)dot - dm*s8 per 32 (Q4_K); Q6_K per 16-group
 * acc += d*sc*d8*(float)dot.  y[t*M+r] = half(acc). ─────────────────── */
static void host_q8_1_group(const uint16_t* x, int8_t* q, float* d8, float* s8) {
    float a = 0.0f;
    for (int i = 0; i < 32; i++) a = fmaxf(a, fabsf(orc_h2f(x[i])));
    float d = a / 127.0f, id = d > 0.0f ? 1.0f / d : 0.0f; int sum = 0;
    for (int i = 0; i < 32; i++) {
        int v = (int)lrintf(orc_h2f(x[i]) * id); v = v > 127 ? 127 : (v < -127 ? -127 : v);
        q[i] = (int8_t)v; sum += v;
    }
    *d8 = d; *s8 = d * (float)sum;
}
void orc_testmodel_float(const uint8_t* W, int t, const uint16_t* X, int M, int N, int K, uint16_t* Y) {
    const int nb = K / QK_K, bb = type_block_bytes(t);
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < M; r++) {
        float* w = (float*)malloc(sizeof(float) * (size_t)K);
        orc_dequant_row(W + (size_t)r * nb * bb, t, nb, w);
        for (int tk = 0; tk < N; tk++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++) acc += w[k] * orc_h2f(X[(size_t)tk * K + k]);
            Y[(size_t)tk * M + r] = orc_f2h(acc);
        }
        free(w);
    }
}
void orc_testmodel_int8(const uint8_t* W, int t, const uint16_t* X, int M, int N, int K, uint16_t* Y) {
    const int nb = K / QK_K;
    #pragma omp parallel for schedule(static)
    for (int tk = 0; tk < N; tk++) {
        int8_t* q8 = (int8_t*)malloc((size_t)K); float* d8 = (float*)malloc(sizeof(float) * (K / 32)); float* s8 = (float*)malloc(sizeof(float) * (K / 32));
        for (int g = 0; g < K / 32; g++) host_q8_1_group(X + (size_t)tk * K + g * 32, q8 + g * 32, &d8[g], &s8[g]);
        for (int r = 0; r < M; r++) {
            float acc = 0.0f;
            for (int b = 0; b < nb; b++) {
                if (t == 12) {
                    const uint8_t* blk = W + ((size_t)r * nb + b) * Q4K_BYTES;
                    float dall = orc_h2f(rd16(blk)), dmin = orc_h2f(rd16(blk + 2));
                    for (int sb = 0; sb < 8; sb++) {
                        uint8_t sc, mn; scale_min_k4(sb, blk + 4, &sc, &mn);
                        float d = dall * sc, dm = dmin * mn; int g = b * 8 + sb, dot = 0;
                        for (int c = 0; c < 32; c++) dot += q4_value(blk, sb * 32 + c) * (int)q8[g * 32 + c];
                        acc += d * d8[g] * (float)dot - dm * s8[g];
                    }
                } else {
                    const uint8_t* blk = W + ((size_t)r * nb + b) * Q6K_BYTES;
                    float dall = orc_h2f(rd16(blk + 208)); const int8_t* scv = (const int8_t*)(blk + 192);
                    for (int g16 = 0; g16 < 16; g16++) {
                        int dot = 0;
                        for (int c = 0; c < 16; c++) dot += (q6_value(blk, g16 * 16 + c) - 32) * (int)q8[b * 256 + g16 * 16 + c];
                        acc += dall * (float)scv[g16] * d8[b * 8 + g16 / 2] * (float)dot;
                    }
                }
            }
            Y[(size_t)tk * M + r] = orc_f2h(acc);
        }
        free(q8); free(d8); free(s8);
    }
}

/* ── Default prefill GEMM model (gemm_quant_batched, gemv_q4.cu:2478-2495):
 * activations quantised per 32 without clamping, Q4_K keeps (half d, half
 * Σx) per group ("DS4", mmq_q4k_llama.cu:383-404), Q6_K keeps fp32 d ("D4",
 * mmq_q6k_llama.cu:424-438).  Q4_K weight scales enter as half products
 * half(d)*half(sc) and -half(dmin)*half(m) (mmq_q4k_llama.cu:159-163) and
 * each 32-group adds dmA.x*dsB.x*C + dmA.y*dsB.y in fp32 (:321-322).  Q6_K
 * adds (Σ_{16-groups} C*sc*d8) * d per 256 (:208, :361).  y[t*M+r] = half. */
static uint16_t hmul(uint16_t a, uint16_t b) { return orc_f2h(orc_h2f(a) * orc_h2f(b)); }
void orc_mmq_quantize(const uint16_t* x, int K, int8_t* q, float* d, float* s, int ds4) {
    for (int g = 0; g < K / 32; g++) {
        float amax = 0.0f, sum = 0.0f;
        /* the kernel reduces amax and sum with an xor-shuffle tree over 32 lanes */
        float v[32], a[32], sm[32];
        for (int i = 0; i < 32; i++) { v[i] = orc_h2f(x[g * 32 + i]); a[i] = fabsf(v[i]); sm[i] = v[i]; }
        for (int off = 16; off > 0; off >>= 1) {
            float ta[32], ts[32];
            for (int l = 0; l < 32; l++) { ta[l] = fmaxf(a[l], a[l ^ off]); ts[l] = sm[l] + sm[l ^ off]; }
            memcpy(a, ta, sizeof a); memcpy(sm, ts, sizeof sm);
        }
        amax = a[0]; sum = sm[0];
        float dd = amax / 127.0f, dinv = dd > 0.0f ? 1.0f / dd : 0.0f;
        for (int i = 0; i < 32; i++) q[g * 32 + i] = (int8_t)lrintf(v[i] * dinv);
        if (ds4) { d[g] = orc_h2f(orc_f2h(dd)); s[g] = orc_h2f(orc_f2h(sum)); }
        else     { d[g] = dd; if (s) s[g] = 0.0f; }
    }
}
void orc_mmq(const uint8_t* W, int t, const uint16_t* X, int M, int N, int K, uint16_t* Y) {
    const int nb = K / QK_K;
    #pragma omp parallel for schedule(static)
    for (int tk = 0; tk < N; tk++) {
        int8_t* q8 = (int8_t*)malloc((size_t)K); float* d8 = (float*)malloc(sizeof(float) * (K / 32)); float* s8 = (float*)malloc(sizeof(float) * (K / 32));
        orc_mmq_quantize(X + (size_t)tk * K, K, q8, d8, s8, t == 12);
        for (int r = 0; r < M; r++) {
            float sum = 0.0f;
            for (int b = 0; b < nb; b++) {
                if (t == 12) {
                    const uint8_t* blk = W + ((size_t)r * nb + b) * Q4K_BYTES;
                    uint16_t dh = rd16(blk), mh = (uint16_t)(rd16(blk + 2) ^ 0x8000u);   /* dm * (1,-1) */
                    for (int sb = 0; sb < 8; sb++) {
                        uint8_t sc, mn; scale_min_k4(sb, blk + 4, &sc, &mn);
                        float ax = orc_h2f(hmul(dh, orc_f2h((float)sc))), ay = orc_h2f(hmul(mh, orc_f2h((float)mn)));
                        int g = b * 8 + sb, dot = 0;
                        for (int c = 0; c < 32; c++) dot += q4_value(blk, sb * 32 + c) * (int)q8[g * 32 + c];
                        sum += ax * d8[g] * (float)dot;
                        sum += ay * s8[g];
                    }
                } else {
                    const uint8_t* blk = W + ((size_t)r * nb + b) * Q6K_BYTES;
                    float dA = orc_h2f(rd16(blk + 208)); const int8_t* scv = (const int8_t*)(blk + 192);
                    float tmp = 0.0f;
                    for (int g16 = 0; g16 < 16; g16++) {
                        int dot = 0;
                        for (int c = 0; c < 16; c++) dot += (q6_value(blk, g16 * 16 + c) - 32) * (int)q8[b * 256 + g16 * 16 + c];
                        tmp += (float)dot * (float)scv[g16] * d8[b * 8 + g16 / 2];
                    }
                    sum += tmp * dA;
                }
            }
            Y[(size_t)tk * M + r] = orc_f2h(sum);
        }
        free(q8); free(d8); free(s8);
    }
}
/* Integer accumulators of the prefill GEMM: dots[t][r][g] per 32 (Q4_K) or 16 (Q6_K). */
void orc_mmq_int_dots(const uint8_t* W, int t, const uint16_t* X, int M, int N, int K, int32_t* dots) {
    const int nb = K / QK_K, G = (t == 12) ? K / 32 : K / 16, gl = (t == 12) ? 32 : 16;
    #pragma omp parallel for schedule(static)
    for (int tk = 0; tk < N; tk++) {
        int8_t* q8 = (int8_t*)malloc((size_t)K); float* d8 = (float*)malloc(sizeof(float) * (K / 32)); float* s8 = (float*)malloc(sizeof(float) * (K / 32));
        orc_mmq_quantize(X + (size_t)tk * K, K, q8, d8, s8, t == 12);
        for (int r = 0; r < M; r++) for (int g = 0; g < G; g++) {
            const uint8_t* blk = W + ((size_t)r * nb + (g * gl) / 256) * type_block_bytes(t);
            int dot = 0, e0 = (g * gl) & 255;
            for (int c = 0; c < gl; c++)
                dot += (t == 12 ? q4_value(blk, e0 + c) : q6_value(blk, e0 + c) - 32) * (int)q8[g * gl + c];
            dots[((size_t)tk * M + r) * G + g] = dot;
        }
        free(q8); free(d8); free(s8);
    }
}

/* ── gemm_quant_batched model: N==1 routes to gemv_quant (gemv_q4.cu:2483). */
void orc_entry_gemm_quant_batched(const uint8_t* W, int t, const uint16_t* X, int M, int N, int K, uint16_t* Y) {
    if (N == 1) { orc_entry_gemv_quant(W, t, X, M, K, Y); return; }
    if (t == 13) { orc_testmodel_float(W, t, X, M, N, K, Y); return; }   /* scalar batched kernel, fp16-x float math */
    orc_mmq(W, t, X, M, N, K, Y);
}

/* ── Embedding row — dequant_embedding_q4k/q6k_kernel, gemv_q4.cu:793-864:
 * val = dall*sc*q - dmin*mn  (Q4_K), val = d*scale*(q-32)  (Q6_K) → half. */
int orc_dequant_embedding_row(const uint8_t* W, int t, int token, int hidden, uint16_t* dst) {
    if (hidden <= 0 || hidden % QK_K || (t != 12 && t != 14)) return 0;
    const int nb = hidden / QK_K;
    const uint8_t* row = W + (size_t)token * nb * type_block_bytes(t);
    for (int b = 0; b < nb; b++) for (int i = 0; i < QK_K; i++) {
        float val;
        if (t == 12) {
            const uint8_t* blk = row + (size_t)b * Q4K_BYTES;
            uint8_t sc, mn; scale_min_k4(i >> 5, blk + 4, &sc, &mn);
            val = orc_h2f(rd16(blk)) * (float)sc * (float)q4_value(blk, i) - orc_h2f(rd16(blk + 2)) * (float)mn;
        } else {
            const uint8_t* blk = row + (size_t)b * Q6K_BYTES;
            val = orc_h2f(rd16(blk + 208)) * (float)((const int8_t*)(blk + 192))[i >> 4] * (float)(q6_value(blk, i) - 32);
        }
        dst[b * QK_K + i] = orc_f2h(val);
    }
    return 1;
}

/* ── RMSNorm (+ optional residual) — CPU path of fused_rmsnorm_residual,
 * src/kernels/fused_norm.cu:147-162: rrms = 1/sqrt(Σv²/dim + eps),
 * out = half(v*rrms*w). ──────────────────────────────────────────────── */
void orc_rmsnorm(const uint16_t* x, const uint16_t* res, const void* w, int w_fp32, int rows, int dim, float eps, uint16_t* out) {
    for (int r = 0; r < rows; r++) {
        float ss = 0.0f;
        for (int i = 0; i < dim; i++) {
            float v = orc_h2f(x[(size_t)r * dim + i]); if (res) v += orc_h2f(res[(size_t)r * dim + i]);
            ss += v * v;
        }
        float rrms = 1.0f / sqrtf(ss / dim + eps);
        for (int i = 0; i < dim; i++) {
            float v = orc_h2f(x[(size_t)r * dim + i]); if (res) v += orc_h2f(res[(size_t)r * dim + i]);
            float wi = w_fp32 ? ((const float*)w)[i] : orc_h2f(((const uint16_t*)w)[i]);
            out[(size_t)r * dim + i] = orc_f2h(v * rrms * wi);
        }
    }
}

/* ── RoPE — rope_kernel, src/kernels/rope.cu:322-367: freq = 1/powf(theta,
 * 2i/hd), angle = pos*freq, (v0,v1) -> (v0 c - v1 s, v0 s + v1 c), pairs
 * (i, i+hd/2) when neox else (2i, 2i+1).  Trigonometry here is evaluated in
 * double and rounded to fp32, which is what the reference's fp32 formula
 * approximates. ──────────────────────────────────────────────────────── */
void orc_rope(uint16_t* q, uint16_t* k, int n_heads, int n_kv_heads, int hd, int pos, float theta, int neox) {
    const int h2 = hd / 2;
    for (int hh = 0; hh < n_heads + n_kv_heads; hh++) {
        uint16_t* p = hh < n_heads ? q + (size_t)hh * hd : k + (size_t)(hh - n_heads) * hd;
        if (hh >= n_heads && !k) break;
        for (int i = 0; i < h2; i++) {
            float freq = 1.0f / powf(theta, (2.0f * i) / hd);
            float angle = (float)pos * freq;
            float c = (float)cos((double)angle), s = (float)sin((double)angle);
            int i0 = neox ? i : 2 * i, i1 = neox ? i + h2 : 2 * i + 1;
            float v0 = orc_h2f(p[i0]), v1 = orc_h2f(p[i1]);
            p[i0] = orc_f2h(v0 * c - v1 * s);
            p[i1] = orc_f2h(v0 * s + v1 * c);
        }
    }
}

/* ── SwiGLU / GeGLU — src/kernels/convert.cu:85-104, :121-143. ─────────── */
void orc_swiglu(const uint16_t* g, const uint16_t* u, int n, uint16_t* out) {
    for (int i = 0; i < n; i++) { float a = orc_h2f(g[i]), b = orc_h2f(u[i]); out[i] = orc_f2h(a / (1.0f + expf(-a)) * b); }
}
void orc_geglu(const uint16_t* g, const uint16_t* u, int n, uint16_t* out) {
    for (int i = 0; i < n; i++) {
        float a = orc_h2f(g[i]), b = orc_h2f(u[i]);
        float ge = 0.5f * a * (1.0f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
        out[i] = orc_f2h(ge * b);
    }
}

/* ── KV quantiser — fp16_to_int8_kernel, src/kernels/convert.cu:26-69:
 * scale = max|x|/127, inv = 127/max, q = clamp(rn(x*inv), ±127). ───────── */
void orc_fp16_to_int8(const uint16_t* src, int rows, int cols, int8_t* dst, float* scale_out) {
    for (int r = 0; r < rows; r++) {
        float mx = 0.0f;
        for (int c = 0; c < cols; c++) mx = fmaxf(mx, fabsf(orc_h2f(src[(size_t)r * cols + c])));
        float scale = mx / 127.0f, inv = scale > 0.0f ? 127.0f / mx : 0.0f;
        if (scale_out) scale_out[r] = scale;
        for (int c = 0; c < cols; c++) {
            int q = (int)lrintf(orc_h2f(src[(size_t)r * cols + c]) * inv);
            dst[(size_t)r * cols + c] = (int8_t)(q > 127 ? 127 : (q < -127 ? -127 : q));
        }
    }
}

/* ── Softmax over logits — src/kernels/softmax.cu:15-74. ───────────────── */
void orc_softmax(float* x, int n) {
    float m = -FLT_MAX, s = 0.0f;
    for (int i = 0; i < n; i++) m = fmaxf(m, x[i]);
    for (int i = 0; i < n; i++) { x[i] = expf(x[i] - m); s += x[i]; }
    for (int i = 0; i < n; i++) x[i] /= s;
}

/* ── Decode attention, one query per head, GQA, optional sliding window.
 * Structure of the scalar CPU path src/kernels/attention.cu:1098-1134 (two
 * passes: scores+max, exp+sum, then Σ p·inv_sum·v), extended to INT8 K/V
 * with the dequantisation of the GPU kernels: k = k8*ks inside the dot
 * (:306-311) and v = v8*vs (:357-360), scales indexed [pos*n_kv+kv_head].
 * kv_int8 == 0 reads fp16 K/V. ──────────────────────────────────────── */
void orc_attention_decode(const uint16_t* q, const void* kc, const void* vc, int n_heads, int n_kv, int hd, int chd,
                          int seq, float scale, int kv_int8, const float* ks, const float* vs, int window, uint16_t* out) {
    const int kv_dim = n_kv * chd, gqa = n_heads / n_kv;
    #pragma omp parallel for schedule(static)
    for (int h = 0; h < n_heads; h++) {
        const int kvh = h / gqa;
        float* sc = (float*)malloc(sizeof(float) * (size_t)(seq > 0 ? seq : 1));
        float mx = -FLT_MAX;
        for (int p = 0; p < seq; p++) {
            if (window > 0 && p < seq - window) { sc[p] = -INFINITY; continue; }
            size_t base = (size_t)p * kv_dim + (size_t)kvh * chd;
            float dot = 0.0f;
            if (kv_int8) {
                float s = ks ? ks[(size_t)p * n_kv + kvh] : 1.0f;
                for (int d = 0; d < hd; d++) dot += orc_h2f(q[h * hd + d]) * ((float)((const int8_t*)kc)[base + d] * s);
            } else {
                for (int d = 0; d < hd; d++) dot += orc_h2f(q[h * hd + d]) * orc_h2f(((const uint16_t*)kc)[base + d]);
            }
            sc[p] = dot * scale; if (sc[p] > mx) mx = sc[p];
        }
        float sum = 0.0f;
        for (int p = 0; p < seq; p++) { sc[p] = expf(sc[p] - mx); sum += sc[p]; }
        float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        for (int d = 0; d < hd; d++) {
            float acc = 0.0f;
            for (int p = 0; p < seq; p++) {
                size_t base = (size_t)p * kv_dim + (size_t)kvh * chd;
                float v = kv_int8 ? (float)((const int8_t*)vc)[base + d] * (vs ? vs[(size_t)p * n_kv + kvh] : 1.0f)
                                  : orc_h2f(((const uint16_t*)vc)[base + d]);
                acc += sc[p] * inv * v;
            }
            out[h * hd + d] = orc_f2h(acc);
        }
        free(sc);
    }
}

/* Prefill attention: token t attends to [0, start+t+1) — kernel at
 * src/kernels/attention.cu:382-514 is the decode loop per (head, token). */
void orc_attention_prefill(const uint16_t* q, const void* kc, const void* vc, int n_heads, int n_kv, int hd, int chd,
                           int N, int start, float scale, int kv_int8, const float* ks, const float* vs, int window, uint16_t* out) {
    for (int t = 0; t < N; t++)
        orc_attention_decode(q + (size_t)t * n_heads * hd, kc, vc, n_heads, n_kv, hd, chd, start + t + 1, scale, kv_int8, ks, vs, window,
                             out + (size_t)t * n_heads * hd);
}

/* ── Whole decoder, decode-step order of Engine::decode_step /
 * transformer_layer / transformer_layer_attn_compute,
 * src/engine/decode.cu:2101-2194, :1169-1246, :1437-1530 (INT8 KV, QK-norm,
 * NeoX RoPE, SwiGLU), greedy argmax = sample_token with temperature<=0,
 * src/engine/sample.cpp:160-184.  KV layout = KVCachePool,
 * src/memory/kv_cache.cpp:96-120, :257-281. ─────────────────────────── */
typedef struct {
    int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_ctx;
    float rope_theta, eps;
} orc_model_cfg;
typedef struct {
    const uint8_t *wq, *wk, *wv, *wo, *gate, *up, *down;
    int t_wq, t_wk, t_wv, t_wo, t_gate, t_up, t_down;
    const float *rms_attn, *rms_ffn, *q_norm, *k_norm;   /* fp32 norm weights */
} orc_layer;
typedef struct {
    orc_model_cfg cfg; const orc_layer* layers;
    const uint8_t* tok_embd; int t_embd; const uint8_t* output; int t_out; const float* out_norm;
    int8_t* kv; float* kv_scales;   /* caller-allocated: 2*L*ctx*n_kv*hd bytes, 2*L*ctx*n_kv floats */
} orc_model;

static int8_t* kv_ptr(const orc_model* m, int l, int pos, int is_v) {
    size_t row = (size_t)m->cfg.n_kv_heads * m->cfg.head_dim, per = (size_t)m->cfg.max_ctx * row;
    return m->kv + (size_t)l * 2 * per + (is_v ? per : 0) + (size_t)pos * row;
}
static float* kvs_ptr(const orc_model* m, int l, int pos, int is_v) {
    size_t per = (size_t)m->cfg.max_ctx * m->cfg.n_kv_heads;
    return m->kv_scales + (size_t)l * 2 * per + (is_v ? per : 0) + (size_t)pos * m->cfg.n_kv_heads;
}

/* One decode step for `token` at position `pos`; writes fp32 logits, returns argmax. */
int orc_decode_step(const orc_model* m, int token, int pos, float* logits) {
    const orc_model_cfg* c = &m->cfg;
    const int H = c->hidden, QD = c->n_heads * c->head_dim, KVD = c->n_kv_heads * c->head_dim, I = c->ffn;
    uint16_t *x = malloc(2 * H), *normed = malloc(2 * H), *x2 = malloc(2 * H);
    uint16_t *qb = malloc(2 * QD), *kb = malloc(2 * KVD), *vb = malloc(2 * KVD), *att = malloc(2 * QD);
    uint16_t *g = malloc(2 * I), *u = malloc(2 * I), *sw = malloc(2 * I);
    orc_dequant_embedding_row(m->tok_embd, m->t_embd, token, H, x);
    for (int l = 0; l < c->n_layers; l++) {
        const orc_layer* w = &m->layers[l];
        orc_rmsnorm(x, NULL, w->rms_attn, 1, 1, H, c->eps, normed);
        const uint8_t* W3[3] = { w->wq, w->wk, w->wv }; int T3[3] = { w->t_wq, w->t_wk, w->t_wv }; int M3[3] = { QD, KVD, KVD };
        uint16_t* Y3[3] = { qb, kb, vb };
        orc_entry_gemv_multi(3, W3, T3, M3, normed, H, Y3);
        if (w->q_norm && w->k_norm) {
            orc_rmsnorm(qb, NULL, w->q_norm, 1, c->n_heads, c->head_dim, c->eps, qb);
            orc_rmsnorm(kb, NULL, w->k_norm, 1, c->n_kv_heads, c->head_dim, c->eps, kb);
        }
        orc_rope(qb, kb, c->n_heads, c->n_kv_heads, c->head_dim, pos, c->rope_theta, 1);
        orc_fp16_to_int8(kb, c->n_kv_heads, c->head_dim, kv_ptr(m, l, pos, 0), kvs_ptr(m, l, pos, 0));
        orc_fp16_to_int8(vb, c->n_kv_heads, c->head_dim, kv_ptr(m, l, pos, 1), kvs_ptr(m, l, pos, 1));
        orc_attention_decode(qb, kv_ptr(m, l, 0, 0), kv_ptr(m, l, 0, 1), c->n_heads, c->n_kv_heads, c->head_dim, c->head_dim,
                             pos + 1, 1.0f / sqrtf((float)c->head_dim), 1, kvs_ptr(m, l, 0, 0), kvs_ptr(m, l, 0, 1), 0, att);
        orc_entry_gemv_quant_add(w->wo, w->t_wo, att, x, H, QD, x2);
        orc_rmsnorm(x2, NULL, w->rms_ffn, 1, 1, H, c->eps, normed);
        const uint8_t* W2[2] = { w->gate, w->up }; int T2[2] = { w->t_gate, w->t_up }; int M2[2] = { I, I };
        uint16_t* Y2[2] = { g, u };
        orc_entry_gemv_multi(2, W2, T2, M2, normed, H, Y2);
        orc_swiglu(g, u, I, sw);
        orc_entry_gemv_quant_add(w->down, w->t_down, sw, x2, H, I, x);
    }
    orc_rmsnorm(x, NULL, m->out_norm, 1, 1, H, c->eps, normed);
    orc_entry_gemv_quant_f32(m->output, m->t_out, normed, c->vocab, H, logits);
    int best = 0;
    for (int i = 1; i < c->vocab; i++) if (logits[i] > logits[best]) best = i;
    free(x); free(normed); free(x2); free(qb); free(kb); free(vb); free(att); free(g); free(u); free(sw);
    return best;
}

/* Batched prompt prefill of n tokens at positions start..start+n-1, layer by layer, in the reference's order
 * (Engine::transformer_prefill, src/engine/decode.cu:1760-1884): RMSNorm over rows, batched K-quant products
 * (the prefill arithmetic: DS4/D4 activation quantiser, not the decode q8_1 one), per-head QK-norm, per-token RoPE
 * and INT8 KV store, causal attention over all n queries, Wo, residual add (fp16), RMSNorm, gate/up, SwiGLU, W_down,
 * residual add; then the final norm and fp32 logits of the LAST token (src/engine/decode.cu:2019-2050 computes the
 * logits of the last prompt token only).  Returns the greedy token. */
static void vec_add_h(const uint16_t* a, const uint16_t* b, int n, uint16_t* out) {      /* src/kernels/convert.cu vec_add: half(a + b) */
    for (int i = 0; i < n; i++) out[i] = orc_f2h(orc_h2f(a[i]) + orc_h2f(b[i]));
}
int orc_prefill(const orc_model* m, const int* tokens, int n, int start, float* logits) {
    const orc_model_cfg* c = &m->cfg;
    const int H = c->hidden, QD = c->n_heads * c->head_dim, KVD = c->n_kv_heads * c->head_dim, I = c->ffn;
    const size_t N = (size_t)n;
    uint16_t *x = malloc(2 * N * H), *normed = malloc(2 * N * H), *x2 = malloc(2 * N * H), *y = malloc(2 * N * H);
    uint16_t *qb = malloc(2 * N * QD), *kb = malloc(2 * N * KVD), *vb = malloc(2 * N * KVD), *att = malloc(2 * N * QD);
    uint16_t *g = malloc(2 * N * I), *u = malloc(2 * N * I), *sw = malloc(2 * N * I);
    for (int t = 0; t < n; t++) orc_dequant_embedding_row(m->tok_embd, m->t_embd, tokens[t], H, x + (size_t)t * H);
    for (int l = 0; l < c->n_layers; l++) {
        const orc_layer* w = &m->layers[l];
        orc_rmsnorm(x, NULL, w->rms_attn, 1, n, H, c->eps, normed);
        orc_entry_gemm_quant_batched(w->wq, w->t_wq, normed, QD, n, H, qb);
        orc_entry_gemm_quant_batched(w->wk, w->t_wk, normed, KVD, n, H, kb);
        orc_entry_gemm_quant_batched(w->wv, w->t_wv, normed, KVD, n, H, vb);
        if (w->q_norm && w->k_norm) {
            orc_rmsnorm(qb, NULL, w->q_norm, 1, n * c->n_heads, c->head_dim, c->eps, qb);
            orc_rmsnorm(kb, NULL, w->k_norm, 1, n * c->n_kv_heads, c->head_dim, c->eps, kb);
        }
        for (int t = 0; t < n; t++) {
            const int pos = start + t;
            orc_rope(qb + (size_t)t * QD, kb + (size_t)t * KVD, c->n_heads, c->n_kv_heads, c->head_dim, pos, c->rope_theta, 1);
            orc_fp16_to_int8(kb + (size_t)t * KVD, c->n_kv_heads, c->head_dim, kv_ptr(m, l, pos, 0), kvs_ptr(m, l, pos, 0));
            orc_fp16_to_int8(vb + (size_t)t * KVD, c->n_kv_heads, c->head_dim, kv_ptr(m, l, pos, 1), kvs_ptr(m, l, pos, 1));
        }
        orc_attention_prefill(qb, kv_ptr(m, l, 0, 0), kv_ptr(m, l, 0, 1), c->n_heads, c->n_kv_heads, c->head_dim, c->head_dim, n, start,
                              1.0f / sqrtf((float)c->head_dim), 1, kvs_ptr(m, l, 0, 0), kvs_ptr(m, l, 0, 1), 0, att);
        orc_entry_gemm_quant_batched(w->wo, w->t_wo, att, H, n, QD, y);
        vec_add_h(x, y, n * H, x2);
        orc_rmsnorm(x2, NULL, w->rms_ffn, 1, n, H, c->eps, normed);
        orc_entry_gemm_quant_batched(w->gate, w->t_gate, normed, I, n, H, g);
        orc_entry_gemm_quant_batched(w->up, w->t_up, normed, I, n, H, u);
        orc_swiglu(g, u, n * I, sw);
        orc_entry_gemm_quant_batched(w->down, w->t_down, sw, H, n, I, y);
        vec_add_h(x2, y, n * H, x);
    }
    orc_rmsnorm(x + (N - 1) * H, NULL, m->out_norm, 1, 1, H, c->eps, normed);
    orc_entry_gemv_quant_f32(m->output, m->t_out, normed, c->vocab, H, logits);
    int best = 0;
    for (int i = 1; i < c->vocab; i++) if (logits[i] > logits[best]) best = i;
    free(x); free(normed); free(x2); free(y); free(qb); free(kb); free(vb); free(att); free(g); free(u); free(sw);
    return best;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
