/* gnf4_oracle.c -- CPU restatement of the grouped 4-bit expert GEMM path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product (the CUDA library and the
 * Python modules that wrap it) links, loads or calls this file; only the test
 * suite, the smoke check and the benchmark's cpu_baseline / reference legs do,
 * and there only as the checker or as the timed CPU arm.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle_*.py)
 * against golden vectors produced by importing the reference's own Python
 * (tests/golden/make_golden.py) and, bit for bit, against the reference's native
 * CPU kernels compiled from its own source into oracle/_ref/.
 *
 * What is restated, with the reference location each function follows
 * (paths are relative to the reference project root):
 *   - NF4 element decode  w = fp32(LUT[code]) * fp32(absmax), element 2j = HIGH
 *     nibble               kernel/nf4_grouped.py:910-929 (dequant_ref), :418-419
 *   - MXFP4 element decode w = ldexp(FP4[code], e8m0 - 127), element 2j = LOW
 *     nibble               kernel/mxfp4_pack_ref.py:46-70 (dequant_mxfp4)
 *   - grouped forward      out[row] = a[row] . W[expert_ids[g]]^T for the rows of
 *     group g              kernel/nf4_grouped.py:697-907, mxfp4_grouped.py:134-172
 *   - grouped dgrad        gi[row] = g[row] . W[expert_ids[g]]
 *                          kernel/nf4_grouped.py:1056-1121
 *   - the CPU tier's locked fp32 summation order (16-lane groups, 4 round-robin
 *     accumulators, mul then add, fixed combine)
 *                          gnf4_native/cpu_kernels.c:14-33, kernel/cpu_grouped.py:53-72
 *   - dgrad locked order (n strictly ascending, mul then add)
 *                          kernel/cpu_grouped.py:119-144
 *   - M-tile table         kernel/nf4_grouped.py:334-362 (build_group_tiles)
 *   - router top-k rule    gnf4_native/cpu_kernels.c:1408-1471
 *
 * Build: gcc -O2 -ffp-contract=off -shared -fPIC (no -ffast-math; contraction
 * off so the locked two-rounding chains stay two roundings).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

static const float kNf4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f,
    0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
    0.7229568362236023f, 1.0f,
};
static const float kFp4[16] = {
    0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
    -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f,
};

enum { FMT_NF4 = 0, FMT_MXFP4 = 1 };
enum { SCALE_F32 = 0, SCALE_BF16 = 1, SCALE_E8M0 = 2 };

static inline float bf16_bits_to_f32(uint16_t h) {
    union { uint32_t u; float f; } v;
    v.u = (uint32_t)h << 16;
    return v.f;
}

/* round-to-nearest-even fp32 -> bf16 bits, NaN kept quiet (torch semantics) */
static inline uint16_t f32_to_bf16_bits(float x) {
    union { float f; uint32_t u; } v = { x };
    if ((v.u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((v.u >> 16) | 0x40);
    return (uint16_t)((v.u + 0x7fffu + ((v.u >> 16) & 1u)) >> 16);
}

API void gnf4o_luts(float *nf4_out16, float *fp4_out16) {
    memcpy(nf4_out16, kNf4, sizeof kNf4);
    memcpy(fp4_out16, kFp4, sizeof kFp4);
}

/* Decode ONE packed weight row of K elements to fp32.
 *   fmt NF4   : scale row has K/64 entries, fp32 (s_dtype 0) or bf16 bits (1)
 *   fmt MXFP4 : scale row has K/32 e8m0 bytes (s_dtype 2)
 * Exactly one rounding per element (NF4) / exact ldexp (MXFP4). */
API int gnf4o_decode_row(int fmt, const uint8_t *packed, const void *scale,
                         int s_dtype, int64_t K, float *w_out) {
    if (fmt == FMT_NF4) {
        if (K % 64) return -1;
        for (int64_t j = 0; j < K / 2; j++) {
            int64_t blk = (2 * j) / 64;
            float am = s_dtype == SCALE_BF16
                           ? bf16_bits_to_f32(((const uint16_t *)scale)[blk])
                           : ((const float *)scale)[blk];
            uint8_t b = packed[j];
            w_out[2 * j] = kNf4[b >> 4] * am;      /* element 2j   = HIGH nibble */
            w_out[2 * j + 1] = kNf4[b & 15] * am;  /* element 2j+1 = LOW nibble  */
        }
        return 0;
    }
    if (fmt == FMT_MXFP4) {
        if (K % 32 || s_dtype != SCALE_E8M0) return -1;
        for (int64_t j = 0; j < K / 2; j++) {
            int ex = (int)((const uint8_t *)scale)[(2 * j) / 32] - 127;
            uint8_t b = packed[j];
            w_out[2 * j] = ldexpf(kFp4[b & 15], ex);      /* 2j   = LOW nibble  */
            w_out[2 * j + 1] = ldexpf(kFp4[b >> 4], ex);  /* 2j+1 = HIGH nibble */
        }
        return 0;
    }
    return -2;
}

static inline int64_t scale_cols(int fmt, int64_t K) {
    return fmt == FMT_NF4 ? K / 64 : K / 32;
}
static inline int64_t scale_elt(int s_dtype) {
    return s_dtype == SCALE_F32 ? 4 : s_dtype == SCALE_BF16 ? 2 : 1;
}

/* Whole stack decode: W [E,N,K/2] (contiguous), S [E,N,K/blk] -> out [E,N,K] fp32 */
API int gnf4o_decode_stack(int fmt, const uint8_t *W, const void *S, int s_dtype,
                           int64_t E, int64_t N, int64_t K, float *out) {
    int64_t sc = scale_cols(fmt, K), se = scale_elt(s_dtype);
    for (int64_t r = 0; r < E * N; r++) {
        int rc = gnf4o_decode_row(fmt, W + r * (K / 2),
                                  (const uint8_t *)S + r * sc * se, s_dtype, K,
                                  out + r * K);
        if (rc) return rc;
    }
    return 0;
}

/* fp64 oracle of the grouped forward.
 *   a [T,K] fp32 (the caller widens bf16/fp16 exactly), sizes[G] (zero allowed),
 *   expert_ids[G] index the stack handed in.  out64 [T,N].
 * Each product and the running sum are fp64, k ascending. */
API int gnf4o_gemm_grouped_f64(int fmt, const float *a, int64_t T,
                               const uint8_t *W, const void *S, int s_dtype,
                               const int32_t *sizes, const int32_t *expert_ids,
                               int32_t G, int32_t E, int64_t N, int64_t K,
                               double *out64) {
    int64_t sc = scale_cols(fmt, K), se = scale_elt(s_dtype);
    float *w = (float *)malloc(sizeof(float) * (size_t)K);
    if (!w) return -3;
    int64_t row0 = 0;
    for (int32_t g = 0; g < G; g++) {
        int32_t e = expert_ids[g];
        if (sizes[g] < 0 || e < 0 || e >= E || row0 + sizes[g] > T) { free(w); return -1; }
        for (int64_t n = 0; n < N && sizes[g] > 0; n++) {
            int64_t r = (int64_t)e * N + n;
            int rc = gnf4o_decode_row(fmt, W + r * (K / 2),
                                      (const uint8_t *)S + r * sc * se, s_dtype, K, w);
            if (rc) { free(w); return rc; }
            for (int64_t t = row0; t < row0 + sizes[g]; t++) {
                const float *at = a + t * K;
                double acc = 0.0;
                for (int64_t k = 0; k < K; k++) acc += (double)at[k] * (double)w[k];
                out64[t * N + n] = acc;
            }
        }
        row0 += sizes[g];
    }
    if (row0 != T) { free(w); return -1; }
    free(w);
    return 0;
}

/* fp64 oracle of the grouped dgrad: gi[t,k] = sum_n g[t,n] * w[e][n,k]. */
API int gnf4o_dgrad_grouped_f64(int fmt, const float *g_in, int64_t T,
                                const uint8_t *W, const void *S, int s_dtype,
                                const int32_t *sizes, const int32_t *expert_ids,
                                int32_t G, int32_t E, int64_t N, int64_t K,
                                double *out64) {
    int64_t sc = scale_cols(fmt, K), se = scale_elt(s_dtype);
    float *w = (float *)malloc(sizeof(float) * (size_t)K);
    if (!w) return -3;
    memset(out64, 0, sizeof(double) * (size_t)(T * K));
    int64_t row0 = 0;
    for (int32_t g = 0; g < G; g++) {
        int32_t e = expert_ids[g];
        if (sizes[g] < 0 || e < 0 || e >= E || row0 + sizes[g] > T) { free(w); return -1; }
        for (int64_t n = 0; n < N && sizes[g] > 0; n++) {
            int64_t r = (int64_t)e * N + n;
            int rc = gnf4o_decode_row(fmt, W + r * (K / 2),
                                      (const uint8_t *)S + r * sc * se, s_dtype, K, w);
            if (rc) { free(w); return rc; }
            for (int64_t t = row0; t < row0 + sizes[g]; t++) {
                double gv = (double)g_in[t * N + n];
                double *o = out64 + t * K;
                for (int64_t k = 0; k < K; k++) o[k] += gv * (double)w[k];
            }
        }
        row0 += sizes[g];
    }
    free(w);
    return row0 == T ? 0 : -1;
}

/* One output element in the CPU tier's locked fp32 order: lane-group q (16
 * consecutive k) feeds accumulator q % 4, each lane doing w*a then +=, then
 * (acc0+acc1)+(acc2+acc3) per lane and a left-to-right sum of the 16 lanes. */
static float locked_dot(const float *a, const float *w, int64_t K) {
    float acc[4][16];
    memset(acc, 0, sizeof acc);
    for (int64_t q = 0; q < K / 16; q++) {
        float *dst = acc[q & 3];
        for (int i = 0; i < 16; i++) {
            float p = w[q * 16 + i] * a[q * 16 + i];
            dst[i] = dst[i] + p;
        }
    }
    float s = 0.0f;
    for (int i = 0; i < 16; i++) {
        float c = (acc[0][i] + acc[1][i]) + (acc[2][i] + acc[3][i]);
        s = s + c;
    }
    return s;
}

/* The CPU tier's forward in its locked order: fp32 in, fp32 out, sizes >= 1. */
API int gnf4o_gemv_grouped_locked(int fmt, const float *a, int64_t T,
                                  const uint8_t *W, const void *S, int s_dtype,
                                  const int32_t *sizes, const int32_t *expert_ids,
                                  int32_t G, int32_t E, int64_t N, int64_t K,
                                  float *out) {
    if (K % 16) return -1;
    int64_t sc = scale_cols(fmt, K), se = scale_elt(s_dtype);
    float *w = (float *)malloc(sizeof(float) * (size_t)K);
    if (!w) return -3;
    int64_t row0 = 0;
    for (int32_t g = 0; g < G; g++) {
        int32_t e = expert_ids[g];
        if (sizes[g] < 1 || e < 0 || e >= E || row0 + sizes[g] > T) { free(w); return -1; }
        for (int64_t n = 0; n < N; n++) {
            int64_t r = (int64_t)e * N + n;
            int rc = gnf4o_decode_row(fmt, W + r * (K / 2),
                                      (const uint8_t *)S + r * sc * se, s_dtype, K, w);
            if (rc) { free(w); return rc; }
            for (int64_t t = row0; t < row0 + sizes[g]; t++)
                out[t * N + n] = locked_dot(a + t * K, w, K);
        }
        row0 += sizes[g];
    }
    free(w);
    return row0 == T ? 0 : -1;
}

/* The CPU tier's dgrad in its locked order: per (t,k) fold over n ascending,
 * p = w*g then acc += p. */
API int gnf4o_dgrad_grouped_locked(int fmt, const float *g_in, int64_t T,
                                   const uint8_t *W, const void *S, int s_dtype,
                                   const int32_t *sizes, const int32_t *expert_ids,
                                   int32_t G, int32_t E, int64_t N, int64_t K,
                                   float *out) {
    int64_t sc = scale_cols(fmt, K), se = scale_elt(s_dtype);
    float *w = (float *)malloc(sizeof(float) * (size_t)K);
    if (!w) return -3;
    memset(out, 0, sizeof(float) * (size_t)(T * K));
    int64_t row0 = 0;
    for (int32_t g = 0; g < G; g++) {
        int32_t e = expert_ids[g];
        if (sizes[g] < 1 || e < 0 || e >= E || row0 + sizes[g] > T) { free(w); return -1; }
        for (int64_t n = 0; n < N; n++) {
            int64_t r = (int64_t)e * N + n;
            int rc = gnf4o_decode_row(fmt, W + r * (K / 2),
                                      (const uint8_t *)S + r * sc * se, s_dtype, K, w);
            if (rc) { free(w); return rc; }
            for (int64_t t = row0; t < row0 + sizes[g]; t++) {
                float gv = g_in[t * N + n];
                float *o = out + t * K;
                for (int64_t k = 0; k < K; k++) {
                    float p = w[k] * gv;
                    o[k] = o[k] + p;
                }
            }
        }
        row0 += sizes[g];
    }
    free(w);
    return row0 == T ? 0 : -1;
}

/* fp32 -> bf16 rounding of a buffer (what the GPU epilogue does once). */
API void gnf4o_round_bf16(const float *in, int64_t n, uint16_t *out_bits) {
    for (int64_t i = 0; i < n; i++) out_bits[i] = f32_to_bf16_bits(in[i]);
}

/* Exclusive prefix sum of the group sizes: offsets[G+1]. */
API int gnf4o_group_offsets(const int32_t *sizes, int32_t G, int32_t *offsets) {
    int64_t run = 0;
    offsets[0] = 0;
    for (int32_t g = 0; g < G; g++) {
        if (sizes[g] < 0) return -1;
        run += sizes[g];
        if (run > INT32_MAX) return -1;
        offsets[g + 1] = (int32_t)run;
    }
    return 0;
}

/* Fixed-height M-tile table: for every group, ceil(size/block_m) tiles of
 * (first row, valid rows, group index); empty groups emit nothing.
 * Returns the tile count (call with NULL outputs to size the arrays). */
API int64_t gnf4o_group_tiles(const int32_t *sizes, int32_t G, int32_t block_m,
                              int32_t *t_row0, int32_t *t_rows, int32_t *t_group) {
    int64_t n = 0, row = 0;
    for (int32_t g = 0; g < G; g++) {
        for (int32_t done = 0; done < sizes[g]; done += block_m) {
            int32_t take = sizes[g] - done < block_m ? sizes[g] - done : block_m;
            if (t_row0) {
                t_row0[n] = (int32_t)(row + done);
                t_rows[n] = take;
                t_group[n] = g;
            }
            n++;
        }
        row += sizes[g];
    }
    return n;
}

/* Router selection: k largest logits per token, descending, ties to the lower
 * index (a stable descending sort).  mode 0: softmax over all E then gather
 * (optionally renormalised over the k); mode 1: softmax over the k selected.
 * Weights are returned in fp32 (the caller rounds to bf16 when it mirrors the
 * reference's bf16 landing rows). */
API int gnf4o_route_topk(const float *logits, int64_t T, int64_t E, int64_t k,
                         int mode, int norm, int32_t *idx_out, float *w_out) {
    if (k < 1 || k > E || k > 64) return -1;
    for (int64_t t = 0; t < T; t++) {
        const float *lg = logits + t * E;
        float bv[64];
        int32_t bi[64];
        int64_t used = 0;
        for (int64_t e = 0; e < E; e++) {
            float v = lg[e];
            int64_t p;
            if (used < k) p = used++;
            else if (v > bv[k - 1]) p = k - 1;
            else continue;
            while (p > 0 && bv[p - 1] < v) { bv[p] = bv[p - 1]; bi[p] = bi[p - 1]; p--; }
            bv[p] = v;
            bi[p] = (int32_t)e;
        }
        float w[64];
        if (mode == 0) {
            float m = lg[0], z = 0.0f, s = 0.0f;
            for (int64_t e = 1; e < E; e++) if (lg[e] > m) m = lg[e];
            for (int64_t e = 0; e < E; e++) z += expf(lg[e] - m);
            for (int64_t j = 0; j < k; j++) { w[j] = expf(bv[j] - m) / z; s += w[j]; }
            if (norm) for (int64_t j = 0; j < k; j++) w[j] /= s;
        } else {
            float m = bv[0], z = 0.0f;
            for (int64_t j = 0; j < k; j++) z += expf(bv[j] - m);
            for (int64_t j = 0; j < k; j++) w[j] = expf(bv[j] - m) / z;
        }
        for (int64_t j = 0; j < k; j++) { idx_out[t * k + j] = bi[j]; w_out[t * k + j] = w[j]; }
    }
    return 0;
}

/* Token-expert pairs -> expert-sorted order (stable), per-expert counts.
 * flat[P] are expert ids in pair order; order_out[P] is the stable argsort,
 * counts_out[E] the histogram.  This is the producer of a_cat / sizes. */
API int gnf4o_sort_pairs(const int32_t *flat, int64_t P, int32_t E,
                         int32_t *order_out, int32_t *counts_out) {
    memset(counts_out, 0, sizeof(int32_t) * (size_t)E);
    for (int64_t p = 0; p < P; p++) {
        if (flat[p] < 0 || flat[p] >= E) return -1;
        counts_out[flat[p]]++;
    }
    int64_t *start = (int64_t *)malloc(sizeof(int64_t) * (size_t)(E + 1));
    if (!start) return -3;
    start[0] = 0;
    for (int32_t e = 0; e < E; e++) start[e + 1] = start[e] + counts_out[e];
    for (int64_t p = 0; p < P; p++) order_out[start[flat[p]]++] = (int32_t)p;
    free(start);
    return 0;
}
