/*
 * CPU oracle for the quantized MoE expert-FFN path (TEST INFRASTRUCTURE, not product code).
 *
 * A plain-C restatement of the arithmetic the reference AscendC kernels perform for
 *   - grouped_matmul, W8A8 per-token mode (int8 x int8 -> int32 -> dequant -> bf16), and
 *   - grouped_matmul_swiglu_quant, A8W8 mode (GEMM -> dequant -> SwiGLU -> per-token int8 requant).
 * Only the test-suite, the smoke check and the CPU-baseline legs of the benchmark may call it.
 * The shipped library never links or loads this file.
 *
 * PARITY UNPINNED: the reference ships no golden vectors and no numerical known-answer test for
 * either operator (its kernel unit tests run on a closed CPU simulator and compare nothing), and
 * the AscendC toolchain it needs (CANN >= 8.3: matmul::MatmulImpl, AscendDequant, SwiGLU, Cast,
 * WholeReduceMax) is closed and absent.  Values are therefore pinned only by the reference kernel
 * sources and README formulas cited beside every function below; what the reference's own tests do
 * pin (group_list semantics, workspace byte counts, tiling keys) is restated at the end of this file
 * and checked against those known answers by the CPU test-suite.
 *
 * Build: gcc -O3 -fopenmp -ffp-contract=off -fno-fast-math (see Makefile).  Every fp32 step is a
 * separately rounded IEEE operation, in the reference's order.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#if defined(__AVX2__)
#include <immintrin.h>
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 27, DT_I32 = 3, DT_NONE = -1 };

/* ------------------------------------------------------------------------------------------- */
/* scalar conversions                                                                            */
/* ------------------------------------------------------------------------------------------- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> bf16, round to nearest even: Cast(..., RoundMode::CAST_RINT) at
 * gmm/grouped_matmul/op_kernel/grouped_matmul_quant_mixcore.h:282 */
static inline uint16_t f32_to_bf16_rne(float f)
{
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
static inline float bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* fp32 -> fp16 round to nearest even (first rounding of CastFp32ToInt8Template,
 * gmm/grouped_matmul_swiglu_quant/op_kernel/grouped_matmul_swiglu_quant_utils.h:312) */
static inline uint16_t f32_to_f16_rne(float f)
{
    uint32_t u = f2u(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);      /* NaN */
    if (a >= 0x47800000u) {                                       /* >= 65536: inf (or overflow) */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);      /* rounds up to 65536 -> inf */
    if (a < 0x33000001u) return (uint16_t)sign;                   /* < 2^-25 (or == 2^-25, tie to 0) */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    if (e < -14) {                                                /* subnormal half */
        int shift = -14 - e + 13;                                 /* 14..24 */
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3ffu);
    uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;       /* carry may bump the exponent: fine */
    return (uint16_t)(sign | q);
}
static inline float f16_to_f32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0) {
        if (m == 0) return u2f(sign);
        float v = (float)m * 5.9604644775390625e-08f; /* m * 2^-24, exact */
        return sign ? -v : v;
    }
    if (e == 31) return u2f(sign | 0x7f800000u | (m << 13));
    return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

/* fp16 -> int8, round to nearest even (second rounding, ..._utils.h:315).  The reference has no
 * clamp; values beyond the int8 range saturate here and NaN maps to 0 (what the GPU cast does). */
static inline int8_t f16_to_i8_rne(uint16_t h)
{
    float v = f16_to_f32(h);
    if (v != v) return 0;
    float r = nearbyintf(v); /* default rounding mode = to nearest even */
    if (r > 127.0f) r = 127.0f;
    if (r < -128.0f) r = -128.0f;
    return (int8_t)(int)r;
}

static inline float load_scale(const void *p, int dtype, int64_t i)
{
    if (dtype == DT_F32) return ((const float *)p)[i];
    if (dtype == DT_BF16) return bf16_to_f32(((const uint16_t *)p)[i]);
    return f16_to_f32(((const uint16_t *)p)[i]);
}

/* ------------------------------------------------------------------------------------------- */
/* group_list -> (first row, row count) per group                                               */
/* ------------------------------------------------------------------------------------------- */

/* gmm/grouped_matmul/op_kernel/grouped_matmul_utils.h:243-257 (GetSplitValueFromGroupList):
 * type 0 = running total (rows = gl[g] - gl[g-1]), type 1 = per-group count; values are narrowed to
 * int32.  gmm/grouped_matmul/op_kernel/grouped_matmul.h:236-247, 263: a group with rows <= 0 is
 * skipped; row offsets advance by the rows of the groups before it.
 * Guard with no reference counterpart: ranges are clipped to [0, M] so that a malformed list can
 * never address memory outside the tensors. */
ORACLE_API int oracle_group_layout(const int64_t *group_list, int64_t len, int type, int64_t M,
                                   int64_t *row_start, int64_t *row_count)
{
    int64_t prev = 0, run = 0;
    for (int64_t g = 0; g < len; ++g) {
        int32_t v = (int32_t)group_list[g];
        int64_t start, rows;
        if (type == 0) { start = prev; rows = (int64_t)v - prev; prev = v; }
        else           { start = run;  rows = v; if (v > 0) run += v; }
        if (rows < 0) rows = 0;
        if (start < 0) { rows += start; start = 0; if (rows < 0) rows = 0; }
        if (start > M) { start = M; rows = 0; }
        if (start + rows > M) rows = M - start;
        row_start[g] = start;
        row_count[g] = rows;
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------- */
/* exact int32 GEMM for one group: acc[r, n] = sum_k x[r,k] * w[k,n]                             */
/* (matmul::MatmulImpl int8 path; gmm/grouped_matmul/op_kernel/grouped_matmul_quant_mixcore.h:175-214, */
/*  gmm/grouped_matmul_swiglu_quant/op_kernel/grouped_matmul_swiglu_quant.h:158-182)             */
/* ------------------------------------------------------------------------------------------- */

/* w element (k, n) lives at w[k * wsk + n * wsn]: (N,1) for the [K,N] layout, (1,K) for a
 * transposed view.  acc is [rows, N] row-major. */
static void gemm_group_generic(const int8_t *x, int64_t rows, int64_t K, int64_t N, const int8_t *w,
                               int64_t wsk, int64_t wsn, int32_t *acc)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        int32_t *a = acc + r * N;
        for (int64_t n = 0; n < N; ++n) a[n] = 0;
        if (wsn == 1) {
            for (int64_t k = 0; k < K; ++k) {
                int32_t xv = x[r * K + k];
                const int8_t *wr = w + k * wsk;
                for (int64_t n = 0; n < N; ++n) a[n] += xv * (int32_t)wr[n];
            }
        } else {
            for (int64_t n = 0; n < N; ++n) {
                int32_t s = 0;
                for (int64_t k = 0; k < K; ++k) s += (int32_t)x[r * K + k] * (int32_t)w[k * wsk + n * wsn];
                a[n] = s;
            }
        }
    }
}

#if defined(__AVX2__)
/* 4 rows x 16 columns register block; k is consumed in pairs through pmaddwd, which is exact here:
 * |x*w| <= 127*128 and a pair sum fits int32 with huge margin. */
static void gemm_group_avx2(const int8_t *x, int64_t rows, int64_t K, int64_t N, const int8_t *w, int32_t *acc)
{
    const int64_t nblk = N / 16, rblk = (rows + 3) / 4;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t rb = 0; rb < rblk; ++rb) {
        for (int64_t nb = 0; nb < nblk; ++nb) {
            const int64_t r0 = rb * 4, n0 = nb * 16;
            const int mr = (int)((rows - r0) < 4 ? (rows - r0) : 4);
            const int8_t *xr[4];
            for (int i = 0; i < 4; ++i) xr[i] = x + (r0 + (i < mr ? i : 0)) * K;
            __m256i c[4][2];
            for (int i = 0; i < 4; ++i) c[i][0] = c[i][1] = _mm256_setzero_si256();
            int64_t k = 0;
            for (; k + 1 < K; k += 2) {
                __m128i w0 = _mm_loadu_si128((const __m128i *)(w + k * N + n0));
                __m128i w1 = _mm_loadu_si128((const __m128i *)(w + (k + 1) * N + n0));
                __m256i lo = _mm256_cvtepi8_epi16(_mm_unpacklo_epi8(w0, w1)); /* cols 0..7, (k,k+1) pairs */
                __m256i hi = _mm256_cvtepi8_epi16(_mm_unpackhi_epi8(w0, w1)); /* cols 8..15 */
                for (int i = 0; i < 4; ++i) {
                    uint32_t p = (uint32_t)(uint16_t)(int16_t)xr[i][k] | ((uint32_t)(uint16_t)(int16_t)xr[i][k + 1] << 16);
                    __m256i xv = _mm256_set1_epi32((int)p);
                    c[i][0] = _mm256_add_epi32(c[i][0], _mm256_madd_epi16(lo, xv));
                    c[i][1] = _mm256_add_epi32(c[i][1], _mm256_madd_epi16(hi, xv));
                }
            }
            if (k < K) {
                __m128i w0 = _mm_loadu_si128((const __m128i *)(w + k * N + n0));
                __m128i z = _mm_setzero_si128();
                __m256i lo = _mm256_cvtepi8_epi16(_mm_unpacklo_epi8(w0, z));
                __m256i hi = _mm256_cvtepi8_epi16(_mm_unpackhi_epi8(w0, z));
                for (int i = 0; i < 4; ++i) {
                    uint32_t p = (uint32_t)(uint16_t)(int16_t)xr[i][k];
                    __m256i xv = _mm256_set1_epi32((int)p);
                    c[i][0] = _mm256_add_epi32(c[i][0], _mm256_madd_epi16(lo, xv));
                    c[i][1] = _mm256_add_epi32(c[i][1], _mm256_madd_epi16(hi, xv));
                }
            }
            for (int i = 0; i < mr; ++i) {
                _mm256_storeu_si256((__m256i *)(acc + (r0 + i) * N + n0), c[i][0]);
                _mm256_storeu_si256((__m256i *)(acc + (r0 + i) * N + n0 + 8), c[i][1]);
            }
        }
    }
    /* column tail */
    const int64_t nt = nblk * 16;
    if (nt < N) {
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; ++r)
            for (int64_t n = nt; n < N; ++n) {
                int32_t s = 0;
                for (int64_t kk = 0; kk < K; ++kk) s += (int32_t)x[r * K + kk] * (int32_t)w[kk * N + n];
                acc[r * N + n] = s;
            }
    }
}
#endif

static int g_force_generic = 0;
ORACLE_API void oracle_force_generic_gemm(int on) { g_force_generic = on; }

static void gemm_group(const int8_t *x, int64_t rows, int64_t K, int64_t N, const int8_t *w, int64_t wsk,
                       int64_t wsn, int32_t *acc)
{
#if defined(__AVX2__)
    if (!g_force_generic && wsn == 1 && wsk == N && N >= 16) { gemm_group_avx2(x, rows, K, N, w, acc); return; }
#endif
    gemm_group_generic(x, rows, K, N, w, wsk, wsn, acc);
}

/* ------------------------------------------------------------------------------------------- */
/* grouped_matmul, W8A8 per-token                                                               */
/* ------------------------------------------------------------------------------------------- */

/* Epilogue of GMMQuantMixCoreCompute (gmm/grouped_matmul/op_kernel/grouped_matmul_quant_mixcore.h):
 *   t = float(acc) * float(scale[e,n])        AscendDequant, :262
 *   t = t * per_token_scale[m]                PerTokenQuant Mul, :300   (order: (acc*w_scale)*x_scale)
 *   t = t + float(bias[e,n])  if bias is bf16 :309-313
 *   act_type 1: t = max(t, 0)                 Relu, :398
 *   act_type 2 / 4 / 5: Gelu / FasterGelu / Silu of the vector library, :394-403.  The library is not part of the
 *             reference's sources; its published definitions are restated in activation() below (parity unpinned).
 *   y = bf16_rne(t)  (or fp16_rne(t))         :282
 * An int32 bias is added inside the matmul to the accumulator (gmm/grouped_matmul/op_kernel/grouped_matmul.h:451-469).
 *
 * y_dtype: 27 = bf16 output; 1 = fp16 output; 3 = raw int32 accumulators (+ int32 bias) written to y.
 * w_trans: 0 = weight stored [E,K,N]; 1 = weight stored [E,N,K] (the transposed view the operator accepts).
 * Rows not covered by group_list are left untouched.  acc_out / pre_cast (both [M,N], optional) receive
 * the int32 accumulators and the fp32 values before the final cast. */
/* Gelu(x) = x / (1 + exp(-1.59576912 (x + 0.044715 x^3))), FasterGelu(x) = x / (1 + exp(-1.702 x)),
 * Silu(x) = x / (1 + exp(-x)); fp32, every operation rounded on its own (-ffp-contract=off). */
static inline float activation(int act_type, float t)
{
    switch (act_type) {
        case 1: return t > 0.0f ? t : 0.0f;
        case 2: {
            const float t3 = (t * t) * t;
            const float u = -1.59576912f * (t + 0.044715f * t3);
            return t / (1.0f + expf(u));
        }
        case 4: return t / (1.0f + expf(-1.702f * t));
        case 5: return t / (1.0f + expf(-t));
        default: return t;
    }
}

ORACLE_API int oracle_gmm_w8a8(const int8_t *x, const int8_t *w, const void *scale, int scale_dtype,
                               const float *per_token_scale, const void *bias, int bias_dtype,
                               const int64_t *group_list, int64_t gl_len, int gl_type, int64_t M, int64_t K,
                               int64_t N, int64_t E, int act_type, int w_trans, int y_dtype, void *y,
                               int32_t *acc_out, float *pre_cast)
{
    if (gl_len > E) return -1;
    int64_t *rs = (int64_t *)malloc(sizeof(int64_t) * (size_t)(2 * gl_len + 2));
    int64_t *rc = rs + gl_len + 1;
    oracle_group_layout(group_list, gl_len, gl_type, M, rs, rc);
    int64_t maxrows = 0;
    for (int64_t g = 0; g < gl_len; ++g) if (rc[g] > maxrows) maxrows = rc[g];
    int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)(maxrows > 0 ? maxrows : 1) * (size_t)N);
    for (int64_t g = 0; g < gl_len; ++g) {
        const int64_t r0 = rs[g], rows = rc[g];
        if (rows <= 0) continue;
        const int8_t *wg = w + g * K * N;
        gemm_group(x + r0 * K, rows, K, N, wg, w_trans ? 1 : N, w_trans ? K : 1, acc);
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const int64_t m = r0 + r;
            const float xs = per_token_scale ? per_token_scale[m] : 1.0f;
            for (int64_t n = 0; n < N; ++n) {
                int32_t a = acc[r * N + n];
                if (bias && bias_dtype == DT_I32) a += ((const int32_t *)bias)[g * N + n];
                if (acc_out) acc_out[m * N + n] = a;
                if (y_dtype == DT_I32) { ((int32_t *)y)[m * N + n] = a; continue; }
                float t = (float)a;                       /* int32 -> fp32, round to nearest even */
                t = t * load_scale(scale, scale_dtype, g * N + n);
                if (per_token_scale) t = t * xs;
                if (bias && bias_dtype == DT_BF16) t = t + bf16_to_f32(((const uint16_t *)bias)[g * N + n]);
                t = activation(act_type, t);
                if (pre_cast) pre_cast[m * N + n] = t;
                ((uint16_t *)y)[m * N + n] = y_dtype == DT_F16 ? f32_to_f16_rne(t) : f32_to_bf16_rne(t);
            }
        }
    }
    free(acc);
    free(rs);
    return 0;
}

/* ------------------------------------------------------------------------------------------- */
/* grouped_matmul_finalize_routing, W8A8                                                        */
/* ------------------------------------------------------------------------------------------- */

/* QuantGroupMatmul<combine = true> of gmm/grouped_matmul_finalize_routing/op_kernel/grouped_matmul_finalize_routing.h:
 *   PreProcess (:208-258), only when shared_input / logit are given ("scatterAdd", base_tiling.cpp:296-300):
 *     y[r, :] = 0 for r outside [shared_offset, shared_offset + shared_rows)
 *     y[shared_offset + r, :] = float(shared_input[r, :]) * shared_weight        Cast CAST_NONE + Muls, :245-249
 *   per row m of group g (groups with no rows skipped, :272-275):
 *     t = float(acc[m, n]) * float(scale[g, n])                                   AscendDequant, :432
 *     s = per_token[m] * logit[m]  (logit[m] alone without per_token)             Mul, :524
 *     t = t * s                                                                   Mul, :441-446
 *     t = t + logit[m] * float(bias[g, n])    if bias (bf16)                      :535-540, :443
 *     y[row_index[m], n] += t   (atomic add, :347-360)   -- or  = t  without shared_input / logit
 * The reference's additions are atomic and unordered; this restatement adds in row order, so a comparison needs a
 * tolerance of a few fp32 ulps of the sum of magnitudes (abs_sum, optional [y_rows, N], receives that sum).
 * Without logits the reference multiplies the bias by a buffer it never filled (:535); here the bias is then added as is.
 * group_list: gl_type 1 (counts, the only value the reference's API admits) or 0.  row_index is int64 (idx_i32 = 0) or int32. */
ORACLE_API int oracle_gmm_finalize_routing(const int8_t *x, const int8_t *w, const void *scale, int scale_dtype,
                                           const uint16_t *bias_bf16, const float *per_token, const int64_t *group_list,
                                           int64_t gl_len, int gl_type, const uint16_t *shared_bf16, int64_t shared_rows,
                                           int64_t shared_offset, float shared_weight, const float *logit,
                                           const void *row_index, int idx_i32, int64_t M, int64_t K, int64_t N, int64_t E,
                                           float *y, int64_t y_rows, double *abs_sum)
{
    if (gl_len > E) return -1;
    const int add = shared_bf16 != NULL || logit != NULL;
    if (add) {
        for (int64_t r = 0; r < y_rows; ++r) {
            const int in_shared = shared_bf16 && r >= shared_offset && r < shared_offset + shared_rows;
            for (int64_t n = 0; n < N; ++n) {
                float v = 0.0f;
                if (in_shared) v = bf16_to_f32(shared_bf16[(r - shared_offset) * N + n]) * shared_weight;
                y[r * N + n] = v;
                if (abs_sum) abs_sum[r * N + n] = fabs((double)v);
            }
        }
    }
    int64_t *rs = (int64_t *)malloc(sizeof(int64_t) * (size_t)(2 * gl_len + 2));
    int64_t *rc = rs + gl_len + 1;
    oracle_group_layout(group_list, gl_len, gl_type, M, rs, rc);
    int64_t maxrows = 0;
    for (int64_t g = 0; g < gl_len; ++g) if (rc[g] > maxrows) maxrows = rc[g];
    int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)(maxrows > 0 ? maxrows : 1) * (size_t)N);
    for (int64_t g = 0; g < gl_len; ++g) {
        const int64_t r0 = rs[g], rows = rc[g];
        if (rows <= 0) continue;
        gemm_group(x + r0 * K, rows, K, N, w + g * K * N, N, 1, acc);
        for (int64_t r = 0; r < rows; ++r) {   /* sequential: rows may share a destination */
            const int64_t m = r0 + r;
            const int64_t dst = idx_i32 ? (int64_t)((const int32_t *)row_index)[m] : ((const int64_t *)row_index)[m];
            if (dst < 0 || dst >= y_rows) continue;
            const float lg = logit ? logit[m] : 1.0f;
            float s;
            if (logit) s = per_token ? per_token[m] * lg : lg;
            else s = per_token ? per_token[m] : 1.0f;
            for (int64_t n = 0; n < N; ++n) {
                float t = (float)acc[r * N + n] * load_scale(scale, scale_dtype, g * N + n);
                t = t * s;
                if (bias_bf16) t = t + lg * bf16_to_f32(bias_bf16[g * N + n]);
                if (add) {
                    y[dst * N + n] = y[dst * N + n] + t;
                    if (abs_sum) abs_sum[dst * N + n] += fabs((double)t);
                } else {
                    y[dst * N + n] = t;
                    if (abs_sum) abs_sum[dst * N + n] = fabs((double)t);
                }
            }
        }
    }
    free(acc);
    free(rs);
    return 0;
}

/* ------------------------------------------------------------------------------------------- */
/* moe_init_routing_v3 (the producer of the path's inputs)                                      */
/* ------------------------------------------------------------------------------------------- */

/* fp32 -> fp16 towards zero (CAST_TRUNC). */
static inline uint16_t f32_to_f16_rz(float f)
{
    uint16_t h = f32_to_f16_rne(f);
    if ((h & 0x7fffu) > 0x7c00u) return h;                        /* NaN */
    const float back = f16_to_f32(h);
    if (fabsf(back) > fabsf(f)) h = (uint16_t)(h - 1);            /* rounded away from zero: step one value back */
    return h;
}

/* Restatement of moe/moe_init_routing_v3/op_kernel:
 *   pair j = token * k + slot; pairs with start <= expert < end are sorted by expert, equal experts by j (key-value sort of
 *   moe_v3_sort_*.h); ExpertTokensCount (moe_v3_expert_tokens_count.h:246-282) gives the counts;
 *   row_idx_type 1: expanded_row_idx[i] = j; 0: expanded_row_idx[j] = i, -1 for filtered pairs (moe_v3_row_idx_gather.h:141-156).
 *   quant = 1 (MoeGatherOutDynamicQuant::Compute, moe_v3_gather_dynamic_quant.h:103-143):
 *     v = float(x) [* smooth[expert - start]]; s = max|v| / 127; q = int8(round_half_away(fp16_towards_zero(v / s)))
 *   quant = 0 (MoeGatherOut, moe_v3_gather_out.h:197-233): row copied, expanded_scale[i] = scale[token] if given.
 * x_dtype: DT_F32 / DT_F16 / DT_BF16 (16-bit types as bit patterns); int8 rows (x_dtype 2) only with quant = 0.
 * Returns the number of output rows. */
ORACLE_API int64_t oracle_moe_init_routing_v3(const void *x, int x_dtype, const int32_t *expert_idx, const float *scale, int64_t n,
                                              int64_t k, int64_t h, int64_t expert_num, int64_t start, int64_t end, int quant,
                                              int row_idx_type, int count_type, void *expanded_x, int32_t *expanded_row_idx,
                                              int64_t *counts_out, float *expanded_scale)
{
    const int64_t pairs = n * k, range = end - start;
    int64_t *count = (int64_t *)calloc((size_t)range + 1, sizeof(int64_t));
    int64_t *first = (int64_t *)calloc((size_t)range + 1, sizeof(int64_t));
    for (int64_t j = 0; j < pairs; ++j) {
        const int64_t e = (int64_t)expert_idx[j] - start;
        if (e >= 0 && e < range) count[e]++;
    }
    int64_t total = 0, nz = 0;
    for (int64_t e = 0; e < range; ++e) {
        first[e] = total;
        total += count[e];
        if (count_type == 1) counts_out[e] = count[e];
        else if (count[e] != 0) { counts_out[2 * nz] = e + start; counts_out[2 * nz + 1] = count[e]; ++nz; }
    }
    if (count_type == 2) {
        const int64_t written = range + 1 < expert_num ? range + 1 : expert_num;
        for (int64_t i = nz; i < written; ++i) { counts_out[2 * i] = 0; counts_out[2 * i + 1] = 0; }
    }
    const size_t eb = x_dtype == DT_F32 ? 4 : (x_dtype == 2 ? 1 : 2);
    float *v = (float *)malloc(sizeof(float) * (size_t)(h > 0 ? h : 1));
    for (int64_t j = 0; j < pairs; ++j) {          /* ascending j inside every expert: the stable order */
        const int64_t e = (int64_t)expert_idx[j] - start;
        if (e < 0 || e >= range) {
            if (row_idx_type == 0) expanded_row_idx[j] = -1;
            continue;
        }
        const int64_t i = first[e]++;
        if (row_idx_type == 1) expanded_row_idx[i] = (int32_t)j;
        else expanded_row_idx[j] = (int32_t)i;
        const int64_t token = j / k;
        const char *src = (const char *)x + (size_t)token * (size_t)h * eb;
        if (!quant) {
            memcpy((char *)expanded_x + (size_t)i * (size_t)h * eb, src, (size_t)h * eb);
            if (scale && expanded_scale) expanded_scale[i] = scale[token];
            continue;
        }
        float amax = 0.0f;
        for (int64_t c = 0; c < h; ++c) {
            float t;
            if (x_dtype == DT_F32) t = ((const float *)src)[c];
            else if (x_dtype == DT_F16) t = f16_to_f32(((const uint16_t *)src)[c]);
            else t = bf16_to_f32(((const uint16_t *)src)[c]);
            if (scale) t = t * scale[e * h + c];
            v[c] = t;
            if (fabsf(t) > amax) amax = fabsf(t);
        }
        const float s = amax / 127.0f;
        expanded_scale[i] = s;
        int8_t *q = (int8_t *)expanded_x + (size_t)i * (size_t)h;
        for (int64_t c = 0; c < h; ++c) {
            const float f = f16_to_f32(f32_to_f16_rz(v[c] / s));
            if (!(f == f)) { q[c] = 0; continue; }
            int r = (int)(f + (f < 0.0f ? -0.5f : 0.5f));
            if (r > 127) r = 127;
            if (r < -128) r = -128;
            q[c] = (int8_t)r;
        }
    }
    free(v);
    free(count);
    free(first);
    return total;
}

/* ------------------------------------------------------------------------------------------- */
/* grouped_matmul_swiglu_quant, A8W8                                                            */
/* ------------------------------------------------------------------------------------------- */

/* Per row m of group e (gmm/grouped_matmul_swiglu_quant/op_kernel/grouped_matmul_swiglu_quant.h):
 *   t[n]  = float(acc[n])                     Cast CAST_NONE, :381
 *   t[n] *= x_scale[m]                        Muls, :392        (order: (acc*x_scale)*w_scale)
 *   t[n] *= float(w_scale[e,n])               Mul, :450
 *   S[j]  = Swish(t[j]) * t[N/2+j]            SwiGLU<float,false>(dst, src0 = t[N/2:], src1 = t[:N/2], beta 1), :468;
 *           Swish(a) = a / (1 + exp(-a))      README.md:61-65 of the operator; first half activated
 *   amax  = max_j |S[j]|                      Abs + ReduceMaxTemplate, :481-490
 *   qs    = amax / 127                        :496, stored to y_scale[m]
 *   r     = 1 / qs ;  u[j] = S[j] * r         :499, :503   (multiply by the reciprocal, not a division)
 *   q[j]  = int8_rne(half_rne(u[j]))          CastFp32ToInt8Template, ..._utils.h:308-316
 * group_list is a running total only (:237-241); it may be shorter than E.  Rows at and beyond
 * group_list[-1] are never written (operator README.md:50-57).
 * The multiplication order inside SwiGLU is not visible (closed toolkit); this file fixes
 * S = gate * (act / (1 + expf(-act))).
 * A row whose amax is 0 gives qs = 0, r = inf, u = NaN in the reference; NaN is mapped to q = 0 here. */
ORACLE_API int oracle_swiglu_quant(const int8_t *x, const int8_t *w, const void *w_scale, int w_scale_dtype,
                                   const float *x_scale, const int64_t *group_list, int64_t gl_len, int64_t M,
                                   int64_t K, int64_t N, int64_t E, int w_trans, int8_t *q, float *q_scale,
                                   int32_t *acc_out, float *s_out)
{
    if (gl_len > E || (N & 1)) return -1;
    const int64_t H = N / 2;
    int64_t *rs = (int64_t *)malloc(sizeof(int64_t) * (size_t)(2 * gl_len + 2));
    int64_t *rc = rs + gl_len + 1;
    oracle_group_layout(group_list, gl_len, 0, M, rs, rc);
    int64_t maxrows = 0;
    for (int64_t g = 0; g < gl_len; ++g) if (rc[g] > maxrows) maxrows = rc[g];
    int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)(maxrows > 0 ? maxrows : 1) * (size_t)N);
    for (int64_t g = 0; g < gl_len; ++g) {
        const int64_t r0 = rs[g], rows = rc[g];
        if (rows <= 0) continue;
        gemm_group(x + r0 * K, rows, K, N, w + g * K * N, w_trans ? 1 : N, w_trans ? K : 1, acc);
#pragma omp parallel
        {
            float *S = (float *)malloc(sizeof(float) * (size_t)H);
#pragma omp for schedule(static)
            for (int64_t r = 0; r < rows; ++r) {
                const int64_t m = r0 + r;
                const float xs = x_scale[m];
                float amax = 0.0f;
                for (int64_t j = 0; j < H; ++j) {
                    float a = (float)acc[r * N + j];
                    float b = (float)acc[r * N + H + j];
                    a = a * xs; b = b * xs;
                    a = a * load_scale(w_scale, w_scale_dtype, g * N + j);
                    b = b * load_scale(w_scale, w_scale_dtype, g * N + H + j);
                    float den = 1.0f + expf(-a);
                    float sw = a / den;
                    float s = b * sw;
                    S[j] = s;
                    float ab = fabsf(s);
                    if (ab > amax) amax = ab;
                }
                if (acc_out) memcpy(acc_out + m * N, acc + r * N, sizeof(int32_t) * (size_t)N);
                if (s_out) memcpy(s_out + m * H, S, sizeof(float) * (size_t)H);
                const float qs = amax / 127.0f;
                q_scale[m] = qs;
                const float rcp = 1.0f / qs;
                for (int64_t j = 0; j < H; ++j) {
                    float u = S[j] * rcp;
                    q[m * H + j] = f16_to_i8_rne(f32_to_f16_rne(u));
                }
            }
            free(S);
        }
    }
    free(acc);
    free(rs);
    return 0;
}

/* ------------------------------------------------------------------------------------------- */
/* Host-side formulas the reference's own unit tests pin                                         */
/* ------------------------------------------------------------------------------------------- */

/* gmm/grouped_matmul_swiglu_quant/op_host/grouped_matmul_swiglu_quant_tiling.cpp:205-232 with the constants
 * of grouped_matmul_swiglu_quant_tiling.h:70-72: mLimit = (64 MiB / 2 / 4) / n; the int32 staging holds
 * min(m, 2*mLimit) rows; 16 MiB are reserved for the system.  Known answers: (m 16, n 512) -> 16809984,
 * (m 16, n 4096) -> 17039360 (tests/ut/op_host/test_grouped_matmul_swiglu_quant_tiling.cpp:70, :99). */
ORACLE_API int64_t oracle_ref_swiglu_workspace_bytes(int64_t m, int64_t n)
{
    const int64_t sys = 16ll * 1024 * 1024, user = 64ll * 1024 * 1024;
    int64_t m_limit = (user / 2 / 4) / n;
    int64_t rows = (m_limit * 2 > m) ? m : m_limit * 2;
    return sys + rows * n * 4;
}

/* Same file :232, :106-118: tiling key 1 (split workspace) iff m > 2*mLimit, else 0. */
ORACLE_API int oracle_ref_swiglu_tiling_key(int64_t m, int64_t n)
{
    const int64_t user = 64ll * 1024 * 1024;
    int64_t m_limit = (user / 2 / 4) / n;
    return m > 2 * m_limit ? 1 : 0;
}

/* Conversions exported so the tests can exercise the rounding rules directly. */
ORACLE_API uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }
ORACLE_API uint16_t oracle_f32_to_f16(float f) { return f32_to_f16_rne(f); }
ORACLE_API int8_t oracle_f16_to_i8(uint16_t h) { return f16_to_i8_rne(h); }
/* A launcher may have exported OMP_NUM_THREADS=1 to every worker (torch.distributed.run does); the timed CPU legs ask
 * for the host's cores explicitly. */
ORACLE_API void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORACLE_API int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
