/*
 * CPU oracle for the uint8 quantized fully-connected path of l-ten.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; it exists so the CUDA path can be checked against a plain
 * restatement of the reference arithmetic.  Parity of this restatement is
 * pinned two ways: against the reference's own object code built from its
 * sources (oracle/_ref, see oracle/Makefile) and against the fixtures under
 * tests/golden that were generated from that build.
 *
 * Every function cites the reference lines it restates (paths are relative to
 * the l-ten project root).
 */
#include <stdint.h>
#include <stddef.h>
#include <math.h>
#include <limits.h>

typedef struct {
    float scale;
    uint8_t zero_point;
} oracle_qparams; /* l-ten/math_fns.h:12-16 */

/* l-ten/utils.cpp:198-226 — min and max, both seeded from element 0. */
void oracle_get_min_max(const float *data, uint64_t len, float *mn, float *mx)
{
    float lo = data[0], hi = data[0];
    for (uint64_t i = 0; i < len; i++) {
        if (data[i] > hi) hi = data[i];
        if (data[i] < lo) lo = data[i];
    }
    *mn = lo;
    *mx = hi;
}

/* l-ten/utils.cpp:266-286 — range widened to hold 0, scale = range/255,
 * zero point = round-half-away(0 - min/scale) cast to uint8. */
void oracle_compute_qparams(float mn, float mx, oracle_qparams *qp)
{
    float zp;
    mn = mn < 0.f ? mn : 0.f;
    mx = mx > 0.f ? mx : 0.f;
    qp->scale = (mx - mn) / (255.f - 0.f);
    zp = 0.f - mn / qp->scale;
    qp->zero_point = (uint8_t)roundf(zp);
}

/* l-ten/utils.cpp:243-254 — zp + x/scale in float, clamp to [0,255], round
 * half away from zero. */
void oracle_quantize_u8(const float *x, uint8_t *q, uint64_t len, const oracle_qparams *qp)
{
    for (uint64_t i = 0; i < len; i++) {
        float v = (float)(int)qp->zero_point + x[i] / qp->scale;
        v = fmaxf(0.f, fminf(255.f, v));
        q[i] = (uint8_t)round((double)v);
    }
}

/* l-ten/utils.cpp:228-241 — same with the int32 clamp (used for the bias with
 * scale s_in*s_wt and zero point 0, tests/nn_tests.cpp:824-826). */
void oracle_quantize_i32(const float *x, int32_t *q, uint64_t len, const oracle_qparams *qp)
{
    const float lowest = (float)INT_MIN, highest = (float)INT_MAX;
    for (uint64_t i = 0; i < len; i++) {
        float v = (float)(int)qp->zero_point + x[i] / qp->scale;
        /* std::max(lowest, std::min(highest, v)) */
        float t = (v < highest) ? v : highest;
        t = (lowest < t) ? t : lowest;
        /* (int)round(2^31) is out of range; x86 cvttsd2si gives INT_MIN. */
        double r = round((double)t);
        q[i] = (r >= 2147483648.0) ? INT_MIN : (int32_t)r;
    }
}

/* l-ten/utils.cpp:256-264 */
void oracle_dequantize(float *x, const uint8_t *q, uint64_t len, const oracle_qparams *qp)
{
    for (uint64_t i = 0; i < len; i++)
        x[i] = qp->scale * (float)((int)q[i] - (int)qp->zero_point);
}

/* Element fetch for the four transpose variants of
 * l-ten/math_fns.cpp:1442-1467. */
static inline int a_at(const uint8_t *A, int tA, uint64_t M, uint64_t K, uint64_t i, uint64_t k)
{
    return tA ? A[k * M + i] : A[i * K + k];
}
static inline int b_at(const uint8_t *B, int tB, uint64_t N, uint64_t K, uint64_t j, uint64_t k)
{
    return tB ? B[j * K + k] : B[j + N * k];
}

/* Operand sums, l-ten/math_fns.cpp:1336-1429: bsum[j] = sum_k B(j,k),
 * asum[i] = sum_k A(i,k) (the reference multiplies them by -z straight away;
 * here the raw sums are kept and the factor is applied in oracle_acc). */
void oracle_operand_sums(int tA, int tB, uint64_t M, uint64_t N, uint64_t K,
                         const uint8_t *A, const uint8_t *B, int32_t *bsum, int32_t *asum)
{
    for (uint64_t j = 0; j < N; j++) {
        int32_t s = 0;
        for (uint64_t k = 0; k < K; k++) s += b_at(B, tB, N, K, j, k);
        bsum[j] = s;
    }
    for (uint64_t i = 0; i < M; i++) {
        int32_t s = 0;
        for (uint64_t k = 0; k < K; k++) s += a_at(A, tA, M, K, i, k);
        asum[i] = s;
    }
}

/* The int32 value the reference holds in `element` just before scaling,
 * l-ten/math_fns.cpp:1433-1473:
 *   sum_k A*B  - zA*bsum[j] - zB*asum[i] + K*zA*zB (+ bias[j]).
 * Unsigned arithmetic gives the same two's-complement wrap as the x86 build.
 * Rows are independent, so the loop is split across OpenMP threads when the
 * file is built with -fopenmp; integer results do not depend on that. */
void oracle_acc_i32(int tA, int tB, uint64_t M, uint64_t N, uint64_t K,
                    const uint8_t *A, const uint8_t *B, int zA, int zB,
                    const int32_t *bias, int32_t *acc)
{
    const uint32_t bc = (uint32_t)((uint64_t)K * (uint64_t)zA * (uint64_t)zB);
    if (!tA && tB) {
        /* FullyConnected_q's case (l-ten/fully_connected.cpp:389-393): both
         * operands walk K contiguously, so the inner loop vectorises. */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < (int64_t)M; i++) {
            const uint8_t *a = A + (uint64_t)i * K;
            uint32_t as = 0;
            for (uint64_t k = 0; k < K; k++) as += a[k];
            for (uint64_t j = 0; j < N; j++) {
                const uint8_t *b = B + j * K;
                uint32_t dot = 0, bs = 0;
                for (uint64_t k = 0; k < K; k++) {
                    dot += (uint32_t)a[k] * (uint32_t)b[k];
                    bs += b[k];
                }
                uint32_t e = dot + (uint32_t)(-zA) * bs + (uint32_t)(-zB) * as + bc;
                if (bias) e += (uint32_t)bias[j];
                acc[(uint64_t)i * N + j] = (int32_t)e;
            }
        }
        return;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)M; i++) {
        uint32_t as = 0;
        for (uint64_t k = 0; k < K; k++) as += (uint32_t)a_at(A, tA, M, K, (uint64_t)i, k);
        for (uint64_t j = 0; j < N; j++) {
            uint32_t dot = 0, bs = 0;
            for (uint64_t k = 0; k < K; k++) {
                uint32_t bv = (uint32_t)b_at(B, tB, N, K, j, k);
                dot += (uint32_t)a_at(A, tA, M, K, (uint64_t)i, k) * bv;
                bs += bv;
            }
            uint32_t e = dot + (uint32_t)(-zA) * bs + (uint32_t)(-zB) * as + bc;
            if (bias) e += (uint32_t)bias[j];
            acc[(uint64_t)i * N + j] = (int32_t)e;
        }
    }
}

/* l-ten/math_fns.cpp:1436 — float, left to right. */
float oracle_real_multiplier(float sA, float sB, float sC)
{
    volatile float p = sA * sB;
    return p / sC;
}

/* The reference's cast `(unsigned char)float` (l-ten/math_fns.cpp:1474):
 * truncation toward zero; outside [0,256) the C++ is undefined and the x86-64
 * build converts to int32 (cvttss2si) and keeps the low byte.  `saturate`
 * selects the clamped alternative instead. */
static inline uint8_t cast_u8(float t, int saturate)
{
    if (saturate) {
        if (!(t > 0.f)) return 0; /* also NaN */
        if (t >= 255.f) return 255;
        return (uint8_t)(int)t;
    }
    if (!(t > -2147483648.f && t < 2147483648.f)) return 0; /* cvttss2si -> 0x80000000 */
    return (uint8_t)((int32_t)t & 0xFF);
}

/* Epilogues applied to acc (int32 [M*N]).
 *   u8 : l-ten/math_fns.cpp:1436,1474   C = (uchar)(rm*acc + zC), no FMA
 *   f32: (sA*sB) * (float)acc — the numerator of real_multiplier applied the
 *        way Dequantize applies a scale (l-ten/utils.cpp:262)
 *   relu: acc = max(acc,0) first (no counterpart in the reference, whose relu
 *        is float-only, l-ten/layers.cpp:9-67). */
void oracle_epilogue_u8(const int32_t *acc, uint64_t len, float sA, float sB, float sC, int zC,
                        int relu, int saturate, uint8_t *out)
{
    const float rm = oracle_real_multiplier(sA, sB, sC);
    for (uint64_t i = 0; i < len; i++) {
        int32_t e = acc[i];
        if (relu && e < 0) e = 0;
        volatile float m = rm * (float)e;
        float t = m + (float)zC;
        out[i] = cast_u8(t, saturate);
    }
}

void oracle_epilogue_f32(const int32_t *acc, uint64_t len, float sA, float sB, int relu, float *out)
{
    volatile float p = sA * sB;
    const float s = p;
    for (uint64_t i = 0; i < len; i++) {
        int32_t e = acc[i];
        if (relu && e < 0) e = 0;
        out[i] = s * (float)e;
    }
}

/* Whole quantized_matmul, l-ten/math_fns.cpp:1311-1478, same argument order;
 * workspace receives the reference's pre-multiplied vectors
 * [ -zA*bsum (N) | -zB*asum (M) ] (l-ten/math_fns.cpp:1325-1326).
 * Returns -1 for alpha != 1 or beta != 0 (reference: LTEN_ERR, :1331-1334). */
int oracle_quantized_matmul(int tA, int tB, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha,
                            const uint8_t *A, const uint8_t *B, uint8_t beta, uint8_t *C,
                            const oracle_qparams *qp, const int32_t *bias, int32_t *workspace)
{
    if (alpha != 1 || beta != 0) return -1;
    int32_t *row = workspace, *col = workspace + N;
    oracle_operand_sums(tA, tB, M, N, K, A, B, row, col);
    for (uint64_t j = 0; j < N; j++) row[j] = (int32_t)((uint32_t)row[j] * (uint32_t)(-(int)qp[0].zero_point));
    for (uint64_t i = 0; i < M; i++) col[i] = (int32_t)((uint32_t)col[i] * (uint32_t)(-(int)qp[1].zero_point));
    const uint32_t bc = (uint32_t)((uint64_t)K * qp[0].zero_point * qp[1].zero_point);
    const float rm = oracle_real_multiplier(qp[0].scale, qp[1].scale, qp[2].scale);
    for (uint64_t i = 0; i < M; i++) {
        for (uint64_t j = 0; j < N; j++) {
            uint32_t e = 0;
            for (uint64_t k = 0; k < K; k++)
                e += (uint32_t)(a_at(A, tA, M, K, i, k) * b_at(B, tB, N, K, j, k));
            e += (uint32_t)row[j] + (uint32_t)col[i] + bc;
            if (bias) e += (uint32_t)bias[j];
            volatile float m = rm * (float)(int32_t)e;
            float t = m + (float)(int)qp[2].zero_point;
            C[i * N + j] = cast_u8(t, 0);
        }
    }
    return 0;
}
