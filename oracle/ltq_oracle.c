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
#include <stdlib.h>

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
static int qmm_core(int tA, int tB, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha, const uint8_t *A,
                    const uint8_t *B, uint8_t beta, uint8_t *C, const oracle_qparams *qp, const int32_t *bias,
                    const int32_t *row_bias, int32_t *workspace)
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
            if (row_bias) e += (uint32_t)row_bias[i];
            volatile float m = rm * (float)(int32_t)e;
            float t = m + (float)(int)qp[2].zero_point;
            C[i * N + j] = cast_u8(t, 0);
        }
    }
    return 0;
}

int oracle_quantized_matmul(int tA, int tB, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha,
                            const uint8_t *A, const uint8_t *B, uint8_t beta, uint8_t *C,
                            const oracle_qparams *qp, const int32_t *bias, int32_t *workspace)
{
    return qmm_core(tA, tB, M, N, K, alpha, A, B, beta, C, qp, bias, NULL, workspace);
}

/* Patch gather, l-ten/im_col.h:5-33: col is [C*kh*kw, Ho*Wo]; row c = (channel, kernel row, kernel column), taps outside
 * the image are 0.  The reference computes the tap position in uint64_t, so a "negative" position wraps to a huge
 * value and fails the `< height` test; signed arithmetic with an explicit >= 0 test says the same. */
void oracle_im2col(const uint8_t *im, uint64_t channels, uint64_t height, uint64_t width, uint64_t kernel_h,
                   uint64_t kernel_w, uint64_t pad_h, uint64_t pad_w, uint64_t stride_h, uint64_t stride_w, uint8_t *col)
{
    const uint64_t hc = (height + 2 * pad_h - kernel_h) / stride_h + 1;
    const uint64_t wc = (width + 2 * pad_w - kernel_w) / stride_w + 1;
    const uint64_t rows = channels * kernel_h * kernel_w;
    for (uint64_t c = 0; c < rows; c++) {
        const uint64_t wo = c % kernel_w, ho = (c / kernel_w) % kernel_h, ci = c / kernel_h / kernel_w;
        for (uint64_t h = 0; h < hc; h++)
            for (uint64_t w = 0; w < wc; w++) {
                const int64_t y = (int64_t)(h * stride_h + ho) - (int64_t)pad_h;
                const int64_t x = (int64_t)(w * stride_w + wo) - (int64_t)pad_w;
                uint8_t v = 0;
                if (y >= 0 && y < (int64_t)height && x >= 0 && x < (int64_t)width) v = im[(ci * height + y) * width + x];
                col[(c * hc + h) * wc + w] = v;
            }
    }
}

/* Conv2d_q::forward, l-ten/conv2d.cpp:266-379: per image, im2col then quantized_matmul(false, false, M = Cout,
 * N = Ho*Wo, K = Cin*kh*kw, weights, col) with qparams {weights, input, output} (:348-350).  `bias` is handed to
 * quantized_matmul as the reference does (added per output POSITION j, so only defined while Ho*Wo <= Cout);
 * bias_per_channel != 0 adds bias[channel] instead, which is what the shipped library offers as an option and has no
 * counterpart in the reference.  Returns -1 if memory runs out. */
int oracle_conv2d_q(const uint8_t *x, uint64_t batches, uint64_t cin, uint64_t height, uint64_t width, const uint8_t *w,
                    const int32_t *bias, int bias_per_channel, uint64_t cout, uint64_t kernel_h, uint64_t kernel_w,
                    uint64_t pad_h, uint64_t pad_w, uint64_t stride_h, uint64_t stride_w, const oracle_qparams *qp_in,
                    const oracle_qparams *qp_wt, const oracle_qparams *qp_out, uint8_t *out)
{
    const uint64_t ho = (height + 2 * pad_h - kernel_h) / stride_h + 1;
    const uint64_t wo = (width + 2 * pad_w - kernel_w) / stride_w + 1;
    const uint64_t M = cout, N = ho * wo, K = cin * kernel_h * kernel_w;
    uint8_t *col = (uint8_t *)malloc(K * N ? K * N : 1);
    int32_t *ws = (int32_t *)malloc((M + N) * sizeof(int32_t));
    if (!col || !ws) {
        free(col);
        free(ws);
        return -1;
    }
    const oracle_qparams qp[3] = {*qp_wt, *qp_in, *qp_out};
    for (uint64_t b = 0; b < batches; b++) {
        oracle_im2col(x + b * cin * height * width, cin, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
                      stride_w, col);
        qmm_core(0, 0, M, N, K, 1, w, col, 0, out + b * M * N, qp, bias_per_channel ? NULL : bias,
                 bias_per_channel ? bias : NULL, ws);
    }
    free(col);
    free(ws);
    return 0;
}
