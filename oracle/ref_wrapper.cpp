// extern "C" doorway into the UNMODIFIED l-ten reference, compiled from its own
// sources where they lie (see oracle/Makefile, target `ref`).  TEST
// INFRASTRUCTURE ONLY: it validates oracle/ltq_oracle.c, generates the fixtures
// under tests/golden and serves as the timed CPU baseline.  Nothing shipped
// links against it.  This file contains no reference code, only calls into it.
#include <cstdint>
#include <cstring>
#include <chrono>
#include "lten.h"   // l-ten/lten.h (reference public umbrella header)
#include "utils.h"  // l-ten/utils.h:23-27
#include "im_col.h" // l-ten/im_col.h:5-33

extern "C" {

struct ref_qparams { float scale; uint8_t zero_point; };

static QuantizationParams to_qp(const ref_qparams& q)
{
    QuantizationParams r;
    r.scale = q.scale;
    r.zero_point = q.zero_point;
    return r;
}

void ref_get_min_max(float* data, uint64_t len, float* mn, float* mx) { GetMinMax(data, len, mn, mx); }

void ref_compute_qparams(float mn, float mx, ref_qparams* out)
{
    QuantizationParams qp;
    ComputeQuantizationParams(mn, mx, &qp);
    out->scale = qp.scale;
    out->zero_point = qp.zero_point;
}

void ref_quantize_u8(float* x, uint8_t* q, uint64_t len, const ref_qparams* qp)
{
    QuantizationParams p = to_qp(*qp);
    Quantize(x, q, len, &p);
}

void ref_quantize_i32(float* x, int* q, uint64_t len, const ref_qparams* qp)
{
    QuantizationParams p = to_qp(*qp);
    Quantize(x, q, len, &p);
}

void ref_dequantize(float* x, uint8_t* q, uint64_t len, const ref_qparams* qp)
{
    QuantizationParams p = to_qp(*qp);
    Dequantize(x, q, len, &p);
}

// l-ten/math_fns.h:104, argument for argument.  Returns -1 if the reference throws.
int ref_quantized_matmul(int tA, int tB, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha, uint8_t* A, uint8_t* B,
                         uint8_t beta, uint8_t* C, const ref_qparams* qp3, int* bias, int* workspace)
{
    QuantizationParams qp[3] = { to_qp(qp3[0]), to_qp(qp3[1]), to_qp(qp3[2]) };
    try {
        quantized_matmul(tA != 0, tB != 0, M, N, K, alpha, A, B, beta, C, qp, bias, workspace);
    } catch (...) {
        return -1;
    }
    return 0;
}

// Whole layer through the reference's public API (l-ten/layers.h:69-106): build a
// FullyConnected_q(K -> N), write weights/bias through get_all_weights() exactly as
// tests/nn_tests.cpp:818-826 does, run forward on a {1, M, K} uint8 tensor.
// Returns seconds spent inside forward() (steady_clock), or -1 on an exception.
double ref_fc_q_forward(uint64_t M, uint64_t N, uint64_t K, const uint8_t* x, const uint8_t* w, const int* bias,
                        const ref_qparams* qp_in, const ref_qparams* qp_wt, const ref_qparams* qp_out, uint8_t* out,
                        int repeats)
{
    try {
        lten::FullyConnected_q fc((int64_t)K, (int64_t)N, bias != nullptr);
        fc.init();
        fc.train(false);
        auto wts = fc.get_all_weights();
        memcpy(wts[0]->get_data_ptr(), w, N * K);
        if (bias) memcpy(wts[1]->get_data_ptr(), bias, N * sizeof(int));
        QuantizationParams qw = to_qp(*qp_wt);
        fc.set_qparams_in(to_qp(*qp_in));
        fc.set_qparams_out(to_qp(*qp_out));
        fc.set_qparams_params(&qw, 1);

        lten::TensorOps opts;
        opts.data_type = lten::UINT8;
        lten::Tensor input = lten::AllocateTensor({ 1, M, K }, &opts);
        memcpy(input.get_data_ptr(), x, M * K);
        lten::Tensor result;
        double best = 1e300;
        if (repeats < 1) repeats = 1;
        for (int r = 0; r < repeats; r++) {
            auto t0 = std::chrono::steady_clock::now();
            result = fc.forward(input);
            auto t1 = std::chrono::steady_clock::now();
            double s = std::chrono::duration<double>(t1 - t0).count();
            if (s < best) best = s;
        }
        memcpy(out, result.get_data_ptr(), M * N);
        return best;
    } catch (...) {
        return -1.0;
    }
}

// The patch gather on its own, l-ten/im_col.h:5-33.
void ref_im2col(const uint8_t* im, uint64_t channels, uint64_t height, uint64_t width, uint64_t kernel_h, uint64_t kernel_w,
                uint64_t pad_h, uint64_t pad_w, uint64_t stride_h, uint64_t stride_w, uint8_t* col)
{
    im2col_cpu<uint8_t>(im, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, col);
}

// Conv2d_q through the reference's public API (l-ten/layers.h:453-524), set up the way tests/nn_tests.cpp:625 and
// :829-840 do: weights through get_all_weights(), qparams through the three setters, forward on an NCHW uint8 tensor.
// Returns 0, or -1 on an exception.
int ref_conv2d_q_forward(uint64_t batches, uint64_t cin, uint64_t height, uint64_t width, uint64_t cout, int kernel_h,
                         int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w, const uint8_t* x, const uint8_t* w,
                         const int* bias, const ref_qparams* qp_in, const ref_qparams* qp_wt, const ref_qparams* qp_out,
                         uint8_t* out)
{
    try {
        lten::Conv2d_q conv((int)cin, (int)cout, bias != nullptr, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w);
        conv.init();
        conv.train(false);
        auto wts = conv.get_all_weights();
        memcpy(wts[0]->get_data_ptr(), w, cout * cin * kernel_h * kernel_w);
        if (bias) memcpy(wts[1]->get_data_ptr(), bias, cout * sizeof(int));
        QuantizationParams qw = to_qp(*qp_wt);
        conv.set_qparams_in(to_qp(*qp_in));
        conv.set_qparams_out(to_qp(*qp_out));
        conv.set_qparams_params(&qw, 1);
        lten::TensorOps opts;
        opts.data_type = lten::UINT8;
        lten::Tensor input = lten::AllocateTensor({ batches, cin, height, width }, &opts);
        memcpy(input.get_data_ptr(), x, batches * cin * height * width);
        lten::Tensor result = conv.forward(input);
        memcpy(out, result.get_data_ptr(), result.get_numels());
        return 0;
    } catch (...) {
        return -1;
    }
}

} // extern "C"
