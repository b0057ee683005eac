// Quantized conv net through the C++ host side, shaped like the network of l-ten's quantized convolution test
// (tests/nn_tests.cpp:620-640): Conv2d_q(1 -> 10, 5 x 5) on 28 x 28 images, reshape to {B, 1, 1, 5760},
// FullyConnected_q(5760 -> 50), FullyConnected_q(50 -> 10), no biases on the convolution.  Activation ranges are calibrated
// from an fp32 run, weights quantized by min/max, every layer output compared byte for byte with the CPU oracle
// (oracle/ltq_oracle.c, test infrastructure), and Conv2d_q's argument checks exercised with the reference's messages.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "lten_q.h"

extern "C" {
struct oracle_qparams { float scale; uint8_t zero_point; };
int oracle_quantized_matmul(int tA, int tB, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha, const uint8_t *A,
                            const uint8_t *B, uint8_t beta, uint8_t *C, const oracle_qparams *qp, const int32_t *bias,
                            int32_t *workspace);
int oracle_conv2d_q(const uint8_t *x, uint64_t batches, uint64_t cin, uint64_t height, uint64_t width, const uint8_t *w,
                    const int32_t *bias, int bias_per_channel, uint64_t cout, uint64_t kernel_h, uint64_t kernel_w,
                    uint64_t pad_h, uint64_t pad_w, uint64_t stride_h, uint64_t stride_w, const oracle_qparams *qp_in,
                    const oracle_qparams *qp_wt, const oracle_qparams *qp_out, uint8_t *out);
void oracle_quantize_u8(const float *x, uint8_t *q, uint64_t len, const oracle_qparams *qp);
}

using namespace lten;

static uint64_t rng_state = 0x2545F4914F6CDD1Dull;
static float uniform01()
{
    rng_state = rng_state * 6364136223846793005ull + 1442695040888963407ull;
    return (float)((rng_state >> 40) & 0xFFFFFF) / 16777216.0f;
}
static float normal(float sigma)
{
    float u1 = uniform01() + 1e-7f, u2 = uniform01();
    return sigma * sqrtf(-2.f * logf(u1)) * cosf(6.2831853f * u2);
}

static int failures = 0;
#define CHECK(cond, what)                                   \
    do {                                                    \
        if (!(cond)) {                                      \
            printf("FAIL: %s (line %d)\n", what, __LINE__); \
            failures++;                                     \
        }                                                   \
    } while (0)

template <typename T>
static Tensor upload(const std::vector<T> &v, std::initializer_list<uint64_t> dims, dtype dt)
{
    TensorOps o;
    o.data_type = dt;
    Tensor host = TensorFromBuffer(dims, (void *)v.data(), false, &o);
    return host.to(GPU, 0);
}

template <typename T>
static std::vector<T> download(const Tensor &t)
{
    Tensor h = t.to(CPU);
    std::vector<T> v(h.get_numels());
    memcpy(v.data(), h.get_data_ptr(), v.size() * sizeof(T));
    return v;
}

static bool throws_with(const char *needle, void (*fn)())
{
    try {
        fn();
    } catch (const ExceptionInfo &e) {
        return strstr(e.get_message(), needle) != nullptr;
    }
    return false;
}

// min/max -> qparams on the device, then quantize on the device; returns the bytes
static std::vector<uint8_t> quantize_by_range(const std::vector<float> &v, QuantizationParams *qp)
{
    Tensor f = upload(v, {(uint64_t)v.size()}, FLOAT32);
    float mn, mx;
    GetMinMax((float *)f.get_data_ptr(), f.get_numels(), &mn, &mx);
    ComputeQuantizationParams(mn, mx, qp);
    TensorOps o;
    o.data_type = UINT8;
    o.device_type = GPU;
    Tensor q = AllocateTensor({(uint64_t)v.size()}, &o);
    Quantize((float *)f.get_data_ptr(), (uint8_t *)q.get_data_ptr(), f.get_numels(), qp);
    return download<uint8_t>(q);
}

static QuantizationParams range_of(const std::vector<float> &v)
{
    Tensor f = upload(v, {(uint64_t)v.size()}, FLOAT32);
    float mn, mx;
    QuantizationParams qp;
    GetMinMax((float *)f.get_data_ptr(), f.get_numels(), &mn, &mx);
    ComputeQuantizationParams(mn, mx, &qp);
    return qp;
}

static Conv2d_q *g_conv = nullptr;

int main()
{
    const int B = 32, IMG = 28, CO = 10, KH = 5, OUTD = 24, FLAT = CO * OUTD * OUTD, H1 = 50, H2 = 10;
    // ---- synthetic fp32 network and images in [0, 1] ----
    std::vector<float> x((size_t)B * IMG * IMG), wc((size_t)CO * KH * KH), w1((size_t)H1 * FLAT), w2((size_t)H2 * H1);
    for (auto &v : x) v = uniform01();
    for (auto &v : wc) v = normal(0.2f);
    for (auto &v : w1) v = normal(0.02f);
    for (auto &v : w2) v = normal(0.1f);
    // ---- fp32 forward for the activation ranges ----
    std::vector<float> a1((size_t)B * FLAT), a2((size_t)B * H1), a3((size_t)B * H2);
    for (int b = 0; b < B; b++)
        for (int c = 0; c < CO; c++)
            for (int i = 0; i < OUTD; i++)
                for (int j = 0; j < OUTD; j++) {
                    float s = 0;
                    for (int u = 0; u < KH; u++)
                        for (int v = 0; v < KH; v++) s += x[((size_t)b * IMG + i + u) * IMG + j + v] * wc[(c * KH + u) * KH + v];
                    a1[(((size_t)b * CO + c) * OUTD + i) * OUTD + j] = s;
                }
    for (int b = 0; b < B; b++)
        for (int j = 0; j < H1; j++) {
            float s = 0;
            for (int k = 0; k < FLAT; k++) s += a1[(size_t)b * FLAT + k] * w1[(size_t)j * FLAT + k];
            a2[(size_t)b * H1 + j] = s;
        }
    for (int b = 0; b < B; b++)
        for (int j = 0; j < H2; j++) {
            float s = 0;
            for (int k = 0; k < H1; k++) s += a2[(size_t)b * H1 + k] * w2[(size_t)j * H1 + k];
            a3[(size_t)b * H2 + j] = s;
        }
    QuantizationParams qp_x = range_of(x), qp_a1 = range_of(a1), qp_a2 = range_of(a2), qp_a3 = range_of(a3);

    // ---- quantized network ----
    QuantizationParams qp_wc, qp_w1, qp_w2;
    std::vector<uint8_t> wcq = quantize_by_range(wc, &qp_wc), w1q = quantize_by_range(w1, &qp_w1),
                         w2q = quantize_by_range(w2, &qp_w2);
    Conv2d_q proto(1, CO, false, KH, KH);
    Conv2d_q *conv1 = new Conv2d_q(proto);  // register_module copy-constructs, then init()s
    conv1->init();
    CHECK(conv1->get_all_weights().size() == 1 && conv1->get_weights()->get_numels() == (uint64_t)CO * KH * KH, "conv weights shape");
    memcpy(conv1->get_all_weights()[0]->get_data_ptr(), wcq.data(), wcq.size());
    conv1->set_qparams_in(qp_x);
    conv1->set_qparams_out(qp_a1);
    conv1->set_qparams_params(&qp_wc, 1);
    conv1->to(GPU, 0);
    FullyConnected_q *fc1 = new FullyConnected_q(FLAT, H1), *fc2 = new FullyConnected_q(H1, H2);
    fc1->init();
    fc2->init();
    memcpy(fc1->get_all_weights()[0]->get_data_ptr(), w1q.data(), w1q.size());
    memcpy(fc2->get_all_weights()[0]->get_data_ptr(), w2q.data(), w2q.size());
    fc1->set_qparams_in(qp_a1);
    fc1->set_qparams_out(qp_a2);
    fc1->set_qparams_params(&qp_w1, 1);
    fc2->set_qparams_in(qp_a2);
    fc2->set_qparams_out(qp_a3);
    fc2->set_qparams_params(&qp_w2, 1);
    fc1->to(GPU, 0);
    fc2->to(GPU, 0);

    // ---- inference: QNet::forward, tests/nn_tests.cpp:630-640 ----
    Tensor input = upload(x, {(uint64_t)B, 1, (uint64_t)IMG, (uint64_t)IMG}, FLOAT32);
    TensorOps o;
    o.data_type = UINT8;
    o.device_type = GPU;
    Tensor q_input = AllocateTensor({(uint64_t)B, 1, (uint64_t)IMG, (uint64_t)IMG}, &o);
    Quantize((float *)input.get_data_ptr(), (uint8_t *)q_input.get_data_ptr(), q_input.get_numels(), &qp_x);
    std::vector<uint8_t> xq = download<uint8_t>(q_input);

    Tensor y1 = conv1->forward(q_input);
    CHECK(y1.get_ndims() == 4 && y1.get_sizes()[0] == (uint64_t)B && y1.get_sizes()[1] == (uint64_t)CO &&
              y1.get_sizes()[2] == (uint64_t)OUTD && y1.get_sizes()[3] == (uint64_t)OUTD, "conv output shape");
    std::vector<uint8_t> got1 = download<uint8_t>(y1), want1(got1.size());
    oracle_qparams oq_x{qp_x.scale, qp_x.zero_point}, oq_wc{qp_wc.scale, qp_wc.zero_point}, oq_a1{qp_a1.scale, qp_a1.zero_point};
    oracle_conv2d_q(xq.data(), B, 1, IMG, IMG, wcq.data(), nullptr, 0, CO, KH, KH, 0, 0, 1, 1, &oq_x, &oq_wc, &oq_a1, want1.data());
    CHECK(got1 == want1, "Conv2d_q output vs oracle");

    y1 = y1.reshape({(uint64_t)B, 1, 1, (uint64_t)FLAT});  // as QNet::forward does: the view must keep the bytes alive
    Tensor y2 = fc1->forward(y1);
    CHECK(y2.row_sums() != nullptr && y2.row_sums()->get_numels() == (uint64_t)B, "fc1 leaves row sums for fc2");
    std::vector<uint8_t> got2 = download<uint8_t>(y2), want2((size_t)B * H1);
    {
        std::vector<int32_t> ws(B + H1);
        oracle_qparams q3[3] = {oq_a1, {qp_w1.scale, qp_w1.zero_point}, {qp_a2.scale, qp_a2.zero_point}};
        oracle_quantized_matmul(0, 1, B, H1, FLAT, 1, got1.data(), w1q.data(), 0, want2.data(), q3, nullptr, ws.data());
    }
    CHECK(got2 == want2, "fc1 output vs oracle");
    Tensor y3 = fc2->forward(y2);
    std::vector<uint8_t> got3 = download<uint8_t>(y3), want3((size_t)B * H2);
    {
        std::vector<int32_t> ws(B + H2);
        oracle_qparams q3[3] = {{qp_a2.scale, qp_a2.zero_point}, {qp_w2.scale, qp_w2.zero_point}, {qp_a3.scale, qp_a3.zero_point}};
        oracle_quantized_matmul(0, 1, B, H2, H1, 1, got2.data(), w2q.data(), 0, want3.data(), q3, nullptr, ws.data());
    }
    CHECK(got3 == want3, "fc2 output vs oracle");
    {
        TensorOps of;
        of.device_type = GPU;
        Tensor out = AllocateTensor({(uint64_t)B, 1, 1, (uint64_t)H2}, &of);
        Dequantize((float *)out.get_data_ptr(), (uint8_t *)y3.get_data_ptr(), y3.get_numels(), &qp_a3);
        std::vector<float> got = download<float>(out);
        double err = 0, ref = 0;
        for (size_t i = 0; i < got.size(); i++) {
            err += fabs(got[i] - a3[i]);
            ref += fabs(a3[i]);
        }
        CHECK(err / ref < 0.15, "uint8 logits close to fp32 logits");
        printf("mean |uint8 - fp32| / mean |fp32| on the logits: %.4f\n", err / ref);
    }

    // ---- argument checks, reference messages (conv2d.cpp:285-301) ----
    g_conv = conv1;
    CHECK(throws_with("only supported for UINT8", [] {
              TensorOps o; o.data_type = FLOAT32; o.device_type = GPU;
              Tensor t = AllocateTensor({1, 1, 28, 28}, &o);
              g_conv->forward(t);
          }), "float input rejected");
    CHECK(throws_with("not the same as this layer's parameters", [] {
              TensorOps o; o.data_type = UINT8;
              Tensor t = AllocateTensor({1, 1, 28, 28}, &o);  // CPU tensor, GPU layer
              g_conv->forward(t);
          }), "device mismatch rejected");
    CHECK(throws_with("exactly 4 dimensions", [] {
              TensorOps o; o.data_type = UINT8; o.device_type = GPU;
              Tensor t = AllocateTensor({1, 28, 28}, &o);
              g_conv->forward(t);
          }), "ndims != 4 rejected");
    CHECK(throws_with("smaller than the kernel", [] {
              TensorOps o; o.data_type = UINT8; o.device_type = GPU;
              Tensor t = AllocateTensor({1, 1, 3, 28}, &o);
              g_conv->forward(t);
          }), "image smaller than the kernel rejected");

    // ---- a 64 -> 32 channel 3 x 3 layer (computed without a patch buffer): NCHW against the oracle, then the same layer
    //      with channels-last input and output, which must hold the same values in the other order ----
    {
        const int B2 = 2, C2 = 64, H2 = 9, W2 = 12, O2 = 32;
        std::vector<uint8_t> x2((size_t)B2 * C2 * H2 * W2), w2((size_t)O2 * C2 * 9);
        uint32_t seed = 12345;
        for (auto &v : x2) { seed = seed * 1664525u + 1013904223u; v = (uint8_t)(seed >> 24); }
        for (auto &v : w2) { seed = seed * 1664525u + 1013904223u; v = (uint8_t)(seed >> 24); }
        Conv2d_q big(C2, O2, false, 3, 3, 1, 1);
        big.init();
        memcpy(big.get_weights()->get_data_ptr(), w2.data(), w2.size());
        QuantizationParams qi{0.02f, 128}, qw{0.005f, 127}, qo{4.0f, 3};
        big.set_qparams_in(qi);
        big.set_qparams_out(qo);
        big.set_qparams_params(&qw, 1);
        big.to(GPU, 0);
        Tensor xin = upload(x2, {(uint64_t)B2, (uint64_t)C2, (uint64_t)H2, (uint64_t)W2}, UINT8);
        Tensor y = big.forward(xin);
        std::vector<uint8_t> got = download<uint8_t>(y), want(got.size());
        oracle_qparams oi{qi.scale, qi.zero_point}, ow{qw.scale, qw.zero_point}, oo{qo.scale, qo.zero_point};
        CHECK(oracle_conv2d_q(x2.data(), B2, C2, H2, W2, w2.data(), nullptr, 0, O2, 3, 3, 1, 1, 1, 1, &oi, &ow, &oo, want.data()) == 0,
              "oracle conv");
        CHECK(got == want, "64-channel Conv2d_q (no patch buffer) vs oracle");
        std::vector<uint8_t> x_cl(x2.size());
        for (int b = 0; b < B2; b++)
            for (int c = 0; c < C2; c++)
                for (int i = 0; i < H2 * W2; i++) x_cl[((size_t)b * H2 * W2 + i) * C2 + c] = x2[((size_t)b * C2 + c) * H2 * W2 + i];
        big.set_layout(true, true);
        Tensor xcl = upload(x_cl, {(uint64_t)B2, (uint64_t)H2, (uint64_t)W2, (uint64_t)C2}, UINT8);
        Tensor ycl = big.forward(xcl);
        CHECK(ycl.get_sizes()[1] == (uint64_t)H2 && ycl.get_sizes()[3] == (uint64_t)O2, "channels-last output shape");
        std::vector<uint8_t> gcl = download<uint8_t>(ycl);
        bool same = gcl.size() == want.size();
        for (int b = 0; same && b < B2; b++)
            for (int o = 0; same && o < O2; o++)
                for (int i = 0; i < H2 * W2; i++)
                    if (gcl[((size_t)b * H2 * W2 + i) * O2 + o] != want[((size_t)b * O2 + o) * H2 * W2 + i]) { same = false; break; }
        CHECK(same, "channels-last in / out holds the NCHW result's values");
    }

    delete conv1;
    delete fc1;
    delete fc2;
    if (failures) {
        printf("%d check(s) FAILED\n", failures);
        return 1;
    }
    printf("PASS\n");
    return 0;
}
