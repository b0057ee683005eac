// Quantized MLP through the C++ host side, written the way l-ten's own quantized test drives its network
// (tests/nn_tests.cpp:786-963): calibrate activation ranges from an fp32 run, quantize weights by min/max and biases to
// int32 with scale s_in * s_wt through get_all_weights(), move the layers to the GPU, Quantize the input, chain
// FullyConnected_q::forward, Dequantize.  Every layer output is compared byte for byte with the CPU oracle
// (oracle/ltq_oracle.c, test infrastructure), and the layer's argument checks are exercised with the reference's messages.
#include <cuda_runtime.h>
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
void oracle_quantize_u8(const float *x, uint8_t *q, uint64_t len, const oracle_qparams *qp);
void oracle_quantize_i32(const float *x, int32_t *q, uint64_t len, const oracle_qparams *qp);
void oracle_dequantize(float *x, const uint8_t *q, uint64_t len, const oracle_qparams *qp);
void oracle_get_min_max(const float *data, uint64_t len, float *mn, float *mx);
void oracle_compute_qparams(float mn, float mx, oracle_qparams *qp);
}

using namespace lten;

static uint64_t rng_state = 0x9E3779B97F4A7C15ull;
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

int main()
{
    const int B = 64, dims[4] = {784, 512, 512, 10};
    // ---- synthetic "trained" fp32 network and input ----
    std::vector<float> x((size_t)B * dims[0]);
    for (auto &v : x) v = uniform01();
    std::vector<std::vector<float>> W(3), bias(3);
    for (int l = 0; l < 3; l++) {
        W[l].resize((size_t)dims[l + 1] * dims[l]);
        bias[l].resize(dims[l + 1]);
        for (auto &v : W[l]) v = normal(0.05f);
        for (auto &v : bias[l]) v = normal(0.01f);
    }
    // ---- calibration: running min/max of the input and of every layer output in fp32 (nn_tests.cpp:562-608) ----
    std::vector<std::vector<float>> act(4);
    act[0] = x;
    for (int l = 0; l < 3; l++) {
        act[l + 1].assign((size_t)B * dims[l + 1], 0.f);
        for (int i = 0; i < B; i++)
            for (int j = 0; j < dims[l + 1]; j++) {
                float s = bias[l][j];
                for (int k = 0; k < dims[l]; k++) s += act[l][(size_t)i * dims[l] + k] * W[l][(size_t)j * dims[l] + k];
                act[l + 1][(size_t)i * dims[l + 1] + j] = s;
            }
    }
    QuantizationParams qp_act[4];
    for (int l = 0; l < 4; l++) {
        Tensor a = upload(act[l], {(uint64_t)act[l].size()}, FLOAT32);
        float mn, mx;
        GetMinMax((float *)a.get_data_ptr(), a.get_numels(), &mn, &mx);
        ComputeQuantizationParams(mn, mx, &qp_act[l]);
        float omn, omx;
        oracle_qparams oq;
        oracle_get_min_max(act[l].data(), act[l].size(), &omn, &omx);
        oracle_compute_qparams(omn, omx, &oq);
        CHECK(mn == omn && mx == omx, "GetMinMax vs oracle");
        CHECK(oq.scale == qp_act[l].scale && oq.zero_point == qp_act[l].zero_point, "ComputeQuantizationParams vs oracle");
    }

    // ---- set up the quantized network (nn_tests.cpp:802-884) ----
    std::vector<FullyConnected_q *> layers;
    std::vector<std::vector<uint8_t>> Wq(3);
    std::vector<std::vector<int32_t>> bq(3);
    QuantizationParams qp_w[3];
    for (int l = 0; l < 3; l++) {
        FullyConnected_q proto(dims[l], dims[l + 1], true);
        FullyConnected_q *fc = new FullyConnected_q(proto);  // register_module copy-constructs, then init()s
        fc->init();
        fc->set_qparams_in(qp_act[l]);
        fc->set_qparams_out(qp_act[l + 1]);
        QuantizationParams qp_wts[2];
        int count = 0;
        for (auto wts : fc->get_all_weights()) {
            if (count == 0) {
                Tensor wf = upload(W[l], {(uint64_t)W[l].size()}, FLOAT32);
                float mn, mx;
                GetMinMax((float *)wf.get_data_ptr(), wf.get_numels(), &mn, &mx);
                ComputeQuantizationParams(mn, mx, &qp_wts[count]);
                TensorOps o;
                o.data_type = UINT8;
                o.device_type = GPU;
                Tensor q = AllocateTensor({(uint64_t)W[l].size()}, &o);
                Quantize((float *)wf.get_data_ptr(), (uint8_t *)q.get_data_ptr(), wf.get_numels(), &qp_wts[count]);
                Wq[l] = download<uint8_t>(q);
                memcpy(wts->get_data_ptr(), Wq[l].data(), Wq[l].size());  // written through get_all_weights()
            } else {
                qp_wts[count].scale = qp_act[l].scale * qp_wts[0].scale;
                qp_wts[count].zero_point = 0;
                Tensor bf = upload(bias[l], {(uint64_t)bias[l].size()}, FLOAT32);
                TensorOps o;
                o.data_type = INT32;
                o.device_type = GPU;
                Tensor q = AllocateTensor({(uint64_t)bias[l].size()}, &o);
                Quantize((float *)bf.get_data_ptr(), (int *)q.get_data_ptr(), bf.get_numels(), &qp_wts[count]);
                bq[l] = download<int32_t>(q);
                memcpy(wts->get_data_ptr(), bq[l].data(), bq[l].size() * sizeof(int32_t));
            }
            count++;
        }
        fc->set_qparams_params(qp_wts, count);
        qp_w[l] = qp_wts[0];
        // oracle agrees on the set-up bytes
        std::vector<uint8_t> wq_o(W[l].size());
        std::vector<int32_t> bq_o(bias[l].size());
        oracle_qparams ow{qp_wts[0].scale, qp_wts[0].zero_point}, ob{qp_wts[1].scale, 0};
        oracle_quantize_u8(W[l].data(), wq_o.data(), wq_o.size(), &ow);
        oracle_quantize_i32(bias[l].data(), bq_o.data(), bq_o.size(), &ob);
        CHECK(wq_o == Wq[l], "weight Quantize vs oracle");
        CHECK(bq_o == bq[l], "bias Quantize vs oracle");
        // the packaged form of the same set-up (lten::quantize_module) writes the same bytes and parameters
        {
            FullyConnected_q twin(dims[l], dims[l + 1], true);
            twin.init();
            Tensor wf = upload(W[l], {(uint64_t)W[l].size()}, FLOAT32);
            Tensor bf = upload(bias[l], {(uint64_t)bias[l].size()}, FLOAT32);
            QuantizationParams got_w = quantize_module(twin, wf, &bf, qp_act[l], qp_act[l + 1]);
            QuantizationParams q3[3];
            twin.get_qparams(q3);
            CHECK(got_w.scale == qp_wts[0].scale && got_w.zero_point == qp_wts[0].zero_point, "quantize_module: weight parameters");
            CHECK(q3[0].scale == qp_act[l].scale && q3[2].scale == qp_act[l + 1].scale && q3[1].scale == qp_wts[0].scale,
                  "quantize_module: layer parameters");
            std::vector<Tensor *> tw = twin.get_all_weights();
            CHECK(memcmp(tw[0]->get_data_ptr(), Wq[l].data(), Wq[l].size()) == 0, "quantize_module: weight bytes");
            CHECK(memcmp(tw[1]->get_data_ptr(), bq[l].data(), bq[l].size() * sizeof(int32_t)) == 0, "quantize_module: bias words");
        }
        fc->train(false);
        fc->to(GPU, 0);
        layers.push_back(fc);
    }
    {   // MinMaxObserver: running statistics over two pieces equal GetMinMax over the whole
        std::vector<float> a(W[0].begin(), W[0].begin() + W[0].size() / 2), b(W[0].begin() + W[0].size() / 2, W[0].end());
        Tensor ta = upload(a, {(uint64_t)a.size()}, FLOAT32), tb = upload(b, {(uint64_t)b.size()}, FLOAT32);
        Tensor tw = upload(W[0], {(uint64_t)W[0].size()}, FLOAT32);
        MinMaxObserver obs;
        CHECK(!obs.seen(), "MinMaxObserver starts empty");
        obs.update(ta);
        obs.update(tb);
        float mn, mx;
        GetMinMax((float *)tw.get_data_ptr(), tw.get_numels(), &mn, &mx);
        QuantizationParams want, got = obs.qparams();
        ComputeQuantizationParams(mn, mx, &want);
        CHECK(obs.min() == mn && obs.max() == mx && got.scale == want.scale && got.zero_point == want.zero_point,
              "MinMaxObserver over two pieces");
    }

    // ---- inference (nn_tests.cpp:930-963) ----
    Tensor input = upload(x, {1, (uint64_t)B, (uint64_t)dims[0]}, FLOAT32);
    TensorOps o;
    o.data_type = UINT8;
    o.device_type = GPU;
    Tensor q_input = AllocateTensor({1, (uint64_t)B, (uint64_t)dims[0]}, &o);
    Quantize((float *)input.get_data_ptr(), (uint8_t *)q_input.get_data_ptr(), q_input.get_numels(), &qp_act[0]);
    std::vector<uint8_t> h = download<uint8_t>(q_input);
    {
        std::vector<uint8_t> xo(x.size());
        oracle_qparams oq{qp_act[0].scale, qp_act[0].zero_point};
        oracle_quantize_u8(x.data(), xo.data(), xo.size(), &oq);
        CHECK(xo == h, "input Quantize vs oracle");
    }
    Tensor cur = q_input;
    layers[0]->set_next(layers[1]);  // a hint only (used by the small-batch kernel): the outputs below must not change
    layers[1]->set_next(layers[2]);
    for (int l = 0; l < 3; l++) {
        Tensor y = layers[l]->forward(cur);
        CHECK(y.get_ndims() == 3 && y.get_sizes()[1] == (uint64_t)B && y.get_sizes()[2] == (uint64_t)dims[l + 1], "output shape");
        CHECK(y.get_data_type() == UINT8 && y.get_device() == GPU, "output dtype/device");
        std::vector<uint8_t> got = download<uint8_t>(y), want((size_t)B * dims[l + 1]);
        std::vector<int32_t> ws(B + dims[l + 1]);
        oracle_qparams qp3[3] = {{qp_act[l].scale, qp_act[l].zero_point}, {qp_w[l].scale, qp_w[l].zero_point},
                                 {qp_act[l + 1].scale, qp_act[l + 1].zero_point}};
        oracle_quantized_matmul(0, 1, B, dims[l + 1], dims[l], 1, h.data(), Wq[l].data(), 0, want.data(), qp3, bq[l].data(), ws.data());
        CHECK(got == want, ("layer " + std::to_string(l) + " output vs oracle").c_str());
        h = got;
        cur = y;
    }
    layers[0]->set_next(nullptr);
    layers[1]->set_next(nullptr);
    {   // the same three layers as one launch: float input in, the last layer's bytes out
        FusedChain_q chain({layers[0], layers[1], layers[2]});
        Tensor y = chain.forward(input);
        CHECK(y.get_ndims() == 3 && y.get_sizes()[1] == (uint64_t)B && y.get_sizes()[2] == (uint64_t)dims[3], "fused chain: output shape");
        CHECK(download<uint8_t>(y) == h, "fused chain (one launch) equals the layer-by-layer result and the oracle");
        Tensor y2 = chain.forward(input);
        CHECK(download<uint8_t>(y2) == h, "fused chain, second call");
    }
    TensorOps of;
    of.device_type = GPU;
    Tensor output = AllocateTensor({1, (uint64_t)B, 10}, &of);
    Dequantize((float *)output.get_data_ptr(), (uint8_t *)cur.get_data_ptr(), cur.get_numels(), &qp_act[3]);
    {
        std::vector<float> got = download<float>(output), want(got.size());
        oracle_qparams oq{qp_act[3].scale, qp_act[3].zero_point};
        oracle_dequantize(want.data(), h.data(), h.size(), &oq);
        CHECK(memcmp(got.data(), want.data(), got.size() * sizeof(float)) == 0, "Dequantize vs oracle");
        // the quantized logits track the fp32 ones
        double err = 0, ref = 0;
        for (size_t i = 0; i < got.size(); i++) {
            err += fabs(got[i] - act[3][i]);
            ref += fabs(act[3][i]);
        }
        CHECK(err / ref < 0.1, "uint8 logits close to fp32 logits");
        printf("mean |uint8 - fp32| / mean |fp32| on the logits: %.4f\n", err / ref);
    }

    // ---- fused extensions: fp32 output with ReLU equals relu(dequantized int32) ----
    {
        layers[0]->set_output(LTQ_OUT_F32, true);
        Tensor y = layers[0]->forward(q_input);
        std::vector<float> got = download<float>(y);
        layers[0]->set_output(LTQ_OUT_I32);
        std::vector<int32_t> acc = download<int32_t>(layers[0]->forward(q_input));
        bool same = true;
        const float s = qp_act[0].scale * qp_w[0].scale;
        for (size_t i = 0; i < got.size(); i++) same = same && got[i] == s * (float)(acc[i] > 0 ? acc[i] : 0);
        CHECK(same, "F32+ReLU epilogue == scale * max(acc, 0)");
        layers[0]->set_output(LTQ_OUT_U8);
    }

    // ---- a stream of the caller's, recycled output buffers ----
    {
        cudaStream_t st;
        cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
        cudaDeviceSynchronize();
        layers[0]->set_stream(st);
        void *first = nullptr;
        std::vector<uint8_t> ref;
        bool same_ptr = true, same_bytes = true;
        for (int it = 0; it < 4; it++) {
            Tensor y = layers[0]->forward(q_input);      // dropped at the end of the iteration: the next one reuses its bytes
            cudaStreamSynchronize(st);
            std::vector<uint8_t> got = download<uint8_t>(y);
            if (it == 0) {
                first = y.get_data_ptr();
                ref = got;
            }
            same_ptr = same_ptr && y.get_data_ptr() == first;
            same_bytes = same_bytes && got == ref;
        }
        CHECK(same_ptr, "forward() recycles the output it handed out before once the caller has dropped it");
        CHECK(same_bytes, "results on a caller stream are the same every time");
        Tensor held = layers[0]->forward(q_input);
        Tensor other = layers[0]->forward(q_input);
        CHECK(held.get_data_ptr() != other.get_data_ptr(), "an output the caller still holds is not reused");
        cudaStreamSynchronize(st);
        CHECK(download<uint8_t>(held) == ref && download<uint8_t>(other) == ref, "both outputs are complete");
        layers[0]->check();
        layers[0]->set_stream(nullptr);
        cudaStreamDestroy(st);
    }

    // ---- one host thread, every visible GPU: row- and column-sharded layer 1 against the oracle ----
    {
        int ndev = 0;
        cudaGetDeviceCount(&ndev);
        if (ndev > 4) ndev = 4;
        std::vector<int> devs;
        for (int d = 0; d < ndev; d++) devs.push_back(d);
        DeviceGroup group(devs);
        const uint64_t K = dims[0], N = 512 / ndev * ndev, nloc = N / ndev;   // layer 1's first N outputs
        const uint64_t Mtot = B;
        oracle_qparams qp3[3] = {{qp_act[0].scale, qp_act[0].zero_point}, {qp_w[0].scale, qp_w[0].zero_point},
                                 {qp_act[1].scale, qp_act[1].zero_point}};
        std::vector<uint8_t> want((size_t)Mtot * N), xin = download<uint8_t>(q_input);
        std::vector<int32_t> ws(Mtot + N);
        oracle_quantized_matmul(0, 1, Mtot, N, K, 1, xin.data(), Wq[0].data(), 0, want.data(), qp3, bq[0].data(), ws.data());
        // rows: full replica on every device, the batch split
        {
            std::vector<FullyConnected_q *> reps;
            std::vector<Tensor> ins;
            for (int d = 0; d < ndev; d++) {
                FullyConnected_q *fc = new FullyConnected_q(K, N, true);
                fc->init();
                memcpy(fc->get_all_weights()[0]->get_data_ptr(), Wq[0].data(), (size_t)N * K);
                memcpy(fc->get_all_weights()[1]->get_data_ptr(), bq[0].data(), (size_t)N * 4);
                fc->set_qparams_in(qp_act[0]);
                fc->set_qparams_out(qp_act[1]);
                fc->set_qparams_params(&qp_w[0], 1);
                fc->to(GPU, d);
                reps.push_back(fc);
                const uint64_t r0 = Mtot * d / ndev, r1 = Mtot * (d + 1) / ndev;
                TensorOps o;
                o.data_type = UINT8;
                Tensor host = TensorFromBuffer({1, r1 - r0, K}, xin.data() + r0 * K, false, &o);
                ins.push_back(host.to(GPU, d));
            }
            std::vector<Tensor> outs = group.forward_rowsharded(reps, ins);
            group.synchronize(20000);
            std::vector<uint8_t> got;
            for (auto &t : outs) {
                std::vector<uint8_t> part = download<uint8_t>(t);
                got.insert(got.end(), part.begin(), part.end());
            }
            CHECK(got == want, "row-sharded layer over the device group vs oracle");
            for (auto fc : reps) delete fc;
        }
        // columns: a slice of the weight rows on every device, the whole batch everywhere, NCCL all-gather
        {
            std::vector<FullyConnected_q *> sl;
            std::vector<Tensor> ins;
            for (int d = 0; d < ndev; d++) {
                FullyConnected_q *fc = new FullyConnected_q(K, nloc, true);
                fc->init();
                memcpy(fc->get_all_weights()[0]->get_data_ptr(), Wq[0].data() + (size_t)d * nloc * K, (size_t)nloc * K);
                memcpy(fc->get_all_weights()[1]->get_data_ptr(), bq[0].data() + (size_t)d * nloc, (size_t)nloc * 4);
                fc->set_qparams_in(qp_act[0]);
                fc->set_qparams_out(qp_act[1]);
                fc->set_qparams_params(&qp_w[0], 1);
                fc->to(GPU, d);
                sl.push_back(fc);
                TensorOps o;
                o.data_type = UINT8;
                Tensor host = TensorFromBuffer({1, Mtot, K}, xin.data(), false, &o);
                ins.push_back(host.to(GPU, d));
            }
            std::vector<Tensor> outs = group.forward_colsharded(sl, ins);
            group.synchronize(20000);
            bool all = true;
            for (auto &t : outs) all = all && download<uint8_t>(t) == want;
            CHECK(all, "column-sharded layer (all-gather over the device group) vs oracle on every device");
            for (auto fc : sl) delete fc;
        }
        printf("device group of %d: row- and column-sharded forward checked\n", ndev);
    }

    // ---- argument checks, reference messages (fully_connected.cpp:330-348) ----
    static FullyConnected_q *L0 = layers[0];
    CHECK(throws_with("at least 3 dimensions", [] {
              TensorOps o; o.data_type = UINT8; o.device_type = GPU;
              Tensor t = AllocateTensor({64, 784}, &o);
              L0->forward(t);
          }), "ndims < 3 rejected");
    CHECK(throws_with("not the same as this layer's parameters", [] {
              TensorOps o; o.data_type = UINT8;
              Tensor t = AllocateTensor({1, 2, 784}, &o);  // CPU tensor, GPU layer
              L0->forward(t);
          }), "device mismatch rejected");
    CHECK(throws_with("not the same as this layer's parameters", [] {
              TensorOps o; o.data_type = FLOAT32; o.device_type = GPU;
              Tensor t = AllocateTensor({1, 2, 784}, &o);
              L0->forward(t);
          }), "dtype mismatch rejected");
    CHECK(throws_with("Last dimension", [] {
              TensorOps o; o.data_type = UINT8; o.device_type = GPU;
              Tensor t = AllocateTensor({1, 2, 100}, &o);
              L0->forward(t);
          }), "feature mismatch rejected");

    for (auto fc : layers) delete fc;
    if (failures) {
        printf("%d check(s) FAILED\n", failures);
        return 1;
    }
    printf("PASS\n");
    return 0;
}
