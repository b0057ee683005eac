// The layer handle behind ltq_layer_* (include/ltq.h): what FullyConnected_q keeps between calls, device side.  Shared by
// the entry points in ltq_api.cu and the multi-device ones in ltq_sharded.cu.
#pragma once
#include "ltq_common.cuh"
#include "ltq_gemm_tc.cuh"
#include "ltq_gemv.cuh"

constexpr int LAYER_MAPS = 8;

struct ltq_layer {
    int device = 0;
    uint64_t K = 0, N = 0;
    const uint8_t *w = nullptr;
    const int32_t *bias = nullptr;
    int32_t *wsum = nullptr;       // [N] sum_k W[j,k]
    int32_t *asum_ws = nullptr;    // activation row sums when the caller supplies none; grows with M like
    uint64_t asum_cap = 0;         // FullyConnected_q::workspace_ (l-ten/fully_connected.cpp:366-371)
    ltq_qparams qp_in{1.f, 0}, qp_wt{1.f, 0}, qp_out{1.f, 0};
    int32_t *rowsum_out = nullptr; // optional: receives the row sums of uint8 outputs (ltq_layer_set_rowsum_output)
    int32_t *clear_ptr = nullptr;  // optional: array cleared by every forward (ltq_layer_set_clear_on_forward)
    uint32_t clear_count = 0;
    ltq::TcOperandMap map_w[LAYER_MAPS];  // weight tensor maps of the tensor-core kernels, one per box height, built on demand
    int map_w_next = 0;
    ltq::GemvWeightMaps map_w_gemv;     // weight tensor maps of the skinny kernel
    ltq::GemvNext next;                 // weights of the layer that runs after this one (ltq_layer_set_next), with
    ltq::GemvWeightMaps map_next_gemv;  // their tensor maps as the skinny kernel of THIS layer needs them
    ltq::GemmDevice *dev = nullptr;  // the device's SM count and status word
};
