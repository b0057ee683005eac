// Host-visible interface of the skinny (M <= 16) weight-streaming kernel (ltq_gemv.cu).
#pragma once
#include "ltq_common.cuh"
#include "ltq_gemm_tc.cuh"

namespace ltq {

// True when the kernel can take the problem: 1 <= M <= 16, K a multiple of 128, 16-byte aligned bases, and a band of at
// most 128 weight rows per tile with at least two ring stages in shared memory, on a device with `sms` SMs (the same
// count launch_gemv is given: the two must agree on the plan).
bool gemv_shape_ok(uint64_t M, uint64_t N, uint64_t K, const void *x, const void *W, int sms);
// x uint8 [M,K], W uint8 [N,K], both K-contiguous.
// Weight tensor maps of the kernel (two box heights, because the row bands of the CTAs differ by at most one group of
// 8 rows).  A caller that keeps one per weight matrix saves the host-side encoding on every call.
struct GemvWeightMaps {
    TcOperandMap lo, hi;
};

// The weight matrix of the launch that will follow this one on the stream (same M, its own N and K): once the kernel has
// issued all of its own loads, every CTA asks the first `boxes` boxes of ITS band of that matrix into L2, so that HBM keeps
// streaming through this launch's tail and the next launch's start.  Only a hint: ignored when the two plans do not
// use the same grid.  `cache` as below.
// Boxes of the next matrix a CTA asks into L2 (~70 KB per SM, ~10 MB per GPU).  Measured on 45 MB matrices, chained
// launches: 8.97 us per launch without, 8.7-8.85 with 1-4 boxes, 9.1-9.4 with 6-9 (M = 16); M = 1: 8.8 / 8.1-8.5 / 8.7-9.2.
constexpr uint32_t GEMV_NEXT_BOXES = 2;
struct GemvNext {
    const uint8_t *W = nullptr;
    uint64_t N = 0, K = 0;
    GemvWeightMaps *cache = nullptr;
    uint32_t boxes = 0;
};

// `status`: device word that receives a code if a bounded wait inside the kernel expires.
// `cache`: optional storage for the weight tensor maps, reused across calls while W, N, K stay the same.
// `early_weights`: the caller guarantees that no work still in flight on `stream` writes W; the kernel is then launched
// as a programmatic dependent of its predecessor and streams weights before that predecessor has finished (x, the
// epilogue's vectors and `out` are only touched after it has).
cudaError_t launch_gemv(const uint8_t *x, const uint8_t *W, uint64_t M, uint64_t N, uint64_t K, const Epilogue &epi,
                        void *out, uint32_t *status, int sms, cudaStream_t stream, GemvWeightMaps *cache,
                        bool early_weights, const GemvNext *next = nullptr);

}  // namespace ltq
