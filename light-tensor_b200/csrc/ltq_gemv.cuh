// Host-visible interface of the skinny (M <= 16) weight-streaming kernel (ltq_gemv.cu).
#pragma once
#include "ltq_common.cuh"

namespace ltq {

// True when the kernel can take the problem: 1 <= M <= 16, K a multiple of 16 whose activation block fits in shared
// memory, 16-byte aligned bases.
bool gemv_shape_ok(uint64_t M, uint64_t N, uint64_t K, const void *x, const void *W);
// x uint8 [M,K], W uint8 [N,K], both K-contiguous.
cudaError_t launch_gemv(const uint8_t *x, const uint8_t *W, uint64_t M, uint64_t N, uint64_t K, const Epilogue &epi,
                        void *out, int sms, cudaStream_t stream);

}  // namespace ltq
