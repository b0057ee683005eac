// Host-visible interface of the patch-buffer-free Conv2d_q path (ltq_conv_direct.cu).
#pragma once
#include "ltq_common.cuh"
#include "ltq_gemm_tc.cuh"

namespace ltq {

// The layer's output channels in blocks of at most 112 (one launch each), with the tensor map of every block's reordered
// weights.
struct ConvDirectPlan {
    static constexpr int MAX_BLOCKS = 8;
    uint32_t blocks = 0;
    uint32_t sh = 1, sw = 1;       // the layer's strides: the channels-last copy is kept as sh * sw planes of equal residues
    uint32_t cout0[MAX_BLOCKS] = {0}, nb[MAX_BLOCKS] = {0}, valid[MAX_BLOCKS] = {0};   // first channel, padded and real count
    TcOperandMap maps[MAX_BLOCKS];
};
// Static eligibility (known when the layer is created) and the block split: stride 1 (input channels are padded to a
// multiple of 64 in the channels-last copy and the reordered weights, output channels to a multiple of 16; at most 8
// blocks), and a block's reordered weights of all kernel taps fit in shared memory beside the ring.  plan->blocks == 0
// and false otherwise.
bool conv_direct_plan(ConvDirectPlan *plan, uint64_t Cin, uint64_t Cout, uint64_t kh, uint64_t kw, uint64_t sh, uint64_t sw);
// Bytes of the channels-last copy of the input (channels padded to a multiple of 64).
size_t conv_direct_input_bytes(const ConvDirectPlan &plan, uint64_t batches, uint64_t Cin, uint64_t H, uint64_t W);
// Bytes of the reordered weight buffer: per block (channels + 16) rows of padded Cin * kh * kw.
size_t conv_direct_weight_bytes(const ConvDirectPlan &plan, uint64_t Cin, uint64_t kh, uint64_t kw);
// Reorders w [Cout][Cin][kh][kw] block by block into wr [channels + 16][kh][kw][Cin] (the extra rows: ones, then zeros) and
// encodes the blocks' maps.
cudaError_t conv_direct_prepare_weights(const uint8_t *w, uint8_t *wr, ConvDirectPlan *plan, uint64_t Cin, uint64_t kh, uint64_t kw,
                                        cudaStream_t stream);
// Per-call eligibility: an output row and the kernel's overhang fit the 128 rows of one tile, and a ring of the tile's
// input regions fits beside the weights.
bool conv_direct_shape_ok(const ConvDirectPlan &plan, uint64_t batches, uint64_t Cin, uint64_t kh, uint64_t kw, uint64_t ph, uint64_t pw,
                          uint64_t H, uint64_t W, uint64_t Ho, uint64_t Wo);
// x [B][Cin][H][W] -> xt [B][H][W][Cin rounded up to a multiple of 64] (zero channels behind the real ones).
cudaError_t launch_nchw_to_nhwc(const uint8_t *x, uint8_t *xt, const ConvDirectPlan &plan, uint64_t batches, uint64_t Cin, uint64_t H,
                                uint64_t W, cudaStream_t stream);
// out [B][Cout][Ho][Wo] (or [B][Ho][Wo][Cout] with nhwc_out, 16-byte aligned) from the transposed input.  `epi`: A = input (patch sums come from the kernel itself: asum
// unused), B = weights (bsum = their sums per output channel, bias per output channel or nullptr).
cudaError_t launch_conv_direct(const uint8_t *xt, const ConvDirectPlan &plan, uint64_t batches, uint64_t Cin, uint64_t H, uint64_t W,
                               uint64_t Cout, uint64_t kh, uint64_t kw, uint64_t ph, uint64_t pw, uint64_t Ho, uint64_t Wo,
                               const Epilogue &epi, void *out, bool nhwc_out, uint32_t *status, int sms, cudaStream_t stream,
                               bool nchw_in = false);
// nchw_in: `xt` is the caller's NCHW input itself and the kernel transposes it into its stages while it loads (no NHWC
// copy, no transposition launch).  Possible when conv_direct_gather_ok says so: strides 1, W a multiple of 8 up to 64, an
// 8-byte aligned input, and shared memory for the gathering warps' scratch buffers beside the weights and three stages.
bool conv_direct_gather_ok(const ConvDirectPlan &plan, uint64_t Cin, uint64_t kh, uint64_t kw, uint64_t ph, uint64_t pw, uint64_t W,
                           uint64_t Wo, const uint8_t *x);

}  // namespace ltq
