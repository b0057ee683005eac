// Patch gather (im2col) for the quantized convolution, laid out for the FullyConnected_q-style GEMM kernels.
//
// The reference (l-ten/im_col.h:5-33) fills a [K, N] buffer, K = C*kh*kw patch taps by N = Ho*Wo output positions, and
// multiplies weights [Cout, K] by it (l-ten/conv2d.cpp:352-367).  The tensor-core kernels here want both operands
// contiguous along K, so this kernel writes the TRANSPOSE, [N, Kp] with one patch per row, Kp = K rounded up to 16 bytes
// and the tail zero (zero bytes add nothing to the products or to the operand sums).  Every image of the batch is
// gathered in one launch.  Taps outside the image are the literal byte 0, as in the reference (not the zero point).
#include "ltq_common.cuh"

namespace ltq {

// One thread = 16 consecutive k of one patch row = one 16-byte store; the gather loads hit L1/L2 (a tap is re-read by up
// to kh*kw patches).  The tap pointer is advanced incrementally (next kernel column, next kernel row, next channel)
// and patches that lie entirely inside the image skip the per-tap bounds test.
__global__ void __launch_bounds__(256) im2col_t_kernel(const uint8_t *__restrict__ im, uint64_t batches, ConvGeom g,
                                                      uint8_t *__restrict__ col_t)
{
    const uint32_t vec_per_row = g.Kp / 16, plane = g.Ho * g.Wo;
    const uint64_t total = batches * plane * vec_per_row;
    const uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    const uint32_t khw = g.kh * g.kw;
    const int64_t next_row = (int64_t)g.W - g.kw, next_chan = (int64_t)(g.H - g.kh) * g.W;
    for (uint64_t v = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += nth) {
        const uint64_t row = v / vec_per_row;
        const uint32_t k0 = (uint32_t)(v - row * vec_per_row) * 16;
        const uint64_t b = row / plane;
        const uint32_t n = (uint32_t)(row - b * plane);
        const uint32_t ho = n / g.Wo, wo = n - ho * g.Wo;
        const int32_t y0 = (int32_t)(ho * g.sh) - (int32_t)g.ph, x0 = (int32_t)(wo * g.sw) - (int32_t)g.pw;
        const bool interior = y0 >= 0 && x0 >= 0 && (uint32_t)y0 + g.kh <= g.H && (uint32_t)x0 + g.kw <= g.W;
        uint32_t c = k0 / khw, r = k0 - c * khw, i = r / g.kw, j = r - i * g.kw;
        // tap (c, i, j) of this patch; may point outside the image (then it is never dereferenced)
        const uint8_t *p = im + ((b * g.C + c) * g.H + (int64_t)y0 + i) * (int64_t)g.W + x0 + j;
        const uint32_t left = g.K > k0 ? g.K - k0 : 0;
        uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
        for (int t = 0; t < 16; t++) {
            uint32_t byte = 0;
            if ((uint32_t)t < left) {
                if (interior || ((uint32_t)(y0 + (int32_t)i) < g.H && (uint32_t)(x0 + (int32_t)j) < g.W)) byte = *p;
                p++;
                if (++j == g.kw) {
                    j = 0;
                    p += next_row;
                    if (++i == g.kh) {
                        i = 0;
                        p += next_chan;
                    }
                }
            }
            w[t >> 2] |= byte << (8 * (t & 3));
        }
        reinterpret_cast<uint4 *>(col_t)[v] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

cudaError_t launch_im2col_t(const uint8_t *im, uint64_t batches, const ConvGeom &g, uint8_t *col_t, cudaStream_t stream)
{
    const uint64_t total = batches * g.Ho * g.Wo * (g.Kp / 16);
    if (total == 0) return cudaSuccess;
    const uint64_t blocks = (total + 255) / 256;
    const unsigned grid = (unsigned)(blocks < 148ull * 32 ? blocks : 148ull * 32);
    im2col_t_kernel<<<grid, 256, 0, stream>>>(im, batches, g, col_t);
    count_launch();
    return cudaGetLastError();
}

}  // namespace ltq
