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

// The fast path.  One CTA per (image, group of R output rows): the C x ((R-1)*stride + kh) input rows that these
// output rows' patches read are staged in shared memory once (zero-padded left, right, above and below), then every
// warp assembles 16-byte units of patch rows from it and stores them.  A warp keeps ONE unit position (its 16 tap offsets
// live in registers, computed once per group of rows) and walks over the output rows and, lane = output column, along
// them: the 32 lanes read 32 neighbouring bytes of the slab per tap (no bank conflicts), a byte costs an add, a
// shared-memory load and its share of the packing, and the patch sums that the GEMM epilogue needs (sum over k of
// every patch) go to one shared-memory counter per patch, which saves a second pass over the patch buffer.  Channels
// are processed in groups of `cg` (a multiple of 16 unless it covers all channels, so that a group's taps fill whole
// 16-byte units).
__global__ void __launch_bounds__(256, 4) im2col_rows_kernel(const uint8_t *__restrict__ im, uint64_t batches, ConvGeom g,
                                                         uint32_t cg, uint32_t Wp, uint32_t R, uint8_t *__restrict__ col_t,
                                                         int32_t *__restrict__ colsum)
{
    extern __shared__ __align__(16) uint8_t sm[];
    const uint32_t khw = g.kh * g.kw;
    const uint32_t RH = (R - 1) * g.sh + g.kh;                         // staged input rows per channel
    const uint32_t zero_idx = cg * RH * Wp;                            // zero bytes: what padding taps read, for every
    const uint32_t zero_len = ((R - 1) * g.sh + 1) * Wp;               // output row and column of the group
    const uint32_t slab_bytes = (zero_idx + zero_len + 15) & ~15u;
    uint8_t *slab = sm;
    int32_t *psum = reinterpret_cast<int32_t *>(sm + slab_bytes);      // [R][Wo]
    const uint32_t vec_per_row = g.Kp / 16;
    const uint32_t groups_per_image = (g.Ho + R - 1) / R;
    const uint64_t groups = batches * groups_per_image;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (uint32_t x = threadIdx.x; x < zero_len; x += 256) slab[zero_idx + x] = 0;
    for (uint64_t gr = blockIdx.x; gr < groups; gr += gridDim.x) {
        const uint64_t b = gr / groups_per_image;
        const uint32_t ho0 = (uint32_t)(gr - b * groups_per_image) * R;
        const uint32_t rv = g.Ho - ho0 < R ? g.Ho - ho0 : R;           // output rows of this group
        const int32_t y0 = (int32_t)(ho0 * g.sh) - (int32_t)g.ph;
        for (uint32_t w = threadIdx.x; w < rv * g.Wo; w += 256) psum[w] = 0;
        for (uint32_t c0 = 0; c0 < g.C; c0 += cg) {
            const uint32_t cn = g.C - c0 < cg ? g.C - c0 : cg;
            const bool last = c0 + cn == g.C;
            __syncthreads();  // the previous channel group's (or row group's) readers are done with the slab
            // stage: one warp per (channel, input row), lanes along the row; eight rows are fetched before any is
            // stored so that the loads overlap (one row at a time this phase is pure global-memory latency)
            {
                constexpr int RB = 8;
                const uint32_t nrows = cn * RH;
                for (uint32_t rb = warp; rb < nrows; rb += 8 * RB) {
                    const uint8_t *src[RB];
                    bool row_ok[RB];
#pragma unroll
                    for (int m = 0; m < RB; m++) {
                        const uint32_t ri = rb + 8 * m;
                        const uint32_t c = ri / RH, i = ri - c * RH;
                        const int32_t y = y0 + (int32_t)i;
                        row_ok[m] = ri < nrows && (uint32_t)y < g.H;
                        src[m] = im + ((b * g.C + c0 + (row_ok[m] ? c : 0u)) * g.H + (row_ok[m] ? (uint32_t)y : 0u)) * (uint64_t)g.W;
                    }
                    for (uint32_t x = lane; x < Wp; x += 32) {
                        const uint32_t xx = x - g.pw;  // wraps for the left padding and then fails the test
                        uint8_t v[RB];
#pragma unroll
                        for (int m = 0; m < RB; m++) v[m] = (row_ok[m] && xx < g.W) ? src[m][xx] : (uint8_t)0;
#pragma unroll
                        for (int m = 0; m < RB; m++)
                            if (rb + 8 * m < nrows) slab[(rb + 8 * m) * Wp + x] = v[m];
                    }
                }
            }
            __syncthreads();
            // 16-byte units of this group: all whole units of its taps; the last group also writes the zero tail up to Kp
            const uint32_t u_lo = c0 * khw / 16;
            const uint32_t units = last ? vec_per_row - u_lo : cn * khw / 16;
            uint8_t *dst0 = col_t + ((b * g.Ho + ho0) * g.Wo) * (uint64_t)g.Kp + (uint64_t)u_lo * 16;
            for (uint32_t u = warp; u < units; u += 8) {
                uint32_t off[16];  // tap offsets for output row 0, column 0; taps beyond the group's channels read zeros
                {
                    const uint32_t k0 = u * 16;
                    uint32_t c = k0 / khw, r = k0 - c * khw, i = r / g.kw, j = r - i * g.kw;
#pragma unroll
                    for (int t = 0; t < 16; t++) {
                        off[t] = c < cn ? (c * RH + i) * Wp + j : zero_idx;
                        if (++j == g.kw) {
                            j = 0;
                            if (++i == g.kh) {
                                i = 0;
                                c++;
                            }
                        }
                    }
                }
                for (uint32_t r = 0; r < rv; r++) {
                    uint8_t *dst_row = dst0 + (uint64_t)r * g.Wo * g.Kp + (uint64_t)u * 16;
                    for (uint32_t wo = lane; wo < g.Wo; wo += 32) {
                        const uint8_t *px = slab + r * g.sh * Wp + wo * g.sw;
                        uint32_t w4[4];
#pragma unroll
                        for (int q = 0; q < 4; q++)
                            w4[q] = (uint32_t)px[off[4 * q]] | ((uint32_t)px[off[4 * q + 1]] << 8) |
                                    ((uint32_t)px[off[4 * q + 2]] << 16) | ((uint32_t)px[off[4 * q + 3]] << 24);
                        *reinterpret_cast<uint4 *>(dst_row + (uint64_t)wo * g.Kp) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                        const uint32_t ones = 0x01010101u;
                        const uint32_t ssum = __dp4a(w4[0], ones, __dp4a(w4[1], ones, __dp4a(w4[2], ones, __dp4a(w4[3], ones, 0u))));
                        if (ssum) atomicAdd(&psum[r * g.Wo + wo], (int32_t)ssum);
                    }
                }
            }
        }
        __syncthreads();
        for (uint32_t w = threadIdx.x; w < rv * g.Wo; w += 256) colsum[(b * g.Ho + ho0) * g.Wo + w] = psum[w];
        __syncthreads();  // psum is cleared again at the top of the loop
    }
}

// Shared-memory plan of the fast path; ok == false -> use the generic kernel and a separate sum pass.
struct Im2colPlan {
    bool ok;
    uint32_t cg, Wp, R;
    size_t smem;
};

static Im2colPlan plan_im2col_rows(const ConvGeom &g, uint64_t batches)
{
    Im2colPlan best{};
    const uint32_t Wp_min = (g.Wo - 1) * g.sw + g.kw;  // columns a patch row can touch, starting at -pw
    const uint32_t Wp = Wp_min < g.W + g.pw ? g.W + g.pw : Wp_min;
    // More output rows per CTA amortise the tap offsets and re-use the overlapping input rows, as long as enough CTAs
    // remain to fill the device and the slab fits.
    for (uint32_t R : {4u, 2u, 1u}) {
        if (R > 1 && batches * ((g.Ho + R - 1) / R) < 2 * 148) continue;
        const uint64_t RH = (uint64_t)(R - 1) * g.sh + g.kh;
        const uint64_t per_channel = RH * Wp, budget = 40 * 1024;
        uint64_t cg = budget / per_channel;
        if (cg >= g.C) cg = g.C;
        else cg = cg / 16 * 16;  // whole 16-byte units per group
        if (cg == 0) continue;
        const uint64_t slab = (cg * per_channel + ((uint64_t)(R - 1) * g.sh + 1) * Wp + 15) & ~15ull;
        Im2colPlan p{};
        p.cg = (uint32_t)cg;
        p.Wp = Wp;
        p.R = R;
        p.smem = slab + 4 * (size_t)R * g.Wo;
        p.ok = p.smem <= 48 * 1024;
        if (p.ok) return p;
    }
    return best;
}

cudaError_t launch_im2col_t_sums(const uint8_t *im, uint64_t batches, const ConvGeom &g, uint8_t *col_t, int32_t *colsum,
                                 cudaStream_t stream)
{
    if (batches == 0 || g.Ho == 0 || g.Wo == 0) return cudaSuccess;
    const Im2colPlan p = plan_im2col_rows(g, batches);
    if (!p.ok) {
        cudaError_t e = launch_im2col_t(im, batches, g, col_t, stream);
        if (e != cudaSuccess) return e;
        return launch_row_sums(col_t, batches * g.Ho * g.Wo, g.Kp, colsum, stream);
    }
    const uint64_t groups = batches * ((g.Ho + p.R - 1) / p.R);
    const unsigned grid = (unsigned)(groups < 148ull * 64 ? groups : 148ull * 64);
    im2col_rows_kernel<<<grid, 256, p.smem, stream>>>(im, batches, g, p.cg, p.Wp, p.R, col_t, colsum);
    count_launch();
    return cudaGetLastError();
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
