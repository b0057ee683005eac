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

// The fast path.  One CTA per (image, output row): the C x kh input rows that this output row's patches read are staged
// in shared memory once (zero-padded left, right, above and below), then every thread assembles 16-byte units of patch
// rows from it through a table of tap offsets and stores them, consecutive units of a patch by consecutive threads.
// The patch sums that the GEMM epilogue needs (sum over k of every patch) are accumulated on the way, which saves a
// second pass over the patch buffer.  Channels are processed in groups of `cg` (a multiple of 16 unless it covers all
// channels, so that a group's taps fill whole 16-byte units).
__global__ void __launch_bounds__(256) im2col_rows_kernel(const uint8_t *__restrict__ im, uint64_t batches, ConvGeom g,
                                                         uint32_t cg, uint32_t Wp, uint8_t *__restrict__ col_t,
                                                         int32_t *__restrict__ colsum)
{
    extern __shared__ __align__(16) uint8_t sm[];
    const uint32_t khw = g.kh * g.kw;
    const uint32_t slab_bytes = (cg * g.kh * Wp + 1 + 15) & ~15u;      // + one zero byte for the padding taps
    const uint32_t table_len = (cg * khw + 15) & ~15u;                // tap offsets of one channel group, padded
    uint8_t *slab = sm;
    uint16_t *koff = reinterpret_cast<uint16_t *>(sm + slab_bytes);
    int32_t *psum = reinterpret_cast<int32_t *>(sm + slab_bytes + 2 * table_len);
    const uint32_t zero_idx = cg * g.kh * Wp;
    const uint32_t vec_per_row = g.Kp / 16;
    const uint64_t pairs = batches * g.Ho;
    uint32_t table_for = 0xFFFFFFFFu;                                  // channel count the table was built for

    for (uint64_t pr = blockIdx.x; pr < pairs; pr += gridDim.x) {
        const uint64_t b = pr / g.Ho;
        const uint32_t ho = (uint32_t)(pr - b * g.Ho);
        const int32_t y0 = (int32_t)(ho * g.sh) - (int32_t)g.ph;
        for (uint32_t w = threadIdx.x; w < g.Wo; w += 256) psum[w] = 0;
        for (uint32_t c0 = 0; c0 < g.C; c0 += cg) {
            const uint32_t cn = g.C - c0 < cg ? g.C - c0 : cg;
            const bool last = c0 + cn == g.C;
            __syncthreads();  // the previous group's (or output row's) readers are done with the slab
            for (uint32_t idx = threadIdx.x; idx < cn * g.kh * Wp; idx += 256) {
                const uint32_t x = idx % Wp, ri = idx / Wp, i = ri % g.kh, c = ri / g.kh;
                const int32_t y = y0 + (int32_t)i, xx = (int32_t)x - (int32_t)g.pw;
                uint8_t v = 0;
                if ((uint32_t)y < g.H && (uint32_t)xx < g.W) v = im[((b * g.C + c0 + c) * g.H + (uint32_t)y) * (uint64_t)g.W + (uint32_t)xx];
                slab[idx] = v;
            }
            if (threadIdx.x == 0) slab[zero_idx] = 0;
            if (table_for != cn) {
                for (uint32_t k = threadIdx.x; k < table_len; k += 256) {
                    uint32_t off = zero_idx;
                    if (k < cn * khw) {
                        const uint32_t c = k / khw, r = k - c * khw, i = r / g.kw, j = r - i * g.kw;
                        off = (c * g.kh + i) * Wp + j;
                    }
                    koff[k] = (uint16_t)off;
                }
                table_for = cn;
            }
            __syncthreads();
            // 16-byte units of this group: all whole units of its taps; the last group also writes the zero tail up to Kp
            const uint32_t u_lo = c0 * khw / 16;
            const uint32_t units = last ? vec_per_row - u_lo : cn * khw / 16;
            uint8_t *dst_row0 = col_t + ((b * g.Ho + ho) * g.Wo) * (uint64_t)g.Kp;
            for (uint32_t item = threadIdx.x; item < g.Wo * units; item += 256) {
                const uint32_t wo = item / units, u = item - wo * units;
                const uint32_t x_base = wo * g.sw;
                uint32_t w4[4] = {0, 0, 0, 0};
                if (u * 16 < table_len) {  // (units of the zero tail beyond the table stay zero)
                    const uint4 o0 = reinterpret_cast<const uint4 *>(koff + u * 16)[0];
                    const uint4 o1 = reinterpret_cast<const uint4 *>(koff + u * 16)[1];
                    const uint32_t ow[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
                    for (int t = 0; t < 16; t++) {
                        const uint32_t off = (ow[t >> 1] >> (16 * (t & 1))) & 0xFFFFu;
                        // the zero byte is shared by all patches: it must not move with the output column
                        const uint32_t byte = slab[off == zero_idx ? off : off + x_base];
                        w4[t >> 2] |= byte << (8 * (t & 3));
                    }
                }
                *reinterpret_cast<uint4 *>(dst_row0 + (uint64_t)wo * g.Kp + (uint64_t)(u_lo + u) * 16) =
                    make_uint4(w4[0], w4[1], w4[2], w4[3]);
                const uint32_t ones = 0x01010101u;
                const uint32_t ssum = __dp4a(w4[0], ones, __dp4a(w4[1], ones, __dp4a(w4[2], ones, __dp4a(w4[3], ones, 0u))));
                if (ssum) atomicAdd(&psum[wo], (int32_t)ssum);
            }
        }
        __syncthreads();
        for (uint32_t w = threadIdx.x; w < g.Wo; w += 256) colsum[(b * g.Ho + ho) * g.Wo + w] = psum[w];
        // (the next iteration's first __syncthreads orders these reads before psum is cleared again? no: clear comes
        // first - so synchronise here)
        __syncthreads();
    }
}

// Shared-memory plan of the fast path; ok == false -> use the generic kernel and a separate sum pass.
struct Im2colPlan {
    bool ok;
    uint32_t cg, Wp;
    size_t smem;
};

static Im2colPlan plan_im2col_rows(const ConvGeom &g)
{
    Im2colPlan p{};
    const uint32_t khw = g.kh * g.kw;
    p.Wp = (g.Wo - 1) * g.sw + g.kw;           // columns a patch row can touch, starting at -pw
    if (p.Wp < g.W + g.pw) p.Wp = g.W + g.pw;  // (never narrower than what is staged)
    const uint64_t per_channel = (uint64_t)g.kh * p.Wp;
    const uint64_t budget = 40 * 1024;
    uint64_t cg = budget / per_channel;
    if (cg >= g.C) cg = g.C;
    else cg = cg / 16 * 16;                     // whole 16-byte units per group
    if (cg == 0) return p;
    const uint64_t slab = (cg * per_channel + 1 + 15) & ~15ull, table = (cg * khw + 15) & ~15ull;
    if (slab > 65535) return p;                 // tap offsets are 16 bit
    p.cg = (uint32_t)cg;
    p.smem = slab + 2 * table + 4 * (size_t)g.Wo;
    p.ok = p.smem <= 48 * 1024;
    return p;
}

cudaError_t launch_im2col_t_sums(const uint8_t *im, uint64_t batches, const ConvGeom &g, uint8_t *col_t, int32_t *colsum,
                                 cudaStream_t stream)
{
    if (batches == 0 || g.Ho == 0 || g.Wo == 0) return cudaSuccess;
    const Im2colPlan p = plan_im2col_rows(g);
    if (!p.ok) {
        cudaError_t e = launch_im2col_t(im, batches, g, col_t, stream);
        if (e != cudaSuccess) return e;
        return launch_row_sums(col_t, batches * g.Ho * g.Wo, g.Kp, colsum, stream);
    }
    const uint64_t pairs = batches * g.Ho;
    const unsigned grid = (unsigned)(pairs < 148ull * 64 ? pairs : 148ull * 64);
    im2col_rows_kernel<<<grid, 256, p.smem, stream>>>(im, batches, g, p.cg, p.Wp, col_t, colsum);
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
