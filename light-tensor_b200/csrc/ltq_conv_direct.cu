// Conv2d_q without a patch buffer (l-ten/conv2d.cpp:352-367 gathers every patch into a [K, Ho*Wo] buffer per image,
// l-ten/im_col.h:5-33, and multiplies; the first GPU form here did the same for the whole batch: 58 MB written and read
// again for 6.4 MB of input).  Here the patches never exist (input channels are padded to a multiple of 64 in the
// channels-last copy and in the reordered weights, output channels to a multiple of 16; zero channels add nothing; the
// description is for stride 1, strides are at the end):
//
//  * the product does not care in which order K is walked as long as both operands agree, so K is taken as
//    (kernel row, kernel column, channel) instead of the reference's (channel, kernel row, kernel column).  The weights
//    are reordered once (ltq_conv2d_set_weights); the input is transposed NCHW -> NHWC per call (6.4 MB for the bench
//    shape, one small kernel).  In NHWC the 64 channels of one pixel are 64 contiguous bytes, and for ONE kernel tap
//    (i, j) the patch slice of every output position of an output row is simply the input row shifted by (i - pad, j - pad);
//  * a tile is `rpt` whole output rows of one image (rpt * Wo <= 128 positions, the MMA's M).  For every tap and every
//    64-channel chunk ONE TMA tensor copy over the 4-D view {channel, x, y, image} brings the [positions][64 bytes]
//    slice into a ring stage, 64-byte swizzled as the MMA descriptor wants it; coordinates that fall outside the image
//    (the padding) are filled with zeros by the copy unit, which is exactly the reference's padding byte.  Only the
//    channel coordinate is the innermost one and it is always a multiple of 64, so the shifts by +-1 pixel cost nothing;
//  * the positions are the MMA's rows, the output channels its columns (the roles l-ten's call has the other way round;
//    the integer sum is the same): tcgen05.mma 128 x (Cout + 16) x 32, two per ring stage.  The reordered weights of all
//    taps stay resident in shared memory.  Sixteen extra weight rows are appended, the first of them all ones: its
//    accumulator column is the sum of the patch's bytes, which the zero-point correction needs - so the patch sums
//    come out of the tensor core too, in the thread that needs them;
//  * epilogue: thread = output position, the usual fused arithmetic of quantized_matmul (l-ten/math_fns.cpp:1433-1474)
//    through the shared helpers, stores straight into NCHW (for one channel the 32 positions of a warp are consecutive
//    addresses).  Accumulators are double buffered in TMEM; one persistent CTA per SM; every wait is bounded.
//
// Strides: the channels-last copy is kept as sh * sw PLANES, plane (y mod sh, x mod sw) holding the pixels of that residue
// as a dense image.  For output position (ho, wo) kernel tap (i, j) reads pixel (sh * ho + i - pad, sw * wo + j - pad), i.e.
// pixel (ho + floor((i - pad) / sh), wo + floor((j - pad) / sw)) of plane ((i - pad) mod sh, (j - pad) mod sw): again a
// constant shift per tap, so a tile loads one region per plane in use (a 5-D tensor copy, the plane being the fifth
// coordinate) and every tap is an MMA over its plane's region with a shifted start.
// More than 112 output channels run as several launches over blocks of channels (each with its own ones row).
// Everything else (rows wider than the 128 slots of a tile, regions or weights too large for shared memory) keeps the
// patch-buffer path in ltq_conv.cu.
#include <cuda.h>

#include <type_traits>

#include "ltq_common.cuh"
#include "ltq_conv_direct.cuh"
#include <string.h>

#include "ltq_gemm_tc.cuh"
#include "ltq_tcgen05.cuh"

namespace ltq {

namespace {

constexpr int GATHER_WARPS = 8;
constexpr int THREADS = 320 + 32 * GATHER_WARPS;   // warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 epilogue (two per TMEM lane
                                                   // quarter), warps 10.. gather an NCHW input straight into the stages (only launched
                                                   // when there is something to gather)
constexpr int GATHER_BUFS = 3;                     // scratch buffers of the gathering warps: copies run GATHER_BUFS - 1 items ahead
static_assert(GATHER_WARPS == 8, "the gathering code gives 16 lanes to a pixel and 16 pixel groups to a row: 256 threads");
constexpr int CCH = 64;                 // channels per K chunk = bytes per row of an operand tile (64-byte swizzle)
constexpr int MAX_STAGES = 8;
constexpr uint32_t MAX_STAGE_BYTES = 96 * 1024;
constexpr int EXTRA = 16;               // weight rows appended behind the output channels (row 0 of them: all ones)
constexpr uint32_t TMEM_COLS = 256;     // two accumulators of up to 128 columns
constexpr size_t SMEM_BUDGET = 200 * 1024;
constexpr uint32_t MAX_TAPS = 256;      // kernel positions (their region offsets are tabulated in shared memory)

struct DirectGeom {
    uint32_t B, Ho, Wo, rpt, tiles_per_image, tiles;
    uint32_t P;                           // pixel slots per row of a region: a power of two >= Wo + dx_span; rpt = 128 / P
    uint32_t kh, kw, ph, pw, cchunks;     // kernel size, padding, padded Cin / 64
    // Strides: the channels-last copy is split into sh * sw PLANES, plane (y mod sh, x mod sw) holding the pixels of that
    // residue as a dense image.  Kernel tap (i, j) then reads plane ((i - ph) mod sh, (j - pw) mod sw) shifted by
    // (floor((i - ph) / sh), floor((j - pw) / sw)) pixels, for every output position alike - stride 1 is the one-plane case.
    uint32_t sh, sw, plane_mask;          // strides; bit p set: plane p is read by some tap
    int32_t dy_min, dx_min;               // smallest shifts (<= 0 with padding)
    uint32_t rows_box, plane_bytes;       // rows of a region (rpt + dy span); rows_box * P * 64 rounded up to 1 KB
    uint32_t Cout, Npad, CoutTotal;       // channels of this launch's block (a multiple of 16), Cout + 16, channels of the layer
    uint32_t CoutValid;                   // channels of the block that exist (the last block may be padded)
    uint32_t stages, stage_bytes;         // ring depth; planes * plane_bytes
    uint32_t nhwc_out;                    // output as [image][row][column][channel] instead of [image][channel][row][column]
    uint32_t gather;                      // 1: the input is NCHW and warps 10 and up transpose it into the stages themselves
    uint32_t Cin, H, W;                   // input geometry (gather only)
};

// Shared-memory matrix descriptor for a K-major operand tile with rows of 64 bytes laid out by TMA with the 64-byte
// swizzle: 8-row groups 512 bytes apart, layout type 4.  The tile base is 512-byte aligned.
__device__ __forceinline__ uint64_t make_smem_desc_sw64(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;
    return d;
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1,
                                            int32_t c2, int32_t c3, int32_t c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
// floor(a / b) and a - b * floor(a / b) for b > 0
__host__ __device__ __forceinline__ int32_t floordiv(int32_t a, int32_t b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }
__host__ __device__ __forceinline__ int32_t floormod(int32_t a, int32_t b) { return a - b * floordiv(a, b); }

// NCHW -> NHWC for `batches` images: one CTA per (image, NHWC_ROWS rows).  The rows' C x W bytes are staged in
// shared memory as 32-bit words (four pixels of one channel each); a thread then takes the words of four consecutive
// channels, transposes the 4 x 4 bytes in registers and writes four words (four channels of one pixel each), so that a
// warp's stores are runs of 64 contiguous bytes.
constexpr uint32_t NHWC_ROWS = 1;        // rows per CTA (measured on 32 x 64 x 56 x 56: 1 row per CTA 9 us, 4 rows per CTA 17 us - the
                                         // kernel lives on the number of warps in flight, not on its instruction count: a
                                         // form without any division, four loads issued ahead per thread, took the same time)
constexpr size_t NHWC_SMEM = 160 * 1024;
template <bool PLANES>   // PLANES = false: strides 1, one plane, none of the residue arithmetic
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ xt, uint32_t Cin,
                                                           uint32_t C, uint32_t H, uint32_t W, uint32_t rows, uint32_t sh, uint32_t sw,
                                                           uint32_t b_first, uint32_t b_total)
{   // C = Cin rounded up to a multiple of 64: the channels-last copy is padded with zero channels.  With strides the copy
    // is split into sh * sw planes [plane][image][ceil(H / sh)][ceil(W / sw)][C], plane = (y mod sh) * sw + (x mod sw).
    griddep_launch_dependents();
    extern __shared__ uint32_t s32[];                    // [rows][C][pitch] words
    const uint32_t h0 = blockIdx.x * rows, b = blockIdx.y;
    const uint32_t nr = H - h0 < rows ? H - h0 : rows;
    const uint32_t ww = (W + 3) / 4, pitch = ww | 1u;    // odd pitch: the column reads below spread over the banks
    griddep_wait();
    const uint8_t *src = x + ((size_t)b * Cin * H + h0) * W;
    const bool words = (W & 3u) == 0 && (reinterpret_cast<uintptr_t>(x) & 3) == 0;
    for (uint32_t i = threadIdx.x; i < nr * C * ww; i += blockDim.x) {
        const uint32_t rc = i / ww, w4 = i - rc * ww, r = rc / C, c = rc - r * C;
        uint32_t v = 0;
        if (c < Cin) {
            const uint8_t *p = src + ((size_t)c * H + r) * W + 4 * w4;
            if (words) {
                v = *reinterpret_cast<const uint32_t *>(p);
            } else {
                for (uint32_t k = 0; k < 4 && 4 * w4 + k < W; k++) v |= (uint32_t)p[k] << (8 * k);
            }
        }
        s32[rc * pitch + w4] = v;
    }
    __syncthreads();
    uint32_t *dst = reinterpret_cast<uint32_t *>(xt);   // C % 64 == 0: word aligned
    const uint32_t cw = C / 4, Hp = (H + sh - 1) / sh, Wp = (W + sw - 1) / sw;
    for (uint32_t j = threadIdx.x; j < nr * ww * cw; j += blockDim.x) {
        const uint32_t rw = j / cw, c4 = j - rw * cw, r = rw / ww, w4 = rw - r * ww;   // consecutive threads: channel groups of one pixel group
        const uint32_t *col = s32 + (r * C + 4 * c4) * pitch + w4;
        const uint32_t r0 = col[0], r1 = col[pitch], r2 = col[2 * pitch], r3 = col[3 * pitch];
        // rK = channel 4*c4+K, bytes = pixels 4*w4 .. +3  ->  oP = pixel 4*w4+P, bytes = channels 4*c4 .. +3
        const uint32_t t0 = __byte_perm(r0, r1, 0x5140), t1 = __byte_perm(r0, r1, 0x7362);   // (r0.b0 r1.b0 r0.b1 r1.b1), (b2, b3)
        const uint32_t u0 = __byte_perm(r2, r3, 0x5140), u1 = __byte_perm(r2, r3, 0x7362);
        const uint32_t o[4] = {__byte_perm(t0, u0, 0x5410), __byte_perm(t0, u0, 0x7632), __byte_perm(t1, u1, 0x5410),
                               __byte_perm(t1, u1, 0x7632)};
#pragma unroll
        for (uint32_t k = 0; k < 4; k++) {
            const uint32_t xx = 4 * w4 + k, yy = h0 + r;
            if (xx < W) {
                if (!PLANES) {   // one plane: no residues to take (the divisions below cost a third of the kernel's time)
                    dst[(((size_t)(b_first + b) * H + yy) * W + xx) * cw + c4] = o[k];
                } else {
                    const uint32_t plane = (yy % sh) * sw + (xx % sw);
                    dst[((((size_t)plane * b_total + b_first + b) * Hp + yy / sh) * Wp + xx / sw) * cw + c4] = o[k];
                }
            }
        }
    }
}

// One block of output channels: wr[n][(i * kw + j) * Cp + c] = w[n][(c * kh + i) * kw + j] for n < valid and c < Cin (w points
// at the block's first channel; Cp = Cin rounded up to 64, the padded channels are zero); rows valid .. Cout-1 (padding of
// the last block): zero; row Cout: all ones; rows Cout+1 .. Cout+15: zero.
__global__ void reorder_weights_kernel(const uint8_t *__restrict__ w, uint8_t *__restrict__ wr, uint32_t Cout, uint32_t valid,
                                       uint32_t Cin, uint32_t Cp, uint32_t kh, uint32_t kw)
{
    const uint32_t K = Cin * kh * kw, Kp = Cp * kh * kw;
    const uint64_t total = (uint64_t)(Cout + EXTRA) * Kp;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t n = (uint32_t)(idx / Kp), k = (uint32_t)(idx - (uint64_t)n * Kp);
        uint8_t v = 0;
        if (n < valid) {
            const uint32_t tap = k / Cp, c = k - tap * Cp, i = tap / kw, j = tap - i * kw;
            if (c < Cin) v = w[(size_t)n * K + ((size_t)c * kh + i) * kw + j];
        } else if (n == Cout) {
            v = 1;
        }
        wr[idx] = v;
    }
}

}  // namespace

// OUT: 0 = uint8, 1 = float, 2 = int32 (ltq_out_mode).
template <int OUT>
__global__ void __launch_bounds__(THREADS, 1)
conv_direct_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const DirectGeom g,
                   const Epilogue epi, void *__restrict__ out, uint32_t *status, const uint8_t *__restrict__ x_nchw)
{
    griddep_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw0 = smem_u32(smem_raw);
    const uint32_t ring = (raw0 + 1023u) & ~1023u;                             // [stages][planes][rows_box][P pixels][64 B]
    const uint32_t wsm = ring + g.stages * g.stage_bytes;                      // [kh * kw * cchunks][Npad rows][64 B]
    const uint32_t taps = g.kh * g.kw, nchunks = taps * g.cchunks, wtile = g.Npad * CCH;
    uint8_t *after = smem_raw + (wsm - raw0) + nchunks * wtile;
    uint32_t *s_col = reinterpret_cast<uint32_t *>(after);                     // [128] column terms
    uint32_t *s_tap = s_col + 128;                                             // [MAX_TAPS] byte offset of every tap's window in a stage
    uint64_t *bars = reinterpret_cast<uint64_t *>(after + (128 + MAX_TAPS) * 4);   // full[S] empty[S] tfull[2] tempty[2] wfull
    uint32_t *s_misc = reinterpret_cast<uint32_t *>(bars + 2 * MAX_STAGES + 5);  // [0] tmem base, [1] abort flag
    volatile uint32_t *abort_flag = s_misc + 1;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * MAX_STAGES;
    const uint32_t tfull0 = empty0 + 8 * MAX_STAGES, tempty0 = tfull0 + 16, wfull = tempty0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < g.stages; s++) {
            mbar_init(full0 + 8 * s, g.gather ? GATHER_WARPS : 1);   // one arrival per gathering warp, or the TMA producer's
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(tfull0 + 8 * s, 1);
            mbar_init(tempty0 + 8 * s, 8);  // one arrival per epilogue warp
        }
        mbar_init(wfull, 1);
        s_misc[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // the reordered weights are static data: on their way before the kernel in front has finished
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        if (!g.gather) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        mbar_expect_tx(wfull, nchunks * wtile);
        for (uint32_t ch = 0; ch < nchunks; ch++) tma_load_2d(wsm + ch * wtile, &map_w, wfull, (int32_t)(ch * CCH), 0);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(s_misc), TMEM_COLS);
        tmem_relinquish();
    }
    // Where every kernel tap's window starts inside a stage: its plane's slot, then (dy * P + dx) pixel slots further on
    // (dy, dx counted from the region's first row and column).  Tabulated once: the MMA-issuing thread is the kernel's
    // critical path and should not divide.
    for (uint32_t tap = threadIdx.x; tap < taps; tap += blockDim.x) {
        const uint32_t i = tap / g.kw, j = tap - i * g.kw;
        const int32_t ti = (int32_t)i - (int32_t)g.ph, tj = (int32_t)j - (int32_t)g.pw;
        const uint32_t pl = (uint32_t)floormod(ti, (int32_t)g.sh) * g.sw + (uint32_t)floormod(tj, (int32_t)g.sw);
        const uint32_t dy = (uint32_t)(floordiv(ti, (int32_t)g.sh) - g.dy_min), dx = (uint32_t)(floordiv(tj, (int32_t)g.sw) - g.dx_min);
        s_tap[tap] = (uint32_t)__popc(g.plane_mask & ((1u << pl) - 1u)) * g.plane_bytes + (dy * g.P + dx) * CCH;
    }
    if (g.gather) {
        // The gathering warps only ever write pixels that exist; the slots left and right of an image row (the padding
        // columns and the unused tail of the P slots) are zero for the whole run.
        uint4 *rz = reinterpret_cast<uint4 *>(smem_raw + (ring - raw0));
        for (uint32_t i = threadIdx.x; i < g.stages * g.stage_bytes / 16; i += blockDim.x) rz[i] = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // plain stores -> tensor-core reads
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_wait();   // the input comes from the kernel in front
    const uint32_t tmem_base = s_misc[0];
    const uint32_t box_bytes = g.rows_box * g.P * CCH;   // a copy always delivers its whole box (zeros outside the image)
    const uint32_t planes = g.sh * g.sw;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && !g.gather) {
            uint32_t st = 0, ph = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < g.tiles; t += gridDim.x) {
                const uint32_t b = t / g.tiles_per_image, ho0 = (t - b * g.tiles_per_image) * g.rpt;
                // per 64-channel chunk one copy per plane in use: the rows_box rows of the plane that the tile's output rows
                // touch, P pixels wide from the leftmost shift on (whatever lies outside the image arrives as zeros)
                for (uint32_t cc = 0; cc < g.cchunks; cc++) {
                    ok = mbar_wait(empty0 + 8 * st, ph ^ 1, abort_flag, status, 0x100u | st);
                    if (!ok) break;
                    mbar_expect_tx(full0 + 8 * st, box_bytes * (uint32_t)__popc(g.plane_mask));
                    for (uint32_t pl = 0; pl < planes; pl++)
                        if (g.plane_mask >> pl & 1u)   // planes in use sit back to back in the stage
                            tma_load_5d(ring + st * g.stage_bytes + (uint32_t)__popc(g.plane_mask & ((1u << pl) - 1u)) * g.plane_bytes,
                                        &map_x, full0 + 8 * st, (int32_t)(cc * CCH), g.dx_min, (int32_t)ho0 + g.dy_min, (int32_t)b, (int32_t)pl);
                    if (++st == g.stages) { st = 0; ph ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
        const uint32_t idesc = make_idesc_i8(128, (int)g.Npad);
        uint32_t st = 0, ph = 0, as = 0, aph = 0;
        bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(wfull, 0, abort_flag, status, 0x600u));
        for (uint32_t t = blockIdx.x; ok && t < g.tiles; t += gridDim.x) {
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(tempty0 + 8 * as, aph ^ 1, abort_flag, status, 0x200u | as));
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + as * 128;
            for (uint32_t cc = 0; cc < g.cchunks; cc++) {
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(full0 + 8 * st, ph, abort_flag, status, 0x300u | st));
                if (!ok) break;
                tc_fence_after();
                if (elect_one()) {
                    // Output position p = (row hh, column ww) sits in slot hh * P + ww, and for kernel tap (i, j) it reads, from
                    // the tap's plane, the pixel in slot (hh + dy) * P + ww + dx: the same 128 rows of 64 bytes, started
                    // (dy * P + dx) slots further on (dy, dx counted from the region's first row and column).  The swizzle is
                    // a function of the shared-memory address, so a shifted start needs nothing else.
                    const uint32_t stage = ring + st * g.stage_bytes;
                    for (uint32_t tap = 0; tap < taps; tap++) {
                        const uint64_t a_desc = make_smem_desc_sw64(stage + s_tap[tap]);
                        const uint64_t b_desc = make_smem_desc_sw64(wsm + (tap * g.cchunks + cc) * wtile);
                        umma_i8(d_tmem, a_desc, b_desc, idesc, (cc | tap) != 0u);
                        umma_i8(d_tmem, a_desc + 2u, b_desc + 2u, idesc, 1u);   // the second 32 bytes of K of the 64-byte rows
                    }
                    umma_commit(empty0 + 8 * st);
                }
                __syncwarp();
                if (++st == g.stages) { st = 0; ph ^= 1; }
            }
            if (!ok) break;
            if (elect_one()) umma_commit(tfull0 + 8 * as);
            __syncwarp();
            if (++as == 2) { as = 0; aph ^= 1; }
        }
    } else if (warp >= 10) {
        // ---------------- gather (warps 10 and up, NCHW input, strides 1, W a multiple of 8 up to 64): what the NHWC copy +
        // the tensor copy do otherwise, in two steps per tile and 64-channel chunk ("item").
        // (1) The item's image rows - rows_box rows x 64 channels x W bytes, as they lie in the NCHW tensor - are fetched
        //     into a scratch buffer with 8-byte asynchronous copies (cp.async; 4-byte ones were measured first and their
        //     sheer number, 3584 per item, set the pace at ~2 us per tile whatever the number of warps and the depth; on
        //     rows of 20 and 28 bytes, which only 4-byte copies can fetch, gathering measured no faster than the NHWC copy
        //     in front, so those keep it),
        //     GATHER_BUFS - 1 items ahead of their use: no registers held, memory latency off the critical path.  Rows
        //     outside the image and channels beyond Cin are not fetched.  A (row, channel) line takes 64 bytes of scratch;
        //     its 8-byte units are rotated by channel / 4 so that the reads of step 2 spread over the banks.
        // (2) A thread takes the words (four pixels each) of four consecutive channels at one place of a row from the
        //     scratch buffer, transposes the 4 x 4 bytes in registers and writes four words - four channels of one pixel
        //     each - into the stage at the addresses the 64-byte swizzle gives them (16-byte unit index XOR bits 7-8 of
        //     the byte address).  Sixteen lanes cover the 64 channels of a pixel, so a warp's stores are two runs of 64
        //     bytes.  Rows outside the image are written as zeros; the columns left and right were zeroed once.
        // The gathering warps meet once per item (named barrier 2): everybody's copies of the item have landed, and everybody is
        // done reading the buffer that the copies issued next will overwrite.  The loop always runs its full count so that
        // the barrier stays matched even after a bounded wait has given up; the work is skipped then.
        if (g.gather) {
            const uint32_t lt = threadIdx.x - 320u, c4 = lt & 15u, wsub = lt >> 4;   // wsub = 0 .. 15: this thread's place (word) in a row
            const uint32_t nw4 = g.W / 4, nw8 = g.W / 8;
            constexpr uint32_t LINE = 16;                                         // words of scratch per (row, channel)
            const size_t chan = (size_t)g.H * g.W;
            uint8_t *ring_ptr = smem_raw + (ring - raw0);
            uint32_t *scratch = reinterpret_cast<uint32_t *>(s_misc + 4);          // [GATHER_BUFS][rows_box * 64 lines]
            const uint32_t scratch_words = g.rows_box * CCH * LINE;
            const uint32_t my_tiles = blockIdx.x < g.tiles ? (g.tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
            const uint32_t items = my_tiles * g.cchunks;
            // cursor of the copies (runs ahead) and of the transposing step
            uint32_t f_t = blockIdx.x, f_cc = 0, f_n = 0;
            // Eight lanes per line; a thread's copies of an item all have the same place in the line and channels a fixed
            // step apart: one address computation per image row, additions after that.
            const uint32_t f_w8 = lt & 7u, f_c0 = lt >> 3, f_cstep = (32u * GATHER_WARPS) >> 3;
            auto fetch_next = [&]() {
                if (f_n < items && f_w8 < nw8) {
                    const uint32_t b = f_t / g.tiles_per_image, ho0 = (f_t - b * g.tiles_per_image) * g.rpt;
                    const uint32_t buf = smem_u32(scratch + (f_n % GATHER_BUFS) * scratch_words);
                    const uint32_t ch0 = f_cc * CCH + f_c0;                      // first channel of this thread
                    for (uint32_t r = 0; r < g.rows_box; r++) {
                        const int32_t y = (int32_t)ho0 + (int32_t)r + g.dy_min;
                        if (y < 0 || y >= (int32_t)g.H) continue;
                        const uint8_t *src = x_nchw + ((size_t)b * g.Cin + ch0) * chan + (size_t)y * g.W + 8 * f_w8;
                        for (uint32_t ch = ch0, c = f_c0; c < (uint32_t)CCH && ch < g.Cin; c += f_cstep, ch += f_cstep) {
                            const uint32_t dst = buf + ((r * CCH + c) * LINE + 2 * ((f_w8 + (c >> 2)) & 7u)) * 4;
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
                            src += (size_t)f_cstep * chan;
                        }
                    }
                }
                if (f_n < items) {
                    f_n++;
                    if (++f_cc == g.cchunks) { f_cc = 0; f_t += gridDim.x; }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");     // (an empty group when nothing is left: the counting stays uniform)
            };
#pragma unroll
            for (int i = 0; i < GATHER_BUFS - 1; i++) fetch_next();
            uint32_t st = 0, ph = 0, t = blockIdx.x, cc = 0;
            bool ok = true;
            for (uint32_t n = 0; n < items; n++) {
                asm volatile("cp.async.wait_group %0;" ::"n"(GATHER_BUFS - 2) : "memory");   // this thread's copies of item n are in place
                asm volatile("bar.sync 2, %0;" ::"n"(32 * GATHER_WARPS) : "memory");   // ... and so are everybody's; item n - 1 has been read by all
                fetch_next();                                             // item n + GATHER_BUFS - 1, into the buffer item n - 1 used
                ok = ok && !*abort_flag;
                if (ok) ok = __all_sync(0xFFFFFFFFu, mbar_wait(empty0 + 8 * st, ph ^ 1, abort_flag, status, 0x700u | st));
                if (ok) {
                    const uint32_t b = t / g.tiles_per_image, ho0 = (t - b * g.tiles_per_image) * g.rpt;
                    (void)b;
                    uint8_t *stage = ring_ptr + st * g.stage_bytes;
                    const uint32_t *sc = scratch + (n % GATHER_BUFS) * scratch_words;
                    const uint32_t c0 = cc * CCH + 4 * c4;                        // this thread's first channel
                    const uint32_t nch = c0 < g.Cin ? (g.Cin - c0 < 4u ? g.Cin - c0 : 4u) : 0u;
                    // this thread's place in a row: words wsub of the lines of channels 4 * c4 .. + 3 (their units rotated by c4)
                    const uint32_t *row = sc + (4 * c4) * LINE + 2 * (((wsub >> 1) + c4) & 7u) + (wsub & 1u);
                    // byte offset of (slot, this thread's four channels) without the swizzle; slot = r * P + 4 * w4 + k - dx_min
                    uint32_t off = (uint32_t)(-g.dx_min) * CCH + (c4 & 3u) * 4 + 4 * wsub * CCH;
                    const uint32_t unit = c4 >> 2;
                    if (wsub < nw4) {
                        for (uint32_t r = 0; r < g.rows_box; r++, row += CCH * LINE, off += g.P * CCH) {
                            const int32_t y = (int32_t)ho0 + (int32_t)r + g.dy_min;
                            const bool row_in = y >= 0 && y < (int32_t)g.H;
                            const uint32_t a0 = row_in && nch > 0 ? row[0] : 0u, a1 = row_in && nch > 1 ? row[LINE] : 0u;
                            const uint32_t a2 = row_in && nch > 2 ? row[2 * LINE] : 0u, a3 = row_in && nch > 3 ? row[3 * LINE] : 0u;
                            const uint32_t t0 = __byte_perm(a0, a1, 0x5140), t1 = __byte_perm(a0, a1, 0x7362);
                            const uint32_t u0 = __byte_perm(a2, a3, 0x5140), u1 = __byte_perm(a2, a3, 0x7362);
                            const uint32_t o[4] = {__byte_perm(t0, u0, 0x5410), __byte_perm(t0, u0, 0x7632), __byte_perm(t1, u1, 0x5410),
                                                   __byte_perm(t1, u1, 0x7632)};
#pragma unroll
                            for (uint32_t k = 0; k < 4; k++) {
                                const uint32_t o_k = off + k * CCH;                 // = slot * 64 + (c4 & 3) * 4
                                // the 16-byte unit of the channels, XORed with bits 7-8 of the byte address (= bits 1-2 of the slot)
                                *reinterpret_cast<uint32_t *>(stage + o_k + ((unit ^ ((o_k >> 7) & 3u)) << 4)) = o[k];
                            }
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // plain stores -> tensor-core reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full0 + 8 * st);
                }
                if (++st == g.stages) { st = 0; ph ^= 1; }
                if (++cc == g.cchunks) { cc = 0; t += gridDim.x; }
            }
            asm volatile("cp.async.wait_all;" ::: "memory");              // nothing of this thread's is still on its way
        }
    } else {
        // ---------------- epilogue (warps 2..9 = 256 threads): thread = output position x half of the channels ----------------
        // A lone warp per scheduler cannot hide its own latencies (measured with four warps: 4.4 us per tile, issue slots
        // 19 % busy), so two warps share each TMEM lane quarter and split the channels.
        const uint32_t q = (uint32_t)warp & 3u, half = (uint32_t)(warp - 2) >> 2;
        const uint32_t et = threadIdx.x - 64;
        const EpilogueConsts c = epilogue_consts(epi);
        const bool relu = epi.flags & LTQ_FLAG_RELU, sat = epi.flags & LTQ_FLAG_SATURATE;
        using OutT = typename std::conditional<OUT == 0, uint8_t, typename std::conditional<OUT == 1, float, int32_t>::type>::type;
        OutT *o = static_cast<OutT *>(out);
        // column terms (-zA * wsum[channel] + bias[channel]): the same for every tile
        for (uint32_t j = et; j < 128u; j += 256) s_col[j] = j < g.CoutValid ? epilogue_col_term(epi, c, j) : 0u;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const uint32_t p = q * 32 + lane;                 // slot inside the tile: output row p / P, column p % P
        const uint32_t hh = p / g.P, wcol = p - hh * g.P;
        const size_t plane = (size_t)g.Ho * g.Wo;
        const uint32_t split = ((g.Cout / 2 + 15) / 16) * 16;
        const uint32_t cb = half ? split : 0u, ce = half ? g.Cout : split;   // this warp's channels
        uint32_t as = 0, aph = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < g.tiles; t += gridDim.x) {
            const uint32_t b = t / g.tiles_per_image, ho0 = (t - b * g.tiles_per_image) * g.rpt;
            const bool valid = wcol < g.Wo && ho0 + hh < g.Ho;
            if (ok) ok = mbar_wait(tfull0 + 8 * as, aph, abort_flag, status, 0x400u | as);
            if (ok) {
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + as * 128;
                uint32_t v[16], vn[16];
                tmem_ld16(taddr + g.Cout, v);             // the all-ones weight row: v[0] = sum of this position's patch bytes
                if (cb < ce) tmem_ld16(taddr + cb, vn);
                tmem_ld_wait();
                // (epi.row_bias: the reference's bias indexing, by output position inside the image)
                const uint32_t rt = c.neg_zB * v[0] + c.bc + (epi.row_bias && valid ? (uint32_t)epi.row_bias[(ho0 + hh) * g.Wo + wcol] : 0u);
                OutT *d = g.nhwc_out ? o + (((size_t)b * g.Ho + ho0 + hh) * g.Wo + wcol) * g.CoutTotal + cb
                                     : o + (size_t)b * g.CoutTotal * plane + (size_t)(ho0 + hh) * g.Wo + wcol + (size_t)cb * plane;
#pragma unroll 1
                for (uint32_t ch = cb; ch < ce; ch += 16) {
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = vn[j];
                    if (ch + 16 < ce) tmem_ld16(taddr + ch + 16, vn);   // the next chunk travels while this one is converted
                    uint32_t res[16];
                    epilogue_convert<OUT, 16>(v, rt, s_col + ch, c, relu, sat, res);
                    if (valid && g.nhwc_out) {
                        // channels-last: the 16 channels of the chunk are consecutive bytes / words of this position
                        uint4 *d4 = reinterpret_cast<uint4 *>(d);
                        if (OUT == 0) {
                            d4[0] = make_uint4(res[0], res[1], res[2], res[3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; j++) d4[j] = make_uint4(res[4 * j], res[4 * j + 1], res[4 * j + 2], res[4 * j + 3]);
                        }
                        d += 16;
                    } else if (valid) {
                        if (ch + 16 <= g.CoutValid) {     // a whole chunk of channels (all but the padded tail of the last block)
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                if (OUT == 0) d[(size_t)j * plane] = (OutT)__byte_perm(res[j >> 2], 0u, 0x4440 + (j & 3));
                                else if (OUT == 1) d[(size_t)j * plane] = (OutT)__uint_as_float(res[j]);
                                else d[(size_t)j * plane] = (OutT)(int32_t)res[j];
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                if (ch + j < g.CoutValid) {
                                    if (OUT == 0) d[(size_t)j * plane] = (OutT)((res[j >> 2] >> (8 * (j & 3))) & 0xFFu);
                                    else if (OUT == 1) d[(size_t)j * plane] = (OutT)__uint_as_float(res[j]);
                                    else d[(size_t)j * plane] = (OutT)(int32_t)res[j];
                                }
                            }
                        }
                        d += 16 * plane;
                    }
                    tmem_ld_wait();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * as);
            }
            if (++as == 2) { as = 0; aph ^= 1; }
        }
    }

    // Teardown: nobody leaves before every role is done with TMEM and shared memory.
    tc_fence_before();
    __syncthreads();
    if (warp == 0 && lane == 0 && *abort_flag) {
        // after a timeout copies issued by this thread may still be landing in this CTA's shared memory
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

size_t direct_smem(uint32_t stages, uint32_t stage_bytes, uint32_t nchunks, uint32_t Npad, uint32_t scratch_bytes = 0)
{
    return 1024 + (size_t)stages * stage_bytes + (size_t)nchunks * Npad * CCH + (128 + MAX_TAPS) * 4 + (2 * MAX_STAGES + 5) * 8 + 16 +
           scratch_bytes;
}
// The gathering warps' scratch buffers: rows_box rows x 64 channels x 64 bytes each.
uint32_t gather_scratch_bytes(uint32_t rows_box, uint64_t) { return (uint32_t)GATHER_BUFS * rows_box * CCH * 64u; }

// What a tile loads: per plane in use a region of rows_box rows x P pixel slots (P a power of two that holds an output
// row and the spread of the kernel's column shifts).  ok = false when a row does not fit the 128 rows of a tile.
struct RegionGeom {
    uint32_t P, rpt, rows_box, plane_bytes, stage_bytes, plane_mask;
    int32_t dy_min, dx_min;
    bool ok;
};
RegionGeom region_geom(uint64_t kh, uint64_t kw, uint64_t ph, uint64_t pw, uint64_t sh, uint64_t sw, uint64_t Wo)
{
    RegionGeom r{};
    r.dy_min = floordiv(-(int32_t)ph, (int32_t)sh);
    r.dx_min = floordiv(-(int32_t)pw, (int32_t)sw);
    const int32_t dy_max = floordiv((int32_t)kh - 1 - (int32_t)ph, (int32_t)sh), dx_max = floordiv((int32_t)kw - 1 - (int32_t)pw, (int32_t)sw);
    const uint64_t need = Wo + (uint64_t)(dx_max - r.dx_min);
    r.P = 8;
    while (r.P < need && r.P < 256) r.P *= 2;
    r.ok = need <= 128;
    if (!r.ok) return r;
    r.rpt = 128 / r.P;
    r.rows_box = r.rpt + (uint32_t)(dy_max - r.dy_min);
    r.plane_bytes = (uint32_t)(((uint64_t)r.rows_box * r.P * CCH + 1023) & ~1023ull);
    for (uint64_t i = 0; i < kh; i++)
        for (uint64_t j = 0; j < kw; j++)
            r.plane_mask |= 1u << (floormod((int32_t)i - (int32_t)ph, (int32_t)sh) * (int32_t)sw + floormod((int32_t)j - (int32_t)pw, (int32_t)sw));
    r.stage_bytes = (uint32_t)__builtin_popcount(r.plane_mask) * r.plane_bytes;
    r.ok = r.rows_box <= 256;
    return r;
}

template <int OUT>
cudaError_t launch_direct(const CUtensorMap &mx, const CUtensorMap &mw, const DirectGeom &g, const Epilogue &epi, void *out,
                          uint32_t *status, int sms, cudaStream_t stream, const uint8_t *x_nchw)
{
    const size_t smem = direct_smem(g.stages, g.stage_bytes, g.kh * g.kw * g.cchunks, g.Npad,
                                    g.gather ? gather_scratch_bytes(g.rows_box, g.W) : 0u);
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_done[dev]) {
        e = cudaFuncSetAttribute(conv_direct_kernel<OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const unsigned grid = g.tiles < (uint32_t)sms ? g.tiles : (unsigned)sms;
    // (the gathering warps are only launched when there is something to gather)
    e = launch_chained(conv_direct_kernel<OUT>, dim3(grid), dim3(g.gather ? THREADS : THREADS - 32 * GATHER_WARPS), smem, stream, mx,
                       mw, g, epi, out, status, x_nchw);
    count_launch();
    note_kernel("conv_direct_kernel<%s> (%u tiles of %u rows x %u slots%s)", out_mode_name(OUT), g.tiles, g.rpt, g.P,
                g.gather ? ", NCHW input gathered in the kernel" : "");
    return e;
}

}  // namespace

static uint64_t padded_channels(uint64_t Cin) { return (Cin + CCH - 1) / CCH * CCH; }

bool conv_direct_plan(ConvDirectPlan *plan, uint64_t Cin, uint64_t Cout, uint64_t kh, uint64_t kw, uint64_t sh, uint64_t sw)
{
    plan->blocks = 0;
    if (sh < 1 || sw < 1 || sh * sw > 16 || kh * kw > MAX_TAPS || encode_fn() == nullptr) return false;
    plan->sh = (uint32_t)sh;
    plan->sw = (uint32_t)sw;
    const uint64_t nchunks = kh * kw * (padded_channels(Cin) / CCH);
    const uint32_t min_stage = region_geom(kh, kw, 0, 0, sh, sw, 1).stage_bytes;   // the smallest a stage can be
    if (nchunks >= (1u << 16)) return false;
    // Output channels (rounded up to a multiple of 16) in blocks of at most 112 (+ 16 extra weight rows = the MMA's 128
    // columns per accumulator), as equal as multiples of 16 allow; a block's weights of all taps stay in shared memory
    // beside a ring of at least 2 of the smallest stages (whether the stages of a given image width fit is decided per call).
    const uint64_t units = (Cout + 15) / 16;
    for (uint32_t blocks = (uint32_t)((units * 16 + 111) / 112); blocks <= (uint32_t)ConvDirectPlan::MAX_BLOCKS; blocks++) {
        const uint32_t nb = (uint32_t)((units + blocks - 1) / blocks) * 16;
        if (direct_smem(2, min_stage, (uint32_t)nchunks, nb + EXTRA) > SMEM_BUDGET) continue;
        uint32_t c0 = 0;
        plan->blocks = 0;
        while (c0 < Cout) {
            const uint32_t left = (uint32_t)(Cout - c0);
            const uint32_t n = left < nb ? (left + 15) / 16 * 16 : nb;
            plan->cout0[plan->blocks] = c0;
            plan->nb[plan->blocks] = n;
            plan->valid[plan->blocks] = left < n ? left : n;
            plan->blocks++;
            c0 += n;
        }
        return true;
    }
    return false;
}

size_t conv_direct_weight_bytes(const ConvDirectPlan &plan, uint64_t Cin, uint64_t kh, uint64_t kw)
{
    size_t rows = 0;
    for (uint32_t i = 0; i < plan.blocks; i++) rows += plan.nb[i] + EXTRA;
    return rows * padded_channels(Cin) * kh * kw;
}

size_t conv_direct_input_bytes(const ConvDirectPlan &plan, uint64_t batches, uint64_t Cin, uint64_t H, uint64_t W)
{
    return (size_t)plan.sh * plan.sw * batches * ((H + plan.sh - 1) / plan.sh) * ((W + plan.sw - 1) / plan.sw) * padded_channels(Cin);
}

cudaError_t conv_direct_prepare_weights(const uint8_t *w, uint8_t *wr, ConvDirectPlan *plan, uint64_t Cin, uint64_t kh, uint64_t kw,
                                        cudaStream_t stream)
{
    const uint64_t K = Cin * kh * kw, Cp = padded_channels(Cin), Kp = Cp * kh * kw;
    size_t row0 = 0;
    for (uint32_t i = 0; i < plan->blocks; i++) {
        uint8_t *dst = wr + row0 * Kp;
        const uint64_t Npad = plan->nb[i] + EXTRA;
        reorder_weights_kernel<<<256, 256, 0, stream>>>(w + (size_t)plan->cout0[i] * K, dst, plan->nb[i], plan->valid[i], (uint32_t)Cin,
                                                        (uint32_t)Cp, (uint32_t)kh, (uint32_t)kw);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        count_launch();
        cuuint64_t dims[2] = {(cuuint64_t)Kp, (cuuint64_t)Npad};
        cuuint64_t strides[1] = {(cuuint64_t)Kp};
        cuuint32_t box[2] = {(cuuint32_t)CCH, (cuuint32_t)Npad};
        cuuint32_t estr[2] = {1, 1};
        TcOperandMap *map = &plan->maps[i];
        CUresult r = encode_fn()(reinterpret_cast<CUtensorMap *>(map->opaque), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, dst, dims, strides,
                                 box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        map->base = dst;
        map->rows = Npad;
        map->K = Kp;
        map->box_rows = (int)Npad;
        map->box_lines = 0;
        row0 += Npad;
    }
    return cudaSuccess;
}

bool conv_direct_shape_ok(const ConvDirectPlan &plan, uint64_t batches, uint64_t Cin, uint64_t kh, uint64_t kw, uint64_t ph, uint64_t pw,
                          uint64_t H, uint64_t W, uint64_t Ho, uint64_t Wo)
{
    if (plan.blocks == 0) return false;
    const uint64_t Cout = plan.nb[0];   // the widest block
    if (!(Wo >= 1 && W <= (1u << 20) && H <= (1u << 20) && ph <= (1u << 20) && pw <= (1u << 20) && batches < (1ull << 31) &&
          Ho < (1ull << 31)))
        return false;
    const RegionGeom r = region_geom(kh, kw, ph, pw, plan.sh, plan.sw, Wo);
    if (!r.ok || r.stage_bytes > MAX_STAGE_BYTES) return false;
    if (padded_channels(Cin) * ((((W + 3) / 4) | 1u) * 4) > NHWC_SMEM) return false;   // one image row of the transposition in shared memory
    return direct_smem(2, r.stage_bytes, (uint32_t)(kh * kw * (padded_channels(Cin) / CCH)), (uint32_t)(Cout + EXTRA)) <= SMEM_BUDGET;
}

bool conv_direct_gather_ok(const ConvDirectPlan &plan, uint64_t Cin, uint64_t kh, uint64_t kw, uint64_t ph, uint64_t pw, uint64_t W,
                           uint64_t Wo, const uint8_t *x)
{
    // strides 1 (one plane), image rows of whole 8-byte units, at most 64 bytes (one scratch line), an 8-byte aligned input ...
    if (!(plan.blocks > 0 && plan.sh == 1 && plan.sw == 1 && W % 8 == 0 && W <= 64 && (reinterpret_cast<uintptr_t>(x) & 7) == 0)) return false;
    // ... and room for the scratch buffers beside the weights and a ring of at least three stages
    const RegionGeom r = region_geom(kh, kw, ph, pw, 1, 1, Wo);
    if (!r.ok) return false;
    return direct_smem(3, r.stage_bytes, (uint32_t)(kh * kw * (padded_channels(Cin) / CCH)), plan.nb[0] + EXTRA,
                       gather_scratch_bytes(r.rows_box, W)) <= SMEM_BUDGET;
}

cudaError_t launch_nchw_to_nhwc(const uint8_t *x, uint8_t *xt, const ConvDirectPlan &plan, uint64_t batches, uint64_t Cin, uint64_t H,
                                uint64_t W, cudaStream_t stream)
{
    const uint64_t C = padded_channels(Cin);
    // planes of different residues have up to one row / column less than ceil(H / sh) x ceil(W / sw): those stay zero
    if (H % plan.sh != 0 || W % plan.sw != 0) {
        cudaError_t e = cudaMemsetAsync(xt, 0, conv_direct_input_bytes(plan, batches, Cin, H, W), stream);
        if (e != cudaSuccess) return e;
    }
    // one CTA per (group of rows, image); the grid's y extent holds 65535 images per launch
    const size_t pitch = ((W + 3) / 4) | 1u, row_bytes = C * pitch * 4;
    if (row_bytes > NHWC_SMEM) return cudaErrorInvalidConfiguration;
    uint32_t rows = (uint32_t)(NHWC_SMEM / row_bytes);
    rows = rows > NHWC_ROWS ? NHWC_ROWS : rows;
    const size_t smem = rows * row_bytes;
    static bool attr_done[64] = {false};                 // the opt-in shared-memory size is a per-device attribute
    int dev = 0;
    cudaError_t ea = cudaGetDevice(&dev);
    if (ea != cudaSuccess) return ea;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_done[dev]) {
        ea = cudaFuncSetAttribute(nchw_to_nhwc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)NHWC_SMEM);
        if (ea == cudaSuccess) ea = cudaFuncSetAttribute(nchw_to_nhwc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)NHWC_SMEM);
        if (ea != cudaSuccess) return ea;
        attr_done[dev] = true;
    }
    const bool one_plane = plan.sh == 1 && plan.sw == 1;
    for (uint64_t b0 = 0; b0 < batches; b0 += 65535) {
        const uint64_t nb = batches - b0 < 65535 ? batches - b0 : 65535;
        const dim3 grid((unsigned)((H + rows - 1) / rows), (unsigned)nb);
        cudaError_t e = one_plane ? launch_chained(nchw_to_nhwc_kernel<false>, grid, dim3(256), smem, stream, x + b0 * Cin * H * W, xt,
                                                   (uint32_t)Cin, (uint32_t)C, (uint32_t)H, (uint32_t)W, rows, 1u, 1u, (uint32_t)b0,
                                                   (uint32_t)batches)
                                  : launch_chained(nchw_to_nhwc_kernel<true>, grid, dim3(256), smem, stream, x + b0 * Cin * H * W, xt,
                                                   (uint32_t)Cin, (uint32_t)C, (uint32_t)H, (uint32_t)W, rows, plan.sh, plan.sw,
                                                   (uint32_t)b0, (uint32_t)batches);
        if (e != cudaSuccess) return e;
        count_launch();
    }
    return cudaSuccess;
}

cudaError_t launch_conv_direct(const uint8_t *xt, const ConvDirectPlan &plan, uint64_t batches, uint64_t Cin, uint64_t H, uint64_t W,
                               uint64_t Cout, uint64_t kh, uint64_t kw, uint64_t ph, uint64_t pw, uint64_t Ho, uint64_t Wo,
                               const Epilogue &epi, void *out, bool nhwc_out, uint32_t *status, int sms, cudaStream_t stream, bool nchw_in)
{
    DirectGeom g;
    g.nhwc_out = nhwc_out ? 1u : 0u;
    g.gather = nchw_in ? 1u : 0u;
    g.Cin = (uint32_t)Cin;
    g.H = (uint32_t)H;
    g.W = (uint32_t)W;
    if (nchw_in && !conv_direct_gather_ok(plan, Cin, kh, kw, ph, pw, W, Wo, xt)) return cudaErrorInvalidConfiguration;
    g.B = (uint32_t)batches;
    g.Ho = (uint32_t)Ho;
    g.Wo = (uint32_t)Wo;
    const RegionGeom rg = region_geom(kh, kw, ph, pw, plan.sh, plan.sw, Wo);
    if (!rg.ok) return cudaErrorInvalidConfiguration;
    g.P = rg.P;
    g.rpt = rg.rpt;
    g.sh = plan.sh;
    g.sw = plan.sw;
    g.plane_mask = rg.plane_mask;
    g.dy_min = rg.dy_min;
    g.dx_min = rg.dx_min;
    g.rows_box = rg.rows_box;
    g.plane_bytes = rg.plane_bytes;
    g.tiles_per_image = (uint32_t)((Ho + g.rpt - 1) / g.rpt);
    if ((uint64_t)g.tiles_per_image * batches >= (1ull << 31)) return cudaErrorInvalidConfiguration;
    g.tiles = g.tiles_per_image * g.B;
    g.kh = (uint32_t)kh;
    g.kw = (uint32_t)kw;
    g.ph = (uint32_t)ph;
    g.pw = (uint32_t)pw;
    const uint64_t Cp = padded_channels(Cin);
    g.cchunks = (uint32_t)(Cp / CCH);
    g.CoutTotal = (uint32_t)Cout;
    g.stage_bytes = rg.stage_bytes;
    // the input as {channel, x, y, image, plane}; a box is 64 channels of the rows of one plane a tile touches, P pixels wide
    alignas(64) CUtensorMap mx;
    const uint64_t Hp = (H + plan.sh - 1) / plan.sh, Wp = (W + plan.sw - 1) / plan.sw;
    cuuint64_t dims[5] = {(cuuint64_t)Cp, (cuuint64_t)Wp, (cuuint64_t)Hp, (cuuint64_t)batches, (cuuint64_t)(plan.sh * plan.sw)};
    cuuint64_t strides[4] = {(cuuint64_t)Cp, (cuuint64_t)(Wp * Cp), (cuuint64_t)(Hp * Wp * Cp), (cuuint64_t)(batches * Hp * Wp * Cp)};
    cuuint32_t box[5] = {(cuuint32_t)CCH, g.P, g.rows_box, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    if (!nchw_in) {   // (with an NCHW input the kernel reads through plain pointers and the map stays unused)
        CUresult r = encode_fn()(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, const_cast<uint8_t *>(xt), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    } else {
        memset(&mx, 0, sizeof(mx));
    }
    const size_t esize = epi.out_mode == LTQ_OUT_U8 ? 1 : 4, plane = (size_t)Ho * Wo;
    // one launch per block of output channels (each reads the input tiles again, out of L2)
    for (uint32_t i = 0; i < plan.blocks; i++) {
        g.Cout = plan.nb[i];
        g.CoutValid = plan.valid[i];
        g.Npad = g.Cout + EXTRA;
        const uint32_t scr = nchw_in ? gather_scratch_bytes(g.rows_box, W) : 0u;
        g.stages = MAX_STAGES;
        while (g.stages > 2 && direct_smem(g.stages, g.stage_bytes, g.kh * g.kw * g.cchunks, g.Npad, scr) > SMEM_BUDGET) g.stages--;
        if (direct_smem(g.stages, g.stage_bytes, g.kh * g.kw * g.cchunks, g.Npad, scr) > SMEM_BUDGET) return cudaErrorInvalidConfiguration;
        Epilogue e = epi;                       // the block's own channel sums and biases
        e.bsum = epi.bsum + plan.cout0[i];
        if (epi.bias) e.bias = epi.bias + plan.cout0[i];
        void *o = static_cast<uint8_t *>(out) + (size_t)plan.cout0[i] * (nhwc_out ? 1 : plane) * esize;
        const CUtensorMap &mw = *reinterpret_cast<const CUtensorMap *>(plan.maps[i].opaque);
        cudaError_t ce;
        switch (epi.out_mode) {
            case LTQ_OUT_U8: ce = launch_direct<0>(mx, mw, g, e, o, status, sms, stream, nchw_in ? xt : nullptr); break;
            case LTQ_OUT_F32: ce = launch_direct<1>(mx, mw, g, e, o, status, sms, stream, nchw_in ? xt : nullptr); break;
            default: ce = launch_direct<2>(mx, mw, g, e, o, status, sms, stream, nchw_in ? xt : nullptr);
        }
        if (ce != cudaSuccess) return ce;
    }
    return cudaSuccess;
}

}  // namespace ltq
