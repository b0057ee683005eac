// Quantisation helpers on the device: min/max, qparams, float->uint8 / int32, uint8->float, and the operand sums the
// GEMM epilogue folds in.  All of them are single-pass, HBM-bound streaming kernels: 16-byte loads, grids sized in
// multiples of the SM count, no shared-memory staging needed.
//
// Arithmetic follows l-ten/utils.cpp:198-286 operation for operation (IEEE divide, separate add, clamp, round half away
// from zero); the file is compiled with -fmad=false so nothing is contracted.
#include "ltq_common.cuh"
#include "ltq_quant.cuh"
#include "ltq_ptx.cuh"

namespace ltq {

static int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// ---- min / max ------------------------------------------------------------------------------------------------------
// Order-preserving map float -> uint32 so that atomicMin/atomicMax on integers order floats.
__device__ __forceinline__ uint32_t f2ord(float f)
{
    uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float ord2f(uint32_t u)
{
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u);
}

// slot[0] = min over ord(x); slot[1] = min over ~ord(x) (i.e. the max, complemented) so both start from 0xFFFFFFFF and a
// single byte-fill initialises them.
__global__ void __launch_bounds__(256) minmax_reduce_kernel(const float *__restrict__ x, uint64_t len, uint32_t *slot)
{
    griddep_launch_dependents();   // the decoding kernel behind may be scheduled; it waits for this grid to finish
    // fminf / fmaxf return the other operand when one is NaN: NaNs never replace a minimum or maximum, as in the
    // reference's compare-and-replace loop.  +inf / -inf as seeds: lo > hi at the end means nothing was comparable.
    float lo = __int_as_float(0x7F800000), hi = __int_as_float(0xFF800000);
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    // 16-byte body when the base pointer allows it, scalar head/tail otherwise.
    const uint64_t mis = ((16 - ((uintptr_t)x & 15)) & 15) / 4;
    const uint64_t head = mis < len ? mis : len;
    const uint64_t nvec = (len - head) / 4;
    const float4 *xv = reinterpret_cast<const float4 *>(x + head);
    auto upd = [&](float v) {
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    };
    auto upd4 = [&](const float4 &v) {
        upd(v.x); upd(v.y); upd(v.z); upd(v.w);
    };
    // four independent 16-byte loads per thread before any arithmetic (the pass lives on bytes in flight), then the rest
    uint64_t i = tid;
    for (; i + 3 * nth < nvec; i += 4 * nth) {
        const float4 a = __ldg(xv + i), b = __ldg(xv + i + nth), c = __ldg(xv + i + 2 * nth), d = __ldg(xv + i + 3 * nth);
        upd4(a); upd4(b); upd4(c); upd4(d);
    }
    for (; i < nvec; i += nth) upd4(__ldg(xv + i));
    for (uint64_t k = tid; k < head; k += nth) upd(x[k]);
    for (uint64_t k = head + nvec * 4 + tid; k < len; k += nth) upd(x[k]);

    for (int o = 16; o; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, o));
    }
    __shared__ float slo[8], shi[8];
    if ((threadIdx.x & 31) == 0) {
        slo[threadIdx.x >> 5] = lo;
        shi[threadIdx.x >> 5] = hi;
    }
    __syncthreads();
    if (threadIdx.x < 8) {
        lo = slo[threadIdx.x];
        hi = shi[threadIdx.x];
        for (int o = 4; o; o >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xFFu, lo, o));
            hi = fmaxf(hi, __shfl_xor_sync(0xFFu, hi, o));
        }
        // Everything above only read x, which was complete before the kernel that seeds the slots started; the slots
        // themselves are ready once that kernel has finished.
        griddep_wait();
        if (threadIdx.x == 0 && lo <= hi) {   // something comparable was seen by this CTA
            atomicMin(slot, f2ord(lo));
            atomicMin(slot + 1, ~f2ord(hi));
        }
    }
}

// Seeds the two slots.  A kernel rather than a memset so that the reduction can be its programmatic dependent and stream
// the data while this one is still being scheduled.
__global__ void minmax_seed_kernel(uint32_t *slot)
{
    griddep_launch_dependents();
    slot[0] = 0xFFFFFFFFu;
    slot[1] = 0xFFFFFFFFu;
}

// Decodes the two slots in place into floats {min, max}.  The reference seeds both with data[0] and replaces them only
// when a comparison is true: an input with no comparable element (all NaN) keeps the seed, and so does an input whose
// first element is NaN, whatever follows (every comparison with the NaN seed is false).
__global__ void minmax_decode_kernel(uint32_t *slot, const float *x)
{
    griddep_wait();                // launched as a programmatic dependent of the reduction
    uint32_t a = slot[0], b = slot[1];
    const float seed = x[0];
    const bool seed_nan = seed != seed;
    float mn = (a == 0xFFFFFFFFu || seed_nan) ? seed : ord2f(a);
    float mx = (b == 0xFFFFFFFFu || seed_nan) ? seed : ord2f(~b);
    reinterpret_cast<float *>(slot)[0] = mn;
    reinterpret_cast<float *>(slot)[1] = mx;
}

cudaError_t launch_min_max(const float *data, uint64_t len, float *minmax, cudaStream_t stream)
{
    uint64_t want = (len / 4 + 255) / 256;
    uint64_t cap = (uint64_t)sm_count() * 8;
    int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    // seed (ordinary launch: starts after everything before it in the stream) -> reduction -> decoding, the last two as
    // programmatic dependents: one launch latency instead of three
    minmax_seed_kernel<<<1, 1, 0, stream>>>(reinterpret_cast<uint32_t *>(minmax));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    e = launch_chained(minmax_reduce_kernel, dim3(blocks), dim3(256), 0, stream, data, len, reinterpret_cast<uint32_t *>(minmax));
    if (e != cudaSuccess) return e;
    e = launch_chained(minmax_decode_kernel, dim3(1), dim3(1), 0, stream, reinterpret_cast<uint32_t *>(minmax), data);
    count_launch(3);
    return e;
}

// ---- qparams from min/max, l-ten/utils.cpp:266-286 -------------------------------------------------------------
__global__ void qparams_kernel(const float *minmax, ltq_qparams *qp)
{
    float mn = fminf(minmax[0], 0.f);
    float mx = fmaxf(minmax[1], 0.f);
    float scale = __fdiv_rn(__fsub_rn(mx, mn), 255.f);
    float zp = __fsub_rn(0.f, __fdiv_rn(mn, scale));
    qp->scale = scale;
    // An all-zero tensor gives scale 0 and zp NaN in the reference (undefined cast); 0 is written here.
    qp->zero_point = (zp == zp) ? (uint8_t)(int)roundf(zp) : (uint8_t)0;
}

cudaError_t launch_qparams_from_minmax(const float *minmax, ltq_qparams *qp, cudaStream_t stream)
{
    qparams_kernel<<<1, 1, 0, stream>>>(minmax, qp);
    count_launch();
    return cudaGetLastError();
}

// ---- Quantize / Dequantize, l-ten/utils.cpp:228-264 -------------------------------------------------------------
// (the uint8 rounding helpers live in ltq_quant.cuh: the fused MLP kernel quantises its input with them too)
__device__ __forceinline__ int32_t quant_i32(float x, float scale, float zpf)
{
    float v = __fadd_rn(zpf, __fdiv_rn(x, scale));
    // std::max((float)INT_MIN, std::min((float)INT_MAX, v)); (float)INT_MAX == 2^31.
    float t = (v < 2147483648.f) ? v : 2147483648.f;
    t = (-2147483648.f < t) ? t : -2147483648.f;
    float r = roundf(t);
    // (int)2^31 is out of range for the reference's conversion, which then yields INT_MIN on x86; NaN likewise.
    if (!(r < 2147483648.f)) return INT32_MIN;
    return (int32_t)r;
}

__global__ void __launch_bounds__(256) quantize_u8_kernel(const float *__restrict__ x, uint8_t *__restrict__ q,
                                                          uint64_t len, float scale, float zpf)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    const bool aligned = (((uintptr_t)x & 15) == 0) && (((uintptr_t)q & 3) == 0);
    uint64_t nvec = aligned ? len / 4 : 0;
    const float inv = quant_screen_inv(scale);
    const float4 *xv = reinterpret_cast<const float4 *>(x);
    uint32_t *qv = reinterpret_cast<uint32_t *>(q);
    uint64_t i = tid;
    for (; i + 3 * nth < nvec; i += 4 * nth) {   // four loads in flight per thread, as in quantize_rows_kernel
        const float4 a = __ldcs(xv + i), b = __ldcs(xv + i + nth), c = __ldcs(xv + i + 2 * nth), d = __ldcs(xv + i + 3 * nth);
        qv[i] = quant4_u8(a, scale, zpf, inv);
        qv[i + nth] = quant4_u8(b, scale, zpf, inv);
        qv[i + 2 * nth] = quant4_u8(c, scale, zpf, inv);
        qv[i + 3 * nth] = quant4_u8(d, scale, zpf, inv);
    }
    for (; i < nvec; i += nth) qv[i] = quant4_u8(__ldcs(xv + i), scale, zpf, inv);
    for (uint64_t i = nvec * 4 + tid; i < len; i += nth) q[i] = (uint8_t)quant_u8(x[i], scale, zpf, inv);
}

__global__ void __launch_bounds__(256) quantize_i32_kernel(const float *__restrict__ x, int32_t *__restrict__ q,
                                                           uint64_t len, float scale, float zpf)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < len; i += nth) q[i] = quant_i32(x[i], scale, zpf);
}

__global__ void __launch_bounds__(256) dequantize_kernel(float *__restrict__ x, const uint8_t *__restrict__ q,
                                                         uint64_t len, float scale, int zp)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    const bool aligned = (((uintptr_t)x & 15) == 0) && (((uintptr_t)q & 3) == 0);
    uint64_t nvec = aligned ? len / 4 : 0;
    auto widen = [&](uint32_t p) {
        float4 v;
        v.x = __fmul_rn(scale, (float)((int)(p & 0xFF) - zp));
        v.y = __fmul_rn(scale, (float)((int)((p >> 8) & 0xFF) - zp));
        v.z = __fmul_rn(scale, (float)((int)((p >> 16) & 0xFF) - zp));
        v.w = __fmul_rn(scale, (float)((int)(p >> 24) - zp));
        return v;
    };
    const uint32_t *qv = reinterpret_cast<const uint32_t *>(q);
    float4 *xv = reinterpret_cast<float4 *>(x);
    uint64_t i = tid;
    for (; i + 3 * nth < nvec; i += 4 * nth) {   // loads first: four words in flight per thread
        const uint32_t a = __ldcs(qv + i), b = __ldcs(qv + i + nth), c = __ldcs(qv + i + 2 * nth), d = __ldcs(qv + i + 3 * nth);
        xv[i] = widen(a);
        xv[i + nth] = widen(b);
        xv[i + 2 * nth] = widen(c);
        xv[i + 3 * nth] = widen(d);
    }
    for (; i < nvec; i += nth) xv[i] = widen(__ldcs(qv + i));
    for (uint64_t i = nvec * 4 + tid; i < len; i += nth) x[i] = __fmul_rn(scale, (float)((int)q[i] - zp));
}

static int stream_grid(uint64_t work_items)
{
    uint64_t want = (work_items + 255) / 256;
    uint64_t cap = (uint64_t)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

cudaError_t launch_quantize_u8(const float *x, uint8_t *q, uint64_t len, const ltq_qparams &qp, cudaStream_t stream)
{
    quantize_u8_kernel<<<stream_grid(len / 4 + 1), 256, 0, stream>>>(x, q, len, qp.scale, (float)(int)qp.zero_point);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_quantize_i32(const float *x, int32_t *q, uint64_t len, const ltq_qparams &qp, cudaStream_t stream)
{
    quantize_i32_kernel<<<stream_grid(len), 256, 0, stream>>>(x, q, len, qp.scale, (float)(int)qp.zero_point);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_dequantize(float *x, const uint8_t *q, uint64_t len, const ltq_qparams &qp, cudaStream_t stream)
{
    dequantize_kernel<<<stream_grid(len / 4 + 1), 256, 0, stream>>>(x, q, len, qp.scale, (int)qp.zero_point);
    count_launch();
    return cudaGetLastError();
}

// ---- activation quantise + row sums -------------------------------------------------------------------------------
// TPR threads cooperate on one row (TPR = 32: a warp; 64: two warps; 256: the whole CTA).  Reads fp32 once, writes uint8 once
// and one int32 per row: 5 bytes per element of HBM traffic, the minimum for this step.
// BACK_TO_FRONT: rows are visited last to first (see the loop below).
template <int TPR, bool BACK_TO_FRONT>
__global__ void __launch_bounds__(256, 8) quantize_rows_kernel(const float *__restrict__ x, uint64_t M, uint64_t K,
                                                            float scale_h, float zpf_h,
                                                            const ltq_qparams *__restrict__ qp_dev,
                                                            uint8_t *__restrict__ q, int32_t *__restrict__ asum)
{
    // launched as a programmatic dependent: release the kernel behind, then wait for the one in front
    griddep_launch_dependents();
    griddep_wait();
    float scale = scale_h, zpf = zpf_h;
    if (qp_dev) {
        scale = qp_dev->scale;
        zpf = (float)(int)qp_dev->zero_point;
    }
    const float inv = quant_screen_inv(scale);
    constexpr int ROWS_PER_CTA = 256 / TPR;
    const int lane = threadIdx.x % TPR;
    const int sub = threadIdx.x / TPR;
    __shared__ int32_t warp_part[2][8];
    int par = 0;
    // BACK_TO_FRONT is chosen when the parameters come from device memory: as a rule they were computed from this very
    // tensor a moment ago (GetMinMax, then ComputeQuantizationParams), that pass went through the rows front to back,
    // and its last rows are what L2 still holds; going back to front reads those from L2 instead of HBM.
    for (uint64_t slot = (uint64_t)blockIdx.x * ROWS_PER_CTA + sub; ; slot += (uint64_t)gridDim.x * ROWS_PER_CTA) {
        // All threads that share a row leave together (slot is uniform among them): the CTA, a pair of warps, or a warp.
        if (slot >= M) break;
        const uint64_t row = BACK_TO_FRONT ? M - 1 - slot : slot;
        const float *xr = x + row * K;
        uint8_t *qr = q + row * K;
        const bool aligned = (((uintptr_t)xr & 15) == 0) && (((uintptr_t)qr & 3) == 0);
        const uint32_t nvec = aligned ? (uint32_t)(K / 4) : 0u;
        uint32_t s = 0;
        const float4 *xv = reinterpret_cast<const float4 *>(xr);
        uint32_t *qv = reinterpret_cast<uint32_t *>(qr);
        // four independent 16-byte loads per thread before any arithmetic: the kernel lives on bytes in flight.  Whole
        // blocks of 4 x TPR vectors run without per-vector bounds checks (eight guards per pass were a tenth of the
        // kernel's instructions); the remainder goes one vector at a time.
        uint32_t i0 = lane;
        for (; i0 + 3u * TPR < nvec; i0 += 4 * TPR) {
            const float4 a = __ldcs(xv + i0), b = __ldcs(xv + i0 + TPR), c = __ldcs(xv + i0 + 2 * TPR), d = __ldcs(xv + i0 + 3 * TPR);
            const uint32_t pa = quant4_u8(a, scale, zpf, inv), pb = quant4_u8(b, scale, zpf, inv);
            const uint32_t pc = quant4_u8(c, scale, zpf, inv), pd = quant4_u8(d, scale, zpf, inv);
            s = __dp4a(pa, 0x01010101u, s);
            s = __dp4a(pb, 0x01010101u, s);
            s = __dp4a(pc, 0x01010101u, s);
            s = __dp4a(pd, 0x01010101u, s);
            qv[i0] = pa;
            qv[i0 + TPR] = pb;
            qv[i0 + 2 * TPR] = pc;
            qv[i0 + 3 * TPR] = pd;
        }
        for (; i0 < nvec; i0 += TPR) {
            const uint32_t p = quant4_u8(__ldcs(xv + i0), scale, zpf, inv);  // read once: first out of L2
            s = __dp4a(p, 0x01010101u, s);
            qv[i0] = p;
        }
        for (uint64_t i = (uint64_t)nvec * 4 + lane; i < K; i += TPR) {
            uint32_t a = quant_u8(xr[i], scale, zpf, inv);
            s += a;
            qr[i] = (uint8_t)a;
        }
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        if (TPR == 32) {
            if (lane == 0) asum[row] = (int32_t)s;
        } else if (TPR == 64) {
            // two warps per row: they meet on a barrier of their own (ids 1-4; 0 is the CTA-wide one), the other three
            // pairs of the CTA run on.  Partial sums alternate between two buffers, so one barrier per row is enough: a
            // warp can only write a buffer again after the barrier of the row in between, which its partner reaches
            // after it has read.
            if ((threadIdx.x & 31) == 0) warp_part[par][threadIdx.x >> 5] = (int32_t)s;
            switch (sub) {   // literal ids: with a register operand the compiler reserves all sixteen barriers
                case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
                case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
                case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
                default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
            }
            if (lane == 0) asum[row] = warp_part[par][2 * sub] + warp_part[par][2 * sub + 1];
            par ^= 1;
        } else {
            if ((threadIdx.x & 31) == 0) warp_part[par][threadIdx.x >> 5] = (int32_t)s;
            __syncthreads();
            if (threadIdx.x == 0) {
                int32_t t = 0;
                for (int w = 0; w < 8; w++) t += warp_part[par][w];
                asum[row] = t;
            }
            par ^= 1;   // the next row writes the other buffer: one barrier per row
        }
    }
}

cudaError_t launch_quantize_rows(const float *x, uint64_t M, uint64_t K, const ltq_qparams *qp_host,
                                 const ltq_qparams *qp_dev, uint8_t *q, int32_t *asum, cudaStream_t stream)
{
    float scale = qp_host ? qp_host->scale : 0.f;
    float zpf = qp_host ? (float)(int)qp_host->zero_point : 0.f;
    const uint64_t cap = (uint64_t)sm_count() * 8;
    cudaError_t e;
    if (K <= 2048) {
        uint64_t want = (M + 7) / 8;
        int blocks = (int)(want > cap ? cap : want);
        e = qp_dev ? launch_chained(quantize_rows_kernel<32, true>, dim3(blocks), dim3(256), 0, stream, x, M, K, scale, zpf, qp_dev, q, asum)
                   : launch_chained(quantize_rows_kernel<32, false>, dim3(blocks), dim3(256), 0, stream, x, M, K, scale, zpf, qp_dev, q, asum);
    } else if (qp_dev && M * K <= (16ull << 20) && K <= 16384 && (M + 3) / 4 >= (uint64_t)sm_count()) {
        // Device parameters and at most 64 MB of fp32: the min / max pass that produced the parameters has left the
        // tensor in L2, the loads return quickly and the work per row (addresses, the sum across lanes, the barrier)
        // is what counts.  Two warps per row pay it once per four passes of the main loop on a 4096-wide row, a whole CTA
        // on the row once per pass, and a barrier only stops the two warps it concerns.  Measured on 4096 x 4096 after
        // GetMinMax: 30.3 us for the whole dynamic step against 32.3 us; on a tensor that comes from HBM the whole-CTA
        // form is the faster one (16.9 us against 18.3 us alone), so it stays the choice everywhere else.
        uint64_t want = (M + 3) / 4;
        int blocks = (int)(want > cap ? cap : want);
        e = qp_dev ? launch_chained(quantize_rows_kernel<64, true>, dim3(blocks), dim3(256), 0, stream, x, M, K, scale, zpf, qp_dev, q, asum)
                   : launch_chained(quantize_rows_kernel<64, false>, dim3(blocks), dim3(256), 0, stream, x, M, K, scale, zpf, qp_dev, q, asum);
    } else {
        int blocks = (int)(M > cap ? cap : M);
        e = qp_dev ? launch_chained(quantize_rows_kernel<256, true>, dim3(blocks), dim3(256), 0, stream, x, M, K, scale, zpf, qp_dev, q, asum)
                   : launch_chained(quantize_rows_kernel<256, false>, dim3(blocks), dim3(256), 0, stream, x, M, K, scale, zpf, qp_dev, q, asum);
    }
    count_launch();
    return e;
}

// ---- operand sums ---------------------------------------------------------------------------------------------------
// One warp per row, 16-byte loads, bytes summed four at a time with dp4a against 0x01010101.
__global__ void __launch_bounds__(256) row_sums_kernel(const uint8_t *__restrict__ m, uint64_t rows, uint64_t cols,
                                                       int32_t *__restrict__ sums)
{
    griddep_launch_dependents();  // launched as a programmatic dependent, see launch_chained
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t r = warp; r < rows; r += nwarps) {
        const uint8_t *p = m + r * cols;
        const uint64_t mis = (16 - ((uintptr_t)p & 15)) & 15;
        const uint64_t head = mis < cols ? mis : cols;
        const uint64_t nvec = (cols - head) / 16;
        const uint4 *pv = reinterpret_cast<const uint4 *>(p + head);
        uint32_t s = 0;
        for (uint64_t i = lane; i < nvec; i += 32) {
            uint4 v = __ldg(pv + i);
            s = __dp4a(v.x, 0x01010101u, s);
            s = __dp4a(v.y, 0x01010101u, s);
            s = __dp4a(v.z, 0x01010101u, s);
            s = __dp4a(v.w, 0x01010101u, s);
        }
        for (uint64_t i = lane; i < head; i += 32) s += p[i];
        for (uint64_t i = head + nvec * 16 + lane; i < cols; i += 32) s += p[i];
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        if (lane == 0) sums[r] = (int32_t)s;
    }
}

// Sums down the columns of a row-major matrix: thread per column, coalesced across threads, rows split over
// blockIdx.y with an atomic combine (sums must be zeroed first).
__global__ void __launch_bounds__(256) col_sums_kernel(const uint8_t *__restrict__ m, uint64_t rows, uint64_t cols,
                                                       int32_t *__restrict__ sums)
{
    const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    int32_t s = 0;
    for (uint64_t r = blockIdx.y; r < rows; r += gridDim.y) s += m[r * cols + c];
    atomicAdd(sums + c, s);
}

__global__ void __launch_bounds__(256) scale_i32_kernel(int32_t *v, uint64_t n, int32_t factor)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n; i += nth) v[i] = (int32_t)((uint32_t)v[i] * (uint32_t)factor);
}

// After an all-gather of column slices the output sits as [G][M][W bytes] (one plane per rank).  This puts it back into
// the row-major [M][G * W] the next layer reads: dst[m][g * W + w] = src[g][m][w].  16-byte copies when W allows.
__global__ void __launch_bounds__(256) interleave_blocks_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                                               uint64_t G, uint64_t M, uint64_t W)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nth = (uint64_t)gridDim.x * blockDim.x;
    if (W % 16 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
        const uint64_t wv = W / 16, total = G * M * wv;
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
        for (uint64_t i = tid; i < total; i += nth) {
            // walk the destination in order (coalesced stores); reads are contiguous runs of W bytes
            const uint64_t m = i / (G * wv), r = i % (G * wv), g = r / wv, w = r % wv;
            d4[i] = __ldg(s4 + (g * M + m) * wv + w);
        }
    } else {
        const uint64_t total = G * M * W;
        for (uint64_t i = tid; i < total; i += nth) {
            const uint64_t m = i / (G * W), r = i % (G * W), g = r / W, w = r % W;
            dst[i] = src[(g * M + m) * W + w];
        }
    }
}

cudaError_t launch_interleave_blocks(const void *src, void *dst, uint64_t G, uint64_t M, uint64_t W, cudaStream_t stream)
{
    const uint64_t work = G * M * ((W + 15) / 16);
    uint64_t want = (work + 255) / 256, cap = (uint64_t)sm_count() * 16;
    int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    interleave_blocks_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), G, M, W);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_row_sums(const uint8_t *m, uint64_t rows, uint64_t cols, int32_t *sums, cudaStream_t stream)
{
    uint64_t want = (rows + 7) / 8;
    uint64_t cap = (uint64_t)sm_count() * 8;
    int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    cudaError_t e = launch_chained(row_sums_kernel, dim3(blocks), dim3(256), 0, stream, m, rows, cols, sums);
    count_launch();
    return e;
}

cudaError_t launch_col_sums(const uint8_t *m, uint64_t rows, uint64_t cols, int32_t *sums, cudaStream_t stream)
{
    cudaError_t e = cudaMemsetAsync(sums, 0, cols * sizeof(int32_t), stream);
    if (e != cudaSuccess) return e;
    uint64_t bx = (cols + 255) / 256;
    uint64_t by = (uint64_t)sm_count() * 4 / bx;
    if (by < 1) by = 1;
    if (by > rows) by = rows ? rows : 1;
    if (by > 65535) by = 65535;
    dim3 grid((unsigned)bx, (unsigned)by);
    col_sums_kernel<<<grid, 256, 0, stream>>>(m, rows, cols, sums);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_scale_i32(int32_t *v, uint64_t n, int32_t factor, cudaStream_t stream)
{
    scale_i32_kernel<<<stream_grid(n), 256, 0, stream>>>(v, n, factor);
    count_launch();
    return cudaGetLastError();
}

}  // namespace ltq
