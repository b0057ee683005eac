// Skinny (M <= 16) quantized linear: out[M,N] = epilogue(x[M,K] . W[N,K]^T).  Decode-like shapes are bound by reading
// the weight matrix once from HBM (N*K bytes against M*N*K MACs), so the kernel is organised around that stream:
//
//  * the whole activation block (<= 16 rows) is staged once per CTA in shared memory, rows padded so that 16-byte
//    reads by a quarter warp hit distinct banks;
//  * a CTA takes units of 8 weight rows; its 8 warps split K in interleaved 64-byte pieces, each lane issuing a batch of
//    independent 16-byte streaming loads (no L1 allocation) before any math, so every SM keeps tens of KB in flight;
//  * the math is warp-level mma.sync m16n8k32 u8 x u8 -> s32 with the activation rows as the 16-row operand and the 8
//    weight rows as the 8-column operand.  K is consumed in a permuted order inside each 64-byte piece (the sum over K
//    does not depend on order), which lets each lane feed the fragments straight from its 16-byte load;
//  * the 8 per-warp partial 16x8 tiles are combined through shared memory and the fused epilogue
//    (l-ten/math_fns.cpp:1469-1474) writes the outputs.
#include "ltq_common.cuh"
#include "ltq_gemv.cuh"

namespace ltq {

namespace {

constexpr int WARPS = 8;
constexpr int UNIT_ROWS = 8;       // weight rows per unit = mma N
constexpr int PIECE = 64;          // bytes of K a warp covers per step (4 lanes x 16 B per weight row)
constexpr int BATCH = 8;           // steps whose loads are issued together

__device__ __forceinline__ void mma_u8(int32_t (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const uint8_t *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

}  // namespace

// HI: rows 8..15 of the activation block are populated (M > 8).
template <bool HI, int OUT>
__global__ void __launch_bounds__(WARPS * 32)
gemv_kernel(const uint8_t *__restrict__ x, const uint8_t *__restrict__ W, uint32_t M, uint32_t N, uint32_t K,
            uint32_t x_pitch, Epilogue epi, void *__restrict__ out)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int XROWS = HI ? 16 : 8;
    uint8_t *xs = smem;                                                         // [XROWS][x_pitch]
    int32_t *red = reinterpret_cast<int32_t *>(smem + (size_t)XROWS * x_pitch);  // [2][WARPS][128]

    // Stage activations, zero-filling rows >= M and the K tail up to the pitch.
    for (uint32_t i = threadIdx.x; i < XROWS * (x_pitch / 16); i += blockDim.x) {
        const uint32_t r = i / (x_pitch / 16), c = (i % (x_pitch / 16)) * 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < M && c < K) v = *reinterpret_cast<const uint4 *>(x + (size_t)r * K + c);
        *reinterpret_cast<uint4 *>(xs + (size_t)r * x_pitch + c) = v;
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const EpilogueConsts c = epilogue_consts(epi);
    const bool relu = epi.flags & LTQ_FLAG_RELU, sat = epi.flags & LTQ_FLAG_SATURATE;
    const uint32_t units = (N + UNIT_ROWS - 1) / UNIT_ROWS;
    const uint8_t *xlo = xs + (size_t)g * x_pitch + 16 * t;
    const uint8_t *xhi = xs + (size_t)(g + 8) * x_pitch + 16 * t;

    int buf = 0;
    for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x, buf ^= 1) {
        const uint32_t n = unit * UNIT_ROWS + g;
        const bool row_ok = n < N;
        const uint8_t *wrow = W + (size_t)(row_ok ? n : 0) * K + 16 * t;
        int32_t acc[4] = {0, 0, 0, 0};
        for (uint32_t k0 = warp * PIECE; k0 < K; k0 += WARPS * PIECE * BATCH) {
            uint4 w[BATCH];
#pragma unroll
            for (int u = 0; u < BATCH; u++) {
                const uint32_t k = k0 + u * WARPS * PIECE;
                // K is a multiple of 16, so a lane's 16 bytes are either wholly inside the row or wholly outside.
                w[u] = (row_ok && k + 16 * t < K) ? ld_stream(wrow + k) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < BATCH; u++) {
                const uint32_t k = k0 + u * WARPS * PIECE;
                if (k < K) {
                    const uint4 lo = *reinterpret_cast<const uint4 *>(xlo + k);
                    uint4 hi = make_uint4(0, 0, 0, 0);
                    if (HI) hi = *reinterpret_cast<const uint4 *>(xhi + k);
                    mma_u8(acc, lo.x, hi.x, lo.y, hi.y, w[u].x, w[u].y);
                    mma_u8(acc, lo.z, hi.z, lo.w, hi.w, w[u].z, w[u].w);
                }
            }
        }
        // Fragment -> [row][col] of the 16x8 partial tile: c0 (g,2t) c1 (g,2t+1) c2 (g+8,2t) c3 (g+8,2t+1).
        int32_t *mine = red + (buf * WARPS + warp) * 128;
        mine[g * 8 + 2 * t] = acc[0];
        mine[g * 8 + 2 * t + 1] = acc[1];
        if (HI) {
            mine[(g + 8) * 8 + 2 * t] = acc[2];
            mine[(g + 8) * 8 + 2 * t + 1] = acc[3];
        }
        __syncthreads();  // partials of this unit visible; the other buffer is free again after the previous sync
        if (threadIdx.x < XROWS * 8) {
            const uint32_t row = threadIdx.x >> 3, col = unit * UNIT_ROWS + (threadIdx.x & 7);
            if (row < M && col < N) {
                uint32_t raw = 0;
#pragma unroll
                for (int w8 = 0; w8 < WARPS; w8++) raw += (uint32_t)red[(buf * WARPS + w8) * 128 + threadIdx.x];
                const int32_t a = epilogue_acc(raw, epilogue_row_term(epi, c, row), epilogue_col_term(epi, c, col), relu);
                const size_t o = (size_t)row * N + col;
                if (OUT == 0)
                    static_cast<uint8_t *>(out)[o] = epilogue_u8(a, c, sat);
                else if (OUT == 1)
                    static_cast<float *>(out)[o] = epilogue_f32(a, c);
                else
                    static_cast<int32_t *>(out)[o] = a;
            }
        }
    }
}

namespace {

uint32_t pitch_for(uint64_t K)
{
    // Rows 128-byte aligned plus 64: consecutive rows start 16 banks apart, so the two rows a quarter warp reads in one
    // 16-byte access never collide.
    return (uint32_t)(((K + 127) / 128) * 128 + 64);
}

size_t smem_for(uint64_t M, uint64_t K)
{
    return (size_t)(M > 8 ? 16 : 8) * pitch_for(K) + 2 * WARPS * 128 * sizeof(int32_t);
}

template <bool HI, int OUT>
cudaError_t launch_t(const uint8_t *x, const uint8_t *W, uint64_t M, uint64_t N, uint64_t K, const Epilogue &epi,
                     void *out, int sms, cudaStream_t stream)
{
    const size_t smem = smem_for(M, K);
    // Attribute and occupancy are looked up once per (device, shared-memory size) and reused: the kernel runs for a few
    // microseconds, so two runtime queries per launch would cost more than the launch itself.
    struct Cached { size_t smem = 0; int per_sm = 0; };
    static Cached cache[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (cache[dev].smem != smem || cache[dev].per_sm == 0) {
        e = cudaFuncSetAttribute(gemv_kernel<HI, OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        int q = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, gemv_kernel<HI, OUT>, WARPS * 32, smem);
        if (e != cudaSuccess) return e;
        if (q < 1) return cudaErrorInvalidConfiguration;
        cache[dev].smem = smem;
        cache[dev].per_sm = q > 4 ? 4 : q;
    }
    const int per_sm = cache[dev].per_sm;
    const uint64_t units = (N + UNIT_ROWS - 1) / UNIT_ROWS;
    uint64_t grid = (uint64_t)sms * per_sm;
    if (grid > units) grid = units;
    gemv_kernel<HI, OUT><<<(unsigned)grid, WARPS * 32, smem, stream>>>(x, W, (uint32_t)M, (uint32_t)N, (uint32_t)K,
                                                                       pitch_for(K), epi, out);
    count_launch();
    return cudaGetLastError();
}

template <bool HI>
cudaError_t launch_o(const uint8_t *x, const uint8_t *W, uint64_t M, uint64_t N, uint64_t K, const Epilogue &epi,
                     void *out, int sms, cudaStream_t stream)
{
    switch (epi.out_mode) {
        case LTQ_OUT_U8: return launch_t<HI, 0>(x, W, M, N, K, epi, out, sms, stream);
        case LTQ_OUT_F32: return launch_t<HI, 1>(x, W, M, N, K, epi, out, sms, stream);
        default: return launch_t<HI, 2>(x, W, M, N, K, epi, out, sms, stream);
    }
}

}  // namespace

bool gemv_shape_ok(uint64_t M, uint64_t N, uint64_t K, const void *x, const void *W)
{
    return M >= 1 && M <= 16 && N >= 1 && N < (1ull << 31) && K >= 16 && K % 16 == 0 &&
           smem_for(M, K) <= 200 * 1024 && (((uintptr_t)x & 15) == 0) && (((uintptr_t)W & 15) == 0);
}

cudaError_t launch_gemv(const uint8_t *x, const uint8_t *W, uint64_t M, uint64_t N, uint64_t K, const Epilogue &epi,
                        void *out, int sms, cudaStream_t stream)
{
    return M > 8 ? launch_o<true>(x, W, M, N, K, epi, out, sms, stream)
                 : launch_o<false>(x, W, M, N, K, epi, out, sms, stream);
}

}  // namespace ltq
