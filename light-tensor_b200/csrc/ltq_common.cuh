// Shared declarations for the ltq CUDA library: error plumbing, launch counting and the epilogue arithmetic that every
// GEMM kernel applies to its raw uint8 x uint8 int32 dot products.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <atomic>

#include "../../include/ltq.h"

namespace ltq {

// ---- host-side error state ---------------------------------------------------------------------------------------
void set_error(const char *fmt, ...);
extern std::atomic<uint64_t> g_launches;
inline void count_launch(uint64_t n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
// Name (with template arguments) of the GEMM kernel the calling thread launched last, for ltq_last_kernel().
void note_kernel(const char *fmt, ...);
inline const char *out_mode_name(int out_mode) { return out_mode == LTQ_OUT_U8 ? "u8" : (out_mode == LTQ_OUT_F32 ? "f32" : "i32"); }

#define LTQ_CUDA_TRY(expr)                                                                                   \
    do {                                                                                                     \
        cudaError_t e__ = (expr);                                                                            \
        if (e__ != cudaSuccess) {                                                                            \
            ::ltq::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__);   \
            return LTQ_ERR_CUDA;                                                                             \
        }                                                                                                    \
    } while (0)

#define LTQ_REQUIRE(cond, status, ...)        \
    do {                                      \
        if (!(cond)) {                        \
            ::ltq::set_error(__VA_ARGS__);    \
            return (status);                  \
        }                                     \
    } while (0)

// Makes `device` current for the lifetime of the guard and restores the caller's device afterwards (l-ten itself never
// calls cudaSetDevice, so the caller's current device must not move under it).
struct DeviceGuard {
    int prev = -1;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int device)
    {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) err = cudaSetDevice(device);
    }
    ~DeviceGuard()
    {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

#define LTQ_ENTER_DEVICE(device)                                                                             \
    ::ltq::DeviceGuard guard__(device);                                                                      \
    if (guard__.err != cudaSuccess) {                                                                        \
        ::ltq::set_error("cannot select CUDA device %d: %s", (device), cudaGetErrorString(guard__.err));     \
        return LTQ_ERR_CUDA;                                                                                 \
    }

// Launches `kernel` as a programmatic dependent of the kernel in front of it in the stream: its CTAs may become
// resident (and run their set-up) while that kernel is still finishing.  The kernel itself must execute
// griddepcontrol.wait before it touches anything the earlier kernel may have written, and griddepcontrol.launch_dependents
// to release the kernel behind it the same way (ltq_ptx.cuh).  After a kernel that never releases its dependents, or
// after anything that is not a kernel, this is an ordinary launch.
bool chained_launches_enabled();  // false when the environment variable LTQ_NO_CHAINED_LAUNCH is set (a debugging switch)
template <typename... P, typename... A>
inline cudaError_t launch_chained(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chained_launches_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// ---- epilogue ------------------------------------------------------------------------------------------------------
// Everything a kernel needs to turn raw = sum_k A[i,k]*B[j,k] into an output element.
//   acc = raw - zA*bsum[j] - zB*asum[i] + K*zA*zB (+ bias[j])            l-ten/math_fns.cpp:1433-1473
// in wrapping 32-bit arithmetic (the reference's int additions wrap the same way on its x86 build).
struct Epilogue {
    const int32_t *bsum;          // [N] raw sums over K of the B operand (weights for the FC layer)
    const int32_t *asum;          // [M] raw sums over K of the A operand (activations)
    const int32_t *bias;          // [N] or nullptr: added per output column (the reference's `bias[j]`)
    const int32_t *row_bias;      // [M] or nullptr: added per output row (Conv2d_q: one value per output channel)
    const ltq_qparams *qpA_dev;   // optional device-resident override of (sA, zA)
    float sA, sB, sC;
    int32_t zA, zB, zC;
    uint32_t K;
    int out_mode;                 // ltq_out_mode
    unsigned flags;               // LTQ_FLAG_RELU | LTQ_FLAG_SATURATE
    // Where results go.  Element (i, j) is written at index i*ldc + j of the kernel's `out` argument and of every
    // further destination (buffers of the same layout, e.g. the peer GPUs' copies of a column-sharded output: the
    // epilogue then IS the all-gather).  ldc = 0 means a dense [M, N] output.
    uint64_t ldc;
    void *more_out[LTQ_MAX_DESTS - 1];
    int n_more;
    int staged;                   // set by a launcher that gave its kernel a PeerStage area (see below)
    // `out` is an NVLink multicast address: one store reaches the buffer of every GPU bound to it (this GPU's included),
    // issued as multimem.st in whole 16-byte pieces.  Set together with `staged` by the tensor-core launchers only.
    int mc;
    // Column blocking (0 = off): output columns come in blocks of col_block, block b starting col_block_stride elements
    // after block b-1, i.e. element (i, j) lives at (j / col_block) * col_block_stride + i*ldc + j % col_block.  This is
    // how one GEMM over the patches of a whole batch writes NCHW: a block is one image's Ho*Wo output positions.
    uint32_t col_block;
    uint64_t col_block_stride;
    // uint8 output only: every kernel also ADDS the sum of each output row's bytes to out_rowsum[row] (atomically; the
    // caller clears the array first).  These are the activation row sums the next layer's epilogue needs, so a chain
    // of layers runs without a sum pass in between.
    int32_t *out_rowsum;
    // Housekeeping for such chains: the first CTA clears clear_count int32 at clear_ptr once the kernel in front has
    // finished (typically the out_rowsum array of ANOTHER layer of the chain, so that no separate clearing launch is
    // needed).  Nothing in this launch may use that array.
    int32_t *clear_ptr;
    uint32_t clear_count;
};

// The epilogue of a plain call: one dense [M, N] destination, no chain hooks.  Callers switch further fields on.
__host__ __device__ inline Epilogue make_epilogue(const int32_t *bsum, const int32_t *asum, const int32_t *bias, const ltq_qparams &qa,
                              const ltq_qparams &qb, const ltq_qparams &qc, uint64_t K, int out_mode, unsigned flags)
{
    Epilogue e;
    e.bsum = bsum;
    e.asum = asum;
    e.bias = bias;
    e.row_bias = nullptr;
    e.ldc = 0;
    e.n_more = 0;
    e.staged = 0;
    e.mc = 0;
    e.col_block = 0;
    e.col_block_stride = 0;
    e.out_rowsum = nullptr;
    e.clear_ptr = nullptr;
    e.clear_count = 0;
    for (auto &m : e.more_out) m = nullptr;
    e.qpA_dev = nullptr;
    e.sA = qa.scale;
    e.sB = qb.scale;
    e.sC = qc.scale;
    e.zA = qa.zero_point;
    e.zB = qb.zero_point;
    e.zC = qc.zero_point;
    e.K = (uint32_t)K;
    e.out_mode = out_mode;
    e.flags = flags & (LTQ_FLAG_RELU | LTQ_FLAG_SATURATE);
    return e;
}

__device__ __forceinline__ void epilogue_housekeeping(const Epilogue &e)
{
    if (e.clear_ptr && blockIdx.x == 0 && blockIdx.y == 0)
        for (uint32_t i = threadIdx.x; i < e.clear_count; i += blockDim.x) e.clear_ptr[i] = 0;
}

// Element offset of (row, col).  With column blocking a chunk of consecutive columns must not straddle a block: the
// tensor-core kernels handle chunks of 16 / 32 columns starting at multiples of 16, so col_block % 32 == 0 there.
__device__ __forceinline__ uint64_t epilogue_offset(const Epilogue &e, uint64_t row, uint64_t col, uint64_t ldc)
{
    if (e.col_block == 0) return row * ldc + col;
    const uint64_t b = col / e.col_block;
    return b * e.col_block_stride + row * ldc + (col - b * e.col_block);
}

__device__ __forceinline__ uint64_t epilogue_pitch(const Epilogue &e, uint64_t N) { return e.ldc ? e.ldc : N; }
// 16-byte stores need every row start aligned in every destination: pitch and bases multiples of 16 bytes.
__device__ __forceinline__ bool epilogue_vec_ok(const Epilogue &e, const void *out, uint64_t N, uint32_t esize)
{
    bool ok = ((epilogue_pitch(e, N) * esize) % 16 == 0) && (((uintptr_t)out & 15) == 0) &&
              ((e.col_block_stride * esize) % 16 == 0) && (e.col_block % 16 == 0);
    for (int d = 0; d < e.n_more; d++) ok = ok && (((uintptr_t)e.more_out[d] & 15) == 0);
    return ok;
}

// Per-launch constants derived once per thread.
struct EpilogueConsts {
    uint32_t neg_zA, neg_zB, bc;  // -zA, -zB, K*zA*zB (mod 2^32)
    float rm, sAB, zCf;
    bool rm_small;                // |rm| <= 0.5: |rm*acc + zC| stays below 2^31 for every int32 acc
};

__device__ __forceinline__ EpilogueConsts epilogue_consts(const Epilogue &e)
{
    float sA = e.sA;
    int32_t zA = e.zA;
    if (e.qpA_dev) {
        sA = e.qpA_dev->scale;
        zA = e.qpA_dev->zero_point;
    }
    EpilogueConsts c;
    c.neg_zA = (uint32_t)(-zA);
    c.neg_zB = (uint32_t)(-e.zB);
    c.bc = e.K * (uint32_t)zA * (uint32_t)e.zB;
    c.sAB = __fmul_rn(sA, e.sB);
    c.rm = __fdiv_rn(c.sAB, e.sC);  // l-ten/math_fns.cpp:1436: float, left to right
    c.zCf = (float)e.zC;
    c.rm_small = fabsf(c.rm) <= 0.5f;  // false for NaN
    return c;
}

// Row part of the correction: -zB*asum[i] + K*zA*zB (+ row_bias[i]).
__device__ __forceinline__ uint32_t epilogue_row_term(const Epilogue &e, const EpilogueConsts &c, uint64_t i)
{
    uint32_t t = c.neg_zB * (uint32_t)e.asum[i] + c.bc;
    if (e.row_bias) t += (uint32_t)e.row_bias[i];
    return t;
}
// Column part: -zA*bsum[j] (+ bias[j]).
__device__ __forceinline__ uint32_t epilogue_col_term(const Epilogue &e, const EpilogueConsts &c, uint64_t j)
{
    uint32_t t = c.neg_zA * (uint32_t)e.bsum[j];
    if (e.bias) t += (uint32_t)e.bias[j];
    return t;
}

__device__ __forceinline__ int32_t epilogue_acc(uint32_t raw, uint32_t row_term, uint32_t col_term, bool relu)
{
    int32_t acc = (int32_t)(raw + row_term + col_term);
    if (relu && acc < 0) acc = 0;
    return acc;
}

// (unsigned char)(rm*acc + zC), l-ten/math_fns.cpp:1474: int->float rounds to nearest, multiply and add are separate
// roundings (the reference is built without FMA), the cast truncates toward zero.  Out of range the reference's x86
// code converts to int32 and keeps the low byte (and yields 0 once |t| >= 2^31); `saturate` clamps instead.
__device__ __forceinline__ uint8_t epilogue_u8(int32_t acc, const EpilogueConsts &c, bool saturate)
{
    float t = __fadd_rn(__fmul_rn(c.rm, __int2float_rn(acc)), c.zCf);
    if (saturate) {
        if (!(t > 0.f)) return 0;
        if (t >= 255.f) return 255;
        return (uint8_t)__float2int_rz(t);
    }
    // The device conversion saturates: t <= -2^31 gives INT_MIN (low byte 0, as on x86) and NaN gives 0 (x86: 0x80000000,
    // low byte 0); only t >= 2^31 needs care, where x86 yields 0x80000000 but the device INT_MAX.
    int32_t r = __float2int_rz(t);
    r = (t >= 2147483648.f) ? 0 : r;
    return (uint8_t)(r & 0xFF);
}

__device__ __forceinline__ float epilogue_f32(int32_t acc, const EpilogueConsts &c)
{
    return __fmul_rn(c.sAB, __int2float_rn(acc));
}

// One chunk of W (32 or 16) accumulator columns of one output row -> output words: W/4 words of packed uint8 (OUT == 0)
// or W words of float / int32 bits.  `res` has room for W words either way.  Written for few instructions per element
// (the epilogue is issue-bound): ReLU is a max against a uniform lower bound, the bytes are gathered with byte
// permutes, and the "t >= 2^31" corner of the wrapping cast is only evaluated when rm is large enough to reach it.
template <int OUT, int W>
__device__ __forceinline__ void epilogue_convert(const uint32_t (&v)[W], uint32_t rt, const uint32_t *col_smem,
                                                 const EpilogueConsts &c, bool relu, bool sat, uint32_t (&res)[W])
{
    // column terms: 16-byte shared loads (the chunk starts at a multiple of 16 columns)
    uint32_t col[W];
#pragma unroll
    for (int g = 0; g < W / 4; g++) {
        const uint4 t4 = reinterpret_cast<const uint4 *>(col_smem)[g];
        col[4 * g] = t4.x;
        col[4 * g + 1] = t4.y;
        col[4 * g + 2] = t4.z;
        col[4 * g + 3] = t4.w;
    }
    const int32_t lo = relu ? 0 : INT32_MIN;
    if (OUT == 0) {
        if (!sat && c.rm_small) {
#pragma unroll
            for (int g = 0; g < W / 4; g++) {
                int32_t r[4];
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const int32_t a = max((int32_t)(v[4 * g + b] + rt + col[4 * g + b]), lo);
                    r[b] = __float2int_rz(__fadd_rn(__fmul_rn(c.rm, __int2float_rn(a)), c.zCf));
                }
                res[g] = __byte_perm(__byte_perm((uint32_t)r[0], (uint32_t)r[1], 0x0040),
                                     __byte_perm((uint32_t)r[2], (uint32_t)r[3], 0x0040), 0x5410);
            }
        } else {
#pragma unroll
            for (int g = 0; g < W / 4; g++) {
                uint32_t w = 0;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const int32_t a = max((int32_t)(v[4 * g + b] + rt + col[4 * g + b]), lo);
                    w |= (uint32_t)epilogue_u8(a, c, sat) << (8 * b);
                }
                res[g] = w;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < W; j++) {
            const int32_t a = max((int32_t)(v[j] + rt + col[j]), lo);
            res[j] = (OUT == 1) ? __float_as_uint(epilogue_f32(a, c)) : (uint32_t)a;
        }
    }
}

// 16 bytes to an ordinary address, or to all GPUs behind a multicast address (the bits travel unchanged).
__device__ __forceinline__ void store16(void *dst, const uint4 &v, bool mc)
{
    if (mc)
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z),
                     "r"(v.w)
                     : "memory");
    else
        *reinterpret_cast<uint4 *>(dst) = v;
}

// The same chunk stored into every destination at element offset `off` (16-byte stores when vec_ok and the chunk is
// complete, element by element otherwise).
template <int OUT, int W>
__device__ __forceinline__ void epilogue_store(const uint32_t (&res)[W], const Epilogue &e, void *out, uint64_t off,
                                               bool vec_ok, int valid)
{
    constexpr int PER16 = OUT == 0 ? 16 : 4;  // elements per 16-byte piece
    const bool mc = e.mc != 0;
    for (int d = -1; d < e.n_more; d++) {
        void *base = d < 0 ? out : e.more_out[d];
        if (vec_ok) {
            // whole 16-byte pieces as vectors (all of them when the chunk is complete), the rest element by element
            uint8_t *dst = static_cast<uint8_t *>(base) + off * (OUT == 0 ? 1 : 4);
#pragma unroll
            for (int g = 0; g < W / PER16; g++)
                if ((g + 1) * PER16 <= valid)
                    store16(dst + 16 * g, make_uint4(res[4 * g], res[4 * g + 1], res[4 * g + 2], res[4 * g + 3]), mc && d < 0);
        }
        const int done = vec_ok ? (valid / PER16) * PER16 : 0;
        if (OUT == 0) {
            uint8_t *dst = static_cast<uint8_t *>(base) + off;
#pragma unroll
            for (int j = 0; j < W; j++)
                if (j >= done && j < valid) dst[j] = (uint8_t)(res[j >> 2] >> (8 * (j & 3)));
        } else {
            uint32_t *dst = static_cast<uint32_t *>(base) + off;
#pragma unroll
            for (int j = 0; j < W; j++)
                if (j >= done && j < valid) dst[j] = res[j];
        }
    }
}

// Sum of the first `valid` output bytes of a converted uint8 chunk (W/4 packed words).
template <int W>
__device__ __forceinline__ uint32_t packed_byte_sum(const uint32_t (&res)[W], int valid)
{
    uint32_t s = 0;
#pragma unroll
    for (int g = 0; g < W / 4; g++) {
        const int left = valid - 4 * g;  // bytes of this word that count
        const uint32_t mask = left >= 4 ? 0xFFFFFFFFu : (left <= 0 ? 0u : (0xFFFFFFFFu >> (8 * (4 - left))));
        s = __dp4a(res[g] & mask, 0x01010101u, s);
    }
    return s;
}

// Converts and stores one chunk; returns the sum of the uint8 values stored (0 for the other output modes).
template <int OUT, int W>
__device__ __forceinline__ uint32_t epilogue_chunk(uint32_t (&v)[W], uint32_t rt, const uint32_t *col_smem,
                                                   const EpilogueConsts &c, bool relu, bool sat, const Epilogue &e, void *out,
                                                   uint64_t off, bool vec_ok, int valid)
{
    uint32_t res[W];
    epilogue_convert<OUT, W>(v, rt, col_smem, c, relu, sat, res);
    epilogue_store<OUT, W>(res, e, out, off, vec_ok, valid);
    return OUT == 0 ? packed_byte_sum<W>(res, valid) : 0u;
}

// Row-coalescing stage for stores that leave the GPU.  In the accumulator layout a thread owns one output row, so a
// direct store instruction writes 32 separate 16-byte pieces, one per row: harmless in local HBM (L2 merges them), but
// over NVLink every piece travels as its own small packet.  A warp therefore parks a block of 32 rows x 128 bytes in
// shared memory (16-byte units XOR-swizzled by row, conflict-free both ways) and writes it back out with each
// instruction covering 4 rows x 128 contiguous bytes.
struct PeerStage {
    static constexpr int BYTES_PER_WARP = 32 * 128;

    // This lane's row: `nunits` 16-byte units starting at unit `u0` of the row's 128 bytes.
    template <int NW>
    static __device__ __forceinline__ void put(uint8_t *stage, int lane, int u0, const uint32_t (&res)[NW], int nunits)
    {
#pragma unroll
        for (int g = 0; g < NW / 4; g++)
            if (g < nunits)
                *reinterpret_cast<uint4 *>(stage + lane * 128 + (((u0 + g) ^ (lane & 7)) << 4)) =
                    make_uint4(res[4 * g], res[4 * g + 1], res[4 * g + 2], res[4 * g + 3]);
    }

    // Writes units [0, units) of all 32 rows to every destination; `off_bytes` is the byte offset of (first row, first
    // unit) and `pitch_bytes` the destinations' row pitch.  Called by the whole warp.
    static __device__ __forceinline__ void flush(const uint8_t *stage, int lane, int units, const Epilogue &e, void *out,
                                                 uint64_t off_bytes, uint64_t pitch_bytes)
    {
        __syncwarp();
        const int u = lane & 7;
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int r = it * 4 + (lane >> 3);
            if (u < units) {
                const uint4 val = *reinterpret_cast<const uint4 *>(stage + r * 128 + ((u ^ (r & 7)) << 4));
                const uint64_t o = off_bytes + (uint64_t)r * pitch_bytes + (uint64_t)u * 16;
                for (int d = -1; d < e.n_more; d++)
                    store16(static_cast<uint8_t *>(d < 0 ? out : e.more_out[d]) + o, val, e.mc != 0 && d < 0);
            }
        }
        __syncwarp();
    }
};

// ---- GEMM dispatch (ltq_api.cu) -------------------------------------------------------------------------------------
// What the dispatcher needs to know about the device: its SM count and the word that bounded waits report into.
struct GemmDevice {
    int sms;
    uint32_t *status;
};
}  // namespace ltq
struct ltq_layer;
namespace ltq {
// Kernel choice and launch for the FullyConnected_q layout (A [M,K], B [N,K], both K-contiguous): skinny kernel,
// tcgen05 kernel (single CTA or CTA pair) or the generic dp4a kernel, by shape and LTQ_FLAG_FORCE_*.  `layer`
// (optional) caches the weight tensor maps.  Allocates nothing.
int run_fc_gemm(const GemmDevice &dev, uint64_t M, uint64_t N, uint64_t K, const uint8_t *A, const uint8_t *B,
                const Epilogue &epi, void *out, unsigned flags, ltq_layer *layer, cudaStream_t stream);

// ---- kernel launchers implemented in the other translation units --------------------------------------------------
// Generic dp4a tile kernel: any M, N, K and any transpose combination.
cudaError_t launch_gemm_simt(bool tA, bool tB, uint64_t M, uint64_t N, uint64_t K, const uint8_t *A, const uint8_t *B,
                             const Epilogue &epi, void *out, cudaStream_t stream);
// Its 64 x 64 tiles are numbered along grid.x: at most 2^31 - 1 of them.
inline bool simt_grid_ok(uint64_t M, uint64_t N)
{
    const uint64_t gx = (M + 63) / 64, gy = (N + 63) / 64;
    return gx <= 0x7FFFFFFFull && gy <= 0x7FFFFFFFull && gx * gy <= 0x7FFFFFFFull;
}

// Operand sums. rows x cols uint8, contiguous along cols: sums[r] = sum_c m[r*cols + c].
cudaError_t launch_row_sums(const uint8_t *m, uint64_t rows, uint64_t cols, int32_t *sums, cudaStream_t stream);
// Same matrix read the other way: sums[c] = sum_r m[r*cols + c].
cudaError_t launch_col_sums(const uint8_t *m, uint64_t rows, uint64_t cols, int32_t *sums, cudaStream_t stream);
// v[i] *= factor (wrapping), used to leave the reference's pre-multiplied workspace behind.
cudaError_t launch_scale_i32(int32_t *v, uint64_t n, int32_t factor, cudaStream_t stream);

// dst[m][g*W + w] = src[g][m][w] over bytes: undoes the plane-per-rank layout an all-gather of column slices leaves.
cudaError_t launch_interleave_blocks(const void *src, void *dst, uint64_t G, uint64_t M, uint64_t W, cudaStream_t stream);

// One warp waits on a barrier nothing arrives on, for at most limit_ns, then records code 0x900 in *status.
cudaError_t launch_bounded_wait_probe(uint32_t *status, uint64_t limit_ns, cudaStream_t stream);

// Patch gather for Conv2d_q over `batches` NCHW images, K-contiguous and zero-padded to Kp (a multiple of 16) bytes per
// row: col_t[b][ho*Wo + wo][k], k = (c*kh + i)*kw + j.  Out-of-image taps and the padding are the byte 0.
struct ConvGeom {
    uint32_t C, H, W, kh, kw, ph, pw, sh, sw, Ho, Wo, K, Kp;
};
cudaError_t launch_im2col_t(const uint8_t *im, uint64_t batches, const ConvGeom &g, uint8_t *col_t, cudaStream_t stream);
// The same gather plus the per-patch sums (colsum[b*Ho*Wo + n] = sum over k of col_t[b][n][k]) in one pass.
cudaError_t launch_im2col_t_sums(const uint8_t *im, uint64_t batches, const ConvGeom &g, uint8_t *col_t, int32_t *colsum,
                                 cudaStream_t stream);

cudaError_t launch_min_max(const float *data, uint64_t len, float *minmax, cudaStream_t stream);
cudaError_t launch_qparams_from_minmax(const float *minmax, ltq_qparams *qp, cudaStream_t stream);
cudaError_t launch_quantize_u8(const float *x, uint8_t *q, uint64_t len, const ltq_qparams &qp, cudaStream_t stream);
cudaError_t launch_quantize_i32(const float *x, int32_t *q, uint64_t len, const ltq_qparams &qp, cudaStream_t stream);
cudaError_t launch_dequantize(float *x, const uint8_t *q, uint64_t len, const ltq_qparams &qp, cudaStream_t stream);
cudaError_t launch_quantize_rows(const float *x, uint64_t M, uint64_t K, const ltq_qparams *qp_host,
                                 const ltq_qparams *qp_dev, uint8_t *q, int32_t *asum, cudaStream_t stream);

}  // namespace ltq
