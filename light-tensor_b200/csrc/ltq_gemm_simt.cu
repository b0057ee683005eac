// Generic uint8 x uint8 -> int32 GEMM on CUDA cores (dp4a) with the full fused epilogue.
//
// This is the kernel for shapes the tensor-core kernel does not take: operands whose K stride is not 16-byte aligned
// and the transposed layouts of quantized_matmul (l-ten/math_fns.cpp:1336-1467) that only Conv2d_q-style callers use.
// It also serves as the on-device cross-check of the tcgen05 kernel at sizes the CPU oracle cannot reach.
//
// 64x64 output tile per 256-thread CTA, 32-deep K slices staged in shared memory as packed 4-byte K groups, each
// thread owning a 4x4 register tile (16 dp4a per 8 shared loads).
#include "ltq_common.cuh"

namespace ltq {

constexpr int TM = 64, TN = 64, TK = 32;
constexpr int LDW = TK / 4 + 1;  // words per staged row, +1 to stagger banks

// Element (r, k) of an operand stored either k-contiguous ([rows, K]) or r-contiguous ([K, rows]).
__device__ __forceinline__ uint8_t fetch(const uint8_t *__restrict__ p, bool k_contig, uint64_t rows, uint64_t K,
                                         uint64_t r, uint64_t k)
{
    if (r >= rows || k >= K) return 0;
    return k_contig ? p[r * K + k] : p[k * rows + r];
}

__device__ __forceinline__ void stage(uint32_t (*dst)[LDW], const uint8_t *__restrict__ p, bool k_contig,
                                      uint64_t rows, uint64_t K, uint64_t r0, uint64_t k0)
{
    uint8_t *d = reinterpret_cast<uint8_t *>(dst);
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
        // Walk memory in its contiguous direction so that neighbouring threads touch neighbouring bytes.
        int r, k;
        if (k_contig) {
            r = e / TK;
            k = e % TK;
        } else {
            k = e / TM;
            r = e % TM;
        }
        d[r * (LDW * 4) + k] = fetch(p, k_contig, rows, K, r0 + r, k0 + k);
    }
}

__global__ void __launch_bounds__(256) gemm_simt_kernel(bool a_kc, bool b_kc, uint64_t M, uint64_t N, uint64_t K,
                                                        const uint8_t *__restrict__ A, const uint8_t *__restrict__ B,
                                                        Epilogue epi, void *__restrict__ out, uint32_t tiles_m)
{
    epilogue_housekeeping(epi);
    __shared__ uint32_t As[TM][LDW];
    __shared__ uint32_t Bs[TN][LDW];
    // tiles are numbered along grid.x (which reaches 2^31 - 1; grid.y stops at 65535), M tiles fastest
    const uint64_t m0 = (uint64_t)(blockIdx.x % tiles_m) * TM, n0 = (uint64_t)(blockIdx.x / tiles_m) * TN;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;

    int32_t acc[4][4] = {};
    for (uint64_t k0 = 0; k0 < K; k0 += TK) {
        stage(As, A, a_kc, M, K, m0, k0);
        stage(Bs, B, b_kc, N, K, n0, k0);
        __syncthreads();
#pragma unroll
        for (int kw = 0; kw < TK / 4; kw++) {
            uint32_t a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[ty + 16 * i][kw];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[tx + 16 * j][kw];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = (int32_t)__dp4a(a[i], b[j], (uint32_t)acc[i][j]);
        }
        __syncthreads();
    }

    const EpilogueConsts c = epilogue_consts(epi);
    const bool relu = epi.flags & LTQ_FLAG_RELU, sat = epi.flags & LTQ_FLAG_SATURATE;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint64_t row = m0 + ty + 16 * i;
        if (row >= M) continue;
        const uint32_t rt = epilogue_row_term(epi, c, row);
        uint32_t rsum = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint64_t col = n0 + tx + 16 * j;
            if (col >= N) continue;
            const int32_t v = epilogue_acc((uint32_t)acc[i][j], rt, epilogue_col_term(epi, c, col), relu);
            const uint64_t o = epilogue_offset(epi, row, col, epilogue_pitch(epi, N));
            for (int d = -1; d < epi.n_more; d++) {
                void *dst = d < 0 ? out : epi.more_out[d];
                if (epi.out_mode == LTQ_OUT_U8) {
                    const uint8_t b = epilogue_u8(v, c, sat);
                    static_cast<uint8_t *>(dst)[o] = b;
                    if (d < 0) rsum += b;
                }
                else if (epi.out_mode == LTQ_OUT_F32)
                    static_cast<float *>(dst)[o] = epilogue_f32(v, c);
                else
                    static_cast<int32_t *>(dst)[o] = v;
            }
        }
        if (epi.out_mode == LTQ_OUT_U8 && epi.out_rowsum) atomicAdd(&epi.out_rowsum[row], (int32_t)rsum);
    }
}

cudaError_t launch_gemm_simt(bool tA, bool tB, uint64_t M, uint64_t N, uint64_t K, const uint8_t *A, const uint8_t *B,
                             const Epilogue &epi, void *out, cudaStream_t stream)
{
    if (M == 0 || N == 0) return cudaSuccess;
    // quantized_matmul's layouts: A is [M,K] unless transposed ([K,M]); B is [K,N] unless transposed ([N,K]).
    const bool a_kc = !tA, b_kc = tB;
    const uint64_t gx = (M + TM - 1) / TM, gy = (N + TN - 1) / TN;
    if (gx > 0x7FFFFFFFull || gy > 0x7FFFFFFFull || gx * gy > 0x7FFFFFFFull) return cudaErrorInvalidConfiguration;
    dim3 grid((unsigned)(gx * gy));
    gemm_simt_kernel<<<grid, 256, 0, stream>>>(a_kc, b_kc, M, N, K, A, B, epi, out, (uint32_t)gx);
    count_launch();
    note_kernel("gemm_simt_kernel");
    return cudaGetLastError();
}

}  // namespace ltq
