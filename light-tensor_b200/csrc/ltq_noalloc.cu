// ltq_quantized_matmul_static: quantized_matmul for callers that are not allowed to allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits -- a plugin called from inside another framework's
// memory-planned region (the host owns every byte of device memory and hands out only the input/output tensors), a
// real-time loop that must not take the allocator's lock or risk an implicit device synchronisation, or a process
// whose device memory was fully reserved up front.  The ordinary entry point makes such callers supply an int32
// workspace of M + N elements for the operand sums; this one keeps that scratch inside the library image instead.
//
// The scratch is a file-scope __device__ array, so every GPU that loads the library carries it (1 MiB + 256 B) until
// the process exits.  It is shared by all calls on a device: two calls whose kernels overlap on the GPU (different
// streams, or different host threads) race on it, and its contents are whatever the previous call left.  Nothing here
// calls cudaMalloc, cudaFree or any routine that allocates.
#include <mutex>

#include "ltq_common.cuh"
#include "ltq_gemm_tc.cuh"
#include "ltq_gemv.cuh"

#define LTQ_STATIC_WS_INTS_IMPL (256 * 1024)
static_assert(LTQ_STATIC_WS_INTS_IMPL == LTQ_STATIC_WS_INTS, "header and implementation disagree on the limit");

// Operand sums: [0, N) sums over K of the B operand, [N, N + M) sums over K of the A operand.
static __device__ __align__(256) int32_t g_static_ws[LTQ_STATIC_WS_INTS_IMPL];
// Status word for the bounded waits inside the GEMM kernels (the ordinary path allocates its own); zero at load,
// read and cleared by ltq_static_check.
static __device__ __align__(256) uint32_t g_static_status[64];

namespace {

struct StaticDevice {
    bool ready = false;
    int sms = 0;
    int32_t *ws = nullptr;       // device address of g_static_ws on this device
    uint32_t *status = nullptr;  // device address of g_static_status on this device
};
StaticDevice g_sdev[64];
std::mutex g_sdev_mu;

// In host code `g_static_ws` is only a handle for the runtime, not an address a kernel can use.  The real device address
// differs per GPU and is looked up once per device, with that device current.
int static_device(int device, StaticDevice **out)
{
    LTQ_REQUIRE(device >= 0 && device < 64, LTQ_ERR_INVALID_ARG, "device index %d out of range", device);
    std::lock_guard<std::mutex> lk(g_sdev_mu);
    StaticDevice &d = g_sdev[device];
    if (!d.ready) {
        int major = 0;
        LTQ_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        LTQ_REQUIRE(major == 10, LTQ_ERR_CUDA, "device %d has compute capability %d.x; this library is built for sm_100a only",
                    device, major);
        LTQ_CUDA_TRY(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device));
        void *p = nullptr;
        LTQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_ws));
        d.ws = static_cast<int32_t *>(p);
        LTQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_status));
        d.status = static_cast<uint32_t *>(p);
        d.ready = true;
    }
    *out = &d;
    return LTQ_OK;
}

}  // namespace

using namespace ltq;

extern "C" int ltq_quantized_matmul_static(int transpose_A, int transpose_B, uint64_t M, uint64_t N, uint64_t K,
                                           uint8_t alpha, const uint8_t *A_dev, const uint8_t *B_dev, uint8_t beta,
                                           uint8_t *C_dev, const ltq_qparams *qparams, const int32_t *bias_dev,
                                           int device, void *stream)
{
    LTQ_REQUIRE(alpha == 1 && beta == 0, LTQ_ERR_UNSUPPORTED, "Support for alpha != 1 and beta != 0 not implemented");
    LTQ_REQUIRE(A_dev && B_dev && C_dev && qparams, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(M + N <= (uint64_t)LTQ_STATIC_WS_INTS && M + N >= M, LTQ_ERR_TOO_LARGE,
                "M + N = %llu exceeds the built-in scratch of %d int32 (use ltq_quantized_matmul with your own workspace)",
                (unsigned long long)(M + N), LTQ_STATIC_WS_INTS);
    if (M == 0 || N == 0) return LTQ_OK;
    const uint64_t bc = K * (uint64_t)qparams[0].zero_point * (uint64_t)qparams[1].zero_point;
    LTQ_REQUIRE(bc <= 0x7FFFFFFFull, LTQ_ERR_UNSUPPORTED, "K*zA*zB = %llu does not fit an int", (unsigned long long)bc);
    LTQ_ENTER_DEVICE(device);
    StaticDevice *sd;
    int rc = static_device(device, &sd);
    if (rc != LTQ_OK) return rc;

    cudaStream_t st = (cudaStream_t)stream;
    const bool tA = transpose_A != 0, tB = transpose_B != 0;
    int32_t *bsum = sd->ws, *asum = sd->ws + N;
    // The scratch still holds the previous call's sums.  Row sums overwrite every element they own; the column-sum
    // kernel accumulates with atomics and is preceded by its own clear (inside launch_col_sums); K == 0 clears here.
    if (K == 0) {
        LTQ_CUDA_TRY(cudaMemsetAsync(sd->ws, 0, (M + N) * sizeof(int32_t), st));
    } else {
        if (tB) LTQ_CUDA_TRY(launch_row_sums(B_dev, N, K, bsum, st));
        else LTQ_CUDA_TRY(launch_col_sums(B_dev, K, N, bsum, st));
        if (!tA) LTQ_CUDA_TRY(launch_row_sums(A_dev, M, K, asum, st));
        else LTQ_CUDA_TRY(launch_col_sums(A_dev, K, M, asum, st));
    }

    // Same epilogue set-up and kernel choice as ltq_quantized_matmul (skinny, tcgen05 single CTA or CTA pair, dp4a):
    // only the scratch and the status word differ.  Tensor maps are encoded on the host into stack objects.
    const Epilogue epi = make_epilogue(bsum, asum, bias_dev, qparams[0], qparams[1], qparams[2], K, LTQ_OUT_U8, 0);
    if (!tA && tB && K > 0) {
        const GemmDevice gd{sd->sms, sd->status};
        rc = run_fc_gemm(gd, M, N, K, A_dev, B_dev, epi, C_dev, 0, nullptr, st);
        if (rc != LTQ_OK) return rc;
    } else {
        LTQ_REQUIRE(simt_grid_ok(M, N), LTQ_ERR_TOO_LARGE, "M x N = %llu x %llu needs more than 2^31 - 1 tiles of 64 x 64",
                    (unsigned long long)M, (unsigned long long)N);
        LTQ_CUDA_TRY(launch_gemm_simt(tA, tB, M, N, K, A_dev, B_dev, epi, C_dev, st));
    }
    return LTQ_OK;
}

// Allocation-free counterpart of ltq_device_check for the calls above: their kernels report an expired bounded wait
// into the library's built-in status word, which this reads back (into a host stack variable) and clears.
extern "C" int ltq_static_check(int device, void *stream)
{
    LTQ_ENTER_DEVICE(device);
    StaticDevice *sd;
    int rc = static_device(device, &sd);
    if (rc != LTQ_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t code = 0;
    LTQ_CUDA_TRY(cudaMemcpyAsync(&code, sd->status, sizeof code, cudaMemcpyDeviceToHost, st));
    LTQ_CUDA_TRY(cudaStreamSynchronize(st));
    if (code) {
        LTQ_CUDA_TRY(cudaMemsetAsync(sd->status, 0, sizeof code, st));
        set_error("a bounded device-side wait expired inside an allocation-free call (code 0x%x: role %u, slot %u)", code,
                  code >> 8, code & 0xFF);
        return LTQ_ERR_DEVICE_TIMEOUT;
    }
    return LTQ_OK;
}

extern "C" int ltq_selftest_bounded_wait_static(int device, uint32_t limit_us, void *stream)
{
    LTQ_REQUIRE(limit_us >= 1 && limit_us <= 1000000, LTQ_ERR_INVALID_ARG, "limit must be between 1 us and 1 s");
    LTQ_ENTER_DEVICE(device);
    StaticDevice *sd;
    int rc = static_device(device, &sd);
    if (rc != LTQ_OK) return rc;
    LTQ_CUDA_TRY(launch_bounded_wait_probe(sd->status, (uint64_t)limit_us * 1000ull, (cudaStream_t)stream));
    return LTQ_OK;
}
