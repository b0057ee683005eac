// C-ABI entry points of libltq (declared in include/ltq.h): argument checking, kernel selection and the layer handle.
// Nothing here computes on the host beyond scalar set-up; every data path is a CUDA kernel and every entry point fails
// with LTQ_ERR_CUDA when no device is usable.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <cmath>
#include <mutex>
#include <new>

#include "ltq_common.cuh"
#include "ltq_gemm_tc.cuh"
#include "ltq_gemv.cuh"
#include "ltq_conv_direct.cuh"
#include "ltq_layer.cuh"

namespace ltq {

std::atomic<uint64_t> g_launches{0};
static thread_local char g_err[512] = "";

static thread_local char g_kernel[96] = "";
void note_kernel(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_kernel, sizeof g_kernel, fmt, ap);
    va_end(ap);
}

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

bool chained_launches_enabled()
{
    static const bool on = getenv("LTQ_NO_CHAINED_LAUNCH") == nullptr;
    return on;
}

namespace {

constexpr int MAX_DEVICES = 64;

// sms; status = device word: 0, or the code of the first bounded wait that expired
using DeviceState = GemmDevice;
DeviceState g_dev[MAX_DEVICES] = {};
std::mutex g_dev_mu;

// Per-device constants and the status word, created on first use with that device current.
int device_state(int device, DeviceState **out)
{
    LTQ_REQUIRE(device >= 0 && device < MAX_DEVICES, LTQ_ERR_INVALID_ARG, "device index %d out of range", device);
    std::lock_guard<std::mutex> lk(g_dev_mu);
    DeviceState &d = g_dev[device];
    if (!d.status) {
        int sms = 0;
        LTQ_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        int major = 0;
        LTQ_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        LTQ_REQUIRE(major == 10, LTQ_ERR_CUDA, "device %d has compute capability %d.x; this library is built for sm_100a only",
                    device, major);
        uint32_t *p = nullptr;
        LTQ_CUDA_TRY(cudaMalloc(&p, 256));
        LTQ_CUDA_TRY(cudaMemset(p, 0, 256));
        d.sms = sms;
        d.status = p;
    }
    *out = &d;
    return LTQ_OK;
}

enum Path { PATH_SIMT, PATH_TC, PATH_SKINNY };

// Kernel choice for the FullyConnected_q layout (A [M,K], B [N,K]).
int choose_path(uint64_t M, uint64_t N, uint64_t K, const void *A, const void *B, unsigned flags, int sms, Path *path)
{
    const bool tc_ok = tc_shape_ok(M, N, K, A, B), sk_ok = gemv_shape_ok(M, N, K, A, B, sms);
    if (flags & LTQ_FLAG_FORCE_SIMT) {
        *path = PATH_SIMT;
    } else if (flags & LTQ_FLAG_FORCE_TC) {
        LTQ_REQUIRE(tc_ok, LTQ_ERR_UNSUPPORTED, "tcgen05 kernel needs K %% 16 == 0 and 16-byte aligned operands (M=%llu N=%llu K=%llu)",
                    (unsigned long long)M, (unsigned long long)N, (unsigned long long)K);
        *path = PATH_TC;
    } else if (flags & LTQ_FLAG_FORCE_SKINNY) {
        LTQ_REQUIRE(sk_ok, LTQ_ERR_UNSUPPORTED, "skinny kernel needs M <= 16, K %% 128 == 0 and 16-byte aligned operands (M=%llu K=%llu)",
                    (unsigned long long)M, (unsigned long long)K);
        *path = PATH_SKINNY;
    } else if (sk_ok) {
        *path = PATH_SKINNY;
    } else if (tc_ok) {
        *path = PATH_TC;
    } else {
        *path = PATH_SIMT;
    }
    return LTQ_OK;
}

}  // namespace
}  // namespace ltq

using namespace ltq;

// Grow-only device buffer, same policy as the reference's col buffer and workspace.
template <typename T>
static int grow(T **buf, uint64_t *cap, uint64_t need, cudaStream_t st, const char *what)
{
    if (need <= *cap) return LTQ_OK;
    T *p = nullptr;
    cudaError_t e = cudaMalloc(&p, need * sizeof(T));
    if (e != cudaSuccess) {
        set_error("cudaMalloc of %llu bytes for %s failed: %s", (unsigned long long)(need * sizeof(T)), what, cudaGetErrorString(e));
        return LTQ_ERR_NO_MEMORY;
    }
    if (*buf) {
        LTQ_CUDA_TRY(cudaStreamSynchronize(st));
        cudaFree(*buf);
    }
    *buf = p;
    *cap = need;
    return LTQ_OK;
}

extern "C" {

int ltq_version(void) { return LTQ_VERSION; }
const char *ltq_last_error(void) { return ltq::g_err; }
const char *ltq_last_kernel(void) { return ltq::g_kernel; }
uint64_t ltq_kernel_launches(void) { return g_launches.load(); }

// ---- helpers ----------------------------------------------------------------------------------------------------------
int ltq_get_min_max(const float *data_dev, uint64_t len, float *minmax_dev, int device, void *stream)
{
    LTQ_REQUIRE(data_dev && minmax_dev && len >= 1, LTQ_ERR_INVALID_ARG, "Invalid argument");  // l-ten/utils.cpp:204-207
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(launch_min_max(data_dev, len, minmax_dev, (cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_compute_qparams(float min_val, float max_val, ltq_qparams *qp)
{
    LTQ_REQUIRE(qp, LTQ_ERR_INVALID_ARG, "Invalid argument");
    // l-ten/utils.cpp:266-286, float arithmetic in the same order.
    min_val = std::fmin(min_val, 0.f);
    max_val = std::fmax(max_val, 0.f);
    volatile float range = max_val - min_val;
    LTQ_REQUIRE(range > 0.f, LTQ_ERR_INVALID_ARG, "empty value range [%g, %g]: scale would be 0", min_val, max_val);
    volatile float scale = range / 255.f;
    volatile float ratio = min_val / scale;
    volatile float zp = 0.f - ratio;
    qp->scale = scale;
    qp->zero_point = (uint8_t)std::round((float)zp);
    return LTQ_OK;
}

int ltq_compute_qparams_dev(const float *minmax_dev, ltq_qparams *qp_dev, int device, void *stream)
{
    LTQ_REQUIRE(minmax_dev && qp_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(launch_qparams_from_minmax(minmax_dev, qp_dev, (cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_quantize_u8(const float *data_dev, uint8_t *q_dev, uint64_t len, const ltq_qparams *qp, int device, void *stream)
{
    LTQ_REQUIRE(data_dev && q_dev && qp, LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (len == 0) return LTQ_OK;
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(launch_quantize_u8(data_dev, q_dev, len, *qp, (cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_quantize_i32(const float *data_dev, int32_t *q_dev, uint64_t len, const ltq_qparams *qp, int device, void *stream)
{
    LTQ_REQUIRE(data_dev && q_dev && qp, LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (len == 0) return LTQ_OK;
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(launch_quantize_i32(data_dev, q_dev, len, *qp, (cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_dequantize(float *data_dev, const uint8_t *q_dev, uint64_t len, const ltq_qparams *qp, int device, void *stream)
{
    LTQ_REQUIRE(data_dev && q_dev && qp, LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (len == 0) return LTQ_OK;
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(launch_dequantize(data_dev, q_dev, len, *qp, (cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_quantize_rows_u8(const float *x_dev, uint64_t M, uint64_t K, const ltq_qparams *qp, const ltq_qparams *qp_dev,
                         uint8_t *q_dev, int32_t *asum_dev, int device, void *stream)
{
    LTQ_REQUIRE(x_dev && q_dev && asum_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE((qp != nullptr) != (qp_dev != nullptr), LTQ_ERR_INVALID_ARG,
                "exactly one of qp (host) and qp_dev (device) must be given");
    if (M == 0) return LTQ_OK;
    LTQ_REQUIRE(K >= 1, LTQ_ERR_INVALID_ARG, "K must be >= 1");
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(launch_quantize_rows(x_dev, M, K, qp, qp_dev, q_dev, asum_dev, (cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_row_sums_u8(const uint8_t *m_dev, uint64_t rows, uint64_t cols, int32_t *sums_dev, int device, void *stream)
{
    LTQ_REQUIRE(m_dev && sums_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (rows == 0) return LTQ_OK;
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(launch_row_sums(m_dev, rows, cols, sums_dev, (cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_interleave_column_blocks(const void *gathered_dev, void *out_dev, uint64_t parts, uint64_t M,
                                 uint64_t part_row_bytes, int device, void *stream)
{
    LTQ_REQUIRE(gathered_dev && out_dev && gathered_dev != out_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (parts == 0 || M == 0 || part_row_bytes == 0) return LTQ_OK;
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(launch_interleave_blocks(gathered_dev, out_dev, parts, M, part_row_bytes, (cudaStream_t)stream));
    return LTQ_OK;
}

}  // extern "C"

// ---- GEMM dispatch shared by the stateless calls and the layer -------------------------------------------------------
int ltq::run_fc_gemm(const GemmDevice &gd, uint64_t M, uint64_t N, uint64_t K, const uint8_t *A, const uint8_t *B,
                     const Epilogue &epi, void *out, unsigned flags, ltq_layer *layer, cudaStream_t stream)
{
    const GemmDevice *dev = &gd;
    Path path;
    int rc = choose_path(M, N, K, A, B, flags, dev->sms, &path);
    if (rc != LTQ_OK) return rc;
    switch (path) {
        case PATH_SKINNY:
            // a layer's weights are fixed between ltq_layer_set_weights calls (which synchronise), so they may be streamed early
            if (layer) layer->next.cache = &layer->map_next_gemv;  // (the handle may have been moved since the hint was set)
            LTQ_CUDA_TRY(launch_gemv(A, B, M, N, K, epi, out, dev->status, dev->sms, stream, layer ? &layer->map_w_gemv : nullptr,
                                     layer != nullptr, layer && layer->next.W ? &layer->next : nullptr));
            break;
        case PATH_TC: {
            const bool pair = !(flags & LTQ_FLAG_FORCE_TC_SINGLE) &&
                              ((flags & LTQ_FLAG_FORCE_TC_PAIR) || tc_pair_preferred(M, N, dev->sms));
            TcOperandMap map_a;
            int er = tc_make_map(&map_a, A, M, K, 128);
            LTQ_REQUIRE(er == 0, LTQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the activation operand (CUresult %d)", er);
            // Weight maps by box height: the tile width for the single-CTA kernel (64, 128, 256), half the width of
            // each class of tiles for the pair kernel.  A layer caches the ones it has needed so far.
            TcOperandMap tmp_b[4];
            int n_tmp = 0;
            auto weight_map = [&](int box_rows, TcOperandMap **res) -> int {
                TcOperandMap *mb = nullptr;
                if (layer) {
                    for (auto &m : layer->map_w)
                        if (m.matches(B, N, K, box_rows)) mb = &m;
                    if (!mb) {
                        mb = &layer->map_w[layer->map_w_next];
                        layer->map_w_next = (layer->map_w_next + 1) % LAYER_MAPS;
                    }
                } else {
                    for (int k = 0; k < n_tmp; k++)
                        if (tmp_b[k].matches(B, N, K, box_rows)) mb = &tmp_b[k];
                    if (!mb) mb = &tmp_b[n_tmp++];
                }
                *res = mb;
                return mb->matches(B, N, K, box_rows) ? 0 : tc_make_map(mb, B, N, K, box_rows);
            };
            if (pair) {
                const PairTiling tl = tc_pair_tiling(M, N, dev->sms, epi.col_block != 0);
                TcOperandMap *maps[4];
                for (int k = 0; k < 4; k++) {
                    er = weight_map((int)tl.width[k] / 2, &maps[k]);
                    LTQ_REQUIRE(er == 0, LTQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the weight operand (CUresult %d)", er);
                }
                LTQ_CUDA_TRY(launch_gemm_tc_pair(map_a, maps, tl, M, N, K, epi, out, dev->status, dev->sms, stream));
            } else {
                const int bn = tc_pick_bn(M, N, dev->sms);
                TcOperandMap *mb;
                er = weight_map(bn, &mb);
                LTQ_REQUIRE(er == 0, LTQ_ERR_CUDA, "cuTensorMapEncodeTiled failed for the weight operand (CUresult %d)", er);
                LTQ_CUDA_TRY(launch_gemm_tc(map_a, *mb, bn, M, N, K, epi, out, dev->status, dev->sms, stream));
            }
            break;
        }
        default:
            LTQ_REQUIRE(simt_grid_ok(M, N), LTQ_ERR_TOO_LARGE, "M x N = %llu x %llu needs more than 2^31 - 1 tiles of 64 x 64",
                        (unsigned long long)M, (unsigned long long)N);
            LTQ_CUDA_TRY(launch_gemm_simt(false, true, M, N, K, A, B, epi, out, stream));
    }
    return LTQ_OK;
}

extern "C" {

int ltq_quantized_matmul_ex(int transpose_A, int transpose_B, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha,
                            const uint8_t *A_dev, const uint8_t *B_dev, uint8_t beta, void *C_dev,
                            const ltq_qparams *qparams, const int32_t *bias_dev, int32_t *workspace_dev, int out_mode,
                            unsigned flags, int device, void *stream)
{
    LTQ_REQUIRE(out_mode == LTQ_OUT_U8 || out_mode == LTQ_OUT_F32 || out_mode == LTQ_OUT_I32, LTQ_ERR_INVALID_ARG,
                "unknown out_mode %d", out_mode);
    LTQ_REQUIRE(alpha == 1 && beta == 0, LTQ_ERR_UNSUPPORTED,
                "Support for alpha != 1 and beta != 0 not implemented");  // l-ten/math_fns.cpp:1331-1334
    LTQ_REQUIRE(A_dev && B_dev && C_dev && qparams && workspace_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (M == 0 || N == 0) return LTQ_OK;
    // l-ten/math_fns.cpp:1433-1434 asserts that K*zA*zB fits an int.
    const uint64_t bc = K * (uint64_t)qparams[0].zero_point * (uint64_t)qparams[1].zero_point;
    LTQ_REQUIRE(bc <= 0x7FFFFFFFull, LTQ_ERR_UNSUPPORTED, "K*zA*zB = %llu does not fit an int", (unsigned long long)bc);
    LTQ_ENTER_DEVICE(device);
    DeviceState *dev;
    int rc = device_state(device, &dev);
    if (rc != LTQ_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const bool tA = transpose_A != 0, tB = transpose_B != 0;
    int32_t *bsum = workspace_dev, *asum = workspace_dev + N;
    if (K == 0) {
        LTQ_CUDA_TRY(cudaMemsetAsync(workspace_dev, 0, (M + N) * sizeof(int32_t), st));
    } else {
        // B is [N,K] when transposed (rows contiguous in K), [K,N] otherwise; A is [M,K] unless transposed ([K,M]).
        if (tB) LTQ_CUDA_TRY(launch_row_sums(B_dev, N, K, bsum, st));
        else LTQ_CUDA_TRY(launch_col_sums(B_dev, K, N, bsum, st));
        if (!tA) LTQ_CUDA_TRY(launch_row_sums(A_dev, M, K, asum, st));
        else LTQ_CUDA_TRY(launch_col_sums(A_dev, K, M, asum, st));
    }
    Epilogue epi = make_epilogue(bsum, asum, bias_dev, qparams[0], qparams[1], qparams[2], K, out_mode, flags);
    if (!tA && tB && K > 0) {
        rc = run_fc_gemm(*dev, M, N, K, A_dev, B_dev, epi, C_dev, flags, nullptr, st);
        if (rc != LTQ_OK) return rc;
    } else {
        LTQ_REQUIRE(simt_grid_ok(M, N), LTQ_ERR_TOO_LARGE, "M x N = %llu x %llu needs more than 2^31 - 1 tiles of 64 x 64",
                (unsigned long long)M, (unsigned long long)N);
        LTQ_CUDA_TRY(launch_gemm_simt(tA, tB, M, N, K, A_dev, B_dev, epi, C_dev, st));
    }
    // Leave the workspace as the reference does: sums already multiplied by the other operand's -zero_point.
    LTQ_CUDA_TRY(launch_scale_i32(bsum, N, -(int32_t)qparams[0].zero_point, st));
    LTQ_CUDA_TRY(launch_scale_i32(asum, M, -(int32_t)qparams[1].zero_point, st));
    return LTQ_OK;
}

int ltq_quantized_matmul(int transpose_A, int transpose_B, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha,
                         const uint8_t *A_dev, const uint8_t *B_dev, uint8_t beta, uint8_t *C_dev,
                         const ltq_qparams *qparams, const int32_t *bias_dev, int32_t *workspace_dev, int device,
                         void *stream)
{
    return ltq_quantized_matmul_ex(transpose_A, transpose_B, M, N, K, alpha, A_dev, B_dev, beta, C_dev, qparams, bias_dev,
                                   workspace_dev, LTQ_OUT_U8, 0, device, stream);
}

// ---- layer handle -----------------------------------------------------------------------------------------------------
int ltq_layer_create(ltq_layer **layer, int device, uint64_t in_features, uint64_t out_features)
{
    LTQ_REQUIRE(layer, LTQ_ERR_INVALID_ARG, "Invalid argument");
    *layer = nullptr;
    LTQ_REQUIRE(in_features >= 1 && out_features >= 1, LTQ_ERR_INVALID_ARG, "feature counts must be >= 1");
    LTQ_REQUIRE(in_features < (1ull << 31) && out_features < (1ull << 31), LTQ_ERR_TOO_LARGE,
                "feature counts must be below 2^31");
    LTQ_ENTER_DEVICE(device);
    DeviceState *dev;
    int rc = device_state(device, &dev);
    if (rc != LTQ_OK) return rc;
    ltq_layer *l = new (std::nothrow) ltq_layer;
    LTQ_REQUIRE(l, LTQ_ERR_NO_MEMORY, "out of host memory");
    l->device = device;
    l->K = in_features;
    l->N = out_features;
    l->dev = dev;
    cudaError_t e = cudaMalloc(&l->wsum, out_features * sizeof(int32_t));
    if (e != cudaSuccess) {
        delete l;
        set_error("cudaMalloc of %llu weight sums failed: %s", (unsigned long long)out_features, cudaGetErrorString(e));
        return LTQ_ERR_NO_MEMORY;
    }
    *layer = l;
    return LTQ_OK;
}

int ltq_layer_destroy(ltq_layer *layer)
{
    if (!layer) return LTQ_OK;
    LTQ_ENTER_DEVICE(layer->device);
    cudaFree(layer->wsum);
    cudaFree(layer->asum_ws);
    delete layer;
    return LTQ_OK;
}

int ltq_layer_set_weights(ltq_layer *layer, const uint8_t *w_dev, const int32_t *bias_dev, void *stream)
{
    LTQ_REQUIRE(layer && w_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_ENTER_DEVICE(layer->device);
    layer->w = w_dev;
    layer->bias = bias_dev;
    for (auto &m : layer->map_w) m = TcOperandMap();
    layer->map_w_gemv = GemvWeightMaps();
    LTQ_CUDA_TRY(launch_row_sums(w_dev, layer->N, layer->K, layer->wsum, (cudaStream_t)stream));
    LTQ_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_layer_set_qparams(ltq_layer *layer, const ltq_qparams *qp_in, const ltq_qparams *qp_wt, const ltq_qparams *qp_out)
{
    LTQ_REQUIRE(layer, LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (qp_in) layer->qp_in = *qp_in;
    if (qp_wt) layer->qp_wt = *qp_wt;
    if (qp_out) layer->qp_out = *qp_out;
    return LTQ_OK;
}

// Shared by ltq_layer_forward (one dense destination) and ltq_layer_forward_scatter.
static int layer_forward_impl(ltq_layer *layer, const uint8_t *x_dev, const int32_t *asum_dev, uint64_t M,
                              const ltq_qparams *qp_in_dev, int out_mode, unsigned flags, void *const *dests, int n_dests,
                              uint64_t ld_out, uint64_t col_offset, void *stream)
{
    LTQ_REQUIRE(layer && x_dev && dests && n_dests >= 1 && n_dests <= LTQ_MAX_DESTS, LTQ_ERR_INVALID_ARG, "Invalid argument");
    for (int d = 0; d < n_dests; d++) LTQ_REQUIRE(dests[d], LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(layer->w, LTQ_ERR_INVALID_ARG, "ltq_layer_set_weights has not been called");
    LTQ_REQUIRE(out_mode == LTQ_OUT_U8 || out_mode == LTQ_OUT_F32 || out_mode == LTQ_OUT_I32, LTQ_ERR_INVALID_ARG,
                "unknown out_mode %d", out_mode);
    LTQ_REQUIRE(M < (1ull << 31), LTQ_ERR_TOO_LARGE, "M must be below 2^31");
    LTQ_REQUIRE(ld_out == 0 || (ld_out >= layer->N && col_offset <= ld_out - layer->N), LTQ_ERR_INVALID_ARG,
                "the layer's %llu columns do not fit at column %llu of a row of %llu", (unsigned long long)layer->N,
                (unsigned long long)col_offset, (unsigned long long)ld_out);
    if (M == 0) return LTQ_OK;
    LTQ_ENTER_DEVICE(layer->device);
    cudaStream_t st = (cudaStream_t)stream;
    if (!asum_dev) {
        // Same policy as the reference's workspace (l-ten/fully_connected.cpp:366-371): reallocate only when the batch grows.
        int rc = grow(&layer->asum_ws, &layer->asum_cap, M, st, "the activation sums");
        if (rc != LTQ_OK) return rc;
        LTQ_CUDA_TRY(launch_row_sums(x_dev, M, layer->K, layer->asum_ws, st));
        asum_dev = layer->asum_ws;
    }
    Epilogue epi = make_epilogue(layer->wsum, asum_dev, layer->bias, layer->qp_in, layer->qp_wt, layer->qp_out, layer->K,
                                 out_mode, flags);
    epi.qpA_dev = qp_in_dev;
    epi.out_rowsum = out_mode == LTQ_OUT_U8 ? layer->rowsum_out : nullptr;
    epi.clear_ptr = layer->clear_ptr;
    epi.clear_count = layer->clear_count;
    const uint64_t esize = out_mode == LTQ_OUT_U8 ? 1 : 4;
    epi.ldc = ld_out;
    if (flags & LTQ_FLAG_MULTICAST_DEST) {
        LTQ_REQUIRE(n_dests == 1, LTQ_ERR_INVALID_ARG, "a multicast destination is the only destination");
        Path path;
        int rc = choose_path(M, layer->N, layer->K, x_dev, layer->w, flags, layer->dev->sms, &path);
        if (rc != LTQ_OK) return rc;
        LTQ_REQUIRE(path == PATH_TC && (ld_out * esize) % 16 == 0 && (col_offset * esize) % 16 == 0 && (layer->N * esize) % 16 == 0 &&
                        ((uintptr_t)dests[0] & 15) == 0,
                    LTQ_ERR_UNSUPPORTED,
                    "multicast stores need the tensor-core kernel (K %% 16 == 0, more than 16 rows) and 16-byte aligned rows, "
                    "column offset and slice width");
        epi.mc = 1;
    }
    epi.n_more = n_dests - 1;
    for (int d = 1; d < n_dests; d++) epi.more_out[d - 1] = static_cast<uint8_t *>(dests[d]) + col_offset * esize;
    return run_fc_gemm(*layer->dev, M, layer->N, layer->K, x_dev, layer->w, epi,
                       static_cast<uint8_t *>(dests[0]) + col_offset * esize, flags, layer, st);
}

int ltq_layer_set_rowsum_output(ltq_layer *layer, int32_t *rowsum_dev)
{
    LTQ_REQUIRE(layer, LTQ_ERR_INVALID_ARG, "Invalid argument");
    layer->rowsum_out = rowsum_dev;
    return LTQ_OK;
}

int ltq_layer_set_clear_on_forward(ltq_layer *layer, int32_t *array_dev, uint64_t count)
{
    LTQ_REQUIRE(layer && (array_dev || count == 0) && count < (1ull << 31), LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(!array_dev || array_dev != layer->rowsum_out, LTQ_ERR_INVALID_ARG,
                "a forward cannot clear the array it accumulates its own row sums into");
    layer->clear_ptr = count ? array_dev : nullptr;
    layer->clear_count = (uint32_t)count;
    return LTQ_OK;
}

int ltq_layer_set_next(ltq_layer *layer, const ltq_layer *next)
{
    LTQ_REQUIRE(layer, LTQ_ERR_INVALID_ARG, "Invalid argument");
    layer->next = ltq::GemvNext();
    layer->map_next_gemv = ltq::GemvWeightMaps();
    if (!next) return LTQ_OK;
    LTQ_REQUIRE(next->device == layer->device, LTQ_ERR_INVALID_ARG, "ltq_layer_set_next: the two layers are on different devices");
    LTQ_REQUIRE(next->w, LTQ_ERR_INVALID_ARG, "ltq_layer_set_next: the next layer has no weights bound");
    layer->next.W = next->w;
    layer->next.N = next->N;
    layer->next.K = next->K;
    layer->next.boxes = ltq::GEMV_NEXT_BOXES;
    return LTQ_OK;
}

int ltq_layer_forward(ltq_layer *layer, const uint8_t *x_dev, const int32_t *asum_dev, uint64_t M,
                      const ltq_qparams *qp_in_dev, int out_mode, unsigned flags, void *out_dev, void *stream)
{
    LTQ_REQUIRE(out_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    void *dests[1] = {out_dev};
    return layer_forward_impl(layer, x_dev, asum_dev, M, qp_in_dev, out_mode, flags, dests, 1, 0, 0, stream);
}

int ltq_layer_forward_scatter(ltq_layer *layer, const uint8_t *x_dev, const int32_t *asum_dev, uint64_t M,
                              const ltq_qparams *qp_in_dev, int out_mode, unsigned flags, void *const *dests, int n_dests,
                              uint64_t ld_out, uint64_t col_offset, void *stream)
{
    LTQ_REQUIRE(ld_out >= 1, LTQ_ERR_INVALID_ARG, "ld_out must be the row length of the destination buffers");
    return layer_forward_impl(layer, x_dev, asum_dev, M, qp_in_dev, out_mode, flags, dests, n_dests, ld_out, col_offset,
                              stream);
}

// ---- buffers that other processes on this node can map (CUDA IPC) -----------------------------------------------------
int ltq_peer_alloc(void **dev_ptr, uint64_t bytes, int device, unsigned char *handle64)
{
    LTQ_REQUIRE(dev_ptr && handle64 && bytes >= 1, LTQ_ERR_INVALID_ARG, "Invalid argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    *dev_ptr = nullptr;
    LTQ_ENTER_DEVICE(device);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        set_error("cudaMalloc of %llu bytes failed: %s", (unsigned long long)bytes, cudaGetErrorString(e));
        return LTQ_ERR_NO_MEMORY;
    }
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        return LTQ_ERR_CUDA;
    }
    memcpy(handle64, &h, sizeof h);
    *dev_ptr = p;
    return LTQ_OK;
}

int ltq_peer_free(void *dev_ptr, int device)
{
    if (!dev_ptr) return LTQ_OK;
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(cudaFree(dev_ptr));
    return LTQ_OK;
}

int ltq_peer_open(const unsigned char *handle64, int device, void **peer_ptr)
{
    LTQ_REQUIRE(handle64 && peer_ptr, LTQ_ERR_INVALID_ARG, "Invalid argument");
    *peer_ptr = nullptr;
    LTQ_ENTER_DEVICE(device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof h);
    LTQ_CUDA_TRY(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return LTQ_OK;
}

int ltq_peer_close(void *peer_ptr, int device)
{
    if (!peer_ptr) return LTQ_OK;
    LTQ_ENTER_DEVICE(device);
    LTQ_CUDA_TRY(cudaIpcCloseMemHandle(peer_ptr));
    return LTQ_OK;
}

// ---- quantized convolution (Conv2d_q) ----------------------------------------------------------------------------------
struct ltq_conv2d {
    int device = 0;
    uint64_t Cin = 0, Cout = 0, kh = 0, kw = 0, ph = 0, pw = 0, sh = 1, sw = 1;
    uint64_t K = 0, Kp = 0;        // patch length C*kh*kw and its 16-byte padded row pitch
    const uint8_t *w = nullptr;    // weights as the GEMM reads them: the caller's buffer, or w_pad when K % 16 != 0
    uint8_t *w_pad = nullptr;      // owned zero-padded copy [Cout, Kp]
    const int32_t *bias = nullptr;
    int32_t *wsum = nullptr;       // [Cout] sums over K of the weights
    uint8_t *col = nullptr;        // transposed patch buffer; grows with the input like Conv2d_q::col_buffer_ptr_
    uint64_t col_cap = 0;          // (l-ten/conv2d.cpp:326-338), but holds several images per pass
    int32_t *colsum = nullptr;     // per-patch sums, the part of Conv2d_q::workspace_ that depends on the input
    uint64_t colsum_cap = 0;
    ltq_qparams qp_in{1.f, 0}, qp_wt{1.f, 0}, qp_out{1.f, 0};
    DeviceState *dev = nullptr;
    // The path without a patch buffer (ltq_conv_direct.cu), where the geometry allows it: the weights reordered to
    // (kernel row, kernel column, channel) with their tensor map, and the NHWC copy of the input, which grows like `col`.
    uint8_t *w_direct = nullptr;
    ltq::ConvDirectPlan direct;
    bool direct_ready = false;
    uint8_t *x_nhwc = nullptr;
    uint64_t x_nhwc_cap = 0;
};

// Patch-buffer budget of one pass over a chunk of the batch.
static constexpr uint64_t CONV_COL_BYTES = 256ull << 20;

int ltq_conv2d_create(ltq_conv2d **conv, int device, uint64_t channels_in, uint64_t channels_out, uint64_t kernel_h,
                      uint64_t kernel_w, uint64_t pad_h, uint64_t pad_w, uint64_t stride_h, uint64_t stride_w)
{
    LTQ_REQUIRE(conv, LTQ_ERR_INVALID_ARG, "Invalid argument");
    *conv = nullptr;
    LTQ_REQUIRE(channels_in >= 1 && channels_out >= 1 && kernel_h >= 1 && kernel_w >= 1 && stride_h >= 1 && stride_w >= 1,
                LTQ_ERR_INVALID_ARG, "channel counts, kernel size and strides must be >= 1");
    const uint64_t lim = 1ull << 20;
    LTQ_REQUIRE(channels_in < lim && channels_out < (1ull << 31) && kernel_h < lim && kernel_w < lim && pad_h < lim &&
                    pad_w < lim && stride_h < lim && stride_w < lim && channels_in * kernel_h * kernel_w < (1ull << 31),
                LTQ_ERR_TOO_LARGE, "convolution geometry out of range");
    LTQ_ENTER_DEVICE(device);
    DeviceState *dev;
    int rc = device_state(device, &dev);
    if (rc != LTQ_OK) return rc;
    ltq_conv2d *c = new (std::nothrow) ltq_conv2d;
    LTQ_REQUIRE(c, LTQ_ERR_NO_MEMORY, "out of host memory");
    c->device = device;
    c->Cin = channels_in;
    c->Cout = channels_out;
    c->kh = kernel_h;
    c->kw = kernel_w;
    c->ph = pad_h;
    c->pw = pad_w;
    c->sh = stride_h;
    c->sw = stride_w;
    c->K = channels_in * kernel_h * kernel_w;
    c->Kp = (c->K + 15) / 16 * 16;
    c->dev = dev;
    cudaError_t e = cudaMalloc(&c->wsum, channels_out * sizeof(int32_t));
    if (e == cudaSuccess && c->Kp != c->K) e = cudaMalloc(&c->w_pad, channels_out * c->Kp);
    if (e == cudaSuccess && conv_direct_plan(&c->direct, channels_in, channels_out, kernel_h, kernel_w, stride_h, stride_w))
        e = cudaMalloc(&c->w_direct, conv_direct_weight_bytes(c->direct, channels_in, kernel_h, kernel_w));
    if (e != cudaSuccess) {
        cudaFree(c->w_pad);
        cudaFree(c->wsum);
        delete c;
        set_error("cudaMalloc of the convolution's weight buffers failed: %s", cudaGetErrorString(e));
        return LTQ_ERR_NO_MEMORY;
    }
    *conv = c;
    return LTQ_OK;
}

int ltq_conv2d_destroy(ltq_conv2d *conv)
{
    if (!conv) return LTQ_OK;
    LTQ_ENTER_DEVICE(conv->device);
    cudaFree(conv->wsum);
    cudaFree(conv->w_pad);
    cudaFree(conv->col);
    cudaFree(conv->colsum);
    cudaFree(conv->w_direct);
    cudaFree(conv->x_nhwc);
    delete conv;
    return LTQ_OK;
}

int ltq_conv2d_set_weights(ltq_conv2d *conv, const uint8_t *w_dev, const int32_t *bias_dev, void *stream)
{
    LTQ_REQUIRE(conv && w_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_ENTER_DEVICE(conv->device);
    cudaStream_t st = (cudaStream_t)stream;
    conv->bias = bias_dev;
    if (conv->w_pad) {
        LTQ_CUDA_TRY(cudaMemsetAsync(conv->w_pad, 0, conv->Cout * conv->Kp, st));
        LTQ_CUDA_TRY(cudaMemcpy2DAsync(conv->w_pad, conv->Kp, w_dev, conv->K, conv->K, conv->Cout, cudaMemcpyDeviceToDevice, st));
        conv->w = conv->w_pad;
    } else {
        conv->w = w_dev;
    }
    LTQ_CUDA_TRY(launch_row_sums(conv->w, conv->Cout, conv->Kp, conv->wsum, st));
    conv->direct_ready = false;
    if (conv->w_direct) {
        LTQ_CUDA_TRY(conv_direct_prepare_weights(w_dev, conv->w_direct, &conv->direct, conv->Cin, conv->kh, conv->kw, st));
        conv->direct_ready = true;
    }
    LTQ_CUDA_TRY(cudaStreamSynchronize(st));
    return LTQ_OK;
}

int ltq_conv2d_set_qparams(ltq_conv2d *conv, const ltq_qparams *qp_in, const ltq_qparams *qp_wt, const ltq_qparams *qp_out)
{
    LTQ_REQUIRE(conv, LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (qp_in) conv->qp_in = *qp_in;
    if (qp_wt) conv->qp_wt = *qp_wt;
    if (qp_out) conv->qp_out = *qp_out;
    return LTQ_OK;
}

int ltq_conv2d_output_size(const ltq_conv2d *conv, uint64_t height_in, uint64_t width_in, uint64_t *height_out,
                           uint64_t *width_out)
{
    LTQ_REQUIRE(conv && height_out && width_out, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(height_in < (1ull << 31) && width_in < (1ull << 31), LTQ_ERR_TOO_LARGE, "image size must be below 2^31");
    LTQ_REQUIRE(height_in + 2 * conv->ph >= conv->kh && width_in + 2 * conv->pw >= conv->kw, LTQ_ERR_INVALID_ARG,
                "padded image (%llu x %llu) smaller than the kernel (%llu x %llu)",
                (unsigned long long)(height_in + 2 * conv->ph), (unsigned long long)(width_in + 2 * conv->pw),
                (unsigned long long)conv->kh, (unsigned long long)conv->kw);
    *height_out = (height_in + 2 * conv->ph - conv->kh) / conv->sh + 1;  // l-ten/conv2d.cpp:313-314
    *width_out = (width_in + 2 * conv->pw - conv->kw) / conv->sw + 1;
    return LTQ_OK;
}

int ltq_conv2d_forward(ltq_conv2d *conv, const uint8_t *x_dev, uint64_t batches, uint64_t height_in, uint64_t width_in,
                       int out_mode, unsigned flags, void *out_dev, void *stream)
{
    LTQ_REQUIRE(conv && (batches == 0 || (x_dev && out_dev)), LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(conv->w, LTQ_ERR_INVALID_ARG, "ltq_conv2d_set_weights has not been called");
    LTQ_REQUIRE(out_mode == LTQ_OUT_U8 || out_mode == LTQ_OUT_F32 || out_mode == LTQ_OUT_I32, LTQ_ERR_INVALID_ARG,
                "unknown out_mode %d", out_mode);
    uint64_t Ho, Wo;
    int rc = ltq_conv2d_output_size(conv, height_in, width_in, &Ho, &Wo);
    if (rc != LTQ_OK) return rc;
    LTQ_REQUIRE(Ho * Wo < (1ull << 31) && batches < (1ull << 31), LTQ_ERR_TOO_LARGE, "output plane or batch too large");
    const uint64_t N = Ho * Wo, M = conv->Cout, K = conv->K, Kp = conv->Kp;
    const bool per_channel = (flags & LTQ_FLAG_BIAS_PER_CHANNEL) != 0;
    // The reference adds bias[j] with j the OUTPUT POSITION (its GEMM's column index, l-ten/math_fns.cpp:1469-1472) out of
    // a tensor that holds channels_out values, which is only defined while Ho*Wo <= channels_out.
    LTQ_REQUIRE(!conv->bias || per_channel || N <= M, LTQ_ERR_UNSUPPORTED,
                "the reference indexes the bias by output position and would read %llu values from a %llu-element tensor; "
                "pass LTQ_FLAG_BIAS_PER_CHANNEL for one bias per output channel",
                (unsigned long long)N, (unsigned long long)M);
    const uint64_t bc = K * (uint64_t)conv->qp_wt.zero_point * (uint64_t)conv->qp_in.zero_point;
    LTQ_REQUIRE(bc <= 0x7FFFFFFFull, LTQ_ERR_UNSUPPORTED, "K*zA*zB = %llu does not fit an int", (unsigned long long)bc);
    if (batches == 0 || N == 0) return LTQ_OK;
    LTQ_ENTER_DEVICE(conv->device);
    cudaStream_t st = (cudaStream_t)stream;

    // Without a patch buffer where the geometry allows (and no kernel is forced, and the bias is per channel or absent):
    // transpose the input to NHWC, then one kernel for the whole batch.
    const bool nhwc_in = (flags & LTQ_FLAG_NHWC_IN) != 0, nhwc_out = (flags & LTQ_FLAG_NHWC_OUT) != 0;
    const bool direct = conv->direct_ready && !(flags & (LTQ_FLAG_FORCE_SIMT | LTQ_FLAG_FORCE_TC | LTQ_FLAG_FORCE_SKINNY)) &&
                        conv_direct_shape_ok(conv->direct, batches, conv->Cin, conv->kh, conv->kw, conv->ph, conv->pw, height_in,
                                             width_in, Ho, Wo);
    LTQ_REQUIRE(!(nhwc_in || nhwc_out) || (direct && conv->Cin % 64 == 0 && conv->Cout % 16 == 0 && (!nhwc_in || (conv->sh == 1 && conv->sw == 1))),
                LTQ_ERR_UNSUPPORTED,
                "channels-last input / output is only available for the layers computed without a patch buffer, with input "
                "channels a multiple of 64 and output channels a multiple of 16 (input: strides 1), and no forced kernel");
    LTQ_REQUIRE(!nhwc_in || ((uintptr_t)x_dev & 15) == 0, LTQ_ERR_INVALID_ARG, "a channels-last input must be 16-byte aligned");
    LTQ_REQUIRE(!nhwc_out || ((uintptr_t)out_dev & 15) == 0, LTQ_ERR_INVALID_ARG, "a channels-last output must be 16-byte aligned");
    if (direct) {
        const uint8_t *x_cl = x_dev;
        // an NCHW input with strides 1 and whole words per row is transposed by the kernel itself while it loads
        const bool gather = !nhwc_in && conv_direct_gather_ok(conv->direct, conv->Cin, conv->kh, conv->kw, conv->ph, conv->pw, width_in,
                                                              Wo, x_dev);
        if (!nhwc_in && !gather) {
            rc = grow(&conv->x_nhwc, &conv->x_nhwc_cap, conv_direct_input_bytes(conv->direct, batches, conv->Cin, height_in, width_in), st,
                      "the NHWC copy of the input");
            if (rc != LTQ_OK) return rc;
            LTQ_CUDA_TRY(launch_nchw_to_nhwc(x_dev, conv->x_nhwc, conv->direct, batches, conv->Cin, height_in, width_in, st));
            x_cl = conv->x_nhwc;
        }
        // positions are the rows here: A = input (its patch sums come out of the kernel), B = weights
        // (bias per channel = per column here; the reference's indexing by output position = per row)
        Epilogue epi = make_epilogue(conv->wsum, nullptr, per_channel ? conv->bias : nullptr, conv->qp_in, conv->qp_wt, conv->qp_out, K,
                                     out_mode, flags);
        epi.row_bias = per_channel ? nullptr : conv->bias;
        LTQ_CUDA_TRY(launch_conv_direct(x_cl, conv->direct, batches, conv->Cin, height_in, width_in, conv->Cout, conv->kh,
                                        conv->kw, conv->ph, conv->pw, Ho, Wo, epi, out_dev, nhwc_out, conv->dev->status,
                                        conv->dev->sms, st, gather));
        return LTQ_OK;
    }

    uint64_t chunk = CONV_COL_BYTES / (N * Kp);
    chunk = chunk < 1 ? 1 : (chunk > batches ? batches : chunk);
    rc = grow(&conv->col, &conv->col_cap, chunk * N * Kp, st, "the patch buffer");
    if (rc != LTQ_OK) return rc;
    rc = grow(&conv->colsum, &conv->colsum_cap, chunk * N, st, "the patch sums");
    if (rc != LTQ_OK) return rc;

    ConvGeom g;
    g.C = (uint32_t)conv->Cin;
    g.H = (uint32_t)height_in;
    g.W = (uint32_t)width_in;
    g.kh = (uint32_t)conv->kh;
    g.kw = (uint32_t)conv->kw;
    g.ph = (uint32_t)conv->ph;
    g.pw = (uint32_t)conv->pw;
    g.sh = (uint32_t)conv->sh;
    g.sw = (uint32_t)conv->sw;
    g.Ho = (uint32_t)Ho;
    g.Wo = (uint32_t)Wo;
    g.K = (uint32_t)K;
    g.Kp = (uint32_t)Kp;
    const uint64_t in_stride = conv->Cin * height_in * width_in;
    const uint64_t esize = out_mode == LTQ_OUT_U8 ? 1 : 4, out_stride = M * N * esize;
    for (uint64_t b0 = 0; b0 < batches; b0 += chunk) {
        const uint64_t nb = batches - b0 < chunk ? batches - b0 : chunk;
        LTQ_CUDA_TRY(launch_im2col_t_sums(x_dev + b0 * in_stride, nb, g, conv->col, conv->colsum, st));
        // out[co, n] = weights[co, :] . patch[n, :]: the weights are the row operand (qparams[0] in the reference's call,
        // l-ten/conv2d.cpp:348-350), the patches the column operand.  When an image's Ho*Wo positions are a multiple of
        // 32 the patches of the whole chunk are ONE GEMM with N = nb*Ho*Wo whose epilogue writes column block b (image b)
        // at out[b]; otherwise one GEMM per image.
        // (the reference's per-position bias indexes by the position inside ONE image, so it keeps the per-image form)
        const bool batched = (N % 32 == 0) && nb > 1 && nb * N < (1ull << 31) && (per_channel || !conv->bias);
        const uint64_t groups = batched ? 1 : nb, per = batched ? nb : 1;
        for (uint64_t i = 0; i < groups; i++) {
            Epilogue epi = make_epilogue(conv->colsum + i * N, conv->wsum, per_channel ? nullptr : conv->bias, conv->qp_wt,
                                         conv->qp_in, conv->qp_out, K, out_mode, flags);
            epi.row_bias = per_channel ? conv->bias : nullptr;
            if (batched) {
                epi.ldc = N;
                epi.col_block = (uint32_t)N;
                epi.col_block_stride = M * N;
            }
            rc = run_fc_gemm(*conv->dev, M, per * N, Kp, conv->w, conv->col + i * N * Kp, epi,
                             static_cast<uint8_t *>(out_dev) + (b0 + i) * out_stride, flags, nullptr, st);
            if (rc != LTQ_OK) return rc;
        }
    }
    return LTQ_OK;
}

int ltq_im2col_t_u8(const uint8_t *im_dev, uint64_t batches, uint64_t channels, uint64_t height, uint64_t width,
                    uint64_t kernel_h, uint64_t kernel_w, uint64_t pad_h, uint64_t pad_w, uint64_t stride_h,
                    uint64_t stride_w, uint8_t *col_t_dev, uint64_t row_pitch, int device, void *stream)
{
    LTQ_REQUIRE(im_dev && col_t_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(kernel_h >= 1 && kernel_w >= 1 && stride_h >= 1 && stride_w >= 1 && channels >= 1, LTQ_ERR_INVALID_ARG,
                "channel count, kernel size and strides must be >= 1");
    const uint64_t lim = 1ull << 20;
    LTQ_REQUIRE(channels < lim && kernel_h < lim && kernel_w < lim && pad_h < lim && pad_w < lim && stride_h < lim &&
                    stride_w < lim && height < (1ull << 31) && width < (1ull << 31) &&
                    channels * kernel_h * kernel_w < (1ull << 31),
                LTQ_ERR_TOO_LARGE, "convolution geometry out of range");
    LTQ_REQUIRE(height + 2 * pad_h >= kernel_h && width + 2 * pad_w >= kernel_w, LTQ_ERR_INVALID_ARG,
                "padded image smaller than the kernel");
    const uint64_t K = channels * kernel_h * kernel_w;
    LTQ_REQUIRE(row_pitch % 16 == 0 && row_pitch >= K && row_pitch < K + 16 && (((uintptr_t)col_t_dev & 15) == 0),
                LTQ_ERR_INVALID_ARG, "row_pitch must be C*kh*kw rounded up to a multiple of 16 and the buffer 16-byte aligned");
    LTQ_ENTER_DEVICE(device);
    ConvGeom g;
    g.C = (uint32_t)channels;
    g.H = (uint32_t)height;
    g.W = (uint32_t)width;
    g.kh = (uint32_t)kernel_h;
    g.kw = (uint32_t)kernel_w;
    g.ph = (uint32_t)pad_h;
    g.pw = (uint32_t)pad_w;
    g.sh = (uint32_t)stride_h;
    g.sw = (uint32_t)stride_w;
    g.Ho = (uint32_t)((height + 2 * pad_h - kernel_h) / stride_h + 1);
    g.Wo = (uint32_t)((width + 2 * pad_w - kernel_w) / stride_w + 1);
    g.K = (uint32_t)K;
    g.Kp = (uint32_t)row_pitch;
    LTQ_REQUIRE((uint64_t)g.Ho * g.Wo < (1ull << 31), LTQ_ERR_TOO_LARGE, "output plane too large");
    LTQ_CUDA_TRY(launch_im2col_t(im_dev, batches, g, col_t_dev, (cudaStream_t)stream));
    return LTQ_OK;
}

int ltq_device_check(int device, void *stream)
{
    LTQ_ENTER_DEVICE(device);
    DeviceState *dev;
    int rc = device_state(device, &dev);
    if (rc != LTQ_OK) return rc;
    uint32_t code = 0;
    LTQ_CUDA_TRY(cudaMemcpyAsync(&code, dev->status, sizeof code, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    LTQ_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    if (code) {
        LTQ_CUDA_TRY(cudaMemsetAsync(dev->status, 0, sizeof code, (cudaStream_t)stream));
        set_error("a bounded device-side wait expired (code 0x%x: role %u, slot %u)", code, code >> 8, code & 0xFF);
        return LTQ_ERR_DEVICE_TIMEOUT;
    }
    return LTQ_OK;
}

int ltq_layer_check(ltq_layer *layer, void *stream)
{
    LTQ_REQUIRE(layer, LTQ_ERR_INVALID_ARG, "Invalid argument");
    return ltq_device_check(layer->device, stream);
}

int ltq_selftest_bounded_wait(int device, uint32_t limit_us, void *stream)
{
    LTQ_REQUIRE(limit_us >= 1 && limit_us <= 1000000, LTQ_ERR_INVALID_ARG, "limit must be between 1 us and 1 s");
    LTQ_ENTER_DEVICE(device);
    DeviceState *dev;
    int rc = device_state(device, &dev);
    if (rc != LTQ_OK) return rc;
    LTQ_CUDA_TRY(launch_bounded_wait_probe(dev->status, (uint64_t)limit_us * 1000ull, (cudaStream_t)stream));
    return LTQ_OK;
}

}  // extern "C"
