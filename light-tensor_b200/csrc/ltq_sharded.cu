// Multi-device entry points for callers that drive every GPU of a box from ONE host thread, the way l-ten itself is
// written (single-threaded API, a device index per tensor, handle arrays of MAX_DEVICES = 8, l-ten/globals.h:15,89-124):
//
//   ltq_comm_init_all / ltq_comm_destroy          one NCCL communicator and one stream per device
//   ltq_linear_forward_rowsharded                 activation rows split over the devices, weights replicated: one
//                                                 ltq_layer_forward per device, nothing exchanged
//   ltq_comm_allreduce_minmax                     the only exchange row sharding ever needs (dynamic quantisation)
//   ltq_linear_forward_colsharded_allgather       weight rows (output columns) split over the devices: per-device
//                                                 forward, ncclAllGather of the slices inside one group, relayout
//   ltq_comm_synchronize                          host-side watchdog: waits for the devices' streams, polls the
//                                                 communicators for asynchronous errors, aborts them on error or timeout
//
// NCCL is bound at run time (dlopen of libnccl.so.2 on first use), so the library itself has no link dependency on it
// and single-device users never load it.  Everything NCCL- or stream-related goes through a table of function pointers
// (ltq_comm_backend) that tests replace with a fake to drive the watchdog and the argument checks without any GPU.
#include <dlfcn.h>
#include <string.h>

#include <chrono>
#include <mutex>
#include <new>
#include <thread>

#include "ltq_common.cuh"
#include "ltq_layer.cuh"

namespace {

// ---- NCCL through dlopen ----------------------------------------------------------------------------------------------
// The few declarations needed, as NCCL 2.x's nccl.h gives them (opaque communicator, int result, enum values).
typedef void *nccl_comm_t;
typedef int (*fn_comm_init_all)(nccl_comm_t *, int, const int *);
typedef int (*fn_comm_op)(nccl_comm_t);
typedef int (*fn_comm_async)(nccl_comm_t, int *);
typedef int (*fn_all_gather)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t);
typedef int (*fn_all_reduce)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t);
typedef int (*fn_void)(void);
typedef const char *(*fn_errstr)(int);
constexpr int NCCL_UINT8 = 1, NCCL_FLOAT32 = 7, NCCL_MAX = 2, NCCL_MIN = 3;

struct NcclLib {
    void *handle = nullptr;
    fn_comm_init_all comm_init_all = nullptr;
    fn_comm_op comm_destroy = nullptr, comm_abort = nullptr;
    fn_comm_async comm_get_async_error = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_all_reduce all_reduce = nullptr;
    fn_void group_start = nullptr, group_end = nullptr;
    fn_errstr error_string = nullptr;
    bool tried = false;
};
NcclLib g_nccl;
std::mutex g_nccl_mu;

bool nccl_load()
{
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (g_nccl.tried) return g_nccl.handle != nullptr;
    g_nccl.tried = true;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);  // the copy a host framework already loaded, if any
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return false;
#define LTQ_SYM(field, type, name)                        \
    g_nccl.field = reinterpret_cast<type>(dlsym(h, name)); \
    if (!g_nccl.field) {                                   \
        dlclose(h);                                        \
        return false;                                      \
    }
    LTQ_SYM(comm_init_all, fn_comm_init_all, "ncclCommInitAll")
    LTQ_SYM(comm_destroy, fn_comm_op, "ncclCommDestroy")
    LTQ_SYM(comm_abort, fn_comm_op, "ncclCommAbort")
    LTQ_SYM(comm_get_async_error, fn_comm_async, "ncclCommGetAsyncError")
    LTQ_SYM(all_gather, fn_all_gather, "ncclAllGather")
    LTQ_SYM(all_reduce, fn_all_reduce, "ncclAllReduce")
    LTQ_SYM(group_start, fn_void, "ncclGroupStart")
    LTQ_SYM(group_end, fn_void, "ncclGroupEnd")
    LTQ_SYM(error_string, fn_errstr, "ncclGetErrorString")
#undef LTQ_SYM
    g_nccl.handle = h;
    return true;
}

// ---- default backend: NCCL + CUDA streams -------------------------------------------------------------------------------
int def_comm_init_all(void **comms, int ndev, const int *devices)
{
    if (!nccl_load()) return -1000;
    return g_nccl.comm_init_all(comms, ndev, devices);
}
int def_comm_destroy(void *c) { return g_nccl.comm_destroy(c); }
int def_comm_abort(void *c) { return g_nccl.comm_abort(c); }
int def_comm_async(void *c, int *err) { return g_nccl.comm_get_async_error(c, err); }
int def_all_gather(const void *send, void *recv, uint64_t bytes, void *c, void *stream)
{
    return g_nccl.all_gather(send, recv, (size_t)bytes, NCCL_UINT8, c, (cudaStream_t)stream);
}
int def_all_reduce_f32(const void *send, void *recv, uint64_t count, int op, void *c, void *stream)
{
    return g_nccl.all_reduce(send, recv, (size_t)count, NCCL_FLOAT32, op == 0 ? NCCL_MIN : NCCL_MAX, c, (cudaStream_t)stream);
}
int def_group_start(void) { return g_nccl.group_start(); }
int def_group_end(void) { return g_nccl.group_end(); }
int def_stream_create(int device, void **stream)
{
    ltq::DeviceGuard g(device);
    if (g.err != cudaSuccess) return (int)g.err;
    cudaStream_t s = nullptr;
    const cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    *stream = s;
    return (int)e;
}
int def_stream_destroy(int device, void *stream)
{
    ltq::DeviceGuard g(device);
    return (int)cudaStreamDestroy((cudaStream_t)stream);
}
int def_stream_query(int device, void *stream)
{
    ltq::DeviceGuard g(device);
    const cudaError_t e = cudaStreamQuery((cudaStream_t)stream);
    if (e == cudaSuccess) return 0;
    if (e == cudaErrorNotReady) return 1;
    return -(int)e;
}
const char *def_error_string(int code)
{
    if (code == -1000) return "libnccl.so.2 could not be loaded";
    return g_nccl.error_string ? g_nccl.error_string(code) : "NCCL error";
}

const ltq_comm_backend g_default_backend = {def_comm_init_all, def_comm_destroy,  def_comm_abort,    def_comm_async,
                                            def_all_gather,    def_all_reduce_f32, def_group_start,   def_group_end,
                                            def_stream_create, def_stream_destroy, def_stream_query,  def_error_string};
ltq_comm_backend g_backend = g_default_backend;
bool g_backend_is_default = true;

}  // namespace

struct ltq_comm {
    int ndev = 0;
    int devices[LTQ_MAX_DESTS] = {0};
    void *comms[LTQ_MAX_DESTS] = {nullptr};
    void *streams[LTQ_MAX_DESTS] = {nullptr};
    bool aborted = false;
    ltq_comm_backend be;
    bool real_devices = true;  // false with a test backend: no CUDA call is made on the devices
};

using namespace ltq;

#define LTQ_BE_TRY(comm, expr, what)                                                                         \
    do {                                                                                                     \
        const int rc__ = (expr);                                                                             \
        if (rc__ != 0) {                                                                                     \
            set_error("%s failed: %s (code %d)", what, (comm)->be.error_string ? (comm)->be.error_string(rc__) : "?", rc__); \
            return LTQ_ERR_CUDA;                                                                             \
        }                                                                                                    \
    } while (0)

static int check_comm(const ltq_comm *comm)
{
    LTQ_REQUIRE(comm, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(!comm->aborted, LTQ_ERR_CUDA, "the communicators of this group were aborted (an earlier error or time-out); destroy it");
    return LTQ_OK;
}

extern "C" {

int ltq_comm_set_backend(const ltq_comm_backend *backend)
{
    if (!backend) {
        g_backend = g_default_backend;
        g_backend_is_default = true;
        return LTQ_OK;
    }
    LTQ_REQUIRE(backend->comm_init_all && backend->comm_destroy && backend->comm_abort && backend->comm_get_async_error &&
                    backend->all_gather && backend->all_reduce_f32 && backend->group_start && backend->group_end &&
                    backend->stream_create && backend->stream_destroy && backend->stream_query,
                LTQ_ERR_INVALID_ARG, "every entry of the backend table but error_string must be set");
    g_backend = *backend;
    g_backend_is_default = false;
    return LTQ_OK;
}

int ltq_comm_init_all(ltq_comm **comm, int ndev, const int *devices)
{
    LTQ_REQUIRE(comm, LTQ_ERR_INVALID_ARG, "Invalid argument");
    *comm = nullptr;
    LTQ_REQUIRE(ndev >= 1 && ndev <= LTQ_MAX_DESTS, LTQ_ERR_INVALID_ARG, "ndev must be between 1 and %d", LTQ_MAX_DESTS);
    ltq_comm *c = new (std::nothrow) ltq_comm;
    LTQ_REQUIRE(c, LTQ_ERR_NO_MEMORY, "out of host memory");
    c->ndev = ndev;
    c->be = g_backend;
    c->real_devices = g_backend_is_default;
    for (int d = 0; d < ndev; d++) {
        c->devices[d] = devices ? devices[d] : d;
        for (int p = 0; p < d; p++)
            if (c->devices[p] == c->devices[d]) {
                delete c;
                set_error("device %d appears twice", devices[d]);
                return LTQ_ERR_INVALID_ARG;
            }
    }
    int rc = c->be.comm_init_all(c->comms, ndev, c->devices);
    if (rc != 0) {
        set_error("ncclCommInitAll failed: %s (code %d)", c->be.error_string ? c->be.error_string(rc) : "?", rc);
        delete c;
        return LTQ_ERR_CUDA;
    }
    for (int d = 0; d < ndev; d++) {
        rc = c->be.stream_create(c->devices[d], &c->streams[d]);
        if (rc != 0) {
            set_error("cannot create a stream on device %d (code %d)", c->devices[d], rc);
            for (int p = 0; p < d; p++) c->be.stream_destroy(c->devices[p], c->streams[p]);
            for (int p = 0; p < ndev; p++) c->be.comm_destroy(c->comms[p]);
            delete c;
            return LTQ_ERR_CUDA;
        }
    }
    *comm = c;
    return LTQ_OK;
}

int ltq_comm_destroy(ltq_comm *comm)
{
    if (!comm) return LTQ_OK;
    for (int d = 0; d < comm->ndev; d++) {
        if (comm->streams[d]) comm->be.stream_destroy(comm->devices[d], comm->streams[d]);
        if (comm->comms[d] && !comm->aborted) comm->be.comm_destroy(comm->comms[d]);  // aborted ones are already gone
    }
    delete comm;
    return LTQ_OK;
}

int ltq_comm_size(const ltq_comm *comm) { return comm ? comm->ndev : 0; }

int ltq_comm_device(const ltq_comm *comm, int index)
{
    return (comm && index >= 0 && index < comm->ndev) ? comm->devices[index] : -1;
}

void *ltq_comm_stream(const ltq_comm *comm, int index)
{
    return (comm && index >= 0 && index < comm->ndev) ? comm->streams[index] : nullptr;
}

int ltq_comm_synchronize(ltq_comm *comm, uint32_t timeout_ms)
{
    int rc = check_comm(comm);
    if (rc != LTQ_OK) return rc;
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        bool busy = false;
        for (int d = 0; d < comm->ndev; d++) {
            const int q = comm->be.stream_query(comm->devices[d], comm->streams[d]);
            if (q < 0) {
                set_error("the stream of device %d reports an error (code %d)", comm->devices[d], -q);
                return LTQ_ERR_CUDA;
            }
            busy = busy || q > 0;
        }
        if (!busy) return LTQ_OK;
        // a communicator that failed asynchronously never finishes its collectives: abort all of them, so that the
        // kernels waiting in them return and the streams drain
        int failed = 0, failed_dev = -1;
        for (int d = 0; d < comm->ndev && !failed; d++) {
            int async = 0;
            const int r = comm->be.comm_get_async_error(comm->comms[d], &async);
            if (r != 0 || async != 0) {
                failed = r != 0 ? r : async;
                failed_dev = comm->devices[d];
            }
        }
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        const bool timed_out = timeout_ms != 0 && (uint64_t)ms >= timeout_ms;
        if (failed || timed_out) {
            for (int d = 0; d < comm->ndev; d++) comm->be.comm_abort(comm->comms[d]);
            comm->aborted = true;
            if (failed) {
                set_error("communicator of device %d failed asynchronously: %s (code %d); all communicators aborted", failed_dev,
                          comm->be.error_string ? comm->be.error_string(failed) : "?", failed);
                return LTQ_ERR_CUDA;
            }
            set_error("the devices' streams did not drain within %u ms; all communicators aborted", timeout_ms);
            return LTQ_ERR_DEVICE_TIMEOUT;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int ltq_comm_allreduce_minmax(ltq_comm *comm, float *const *minmax_dev)
{
    int rc = check_comm(comm);
    if (rc != LTQ_OK) return rc;
    LTQ_REQUIRE(minmax_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    for (int d = 0; d < comm->ndev; d++) LTQ_REQUIRE(minmax_dev[d], LTQ_ERR_INVALID_ARG, "Invalid argument");
    if (comm->ndev == 1) return LTQ_OK;
    LTQ_BE_TRY(comm, comm->be.group_start(), "ncclGroupStart");
    for (int d = 0; d < comm->ndev; d++) {
        LTQ_BE_TRY(comm, comm->be.all_reduce_f32(minmax_dev[d], minmax_dev[d], 1, 0, comm->comms[d], comm->streams[d]),
                   "ncclAllReduce(min)");
        LTQ_BE_TRY(comm, comm->be.all_reduce_f32(minmax_dev[d] + 1, minmax_dev[d] + 1, 1, 1, comm->comms[d], comm->streams[d]),
                   "ncclAllReduce(max)");
    }
    LTQ_BE_TRY(comm, comm->be.group_end(), "ncclGroupEnd");
    return LTQ_OK;
}

static int check_layers(const ltq_comm *comm, ltq_layer *const *layers, bool same_n)
{
    LTQ_REQUIRE(layers, LTQ_ERR_INVALID_ARG, "Invalid argument");
    for (int d = 0; d < comm->ndev; d++) {
        LTQ_REQUIRE(layers[d], LTQ_ERR_INVALID_ARG, "Invalid argument");
        LTQ_REQUIRE(layers[d]->device == comm->devices[d], LTQ_ERR_INVALID_ARG,
                    "layer %d lives on device %d, the group's device %d is %d", d, layers[d]->device, d, comm->devices[d]);
        LTQ_REQUIRE(layers[d]->K == layers[0]->K && (!same_n || layers[d]->N == layers[0]->N), LTQ_ERR_INVALID_ARG,
                    "layer %d has other dimensions than layer 0", d);
    }
    return LTQ_OK;
}

int ltq_linear_forward_rowsharded(ltq_comm *comm, ltq_layer *const *layers, const uint8_t *const *x_dev,
                                  const int32_t *const *asum_dev, const uint64_t *rows, const ltq_qparams *const *qp_in_dev,
                                  int out_mode, unsigned flags, void *const *out_dev)
{
    int rc = check_comm(comm);
    if (rc != LTQ_OK) return rc;
    LTQ_REQUIRE(x_dev && rows && out_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    rc = check_layers(comm, layers, true);
    if (rc != LTQ_OK) return rc;
    for (int d = 0; d < comm->ndev; d++) {
        if (rows[d] == 0) continue;
        rc = ltq_layer_forward(layers[d], x_dev[d], asum_dev ? asum_dev[d] : nullptr, rows[d], qp_in_dev ? qp_in_dev[d] : nullptr,
                               out_mode, flags, out_dev[d], comm->streams[d]);
        if (rc != LTQ_OK) return rc;
    }
    return LTQ_OK;
}

int ltq_linear_forward_colsharded_allgather(ltq_comm *comm, ltq_layer *const *layers, const uint8_t *const *x_dev,
                                            const int32_t *const *asum_dev, uint64_t M, const ltq_qparams *const *qp_in_dev,
                                            int out_mode, unsigned flags, void *const *local_dev, void *const *gathered_dev,
                                            void *const *out_dev)
{
    int rc = check_comm(comm);
    if (rc != LTQ_OK) return rc;
    LTQ_REQUIRE(x_dev && local_dev && out_dev && (comm->ndev == 1 || gathered_dev), LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(out_mode == LTQ_OUT_U8 || out_mode == LTQ_OUT_F32 || out_mode == LTQ_OUT_I32, LTQ_ERR_INVALID_ARG,
                "unknown out_mode %d", out_mode);
    rc = check_layers(comm, layers, true);  // equal slices: the all-gather wants equal contributions
    if (rc != LTQ_OK) return rc;
    if (M == 0) return LTQ_OK;
    const uint64_t esize = out_mode == LTQ_OUT_U8 ? 1 : 4, n_loc = layers[0]->N, slice_bytes = M * n_loc * esize;
    // this device's columns: straight into `out` when there is nothing to gather
    for (int d = 0; d < comm->ndev; d++) {
        rc = ltq_layer_forward(layers[d], x_dev[d], asum_dev ? asum_dev[d] : nullptr, M, qp_in_dev ? qp_in_dev[d] : nullptr,
                               out_mode, flags, comm->ndev == 1 ? out_dev[d] : local_dev[d], comm->streams[d]);
        if (rc != LTQ_OK) return rc;
    }
    if (comm->ndev == 1) return LTQ_OK;
    LTQ_BE_TRY(comm, comm->be.group_start(), "ncclGroupStart");
    for (int d = 0; d < comm->ndev; d++)
        LTQ_BE_TRY(comm, comm->be.all_gather(local_dev[d], gathered_dev[d], slice_bytes, comm->comms[d], comm->streams[d]),
                   "ncclAllGather");
    LTQ_BE_TRY(comm, comm->be.group_end(), "ncclGroupEnd");
    // [ndev][M][n_loc] -> row-major [M][ndev * n_loc]
    for (int d = 0; d < comm->ndev; d++) {
        rc = ltq_interleave_column_blocks(gathered_dev[d], out_dev[d], (uint64_t)comm->ndev, M, n_loc * esize, comm->devices[d],
                                          comm->streams[d]);
        if (rc != LTQ_OK) return rc;
    }
    return LTQ_OK;
}

}  // extern "C"
