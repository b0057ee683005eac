/*
 * ltq — B200 (sm_100a) CUDA implementation of l-ten's uint8 quantized
 * fully-connected forward path, behind a C ABI.
 *
 * Every pointer named *_dev is device memory on `device`; everything else is
 * host memory.  All entry points return 0 on success or a negative ltq_status;
 * ltq_last_error() gives the message of the calling thread's last failure.
 * No exception crosses this boundary and no entry point has a CPU fallback:
 * without a usable CUDA device every compute call fails with
 * LTQ_ERR_CUDA.
 *
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 * stream, which keeps ordering with l-ten's own synchronous CUDA calls).
 * Work is enqueued on it and the call returns without synchronising unless
 * stated otherwise.
 *
 * Reference interfaces are cited as file:line inside the l-ten project.
 */
#ifndef LTQ_H
#define LTQ_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LTQ_VERSION 1

/* Mirrors `struct QuantizationParams`, l-ten/math_fns.h:12-16 (same layout:
 * float at 0, uint8 at 4, size 8): real = scale * (q - zero_point). */
typedef struct ltq_qparams {
    float scale;
    uint8_t zero_point;
} ltq_qparams;

typedef enum ltq_status {
    LTQ_OK = 0,
    LTQ_ERR_INVALID_ARG = -1,   /* null pointer, bad size, bad enum */
    LTQ_ERR_UNSUPPORTED = -2,   /* alpha != 1 / beta != 0 (l-ten/math_fns.cpp:1331-1334), K*255^2 overflow */
    LTQ_ERR_CUDA = -3,          /* a CUDA runtime/driver call failed; message has the CUDA error string */
    LTQ_ERR_DEVICE_TIMEOUT = -4,/* a bounded device-side wait gave up (status word read back on request) */
    LTQ_ERR_NO_MEMORY = -5,
    LTQ_ERR_TOO_LARGE = -6      /* size beyond a documented fixed limit */
} ltq_status;

/* What the epilogue writes (out_dev element type follows). */
typedef enum ltq_out_mode {
    LTQ_OUT_U8 = 0,  /* (uchar)(rm*acc + z_out), rm = s_a*s_w/s_out — the reference's only mode, l-ten/math_fns.cpp:1436,1474 */
    LTQ_OUT_F32 = 1, /* (s_a*s_w) * (float)acc — what Dequantize would recover, without the uint8 round trip */
    LTQ_OUT_I32 = 2  /* acc itself: sum (a-z_a)(w-z_w) + bias, l-ten/math_fns.cpp:1469-1473 */
} ltq_out_mode;

/* Epilogue flags (bit-or). */
#define LTQ_FLAG_RELU 1u     /* acc = max(acc,0) before scaling; no counterpart in the reference (its relu is float-only) */
#define LTQ_FLAG_SATURATE 2u /* U8 cast clamps to [0,255]. Default (flag clear) reproduces the reference build's cast:
                                truncate toward zero, keep the low byte when out of range */
/* Kernel selection override, for tests and profiling (default: by shape). */
#define LTQ_FLAG_BIAS_PER_CHANNEL 4u /* ltq_conv2d_forward only: bias[c] per output channel instead of the reference's
                                       indexing by output position (see ltq_conv2d_forward) */
#define LTQ_MAX_DESTS 8  /* destinations of one ltq_layer_forward_scatter call (this GPU's buffer + 7 peers) */
#define LTQ_FLAG_FORCE_SIMT 0x100u  /* generic dp4a tile kernel */
#define LTQ_FLAG_FORCE_TC 0x200u    /* tcgen05 kernel (needs K % 16 == 0) */
#define LTQ_FLAG_FORCE_TC_PAIR 0x800u   /* with the tcgen05 path: the 2-CTA (cta_group::2) 256 x 256 tile kernel */
#define LTQ_FLAG_FORCE_TC_SINGLE 0x1000u/* with the tcgen05 path: the single-CTA kernel */
#define LTQ_FLAG_FORCE_SKINNY 0x400u/* weight-streaming kernel (needs M <= 16, K % 128 == 0) */
#define LTQ_FLAG_MULTICAST_DEST 0x2000u /* ltq_layer_forward_scatter only: dests[0] is an NVLink multicast address */
#define LTQ_FLAG_NHWC_IN 0x4000u   /* ltq_conv2d_forward only: x_dev is [batches, height, width, channels] */
#define LTQ_FLAG_NHWC_OUT 0x8000u  /* ltq_conv2d_forward only: out_dev is [batches, height_out, width_out, channels_out] */

int ltq_version(void);
const char *ltq_last_error(void);
/* Number of kernels this library has launched since load (all threads). */
uint64_t ltq_kernel_launches(void);
/* Name of the GEMM kernel the calling thread launched last, with its template arguments (tile width, output type), e.g.
 * "gemm_tc_pair_kernel<256,u8>"; "" before the first one.  For tests, profiling and benchmark records: it names what
 * the shape-based dispatch of ltq_layer_forward / ltq_quantized_matmul* actually chose.  No counterpart in the
 * reference. */
const char *ltq_last_kernel(void);

/* ---- quantisation helpers (replace l-ten/utils.h:23-27 for device data) -------------------------------------- */

/* GetMinMax, l-ten/utils.cpp:198-226.  minmax_dev[0]=min, [1]=max (floats, device).  len >= 1.  NaNs behave as in the
 * reference's compare-and-replace loop: a NaN in data[0] makes both results NaN, NaNs elsewhere are skipped.  When the
 * minimum or maximum is a zero and the data hold zeros of both signs, the reference returns the one met first; which of
 * the two this call returns is unspecified (they are equal as numbers, and ComputeQuantizationParams maps both to the
 * same result). */
int ltq_get_min_max(const float *data_dev, uint64_t len, float *minmax_dev, int device, void *stream);

/* ComputeQuantizationParams, l-ten/utils.cpp:266-286.  Pure host arithmetic on two scalars.
 * Returns LTQ_ERR_INVALID_ARG when the widened range is empty (min = max = 0), where the reference divides by 0. */
int ltq_compute_qparams(float min_val, float max_val, ltq_qparams *qp);

/* Same rule evaluated on the device from minmax_dev into qp_dev (no host round trip). */
int ltq_compute_qparams_dev(const float *minmax_dev, ltq_qparams *qp_dev, int device, void *stream);

/* Quantize(float*, uint8_t*, len, qp), l-ten/utils.cpp:243-254. */
int ltq_quantize_u8(const float *data_dev, uint8_t *q_dev, uint64_t len, const ltq_qparams *qp, int device,
                    void *stream);
/* Quantize(float*, int*, len, qp), l-ten/utils.cpp:228-241 (bias: scale s_in*s_wt, zero point 0). */
int ltq_quantize_i32(const float *data_dev, int32_t *q_dev, uint64_t len, const ltq_qparams *qp, int device,
                     void *stream);
/* Dequantize(float*, uint8_t*, len, qp), l-ten/utils.cpp:256-264. */
int ltq_dequantize(float *data_dev, const uint8_t *q_dev, uint64_t len, const ltq_qparams *qp, int device,
                   void *stream);

/* Activation quantise step fused with the per-row sums the GEMM epilogue needs: q = Quantize(x) over [M,K] and
 * asum[i] = sum_k q[i,k] (the col_vector of l-ten/math_fns.cpp:1372-1380 before its -z_w factor).
 * Exactly one of qp (host) / qp_dev (device, e.g. from ltq_compute_qparams_dev) must be non-NULL. */
int ltq_quantize_rows_u8(const float *x_dev, uint64_t M, uint64_t K, const ltq_qparams *qp, const ltq_qparams *qp_dev,
                         uint8_t *q_dev, int32_t *asum_dev, int device, void *stream);

/* Per-row sums of a uint8 [rows, cols] matrix into int32 [rows] (row_vector / col_vector of
 * l-ten/math_fns.cpp:1362-1380 before their -z factors). */
int ltq_row_sums_u8(const uint8_t *m_dev, uint64_t rows, uint64_t cols, int32_t *sums_dev, int device, void *stream);

/* Column (N) sharding support; no counterpart in the reference, which has no multi-device code at all.  After an
 * all-gather of per-rank output slices [M, N/parts] the data sits as [parts][M][part_row_bytes]; this writes the
 * row-major [M][parts * part_row_bytes] that the next layer (or the caller) expects.  Element type does not matter:
 * part_row_bytes = (N / parts) * sizeof(element). */
int ltq_interleave_column_blocks(const void *gathered_dev, void *out_dev, uint64_t parts, uint64_t M,
                                 uint64_t part_row_bytes, int device, void *stream);

/* ---- the reference kernel call, argument for argument ---------------------------------------------------------- */

/* quantized_matmul, l-ten/math_fns.h:104 / l-ten/math_fns.cpp:1311-1478, all four transpose variants.
 * A, B, C, bias, workspace are device pointers; qparams is a HOST array of 3 (A-operand, B-operand, output).
 * workspace_dev holds at least (M + N) int32 and receives [-z_A*sum_k B(j,.) (N) | -z_B*sum_k A(i,.) (M)] exactly as
 * the reference leaves it.  alpha != 1 or beta != 0 -> LTQ_ERR_UNSUPPORTED (reference: LTEN_ERR).
 * C = (uchar)(rm * acc + z_C) with the reference build's truncating, wrapping cast. */
int ltq_quantized_matmul(int transpose_A, int transpose_B, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha,
                         const uint8_t *A_dev, const uint8_t *B_dev, uint8_t beta, uint8_t *C_dev,
                         const ltq_qparams *qparams, const int32_t *bias_dev, int32_t *workspace_dev, int device,
                         void *stream);

/* The same product with the output modes and flags of ltq_layer_forward: int32 (the corrected accumulator; with zero
 * points 0 the plain uint8 x uint8 -> int32 matrix product that Tensor::matmul lacks for UINT8,
 * l-ten/math_fns.cpp:1295-1305), float ((sA*sB) * acc) or requantized uint8; LTQ_FLAG_RELU / LTQ_FLAG_SATURATE /
 * LTQ_FLAG_FORCE_*.  C_dev holds M*N elements of the mode's type. */
int ltq_quantized_matmul_ex(int transpose_A, int transpose_B, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha,
                            const uint8_t *A_dev, const uint8_t *B_dev, uint8_t beta, void *C_dev,
                            const ltq_qparams *qparams, const int32_t *bias_dev, int32_t *workspace_dev, int out_mode,
                            unsigned flags, int device, void *stream);

/* No counterpart in the reference: the same computation as ltq_quantized_matmul for callers that must not allocate
 * device memory and therefore have no workspace to pass -- code running inside another framework's pre-planned memory
 * region, latency-critical loops that cannot take the allocator's lock or an implicit synchronisation, processes
 * whose device memory is fully reserved.  The (M + N) int32 of scratch live in a fixed array inside the library image
 * (every GPU that loads the library holds LTQ_STATIC_WS_INTS * 4 bytes until exit), so M + N must not exceed
 * LTQ_STATIC_WS_INTS (LTQ_ERR_TOO_LARGE otherwise).  The call performs no cudaMalloc / cudaFree and calls no
 * allocating routine.  The first call on each device looks up the array's device address; make that first call
 * outside any stream capture.  All calls on a device share the scratch: it holds the previous call's sums on entry
 * (they are overwritten or cleared before use), and two calls whose kernels overlap on the GPU race on it -- issue
 * them on one stream, or otherwise order them.  Output C is identical to ltq_quantized_matmul's, and so is the kernel
 * choice (weight-streaming, tcgen05 single CTA or CTA pair, dp4a).
 * Failure path: the bounded waits inside these kernels report into a status word that also lives in the library
 * image, not into the one ltq_device_check reads (creating that one allocates).  ltq_static_check reads and clears it
 * without allocating: LTQ_OK, or LTQ_ERR_DEVICE_TIMEOUT when a wait ran out since the last check (C is then
 * incomplete).  It synchronises `stream`. */
#define LTQ_STATIC_WS_INTS (256 * 1024)
int ltq_quantized_matmul_static(int transpose_A, int transpose_B, uint64_t M, uint64_t N, uint64_t K, uint8_t alpha,
                                const uint8_t *A_dev, const uint8_t *B_dev, uint8_t beta, uint8_t *C_dev,
                                const ltq_qparams *qparams, const int32_t *bias_dev, int device, void *stream);
int ltq_static_check(int device, void *stream);

/* ---- layer handle: what FullyConnected_q (l-ten/layers.h:69-106) keeps between calls ------------------------- */

typedef struct ltq_layer ltq_layer;

/* FullyConnected_q::init, l-ten/fully_connected.cpp:295-320, device side.  The handle owns only derived state
 * (weight row sums, tensor maps, the activation-sum workspace that l-ten keeps in workspace_); weights and bias stay
 * the caller's. */
int ltq_layer_create(ltq_layer **layer, int device, uint64_t in_features, uint64_t out_features);
int ltq_layer_destroy(ltq_layer *layer);

/* Bind device weights uint8 [N,K] (K contiguous: the {1,1,N,K} tensor of l-ten/fully_connected.cpp:303) and
 * optional int32 bias [N]; computes sum_k W[j,k] once (the reference recomputes it on every call,
 * l-ten/math_fns.cpp:1362-1370).  Call again whenever the weight bytes change or move.  Synchronises `stream`. */
int ltq_layer_set_weights(ltq_layer *layer, const uint8_t *w_dev, const int32_t *bias_dev, void *stream);

/* set_qparams_in / set_qparams_out / set_qparams_params, l-ten/layers.h:89-91, fully_connected.cpp:440-446. */
int ltq_layer_set_qparams(ltq_layer *layer, const ltq_qparams *qp_in, const ltq_qparams *qp_wt,
                          const ltq_qparams *qp_out);

/* FullyConnected_q::forward's compute, l-ten/fully_connected.cpp:364-395, with all leading dims folded into M.
 *   x_dev     uint8 [M,K]
 *   asum_dev  int32 [M] row sums of x (from ltq_quantize_rows_u8), or NULL: computed here into the layer's workspace
 *   qp_in_dev optional DEVICE qparams overriding the layer's input qparams (dynamic activation quantisation
 *             without a host round trip); NULL = use the value set by ltq_layer_set_qparams
 *   out_dev   uint8 / float / int32 [M,N] by out_mode
 * Kernel choice: M <= 16 with K % 128 == 0 -> weight-streaming kernel; otherwise the tcgen05 kernel
 * when K % 16 == 0; else the generic kernel.
 * Stream capture: with asum_dev == NULL the layer's own workspace grows (cudaMalloc) the first time a larger M is seen;
 * pass asum_dev, or run the largest M once before capturing. */
int ltq_layer_forward(ltq_layer *layer, const uint8_t *x_dev, const int32_t *asum_dev, uint64_t M,
                      const ltq_qparams *qp_in_dev, int out_mode, unsigned flags, void *out_dev, void *stream);

/* Chains of layers without a sum pass in between (no counterpart in the reference, which recomputes all sums inside
 * every quantized_matmul call): with rowsum_dev set (int32 [M], NULL switches it off again), every later uint8-output
 * forward of this layer also ADDS the sum of each output row's bytes to rowsum_dev[row] -- exactly the asum_dev the
 * next layer's ltq_layer_forward wants.  The additions are atomic and accumulate: clear the array (cudaMemsetAsync on
 * the same stream) before each forward.  Ignored for float / int32 output. */
int ltq_layer_set_rowsum_output(ltq_layer *layer, int32_t *rowsum_dev);

/* Housekeeping for such chains, so that they need no clearing launch either: every later forward of this layer also
 * clears count int32 at array_dev (count 0 / NULL switches it off), after everything in front of it in the stream has
 * finished and before anything behind it starts.  Meant for the rowsum array of ANOTHER layer of the chain whose
 * consumer has already run: e.g. with layers L1 -> L2 -> L3, sums1 = rows of L1's output and sums2 = rows of L2's
 * output, let L3 clear sums1 and L1 clear sums2.  The array must not be the one this layer accumulates into, nor the
 * asum_dev passed to the same forward. */
int ltq_layer_set_clear_on_forward(ltq_layer *layer, int32_t *array_dev, uint64_t count);

/* A hint for chains of layers at small batch (M <= 16), where each forward is bound by reading the layer's weights
 * once from device memory: `next` is the layer whose forward follows `layer`'s on the same stream (QNet::forward,
 * tests/nn_tests.cpp:630-640, calls its layers in a fixed order).  The weight-streaming kernel of `layer` then asks
 * the first part of `next`'s weights into the L2 cache once all of its own reads are on their way, so that memory
 * keeps streaming while `layer` finishes and `next` starts.  Purely a performance hint: results are unchanged, and it
 * is ignored by the other kernels and when the two layers' shapes do not divide over the SMs alike.  The hint
 * records next's weight pointer and shape as they are NOW; set it again after rebinding next's weights, and clear it
 * (next = NULL) before those weights are freed.  Both layers must be on the same device. */
int ltq_layer_set_next(ltq_layer *layer, const ltq_layer *next);

/* ltq_layer_forward with the result written into several buffers at once, each holding rows of ld_out elements, at
 * column col_offset: element (i, j) of this layer's output goes to dests[d][i * ld_out + col_offset + j] for every d.
 * No counterpart in the reference (which runs on one device).  This is the exchange step of a COLUMN-SHARDED layer
 * done by the GEMM epilogue itself: each rank owns out_features / world columns, dests[0] is its own [M, ld_out]
 * buffer and dests[1 .. n_dests-1] are the other ranks' buffers mapped into this process (ltq_peer_open), so the
 * stores travel over NVLink while the tiles are still being computed and no all-gather or relayout pass follows.
 * n_dests <= LTQ_MAX_DESTS.  The call only orders its own stores: before any rank READS its buffer, every rank's
 * call must have completed (a stream-ordered collective of any size, or a host barrier after a stream sync), and a
 * buffer must not be rewritten while another rank may still read it (alternate two buffers).
 * 16-byte stores are used when ld_out * element size, col_offset * element size and all bases are multiples of 16.
 * With LTQ_FLAG_MULTICAST_DEST, dests holds ONE address of an NVLink multicast mapping (NVSwitch replicates every store
 * into the buffer of each GPU bound to it, this GPU's included; e.g. the multicast pointer of a symmetric-memory
 * allocation): every rank then sends its columns once instead of once per peer.  Stores are issued as multimem.st in
 * 16-byte pieces, so the 16-byte conditions above must hold and out_features * element size must be a multiple of 16;
 * only the tensor-core kernels take it (K % 16 == 0, M > 16 or K % 128 != 0), anything else is LTQ_ERR_UNSUPPORTED. */
int ltq_layer_forward_scatter(ltq_layer *layer, const uint8_t *x_dev, const int32_t *asum_dev, uint64_t M,
                              const ltq_qparams *qp_in_dev, int out_mode, unsigned flags, void *const *dests, int n_dests,
                              uint64_t ld_out, uint64_t col_offset, void *stream);

/* Device buffers that other processes on the same node can map (CUDA IPC: cudaMalloc + cudaIpcGetMemHandle on the
 * owner, cudaIpcOpenMemHandle with lazy peer access on the others).  handle64 is 64 opaque bytes to be carried to the
 * other process by any means (torch.distributed's object collectives in this repository).  No counterpart in the
 * reference. */
int ltq_peer_alloc(void **dev_ptr, uint64_t bytes, int device, unsigned char *handle64);
int ltq_peer_free(void *dev_ptr, int device);
int ltq_peer_open(const unsigned char *handle64, int device, void **peer_ptr);
int ltq_peer_close(void *peer_ptr, int device);

/* ---- a chain of layers in one launch ----------------------------------------------------------------------------------
 * The reference runs a quantized network as one kernel-sized step per layer with the activations going through memory
 * in between (tests/nn_tests.cpp:630-640, 930-963).  For a small multi-layer perceptron that is all launch latency.  A
 * fused chain runs Quantize(input) and 2 to 4 FullyConnected_q layers as ONE launch per batch: clusters of 8 CTAs keep
 * the weights and the activations in (distributed) shared memory, every 64 rows of the batch one cluster.  The result
 * is bit-identical to ltq_quantize_rows_u8 + ltq_layer_forward layer by layer.  No counterpart in the reference.
 *
 * layers: handles with weights bound (ltq_layer_set_weights) on one device, layer l+1 taking layer l's outputs; the chain
 * borrows them (keep them alive, and create the chain again after rebinding weights).  Quantisation parameters are read
 * from the layers at every forward: qp_in of layers[0] quantises the input, qp_out of layer l must equal qp_in of layer
 * l+1 for the chain to mean what the layer-by-layer path means.  LTQ_ERR_UNSUPPORTED when a chain does not fit (K not a
 * multiple of 16, a layer wider than 2048 outputs, or weights + activations beyond one cluster's shared memory: a chain
 * of about 0.75 M weights fits); run it layer by layer then. */
typedef struct ltq_mlp ltq_mlp;
int ltq_mlp_create(ltq_mlp **mlp, ltq_layer *const *layers, int n_layers);
int ltq_mlp_destroy(ltq_mlp *mlp);
/* x_dev float32 [M, in_features of layers[0]]; hidden layers write uint8 (kept on chip), the last layer writes out_dev
 * [M, out_features] in out_mode.  layer_flags: n_layers entries of LTQ_FLAG_RELU / LTQ_FLAG_SATURATE, or NULL for none. */
int ltq_mlp_forward(ltq_mlp *mlp, const float *x_dev, uint64_t M, const unsigned *layer_flags, int out_mode, void *out_dev,
                    void *stream);

/* ---- one host thread, several devices ---------------------------------------------------------------------------------
 * l-ten's API is single-threaded and names a device per tensor (TensorOps::device_index, handle arrays of MAX_DEVICES = 8,
 * l-ten/globals.h:15,89-124) but has no multi-device code for this path.  These entry points let such a caller run a
 * sharded quantized layer: one NCCL communicator and one stream per device, created together (ncclCommInitAll), and
 * calls that take one pointer per device.  NCCL is loaded at run time (libnccl.so.2) the first time a group is created.
 * Work is enqueued on the group's own streams (ltq_comm_stream) and the calls return without waiting; whatever produced
 * the inputs on other streams must have finished, or be ordered before, by the caller.  ltq_comm_synchronize waits. */
typedef struct ltq_comm ltq_comm;

/* devices: ndev distinct device indices, or NULL for 0 .. ndev-1.  1 <= ndev <= LTQ_MAX_DESTS. */
int ltq_comm_init_all(ltq_comm **comm, int ndev, const int *devices);
int ltq_comm_destroy(ltq_comm *comm);
int ltq_comm_size(const ltq_comm *comm);
int ltq_comm_device(const ltq_comm *comm, int index);      /* device index of member `index`, -1 if out of range */
void *ltq_comm_stream(const ltq_comm *comm, int index);    /* its cudaStream_t */

/* Waits until every device's stream has drained.  While waiting it polls the communicators (ncclCommGetAsyncError): on
 * an asynchronous error, or when timeout_ms (0 = no limit) runs out, every communicator is aborted (ncclCommAbort), so
 * that collectives stuck on a lost peer return, and the call fails with LTQ_ERR_CUDA / LTQ_ERR_DEVICE_TIMEOUT.  After
 * that the group only accepts ltq_comm_destroy. */
int ltq_comm_synchronize(ltq_comm *comm, uint32_t timeout_ms);

/* Row (M) sharding: device d holds a full replica of the layer (layers[d], created on that device) and rows[d] rows of
 * the activations x_dev[d] uint8 [rows[d], K]; it writes the same rows of the output to out_dev[d].  Nothing is
 * exchanged (parameters are per tensor, rows are independent).  asum_dev / qp_in_dev: per-device arrays as in
 * ltq_layer_forward, or NULL. */
int ltq_linear_forward_rowsharded(ltq_comm *comm, ltq_layer *const *layers, const uint8_t *const *x_dev,
                                  const int32_t *const *asum_dev, const uint64_t *rows, const ltq_qparams *const *qp_in_dev,
                                  int out_mode, unsigned flags, void *const *out_dev);

/* The one exchange row sharding needs, and only under dynamic activation quantisation: the per-tensor min / max must be
 * those of ALL rows for the sharded result to equal the single-device one.  minmax_dev[d]: two floats on device d
 * (from ltq_get_min_max over its rows, enqueued on the group's stream); replaced in place by the global {min, max}. */
int ltq_comm_allreduce_minmax(ltq_comm *comm, float *const *minmax_dev);

/* Column (N) sharding: device d holds weight rows (output features) [d*n, (d+1)*n) as layers[d] (all with the same n =
 * N / ndev and the same K) and the FULL activations x_dev[d] uint8 [M, K].  Each device computes its [M, n] slice into
 * local_dev[d], the slices are all-gathered (ncclAllGather inside one group) into gathered_dev[d] ([ndev][M][n]) and
 * re-laid out into out_dev[d], row-major [M, N], on every device.  With ndev = 1 the result goes straight to out_dev. */
int ltq_linear_forward_colsharded_allgather(ltq_comm *comm, ltq_layer *const *layers, const uint8_t *const *x_dev,
                                            const int32_t *const *asum_dev, uint64_t M, const ltq_qparams *const *qp_in_dev,
                                            int out_mode, unsigned flags, void *const *local_dev, void *const *gathered_dev,
                                            void *const *out_dev);

/* What a group does with its devices and communicators, as a table of functions.  The default (backend = NULL) is NCCL
 * and CUDA streams.  Tests install a fake to exercise the watchdog of ltq_comm_synchronize and the bookkeeping without a
 * GPU: groups created while a fake is installed make no CUDA or NCCL call at all.  Return values: 0 = success;
 * stream_query: 0 = idle, 1 = busy, negative = error; comm_get_async_error stores a non-zero code when the
 * communicator has failed.  all_reduce_f32's op: 0 = min, 1 = max. */
typedef struct ltq_comm_backend {
    int (*comm_init_all)(void **comms, int ndev, const int *devices);
    int (*comm_destroy)(void *comm);
    int (*comm_abort)(void *comm);
    int (*comm_get_async_error)(void *comm, int *async_error);
    int (*all_gather)(const void *send, void *recv, uint64_t bytes, void *comm, void *stream);
    int (*all_reduce_f32)(const void *send, void *recv, uint64_t count, int op, void *comm, void *stream);
    int (*group_start)(void);
    int (*group_end)(void);
    int (*stream_create)(int device, void **stream);
    int (*stream_destroy)(int device, void *stream);
    int (*stream_query)(int device, void *stream);
    const char *(*error_string)(int code);
} ltq_comm_backend;
int ltq_comm_set_backend(const ltq_comm_backend *backend);

/* Reads (and clears) the layer's device status word: LTQ_OK, or LTQ_ERR_DEVICE_TIMEOUT when a bounded wait inside a
 * kernel ran out since the last check.  Synchronises `stream`. */
int ltq_layer_check(ltq_layer *layer, void *stream);

/* ---- quantized convolution: Conv2d_q (l-ten/layers.h:453-524, l-ten/conv2d.cpp:238-379) -------------------------
 * The reference runs this layer on the CPU only ("Conv2d_q only supports the CPU device type", conv2d.cpp:371); here
 * it is an im2col pass over the whole batch followed by one GEMM per image on the kernels of the linear path. */

typedef struct ltq_conv2d ltq_conv2d;

/* Conv2d_q's constructor + init (l-ten/layers.h:456-472, conv2d.cpp:238-264).  The handle owns derived state only:
 * weight row sums, a zero-padded weight copy when C*kh*kw is not a multiple of 16, the patch buffer and patch sums
 * (the reference's col_buffer_ptr_ and workspace_, grown on demand the same way). */
int ltq_conv2d_create(ltq_conv2d **conv, int device, uint64_t channels_in, uint64_t channels_out, uint64_t kernel_h,
                      uint64_t kernel_w, uint64_t pad_h, uint64_t pad_w, uint64_t stride_h, uint64_t stride_w);
int ltq_conv2d_destroy(ltq_conv2d *conv);

/* Bind device weights uint8 [channels_out, channels_in * kernel_h * kernel_w] (the {Cout, Cin, kh*kw} tensor of
 * conv2d.cpp:247) and optional int32 bias [channels_out].  Synchronises `stream`. */
int ltq_conv2d_set_weights(ltq_conv2d *conv, const uint8_t *w_dev, const int32_t *bias_dev, void *stream);

/* set_qparams_in / set_qparams_out / set_qparams_params, l-ten/layers.h:505-507. */
int ltq_conv2d_set_qparams(ltq_conv2d *conv, const ltq_qparams *qp_in, const ltq_qparams *qp_wt,
                           const ltq_qparams *qp_out);

/* height_out = (height_in + 2*pad_h - kernel_h) / stride_h + 1 and likewise for the width (conv2d.cpp:313-314). */
int ltq_conv2d_output_size(const ltq_conv2d *conv, uint64_t height_in, uint64_t width_in, uint64_t *height_out,
                           uint64_t *width_out);

/* Conv2d_q::forward (conv2d.cpp:266-379): x_dev uint8 NCHW [batches, channels_in, height_in, width_in] ->
 * out_dev [batches, channels_out, height_out, width_out], uint8 (LTQ_OUT_U8, what the reference returns), float or
 * int32 by out_mode.  Arithmetic per image is quantized_matmul(false, false, M = channels_out, N = Ho*Wo,
 * K = Cin*kh*kw, weights, im2col(image)) with qparams {weights, input, output}; padding taps are the byte 0
 * (l-ten/im_col.h:27-28), not the input zero point.
 * Bias: the reference adds bias[j] with j the output POSITION (math_fns.cpp:1469-1472) although the tensor holds
 * channels_out values; that is reproduced as long as Ho*Wo <= channels_out and refused (LTQ_ERR_UNSUPPORTED) beyond,
 * where the reference reads past the tensor.  LTQ_FLAG_BIAS_PER_CHANNEL adds bias[c] per output channel instead.
 * LTQ_FLAG_RELU / LTQ_FLAG_SATURATE / LTQ_FLAG_FORCE_* act as in ltq_layer_forward.
 * Layout, additive: the reference knows NCHW only.  Most layers are computed from a channels-last form of the
 * input (made tile by tile inside the kernel, or as a copy by a kernel in front); where the input channels are a multiple of 64 and the output channels a multiple of 16, LTQ_FLAG_NHWC_IN
 * hands that layout in directly (nothing to transpose; x_dev 16-byte aligned) and LTQ_FLAG_NHWC_OUT writes it (out_dev
 * 16-byte aligned; LTQ_FLAG_NHWC_IN needs strides 1), so that a chain of such layers never leaves it.  The values are
 * the same, only their place in memory differs.  For any other geometry or a forced kernel the two flags give
 * LTQ_ERR_UNSUPPORTED. */
int ltq_conv2d_forward(ltq_conv2d *conv, const uint8_t *x_dev, uint64_t batches, uint64_t height_in, uint64_t width_in,
                       int out_mode, unsigned flags, void *out_dev, void *stream);

/* The patch gather on its own: im2col_cpu (l-ten/im_col.h:5-33) for `batches` images in one launch, written
 * TRANSPOSED and padded: col_t[b][ho*Wo + wo][k], k = (c*kernel_h + i)*kernel_w + j, each row row_pitch bytes
 * (= C*kh*kw rounded up to a multiple of 16) with a zero tail.  col_t_dev must be 16-byte aligned. */
int ltq_im2col_t_u8(const uint8_t *im_dev, uint64_t batches, uint64_t channels, uint64_t height, uint64_t width,
                    uint64_t kernel_h, uint64_t kernel_w, uint64_t pad_h, uint64_t pad_w, uint64_t stride_h,
                    uint64_t stride_w, uint8_t *col_t_dev, uint64_t row_pitch, int device, void *stream);

/* Same check for a device without a layer at hand (the stateless entry points share the device's status word). */
int ltq_device_check(int device, void *stream);

/* Failure-path self-test, no counterpart in the reference: launches one warp that waits on a barrier nothing will
 * ever arrive on.  The wait gives up after limit_us (1 .. 1 000 000), leaves code 0x900 in the device status word and
 * the kernel returns normally; the next ltq_device_check / ltq_layer_check then reports LTQ_ERR_DEVICE_TIMEOUT and
 * clears it.  Nothing hangs or faults: this is how the bounded waits inside the GEMM kernels are exercised. */
int ltq_selftest_bounded_wait(int device, uint32_t limit_us, void *stream);
/* The same probe reporting into the status word of the allocation-free entry points (read by ltq_static_check). */
int ltq_selftest_bounded_wait_static(int device, uint32_t limit_us, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LTQ_H */
