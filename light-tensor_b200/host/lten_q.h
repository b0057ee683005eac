// C++ host side of the quantized fully-connected path: a self-contained mirror of the part of l-ten's public surface
// that this path touches, driving libltq (include/ltq.h) for everything that computes.
//
//   lten::Tensor / TensorOps / AllocateTensor / TensorFromBuffer      l-ten/tensor.h:33-81,1478-1482, tensorimpl.h:46-63
//   lten::Module, lten::FullyConnected_q, lten::Conv2d_q              l-ten/layers.h:14-31,69-106,453-524
//   QuantizationParams                                                l-ten/math_fns.h:12-16
//   GetMinMax / ComputeQuantizationParams / Quantize / Dequantize     l-ten/utils.h:23-27
//
// Same names, argument meaning and error behaviour (LTEN_ERR prints to stderr and throws lten::ExceptionInfo,
// l-ten/error.h:78-93), so code written against l-ten's quantized layer compiles against this header.  What differs:
// FullyConnected_q::to(GPU, idx) works, forward() takes GPU tensors, and the free functions take DEVICE pointers
// (classified with cudaPointerGetAttributes).  There is no CPU compute path: forward() on a CPU tensor and the free
// functions on host buffers throw; only ComputeQuantizationParams, which works on two scalars, runs on the host.
#ifndef LTEN_Q_H
#define LTEN_Q_H

#include <stdint.h>

#include <initializer_list>
#include <memory>
#include <string>
#include <vector>

#include "../../include/ltq.h"

typedef ltq_qparams QuantizationParams;  // same layout as l-ten/math_fns.h:12-16

namespace lten {

enum device { CPU, GPU };
enum dtype { FLOAT32, INT32, UINT8 };
enum { MAX_DIMS = 16 };

class ExceptionInfo : public std::exception {
public:
    ExceptionInfo(const char *msg, const char *file, const char *func, int line);
    const char *what() const noexcept override { return text_.c_str(); }
    const char *get_message() const { return msg_.c_str(); }

private:
    std::string msg_, text_;
};

struct TensorOps {
    dtype data_type = FLOAT32;
    device device_type = CPU;
    int device_index = 0;
    bool alloc_gradient_buffer = false;
};

// Value handle over reference-counted storage (the role of intrusive_ptr<TensorImplBase> in l-ten).
class Tensor {
public:
    Tensor() {}
    void *get_data_ptr() const;
    uint64_t get_numels() const;
    const uint64_t *get_sizes() const;
    int get_ndims() const;
    dtype get_data_type() const;
    device get_device() const;
    int get_device_index() const;
    // Copies to the target device (synchronous cudaMemcpy, as l-ten/tensorimpl.cpp:311-412 does).
    Tensor to(device target_device, int target_device_index = 0) const;
    Tensor reshape(const std::initializer_list<uint64_t> &dims) const;
    bool defined() const { return impl_ != nullptr; }
    // Additive: int32 sums over the last dimension (one per row) that a quantized layer leaves on its uint8 output, and
    // the next quantized layer picks up instead of running a sum pass.  A reshape that changes the last dimension
    // drops them; writing into the tensor's bytes by hand does not (detach them with attach_row_sums(Tensor())).
    void attach_row_sums(const Tensor &sums);
    const Tensor *row_sums() const;
    // Additive: true when this handle is the only one referring to its bytes, and whether it has the given shape and
    // placement (what a layer asks before it recycles an output it handed out earlier).
    bool unique() const;
    bool matches(const uint64_t *dims, int ndims, const TensorOps &ops) const;

private:
    struct Impl;
    std::shared_ptr<Impl> impl_;
    friend Tensor AllocateTensor(const uint64_t *, int, TensorOps *);
    friend Tensor TensorFromBuffer(const uint64_t *, int, void *, bool, TensorOps *);
};

Tensor AllocateTensor(const std::initializer_list<uint64_t> &dims, TensorOps *options_ptr = nullptr);
Tensor AllocateTensor(const uint64_t *dims_ptr, int ndims, TensorOps *options_ptr = nullptr);
Tensor TensorFromBuffer(const std::initializer_list<uint64_t> &dims, void *data_ptr, bool own_memory = false,
                        TensorOps *options_ptr = nullptr);
Tensor TensorFromBuffer(const uint64_t *dims_ptr, int ndims, void *data_ptr, bool own_memory = false,
                        TensorOps *options_ptr = nullptr);

class Module {
public:
    Module() {}
    virtual ~Module() {}
    virtual bool init() = 0;
    virtual std::vector<Tensor *> get_all_weights() = 0;
    virtual void clear_gradients() = 0;
    virtual void to(device target_device, int target_device_index = 0) = 0;
    void train(bool is_training) { is_training_ = is_training; }
    virtual void set_qparams_in(QuantizationParams) {}
    virtual void set_qparams_out(QuantizationParams) {}
    virtual void set_qparams_params(QuantizationParams *, int) {}
    // Additive: input, weight and output parameters of a quantized module (what a checkpoint has to carry).
    virtual void get_qparams(QuantizationParams out[3]) const
    {
        out[0] = out[1] = out[2] = QuantizationParams{1.f, 0};
    }

protected:
    bool is_training_ = true;
};

class FullyConnected_q : public Module {
public:
    FullyConnected_q(int64_t input_features, int64_t output_features, bool use_bias = false, dtype data_type = FLOAT32);
    FullyConnected_q(const FullyConnected_q &other);             // copyable before init(), as register_module needs
    FullyConnected_q &operator=(const FullyConnected_q &other);  // (l-ten/net.h:37-76)
    ~FullyConnected_q();

    bool init();
    Tensor forward(Tensor &input);
    Tensor *get_weights() { return weight_ptr_; }
    Tensor *get_bias() { return bias_ptr_; }
    void clear_gradients() {}
    std::vector<Tensor *> get_all_weights();
    void to(device target_device, int target_device_index = 0);
    bool is_using_bias() { return use_bias_; }

    void set_qparams_in(QuantizationParams qparams_in) { qparams_in_ = qparams_in; }
    void set_qparams_out(QuantizationParams qparams_out) { qparams_out_ = qparams_out; }
    void set_qparams_params(QuantizationParams *qparams, int count);
    void get_qparams(QuantizationParams out[3]) const override
    {
        out[0] = qparams_in_;
        out[1] = qparams_wt_;
        out[2] = qparams_out_;
    }

    // Additive: what the fused epilogue writes.  Defaults reproduce the reference (uint8, no ReLU, wrapping cast).
    void set_output(ltq_out_mode mode, bool relu = false, bool saturate = false);
    // Additive: the CUDA stream (cudaStream_t) forward() enqueues its kernels on.  Default NULL: the legacy default
    // stream, which orders them with l-ten's own synchronous CUDA calls.  forward() never synchronises; with a
    // stream of its own a layer overlaps with copies and with other layers, and can be captured into a CUDA graph once
    // a forward of the same shape has run (output buffers are recycled, see forward()).
    void set_stream(void *stream) { stream_ = stream; }
    void *get_stream() const { return stream_; }
    // Additive: LTQ_ERR_DEVICE_TIMEOUT surfaced as an exception if a bounded device-side wait expired since the last call.
    void check();
    // Additive, a performance hint for networks run at small batch: `next` is the layer whose forward() follows this
    // one's (nullptr clears).  Both must already be on the GPU; call again after either moves, and clear it before
    // `next` is destroyed.  Results are unchanged (ltq_layer_set_next).
    void set_next(const FullyConnected_q *next);

private:
    friend class DeviceGroup;
    friend class FusedChain_q;
    // Result (and, for uint8 results, row-sum) tensors of the shape asked for: the ones handed out by the previous
    // forward when the caller has dropped them by now, fresh ones otherwise.
    Tensor take_output(const uint64_t *dims, int ndims, const TensorOps &ops, Tensor *cache);
    uint64_t input_features_, output_features_;
    Tensor *weight_ptr_ = nullptr, *bias_ptr_ = nullptr;
    bool use_bias_;
    QuantizationParams qparams_in_{1.f, 0}, qparams_out_{1.f, 0}, qparams_wt_{1.f, 0};
    ltq_layer *handle_ = nullptr;  // created by to(GPU), never by the constructor
    ltq_out_mode out_mode_ = LTQ_OUT_U8;
    unsigned flags_ = 0;
    void *stream_ = nullptr;
    Tensor cached_result_, cached_sums_;
};

// A chain of 2-4 FullyConnected_q layers run as ONE kernel launch per batch, input quantisation included (additive: the
// reference's QNet::forward, tests/nn_tests.cpp:630-640, quantises the input and calls layer after layer, which for a
// small network is all launch latency).  The layers stay owned by the caller, must be on the same GPU, and keep their
// parameters and output settings: layer i's ReLU / saturate flags apply to it, the LAST layer's output mode is the
// chain's.  forward() takes the FLOAT32 GPU input {.., rows, in_features of the first layer} and returns what the last
// layer's forward() would return after Quantize(input) and the layers in turn, bit for bit.  Throws where the chain
// does not fit one cluster's shared memory (then run the layers one by one).
class FusedChain_q {
public:
    explicit FusedChain_q(const std::vector<FullyConnected_q *> &layers);
    ~FusedChain_q();
    FusedChain_q(const FusedChain_q &) = delete;
    FusedChain_q &operator=(const FusedChain_q &) = delete;
    Tensor forward(Tensor &input);
    void set_stream(void *stream) { stream_ = stream; }

private:
    std::vector<FullyConnected_q *> layers_;
    ltq_mlp *handle_ = nullptr;
    void *stream_ = nullptr;
};

// One host thread driving a quantized layer over several GPUs (additive: l-ten has no multi-device code on this path,
// but its API is exactly this model - a device index per tensor, handle arrays of MAX_DEVICES, l-ten/globals.h:15,89-124).
// Wraps ltq_comm: one NCCL communicator and one stream per device.  Work is enqueued on the group's streams; call
// synchronize() before reading results on the host or from other streams.
class DeviceGroup {
public:
    explicit DeviceGroup(const std::vector<int> &device_indices);
    ~DeviceGroup();
    DeviceGroup(const DeviceGroup &) = delete;
    DeviceGroup &operator=(const DeviceGroup &) = delete;
    int size() const { return (int)devices_.size(); }
    int device(int i) const { return devices_[i]; }
    void *stream(int i) const;
    // Waits for every device; on an NCCL error or after timeout_ms (0 = none) aborts the communicators and throws.
    void synchronize(uint32_t timeout_ms = 0);
    // Row (M) sharding: replicas[d] is a copy of the layer moved to device(d) (full weights), inputs[d] holds that
    // device's rows, {..., rows_d, K} uint8.  Returns each device's rows of the output.  Nothing is exchanged.
    std::vector<Tensor> forward_rowsharded(const std::vector<FullyConnected_q *> &replicas, std::vector<Tensor> &inputs);
    // Column (N) sharding: slices[d] is a layer of out_features / size() outputs holding weight rows
    // [d * n, (d + 1) * n) on device(d); inputs[d] is the FULL activation tensor on that device.  The slices' outputs are
    // all-gathered over NCCL and re-laid out: every device gets the full {..., M, N} result.
    std::vector<Tensor> forward_colsharded(const std::vector<FullyConnected_q *> &slices, std::vector<Tensor> &inputs);

private:
    std::vector<int> devices_;
    ltq_comm *comm_ = nullptr;
};

// Quantized 2-D convolution, l-ten/layers.h:453-524 and l-ten/conv2d.cpp:238-406.  The reference computes it on the CPU
// only (its to() throws "Only CPU device supported"); here to(GPU, idx) builds the device state and forward() takes an
// NCHW uint8 GPU tensor.
class Conv2d_q : public Module {
public:
    Conv2d_q(const int channels_in, const int channels_out, bool use_bias, const int kernel_h, const int kernel_w,
             const int pad_h = 0, const int pad_w = 0, const int stride_h = 1, const int stride_w = 1);
    Conv2d_q(const Conv2d_q &other);             // copyable before init(), as register_module needs
    Conv2d_q &operator=(const Conv2d_q &other);
    ~Conv2d_q();

    uint64_t get_channels_out() { return channels_out_; }
    uint64_t get_channels_in() { return channels_in_; }
    uint64_t get_kernel_h() { return kernel_h_; }
    uint64_t get_kernel_w() { return kernel_w_; }
    uint64_t get_pad_h() { return pad_h_; }
    uint64_t get_pad_w() { return pad_w_; }
    uint64_t get_stride_h() { return stride_h_; }
    uint64_t get_stride_w() { return stride_w_; }

    bool init();
    Tensor forward(Tensor &input);
    std::vector<Tensor *> get_all_weights();
    Tensor *get_weights() { return weight_ptr_; }
    Tensor *get_bias() { return bias_ptr_; }
    void clear_gradients() {}
    void to(device target_device, int target_device_index = 0);

    void set_qparams_in(QuantizationParams qparams_in) { qparams_in_ = qparams_in; }
    void set_qparams_out(QuantizationParams qparams_out) { qparams_out_ = qparams_out; }
    void set_qparams_params(QuantizationParams *qparams, int count);
    void get_qparams(QuantizationParams out[3]) const override
    {
        out[0] = qparams_in_;
        out[1] = qparams_wt_;
        out[2] = qparams_out_;
    }

    // Additive.  bias_per_channel adds bias[c] per output channel; the default applies the bias the way the reference's
    // GEMM does, per output position, which it only defines while Ho*Wo <= channels_out.
    void set_output(ltq_out_mode mode, bool relu = false, bool saturate = false, bool bias_per_channel = false);
    // Additive: channels-last placement ({N, H, W, C}) of the input and / or the output, for chains of layers that are
    // computed from a channels-last copy anyway (stride 1, input channels a multiple of 64, output channels a multiple
    // of 16); forward() throws for other layers.  The values are those of the NCHW call.
    void set_layout(bool channels_last_in, bool channels_last_out);

private:
    uint64_t channels_in_, channels_out_, kernel_h_, kernel_w_, pad_h_, pad_w_, stride_h_, stride_w_;
    bool use_bias_;
    Tensor *weight_ptr_ = nullptr, *bias_ptr_ = nullptr;
    QuantizationParams qparams_in_{1.f, 0}, qparams_out_{1.f, 0}, qparams_wt_{1.f, 0};
    ltq_conv2d *handle_ = nullptr;
    ltq_out_mode out_mode_ = LTQ_OUT_U8;
    unsigned flags_ = 0;
};

// Checkpoint of quantized modules: every tensor of get_all_weights() with its own element size, then the three
// QuantizationParams.  l-ten's NeuralNetwork::save_checkpoint / load_checkpoint (l-ten/net.h:130-265) assume four bytes
// per element and keep no quantisation parameters; same return convention (0 = ok, -1 = failure).  Layout (little
// endian): "LTQCKPT1", uint32 modules, per module { uint32 tensors, per tensor { uint8 dtype (0 uint8, 1 int32,
// 2 float32), 3 zero bytes, uint32 ndims, uint64 dims[], data }, 3 x { float scale, uint8 zero_point, 3 zero bytes } }.
// Modules may be on the CPU or on a GPU; after loading into GPU modules call to(GPU, index) again (or load before to()).
// Calibration and quantisation set-up, the step in front of the quantized layers.  l-ten has no helper for this: its
// quantized test repeats it per network (tests/nn_tests.cpp:538-608 for the running statistics, :786-884 for the
// per-layer set-up).  These two package exactly that recipe, computing on the device.
//
// Running minimum / maximum over the FLOAT32 GPU tensors shown to update() (the test's blob_statistics +
// update_statistics, seeded with +/-FLT_MAX), turned into QuantizationParams by ComputeQuantizationParams.
class MinMaxObserver {
public:
    void update(const Tensor &x);
    bool seen() const { return min_ <= max_; }
    float min() const { return min_; }
    float max() const { return max_; }
    QuantizationParams qparams() const;  // throws if nothing has been observed

private:
    float min_ = 3.402823466e+38f, max_ = -3.402823466e+38f;
};

// Fills a freshly init()-ed quantized module (FullyConnected_q or Conv2d_q) from float parameters held on a GPU, the
// way tests/nn_tests.cpp:808-834 does for each layer: weights -> GetMinMax -> ComputeQuantizationParams -> Quantize
// (uint8) written through get_all_weights()[0]; bias -> int32 with scale s_in * s_wt and zero point 0 written through
// get_all_weights()[1]; then set_qparams_in / set_qparams_out / set_qparams_params.  Returns the weight parameters.
// `bias` may be nullptr only for a module built without one.  Call to(GPU, idx) afterwards, as the reference's flow does.
QuantizationParams quantize_module(Module &q_mod, const Tensor &weight, const Tensor *bias, QuantizationParams qp_in,
                                   QuantizationParams qp_out);

int save_checkpoint(const std::vector<Module *> &modules, const char *checkpoint_path);
int load_checkpoint(const std::vector<Module *> &modules, const char *checkpoint_path);

}  // namespace lten

// l-ten/utils.h:23-27 with device pointers (both buffers of a call on the same device).  Results that the reference
// returns through host scalars (min, max, the parameters) come back to the host.
void GetMinMax(float *data, uint64_t len, float *min_val, float *max_val);
void Quantize(float *data, int *q_data, uint64_t len, QuantizationParams *qp);
void Quantize(float *data, uint8_t *q_data, uint64_t len, QuantizationParams *qp);
void Dequantize(float *data, uint8_t *q_data, uint64_t len, QuantizationParams *qp);
void ComputeQuantizationParams(float min_val, float max_val, QuantizationParams *qp);

#endif  // LTEN_Q_H
