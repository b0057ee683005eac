// Implementation of lten_q.h on top of libltq and the CUDA runtime.
#include "lten_q.h"

#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace lten {

// l-ten/error.h:78-93 + l-ten/utils.cpp:303-322: print, then throw.
ExceptionInfo::ExceptionInfo(const char *msg, const char *file, const char *func, int line) : msg_(msg)
{
    text_ = std::string(msg) + " [" + file + ":" + std::to_string(line) + " " + func + "]";
}

#define LTEN_ERR(msg)                                                                                          \
    do {                                                                                                       \
        fprintf(stderr, "[Error] File: %s Function: %s Line:%d Msg: %s\n", __FILE__, __func__, __LINE__, msg); \
        throw lten::ExceptionInfo(msg, __FILE__, __func__, __LINE__);                                          \
    } while (0)

#define LTEN_CUDA(expr)                                           \
    do {                                                          \
        cudaError_t e__ = (expr);                                 \
        if (e__ != cudaSuccess) LTEN_ERR(cudaGetErrorString(e__)); \
    } while (0)

#define LTQ_CALL(expr)                          \
    do {                                        \
        if ((expr) != LTQ_OK) LTEN_ERR(ltq_last_error()); \
    } while (0)

static size_t dtype_size(dtype t) { return t == UINT8 ? 1 : 4; }

// Device or host bytes shared by every handle and view that refers to them (the role of the reference-counted
// TensorImpl storage in l-ten: `output = output.reshape(...)` must keep the bytes alive).
struct Storage {
    void *data = nullptr;
    bool own = true;
    device dev = CPU;
    int index = 0;
    ~Storage()
    {
        if (!own || !data) return;
        if (dev == GPU) {
            int prev = 0;
            cudaGetDevice(&prev);
            cudaSetDevice(index);
            cudaFree(data);
            cudaSetDevice(prev);
        } else {
            free(data);
        }
    }
};

struct Tensor::Impl {
    std::shared_ptr<Storage> storage;
    void *data = nullptr;  // == storage->data
    uint64_t dims[MAX_DIMS] = {0};
    int ndims = 0;
    uint64_t numels = 0;
    TensorOps ops;
    // Optional side-car left by the quantized layer that produced this tensor: int32 sums over the last dimension, one
    // per row (numels / dims[ndims-1] of them).  The next quantized layer uses them instead of a sum pass.
    std::shared_ptr<Tensor> row_sums;
};

void *Tensor::get_data_ptr() const { return impl_ ? impl_->data : nullptr; }
uint64_t Tensor::get_numels() const { return impl_ ? impl_->numels : 0; }
const uint64_t *Tensor::get_sizes() const { return impl_->dims; }
int Tensor::get_ndims() const { return impl_ ? impl_->ndims : 0; }
dtype Tensor::get_data_type() const { return impl_->ops.data_type; }
device Tensor::get_device() const { return impl_->ops.device_type; }
int Tensor::get_device_index() const { return impl_->ops.device_index; }

void Tensor::attach_row_sums(const Tensor &sums)
{
    if (!impl_) LTEN_ERR("Invalid argument");
    impl_->row_sums = sums.defined() ? std::make_shared<Tensor>(sums) : nullptr;
}

const Tensor *Tensor::row_sums() const { return impl_ && impl_->row_sums ? impl_->row_sums.get() : nullptr; }

bool Tensor::unique() const { return impl_ && impl_.use_count() == 1 && impl_->storage.use_count() == 1; }

bool Tensor::matches(const uint64_t *dims, int ndims, const TensorOps &ops) const
{
    if (!impl_ || impl_->ndims != ndims || impl_->ops.data_type != ops.data_type || impl_->ops.device_type != ops.device_type ||
        impl_->ops.device_index != ops.device_index)
        return false;
    return memcmp(impl_->dims, dims, sizeof(uint64_t) * ndims) == 0;
}

Tensor AllocateTensor(const uint64_t *dims_ptr, int ndims, TensorOps *options_ptr)
{
    if (ndims < 1 || ndims > MAX_DIMS) LTEN_ERR("Invalid number of dimensions");
    Tensor t;
    t.impl_ = std::make_shared<Tensor::Impl>();
    Tensor::Impl &im = *t.impl_;
    if (options_ptr) im.ops = *options_ptr;
    im.ndims = ndims;
    im.numels = 1;
    for (int i = 0; i < ndims; i++) {
        im.dims[i] = dims_ptr[i];
        im.numels *= dims_ptr[i];
    }
    const size_t bytes = im.numels * dtype_size(im.ops.data_type);
    im.storage = std::make_shared<Storage>();
    im.storage->dev = im.ops.device_type;
    im.storage->index = im.ops.device_index;
    if (im.ops.device_type == GPU) {
        int prev = 0;
        LTEN_CUDA(cudaGetDevice(&prev));
        LTEN_CUDA(cudaSetDevice(im.ops.device_index));
        LTEN_CUDA(cudaMalloc(&im.storage->data, bytes ? bytes : 1));
        LTEN_CUDA(cudaMemset(im.storage->data, 0, bytes));
        LTEN_CUDA(cudaSetDevice(prev));
    } else {
        im.storage->data = calloc(bytes ? bytes : 1, 1);
        if (!im.storage->data) LTEN_ERR("out of memory");
    }
    im.data = im.storage->data;
    return t;
}

Tensor AllocateTensor(const std::initializer_list<uint64_t> &dims, TensorOps *options_ptr)
{
    return AllocateTensor(dims.begin(), (int)dims.size(), options_ptr);
}

Tensor TensorFromBuffer(const uint64_t *dims_ptr, int ndims, void *data_ptr, bool own_memory, TensorOps *options_ptr)
{
    if (ndims < 1 || ndims > MAX_DIMS) LTEN_ERR("Invalid number of dimensions");
    Tensor t;
    t.impl_ = std::make_shared<Tensor::Impl>();
    Tensor::Impl &im = *t.impl_;
    if (options_ptr) im.ops = *options_ptr;
    im.ndims = ndims;
    im.numels = 1;
    for (int i = 0; i < ndims; i++) {
        im.dims[i] = dims_ptr[i];
        im.numels *= dims_ptr[i];
    }
    im.storage = std::make_shared<Storage>();
    im.storage->data = data_ptr;
    im.storage->own = own_memory;
    im.storage->dev = im.ops.device_type;
    im.storage->index = im.ops.device_index;
    im.data = data_ptr;
    return t;
}

Tensor TensorFromBuffer(const std::initializer_list<uint64_t> &dims, void *data_ptr, bool own_memory, TensorOps *options_ptr)
{
    return TensorFromBuffer(dims.begin(), (int)dims.size(), data_ptr, own_memory, options_ptr);
}

Tensor Tensor::to(device target_device, int target_device_index) const
{
    if (!impl_) LTEN_ERR("Invalid argument");
    TensorOps ops = impl_->ops;
    ops.device_type = target_device;
    ops.device_index = target_device == GPU ? target_device_index : 0;
    Tensor r = AllocateTensor(impl_->dims, impl_->ndims, &ops);
    const size_t bytes = impl_->numels * dtype_size(ops.data_type);
    if (bytes == 0) return r;
    if (impl_->ops.device_type == CPU && target_device == CPU) {
        memcpy(r.get_data_ptr(), impl_->data, bytes);
    } else {
        // cudaMemcpyDefault resolves host / device / peer copies from the pointers (unified addressing)
        LTEN_CUDA(cudaMemcpy(r.get_data_ptr(), impl_->data, bytes, cudaMemcpyDefault));
    }
    return r;
}

Tensor Tensor::reshape(const std::initializer_list<uint64_t> &dims) const
{
    uint64_t n = 1;
    for (uint64_t d : dims) n *= d;
    if (!impl_ || n != impl_->numels) LTEN_ERR("Invalid reshape dimensions");
    Tensor r = *this;
    r.impl_ = std::make_shared<Impl>(*impl_);  // a view: shares the storage, which lives as long as any handle does
    r.impl_->ndims = (int)dims.size();
    int i = 0;
    for (uint64_t d : dims) r.impl_->dims[i++] = d;
    // sums over the last dimension stay valid only while the last dimension does
    if (r.impl_->dims[r.impl_->ndims - 1] != impl_->dims[impl_->ndims - 1]) r.impl_->row_sums.reset();
    return r;
}

// ---- FullyConnected_q ------------------------------------------------------------------------------------------------
FullyConnected_q::FullyConnected_q(int64_t input_features, int64_t output_features, bool use_bias, dtype)
    : input_features_((uint64_t)input_features), output_features_((uint64_t)output_features), use_bias_(use_bias)
{
}

FullyConnected_q::FullyConnected_q(const FullyConnected_q &o) : Module(o) { *this = o; }

FullyConnected_q &FullyConnected_q::operator=(const FullyConnected_q &o)
{
    if (this == &o) return *this;
    if (o.weight_ptr_ || o.handle_) LTEN_ERR("FullyConnected_q can only be copied before init()");
    input_features_ = o.input_features_;
    output_features_ = o.output_features_;
    use_bias_ = o.use_bias_;
    qparams_in_ = o.qparams_in_;
    qparams_out_ = o.qparams_out_;
    qparams_wt_ = o.qparams_wt_;
    out_mode_ = o.out_mode_;
    flags_ = o.flags_;
    is_training_ = o.is_training_;
    return *this;
}

FullyConnected_q::~FullyConnected_q()
{
    ltq_layer_destroy(handle_);
    delete weight_ptr_;
    delete bias_ptr_;
}

// l-ten/fully_connected.cpp:295-320: uint8 weights {1,1,N,K}, int32 bias {N}, on the CPU, left for the quantisation
// set-up code to fill.
bool FullyConnected_q::init()
{
    TensorOps options;
    options.data_type = UINT8;
    weight_ptr_ = new Tensor;
    *weight_ptr_ = AllocateTensor({1, 1, output_features_, input_features_}, &options);
    if (use_bias_) {
        bias_ptr_ = new Tensor;
        options.data_type = INT32;
        *bias_ptr_ = AllocateTensor({output_features_}, &options);
    }
    return true;
}

std::vector<Tensor *> FullyConnected_q::get_all_weights()
{
    std::vector<Tensor *> weights;
    weights.push_back(weight_ptr_);
    if (use_bias_) weights.push_back(bias_ptr_);
    return weights;
}

void FullyConnected_q::set_qparams_params(QuantizationParams *qparams, int count)
{
    if (qparams && count) qparams_wt_ = qparams[0];  // l-ten/fully_connected.cpp:440-446: only [0] is kept
}

void FullyConnected_q::set_output(ltq_out_mode mode, bool relu, bool saturate)
{
    out_mode_ = mode;
    flags_ = (relu ? LTQ_FLAG_RELU : 0u) | (saturate ? LTQ_FLAG_SATURATE : 0u);
}

void FullyConnected_q::set_next(const FullyConnected_q *next)
{
    if (!handle_) LTEN_ERR("set_next: the layer is not on the GPU");
    if (next && !next->handle_) LTEN_ERR("set_next: the next layer is not on the GPU");
    if (ltq_layer_set_next(handle_, next ? next->handle_ : nullptr) != LTQ_OK) LTEN_ERR(ltq_last_error());
}

void FullyConnected_q::to(device target_device, int target_device_index)
{
    if (!weight_ptr_) LTEN_ERR("init() has not been called");
    *weight_ptr_ = weight_ptr_->to(target_device, target_device_index);
    if (bias_ptr_) *bias_ptr_ = bias_ptr_->to(target_device, target_device_index);
    ltq_layer_destroy(handle_);
    handle_ = nullptr;
    if (target_device == GPU) {
        LTQ_CALL(ltq_layer_create(&handle_, target_device_index, input_features_, output_features_));
        LTQ_CALL(ltq_layer_set_weights(handle_, static_cast<const uint8_t *>(weight_ptr_->get_data_ptr()),
                                       bias_ptr_ ? static_cast<const int32_t *>(bias_ptr_->get_data_ptr()) : nullptr,
                                       nullptr));
    }
}

// Output buffers are recycled: a forward hands out the tensor it handed out last time if the caller has let go of it
// (no cudaMalloc, no synchronising cudaMemset per call, and the addresses stay the same from call to call, which is
// what stream overlap and graph capture need).  A tensor the caller still holds is never touched.
Tensor FullyConnected_q::take_output(const uint64_t *dims, int ndims, const TensorOps &ops, Tensor *cache)
{
    if (cache->defined() && cache->unique() && cache->matches(dims, ndims, ops)) {
        cache->attach_row_sums(Tensor());
        return *cache;
    }
    *cache = AllocateTensor(dims, ndims, const_cast<TensorOps *>(&ops));
    return *cache;
}

void FullyConnected_q::check()
{
    if (handle_) LTQ_CALL(ltq_layer_check(handle_, stream_));
}

Tensor FullyConnected_q::forward(Tensor &input)
{
    // the reference's checks, messages and order: l-ten/fully_connected.cpp:330-348
    const int ndims = input.get_ndims();
    if (ndims < 3) LTEN_ERR("FullyConnected_q requires tensors with at least 3 dimensions");
    if (input.get_device() != weight_ptr_->get_device() || input.get_device_index() != weight_ptr_->get_device_index() ||
        input.get_data_type() != weight_ptr_->get_data_type())
        LTEN_ERR("Input tensor device type or data type are not the same as this layer's parameters");
    uint64_t dims[MAX_DIMS];
    memcpy(dims, input.get_sizes(), sizeof(uint64_t) * ndims);
    if (dims[ndims - 1] != input_features_) LTEN_ERR("Last dimension must be equal to the number of input features");
    if (input.get_device() != GPU)
        LTEN_ERR("FullyConnected_q: this build computes on GPU tensors only; call to(GPU, index) first");
    dims[ndims - 1] = output_features_;

    TensorOps options;
    options.data_type = out_mode_ == LTQ_OUT_U8 ? UINT8 : (out_mode_ == LTQ_OUT_F32 ? FLOAT32 : INT32);
    options.device_type = GPU;
    options.device_index = input.get_device_index();
    Tensor result = take_output(dims, ndims, options, &cached_result_);

    uint64_t rows = 1;  // every leading dimension folds into M: parameters are per tensor, rows are independent
    for (int d = 0; d < ndims - 1; d++) rows *= dims[d];
    // Row sums: taken from the tensor if the layer that produced it left them, and left on the result for the next layer
    // (uint8 output only), so that a chain of quantized layers runs without a sum pass in between.
    const Tensor *in_sums = input.row_sums();
    const int32_t *asum = in_sums && in_sums->get_numels() == rows ? static_cast<const int32_t *>(in_sums->get_data_ptr()) : nullptr;
    Tensor out_sums;
    if (out_mode_ == LTQ_OUT_U8) {
        TensorOps so;
        so.data_type = INT32;
        so.device_type = GPU;
        so.device_index = input.get_device_index();
        const uint64_t sdims[1] = {rows};
        out_sums = take_output(sdims, 1, so, &cached_sums_);
        // the epilogue accumulates into it: cleared in stream order, without stopping the host
        int prev = 0;
        LTEN_CUDA(cudaGetDevice(&prev));
        LTEN_CUDA(cudaSetDevice(so.device_index));
        LTEN_CUDA(cudaMemsetAsync(out_sums.get_data_ptr(), 0, rows * sizeof(int32_t), static_cast<cudaStream_t>(stream_)));
        LTEN_CUDA(cudaSetDevice(prev));
    }
    LTQ_CALL(ltq_layer_set_rowsum_output(handle_, out_sums.defined() ? static_cast<int32_t *>(out_sums.get_data_ptr()) : nullptr));
    LTQ_CALL(ltq_layer_set_qparams(handle_, &qparams_in_, &qparams_wt_, &qparams_out_));
    LTQ_CALL(ltq_layer_forward(handle_, static_cast<const uint8_t *>(input.get_data_ptr()), asum, rows, nullptr, out_mode_,
                               flags_, result.get_data_ptr(), stream_));
    if (out_sums.defined()) result.attach_row_sums(out_sums);
    return result;
}

// ---- FusedChain_q -----------------------------------------------------------------------------------------------------
FusedChain_q::FusedChain_q(const std::vector<FullyConnected_q *> &layers) : layers_(layers)
{
    std::vector<ltq_layer *> hs;
    for (FullyConnected_q *l : layers_) {
        if (!l || !l->handle_) LTEN_ERR("FusedChain_q: every layer must be on the GPU (call to(GPU, index) first)");
        hs.push_back(l->handle_);
    }
    LTQ_CALL(ltq_mlp_create(&handle_, hs.data(), (int)hs.size()));
}

FusedChain_q::~FusedChain_q() { ltq_mlp_destroy(handle_); }

Tensor FusedChain_q::forward(Tensor &input)
{
    const int ndims = input.get_ndims();
    if (ndims < 3) LTEN_ERR("FullyConnected_q requires tensors with at least 3 dimensions");
    FullyConnected_q *first = layers_.front(), *last = layers_.back();
    if (input.get_device() != GPU || input.get_data_type() != FLOAT32 ||
        input.get_device_index() != first->weight_ptr_->get_device_index())
        LTEN_ERR("FusedChain_q: FLOAT32 input on the layers' GPU expected");
    uint64_t dims[MAX_DIMS];
    memcpy(dims, input.get_sizes(), sizeof(uint64_t) * ndims);
    if (dims[ndims - 1] != first->input_features_) LTEN_ERR("Last dimension must be equal to the number of input features");
    dims[ndims - 1] = last->output_features_;
    uint64_t rows = 1;
    for (int d = 0; d < ndims - 1; d++) rows *= dims[d];
    TensorOps options;
    options.data_type = last->out_mode_ == LTQ_OUT_U8 ? UINT8 : (last->out_mode_ == LTQ_OUT_F32 ? FLOAT32 : INT32);
    options.device_type = GPU;
    options.device_index = input.get_device_index();
    Tensor result = AllocateTensor(dims, ndims, &options);
    std::vector<unsigned> flags;
    for (FullyConnected_q *l : layers_) {   // the parameters may have been set after the chain was built
        LTQ_CALL(ltq_layer_set_qparams(l->handle_, &l->qparams_in_, &l->qparams_wt_, &l->qparams_out_));
        flags.push_back(l->flags_);
    }
    LTQ_CALL(ltq_mlp_forward(handle_, static_cast<const float *>(input.get_data_ptr()), rows, flags.data(), last->out_mode_,
                             result.get_data_ptr(), stream_));
    return result;
}

// ---- DeviceGroup -------------------------------------------------------------------------------------------------------
DeviceGroup::DeviceGroup(const std::vector<int> &device_indices) : devices_(device_indices)
{
    LTQ_CALL(ltq_comm_init_all(&comm_, (int)devices_.size(), devices_.data()));
}

DeviceGroup::~DeviceGroup() { ltq_comm_destroy(comm_); }

void *DeviceGroup::stream(int i) const { return ltq_comm_stream(comm_, i); }

void DeviceGroup::synchronize(uint32_t timeout_ms) { LTQ_CALL(ltq_comm_synchronize(comm_, timeout_ms)); }

static uint64_t fold_rows(const Tensor &t)
{
    uint64_t rows = 1;
    for (int d = 0; d < t.get_ndims() - 1; d++) rows *= t.get_sizes()[d];
    return rows;
}

std::vector<Tensor> DeviceGroup::forward_rowsharded(const std::vector<FullyConnected_q *> &replicas, std::vector<Tensor> &inputs)
{
    const int n = size();
    if ((int)replicas.size() != n || (int)inputs.size() != n) LTEN_ERR("one layer replica and one input per device of the group");
    std::vector<ltq_layer *> layers(n);
    std::vector<const uint8_t *> xs(n);
    std::vector<uint64_t> rows(n);
    std::vector<void *> outs(n);
    std::vector<Tensor> results(n);
    const ltq_out_mode mode = replicas[0]->out_mode_;
    for (int d = 0; d < n; d++) {
        FullyConnected_q *fc = replicas[d];
        const Tensor &x = inputs[d];
        if (!fc->handle_ || x.get_ndims() < 2 || x.get_device() != GPU || x.get_device_index() != devices_[d] ||
            x.get_data_type() != UINT8 || x.get_sizes()[x.get_ndims() - 1] != fc->input_features_ || fc->out_mode_ != mode)
            LTEN_ERR("Input tensor device type or data type are not the same as this layer's parameters");
        uint64_t dims[MAX_DIMS];
        memcpy(dims, x.get_sizes(), sizeof(uint64_t) * x.get_ndims());
        dims[x.get_ndims() - 1] = fc->output_features_;
        TensorOps o;
        o.data_type = mode == LTQ_OUT_U8 ? UINT8 : (mode == LTQ_OUT_F32 ? FLOAT32 : INT32);
        o.device_type = GPU;
        o.device_index = devices_[d];
        results[d] = fc->take_output(dims, x.get_ndims(), o, &fc->cached_result_);
        LTQ_CALL(ltq_layer_set_rowsum_output(fc->handle_, nullptr));
        LTQ_CALL(ltq_layer_set_qparams(fc->handle_, &fc->qparams_in_, &fc->qparams_wt_, &fc->qparams_out_));
        layers[d] = fc->handle_;
        xs[d] = static_cast<const uint8_t *>(x.get_data_ptr());
        rows[d] = fold_rows(x);
        outs[d] = results[d].get_data_ptr();
    }
    LTQ_CALL(ltq_linear_forward_rowsharded(comm_, layers.data(), xs.data(), nullptr, rows.data(), nullptr, mode,
                                           replicas[0]->flags_, outs.data()));
    return results;
}

std::vector<Tensor> DeviceGroup::forward_colsharded(const std::vector<FullyConnected_q *> &slices, std::vector<Tensor> &inputs)
{
    const int n = size();
    if ((int)slices.size() != n || (int)inputs.size() != n) LTEN_ERR("one layer slice and one input per device of the group");
    const ltq_out_mode mode = slices[0]->out_mode_;
    const dtype dt = mode == LTQ_OUT_U8 ? UINT8 : (mode == LTQ_OUT_F32 ? FLOAT32 : INT32);
    const uint64_t M = fold_rows(inputs[0]), n_loc = slices[0]->output_features_;
    std::vector<ltq_layer *> layers(n);
    std::vector<const uint8_t *> xs(n);
    std::vector<void *> locals(n), gathered(n), outs(n);
    std::vector<Tensor> results(n), keep;
    for (int d = 0; d < n; d++) {
        FullyConnected_q *fc = slices[d];
        const Tensor &x = inputs[d];
        if (!fc->handle_ || x.get_ndims() < 2 || x.get_device() != GPU || x.get_device_index() != devices_[d] ||
            x.get_data_type() != UINT8 || x.get_sizes()[x.get_ndims() - 1] != fc->input_features_ || fc->out_mode_ != mode ||
            fc->output_features_ != n_loc || fold_rows(x) != M)
            LTEN_ERR("Input tensor device type or data type are not the same as this layer's parameters");
        uint64_t dims[MAX_DIMS];
        memcpy(dims, x.get_sizes(), sizeof(uint64_t) * x.get_ndims());
        dims[x.get_ndims() - 1] = n_loc * (uint64_t)n;
        TensorOps o;
        o.data_type = dt;
        o.device_type = GPU;
        o.device_index = devices_[d];
        results[d] = AllocateTensor(dims, x.get_ndims(), &o);
        Tensor loc = AllocateTensor({M, n_loc}, &o), gat = AllocateTensor({(uint64_t)n, M, n_loc}, &o);
        keep.push_back(loc);
        keep.push_back(gat);
        LTQ_CALL(ltq_layer_set_rowsum_output(fc->handle_, nullptr));
        LTQ_CALL(ltq_layer_set_qparams(fc->handle_, &fc->qparams_in_, &fc->qparams_wt_, &fc->qparams_out_));
        layers[d] = fc->handle_;
        xs[d] = static_cast<const uint8_t *>(x.get_data_ptr());
        locals[d] = loc.get_data_ptr();
        gathered[d] = gat.get_data_ptr();
        outs[d] = results[d].get_data_ptr();
    }
    LTQ_CALL(ltq_linear_forward_colsharded_allgather(comm_, layers.data(), xs.data(), nullptr, M, nullptr, mode,
                                                     slices[0]->flags_, locals.data(), gathered.data(), outs.data()));
    // the scratch tensors are released when this returns: their kernels must have run by then
    synchronize();
    return results;
}

// ---- Conv2d_q ----------------------------------------------------------------------------------------------------------
Conv2d_q::Conv2d_q(const int channels_in, const int channels_out, bool use_bias, const int kernel_h, const int kernel_w,
                   const int pad_h, const int pad_w, const int stride_h, const int stride_w)
    : channels_in_((uint64_t)channels_in), channels_out_((uint64_t)channels_out), kernel_h_((uint64_t)kernel_h),
      kernel_w_((uint64_t)kernel_w), pad_h_((uint64_t)pad_h), pad_w_((uint64_t)pad_w), stride_h_((uint64_t)stride_h),
      stride_w_((uint64_t)stride_w), use_bias_(use_bias)
{
}

Conv2d_q::Conv2d_q(const Conv2d_q &o) : Module(o) { *this = o; }

Conv2d_q &Conv2d_q::operator=(const Conv2d_q &o)
{
    if (this == &o) return *this;
    if (o.weight_ptr_ || o.handle_) LTEN_ERR("Conv2d_q can only be copied before init()");
    channels_in_ = o.channels_in_;
    channels_out_ = o.channels_out_;
    kernel_h_ = o.kernel_h_;
    kernel_w_ = o.kernel_w_;
    pad_h_ = o.pad_h_;
    pad_w_ = o.pad_w_;
    stride_h_ = o.stride_h_;
    stride_w_ = o.stride_w_;
    use_bias_ = o.use_bias_;
    qparams_in_ = o.qparams_in_;
    qparams_out_ = o.qparams_out_;
    qparams_wt_ = o.qparams_wt_;
    out_mode_ = o.out_mode_;
    flags_ = o.flags_;
    is_training_ = o.is_training_;
    return *this;
}

Conv2d_q::~Conv2d_q()
{
    ltq_conv2d_destroy(handle_);
    delete weight_ptr_;
    delete bias_ptr_;
}

// l-ten/conv2d.cpp:238-264: uint8 weights {Cout, Cin, kh*kw}, int32 bias {1, Cout, 1, 1}, on the CPU, no initialisation.
bool Conv2d_q::init()
{
    TensorOps options;
    options.data_type = UINT8;
    weight_ptr_ = new Tensor;
    *weight_ptr_ = AllocateTensor({channels_out_, channels_in_, kernel_h_ * kernel_w_}, &options);
    if (use_bias_) {
        options.data_type = INT32;
        bias_ptr_ = new Tensor;
        *bias_ptr_ = AllocateTensor({1, channels_out_, 1, 1}, &options);
    }
    return true;
}

std::vector<Tensor *> Conv2d_q::get_all_weights()
{
    std::vector<Tensor *> weights;
    weights.push_back(weight_ptr_);
    if (use_bias_) weights.push_back(bias_ptr_);
    return weights;
}

void Conv2d_q::set_qparams_params(QuantizationParams *qparams, int count)
{
    if (qparams && count) qparams_wt_ = qparams[0];  // l-ten/conv2d.cpp:400-406
}

void Conv2d_q::set_output(ltq_out_mode mode, bool relu, bool saturate, bool bias_per_channel)
{
    out_mode_ = mode;
    flags_ = (flags_ & (LTQ_FLAG_NHWC_IN | LTQ_FLAG_NHWC_OUT)) | (relu ? LTQ_FLAG_RELU : 0u) | (saturate ? LTQ_FLAG_SATURATE : 0u) |
             (bias_per_channel ? LTQ_FLAG_BIAS_PER_CHANNEL : 0u);
}

void Conv2d_q::to(device target_device, int target_device_index)
{
    if (!weight_ptr_) LTEN_ERR("init() has not been called");
    *weight_ptr_ = weight_ptr_->to(target_device, target_device_index);
    if (bias_ptr_) *bias_ptr_ = bias_ptr_->to(target_device, target_device_index);
    ltq_conv2d_destroy(handle_);
    handle_ = nullptr;
    if (target_device == GPU) {
        LTQ_CALL(ltq_conv2d_create(&handle_, target_device_index, channels_in_, channels_out_, kernel_h_, kernel_w_, pad_h_,
                                   pad_w_, stride_h_, stride_w_));
        LTQ_CALL(ltq_conv2d_set_weights(handle_, static_cast<const uint8_t *>(weight_ptr_->get_data_ptr()),
                                        bias_ptr_ ? static_cast<const int32_t *>(bias_ptr_->get_data_ptr()) : nullptr,
                                        nullptr));
    }
}

void Conv2d_q::set_layout(bool channels_last_in, bool channels_last_out)
{
    flags_ = (flags_ & ~(LTQ_FLAG_NHWC_IN | LTQ_FLAG_NHWC_OUT)) | (channels_last_in ? LTQ_FLAG_NHWC_IN : 0u) |
             (channels_last_out ? LTQ_FLAG_NHWC_OUT : 0u);
}

Tensor Conv2d_q::forward(Tensor &input)
{
    // the reference's checks, messages and order: l-ten/conv2d.cpp:285-301
    if (input.get_data_type() != UINT8) LTEN_ERR("Conv2d_q is only supported for UINT8 tensors");
    if (input.get_device() != weight_ptr_->get_device() || input.get_device_index() != weight_ptr_->get_device_index() ||
        input.get_data_type() != weight_ptr_->get_data_type())
        LTEN_ERR("Input tensor device type or data type are not the same as this layer's parameters");
    if (input.get_ndims() != 4) LTEN_ERR("Conv2d_q requires tensors with exactly 4 dimensions (NCHW)");
    if (input.get_device() != GPU) LTEN_ERR("Conv2d_q: this build computes on GPU tensors only; call to(GPU, index) first");
    const uint64_t *in = input.get_sizes();
    const bool cl_in = (flags_ & LTQ_FLAG_NHWC_IN) != 0, cl_out = (flags_ & LTQ_FLAG_NHWC_OUT) != 0;
    const uint64_t h_in = cl_in ? in[1] : in[2], w_in = cl_in ? in[2] : in[3];
    if ((cl_in ? in[3] : in[1]) != channels_in_) LTEN_ERR("Conv2d_q: the input's channel count is not the layer's");
    uint64_t ho = 0, wo = 0;
    LTQ_CALL(ltq_conv2d_output_size(handle_, h_in, w_in, &ho, &wo));

    TensorOps options;
    options.data_type = out_mode_ == LTQ_OUT_U8 ? UINT8 : (out_mode_ == LTQ_OUT_F32 ? FLOAT32 : INT32);
    options.device_type = GPU;
    options.device_index = input.get_device_index();
    Tensor result = cl_out ? AllocateTensor({in[0], ho, wo, channels_out_}, &options) : AllocateTensor({in[0], channels_out_, ho, wo}, &options);
    LTQ_CALL(ltq_conv2d_set_qparams(handle_, &qparams_in_, &qparams_wt_, &qparams_out_));
    LTQ_CALL(ltq_conv2d_forward(handle_, static_cast<const uint8_t *>(input.get_data_ptr()), in[0], h_in, w_in, out_mode_,
                                flags_, result.get_data_ptr(), nullptr));
    return result;
}

// ---- checkpoint I/O -------------------------------------------------------------------------------------------------------
namespace {
const char CKPT_MAGIC[8] = {'L', 'T', 'Q', 'C', 'K', 'P', 'T', '1'};
uint8_t dtype_code(dtype d) { return d == UINT8 ? 0 : (d == INT32 ? 1 : 2); }
}  // namespace

int save_checkpoint(const std::vector<Module *> &modules, const char *checkpoint_path)
{
    FILE *f = fopen(checkpoint_path, "wb");
    if (!f) return -1;
    bool ok = fwrite(CKPT_MAGIC, 1, 8, f) == 8;
    const uint32_t n = (uint32_t)modules.size();
    ok = ok && fwrite(&n, 4, 1, f) == 1;
    for (Module *m : modules) {
        std::vector<Tensor *> ts = m->get_all_weights();
        const uint32_t nt = (uint32_t)ts.size();
        ok = ok && fwrite(&nt, 4, 1, f) == 1;
        for (Tensor *t : ts) {
            Tensor host = t->to(CPU);
            const uint8_t head[4] = {dtype_code(host.get_data_type()), 0, 0, 0};
            const uint32_t nd = (uint32_t)host.get_ndims();
            ok = ok && fwrite(head, 1, 4, f) == 4 && fwrite(&nd, 4, 1, f) == 1;
            ok = ok && fwrite(host.get_sizes(), 8, nd, f) == nd;
            const size_t bytes = host.get_numels() * dtype_size(host.get_data_type());
            ok = ok && fwrite(host.get_data_ptr(), 1, bytes, f) == bytes;
        }
        QuantizationParams q[3];
        m->get_qparams(q);
        for (int i = 0; i < 3; i++) {
            const uint8_t tail[4] = {q[i].zero_point, 0, 0, 0};
            ok = ok && fwrite(&q[i].scale, 4, 1, f) == 1 && fwrite(tail, 1, 4, f) == 4;
        }
    }
    ok = (fclose(f) == 0) && ok;
    return ok ? 0 : -1;
}

int load_checkpoint(const std::vector<Module *> &modules, const char *checkpoint_path)
{
    FILE *f = fopen(checkpoint_path, "rb");
    if (!f) return -1;
    char magic[8];
    uint32_t n = 0;
    bool ok = fread(magic, 1, 8, f) == 8 && memcmp(magic, CKPT_MAGIC, 8) == 0 && fread(&n, 4, 1, f) == 1 &&
              n == modules.size();
    for (size_t mi = 0; ok && mi < modules.size(); mi++) {
        Module *m = modules[mi];
        std::vector<Tensor *> ts = m->get_all_weights();
        uint32_t nt = 0;
        ok = fread(&nt, 4, 1, f) == 1 && nt == ts.size();
        for (size_t ti = 0; ok && ti < ts.size(); ti++) {
            Tensor *t = ts[ti];
            uint8_t head[4];
            uint32_t nd = 0;
            uint64_t dims[MAX_DIMS];
            ok = fread(head, 1, 4, f) == 4 && fread(&nd, 4, 1, f) == 1 && nd == (uint32_t)t->get_ndims() && nd <= MAX_DIMS &&
                 head[0] == dtype_code(t->get_data_type()) && fread(dims, 8, nd, f) == nd &&
                 memcmp(dims, t->get_sizes(), 8 * nd) == 0;
            if (!ok) break;
            const size_t bytes = t->get_numels() * dtype_size(t->get_data_type());
            if (t->get_device() == CPU) {
                ok = fread(t->get_data_ptr(), 1, bytes, f) == bytes;
            } else {
                std::vector<uint8_t> buf(bytes);
                ok = fread(buf.data(), 1, bytes, f) == bytes &&
                     cudaMemcpy(t->get_data_ptr(), buf.data(), bytes, cudaMemcpyHostToDevice) == cudaSuccess;
            }
        }
        QuantizationParams q[3];
        for (int i = 0; ok && i < 3; i++) {
            uint8_t tail[4];
            ok = fread(&q[i].scale, 4, 1, f) == 1 && fread(tail, 1, 4, f) == 4;
            q[i].zero_point = tail[0];
        }
        if (ok) {
            m->set_qparams_in(q[0]);
            m->set_qparams_params(&q[1], 1);
            m->set_qparams_out(q[2]);
        }
    }
    fclose(f);
    return ok ? 0 : -1;
}

// ---- calibration / quantisation set-up -----------------------------------------------------------------------------------
void MinMaxObserver::update(const Tensor &x)
{
    if (!x.defined() || x.get_device() != GPU || x.get_data_type() != FLOAT32) LTEN_ERR("MinMaxObserver: FLOAT32 GPU tensor expected");
    float mn, mx;
    ::GetMinMax((float *)x.get_data_ptr(), x.get_numels(), &mn, &mx);
    if (mn < min_) min_ = mn;
    if (mx > max_) max_ = mx;
}

QuantizationParams MinMaxObserver::qparams() const
{
    if (!seen()) LTEN_ERR("MinMaxObserver: no data has been observed");
    QuantizationParams qp;
    ::ComputeQuantizationParams(min_, max_, &qp);
    return qp;
}

QuantizationParams quantize_module(Module &q_mod, const Tensor &weight, const Tensor *bias, QuantizationParams qp_in,
                                   QuantizationParams qp_out)
{
    std::vector<Tensor *> tensors = q_mod.get_all_weights();
    if (tensors.empty() || !tensors[0] || !tensors[0]->defined()) LTEN_ERR("quantize_module: init() has not been called");
    if (!weight.defined() || weight.get_device() != GPU || weight.get_data_type() != FLOAT32)
        LTEN_ERR("quantize_module: FLOAT32 GPU weight tensor expected");
    if (weight.get_numels() != tensors[0]->get_numels()) LTEN_ERR("quantize_module: weight size does not match the module");
    QuantizationParams qps[2];
    int count = 0;
    float mn, mx;
    ::GetMinMax((float *)weight.get_data_ptr(), weight.get_numels(), &mn, &mx);
    ::ComputeQuantizationParams(mn, mx, &qps[0]);
    TensorOps o;
    o.device_type = GPU;
    o.device_index = weight.get_device_index();
    o.data_type = UINT8;
    Tensor wq = AllocateTensor({weight.get_numels()}, &o);
    ::Quantize((float *)weight.get_data_ptr(), (uint8_t *)wq.get_data_ptr(), weight.get_numels(), &qps[0]);
    LTEN_CUDA(cudaMemcpy(tensors[0]->get_data_ptr(), wq.get_data_ptr(), weight.get_numels(), cudaMemcpyDefault));
    count = 1;
    if (tensors.size() > 1) {
        if (!bias) LTEN_ERR("quantize_module: the module uses a bias but none was given");
        if (!bias->defined() || bias->get_device() != GPU || bias->get_data_type() != FLOAT32)
            LTEN_ERR("quantize_module: FLOAT32 GPU bias tensor expected");
        if (bias->get_numels() != tensors[1]->get_numels()) LTEN_ERR("quantize_module: bias size does not match the module");
        // arXiv:1712.05877: the bias shares the accumulator's scale, s_in * s_wt, with zero point 0 (nn_tests.cpp:824-826)
        qps[1].scale = qp_in.scale * qps[0].scale;
        qps[1].zero_point = 0;
        o.data_type = INT32;
        Tensor bq = AllocateTensor({bias->get_numels()}, &o);
        ::Quantize((float *)bias->get_data_ptr(), (int *)bq.get_data_ptr(), bias->get_numels(), &qps[1]);
        LTEN_CUDA(cudaMemcpy(tensors[1]->get_data_ptr(), bq.get_data_ptr(), bias->get_numels() * sizeof(int32_t), cudaMemcpyDefault));
        count = 2;
    }
    q_mod.set_qparams_in(qp_in);
    q_mod.set_qparams_out(qp_out);
    q_mod.set_qparams_params(qps, count);
    return qps[0];
}

}  // namespace lten

// ---- free functions ----------------------------------------------------------------------------------------------------
namespace {

// -1: host memory; otherwise the CUDA device that owns the pointer.
int device_of(const void *p)
{
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return (a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged) ? a.device : -1;
}

void fail(const char *msg, const char *func)
{
    fprintf(stderr, "[Error] Function: %s Msg: %s\n", func, msg);
    throw lten::ExceptionInfo(msg, __FILE__, func, 0);
}

#define FREE_LTQ_CALL(expr) \
    do {                    \
        if ((expr) != LTQ_OK) fail(ltq_last_error(), __func__); \
    } while (0)

}  // namespace

void ComputeQuantizationParams(float min_val, float max_val, QuantizationParams *qp)
{
    FREE_LTQ_CALL(ltq_compute_qparams(min_val, max_val, qp));
}

void GetMinMax(float *data, uint64_t len, float *min_val, float *max_val)
{
    if (!data || !min_val || !max_val) fail("Invalid argument", __func__);  // l-ten/utils.cpp:204-207
    const int dev = device_of(data);
    if (dev < 0) fail("GetMinMax: host data is not computed by this build; pass a device pointer", __func__);
    float *mm = nullptr, h[2];
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(dev);
    if (cudaMalloc(&mm, 2 * sizeof(float)) != cudaSuccess) fail("cudaMalloc failed", __func__);
    const int rc = ltq_get_min_max(data, len, mm, dev, nullptr);
    const cudaError_t ce = cudaMemcpy(h, mm, sizeof h, cudaMemcpyDeviceToHost);
    cudaFree(mm);
    cudaSetDevice(prev);
    if (rc != LTQ_OK) fail(ltq_last_error(), __func__);
    if (ce != cudaSuccess) fail(cudaGetErrorString(ce), __func__);
    *min_val = h[0];
    *max_val = h[1];
}

void Quantize(float *data, uint8_t *q_data, uint64_t len, QuantizationParams *qp)
{
    const int dev = device_of(data);
    if (dev < 0 || device_of(q_data) != dev) fail("Quantize: both buffers must be on the same CUDA device", __func__);
    FREE_LTQ_CALL(ltq_quantize_u8(data, q_data, len, qp, dev, nullptr));
}

void Quantize(float *data, int *q_data, uint64_t len, QuantizationParams *qp)
{
    const int dev = device_of(data);
    if (dev < 0 || device_of(q_data) != dev) fail("Quantize: both buffers must be on the same CUDA device", __func__);
    FREE_LTQ_CALL(ltq_quantize_i32(data, q_data, len, qp, dev, nullptr));
}

void Dequantize(float *data, uint8_t *q_data, uint64_t len, QuantizationParams *qp)
{
    const int dev = device_of(q_data);
    if (dev < 0 || device_of(data) != dev) fail("Dequantize: both buffers must be on the same CUDA device", __func__);
    FREE_LTQ_CALL(ltq_dequantize(data, q_data, len, qp, dev, nullptr));
}
