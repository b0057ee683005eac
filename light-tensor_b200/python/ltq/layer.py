"""``FullyConnected_q`` (l-ten/layers.h:69-106) and ``Conv2d_q`` (l-ten/layers.h:453-524) with the reference's method
names, driving the CUDA library."""
import ctypes as C

import torch

from ._binding import (OUT_F32, OUT_I32, OUT_U8, FLAG_BIAS_PER_CHANNEL, FLAG_NHWC_IN, FLAG_NHWC_OUT, FLAG_RELU, FLAG_SATURATE, QParams, check,
                       lib)

_OUT_DTYPE = {OUT_U8: torch.uint8, OUT_F32: torch.float32, OUT_I32: torch.int32}


class LayerHandle:
    """Owns one ``ltq_layer`` (device-side derived state of a quantized linear layer)."""

    def __init__(self, device_index, in_features, out_features):
        self._h = C.c_void_p()
        self.device_index = device_index
        self.K, self.N = in_features, out_features
        check(lib().ltq_layer_create(C.byref(self._h), device_index, in_features, out_features))

    def close(self):
        if self._h:
            lib().ltq_layer_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device_index).cuda_stream)

    def set_weights(self, w, bias=None):
        assert w.is_cuda and w.dtype == torch.uint8 and w.is_contiguous() and w.numel() == self.N * self.K
        if bias is not None:
            assert bias.is_cuda and bias.dtype == torch.int32 and bias.numel() == self.N
        self._keep = (w, bias)  # the library borrows these pointers
        check(lib().ltq_layer_set_weights(self._h, w.data_ptr(), None if bias is None else bias.data_ptr(),
                                          self._stream()))

    def set_qparams(self, qp_in=None, qp_wt=None, qp_out=None):
        ref = lambda q: None if q is None else C.byref(q)
        check(lib().ltq_layer_set_qparams(self._h, ref(qp_in), ref(qp_wt), ref(qp_out)))

    def forward(self, x, out_mode=OUT_U8, flags=0, asum=None, qp_in_dev=None, out=None):
        """x: uint8 CUDA [M,K] (contiguous).  Returns [M,N] in the dtype of out_mode."""
        assert x.is_cuda and x.dtype == torch.uint8 and x.is_contiguous()
        M = x.numel() // self.K
        if out is None:
            out = torch.empty((M, self.N), dtype=_OUT_DTYPE[out_mode], device=x.device)
        check(lib().ltq_layer_forward(self._h, x.data_ptr(), None if asum is None else asum.data_ptr(), M,
                                      None if qp_in_dev is None else qp_in_dev.data_ptr(), out_mode, flags,
                                      out.data_ptr(), self._stream()))
        return out

    def set_rowsum_output(self, rowsum):
        """int32 CUDA tensor [M] (or None): later uint8-output forwards add each output row's byte sum to it, which is the
        ``asum`` the next layer wants.  Clear it before each forward (``rowsum.zero_()`` on the same stream)."""
        self._rowsum = rowsum
        check(lib().ltq_layer_set_rowsum_output(self._h, None if rowsum is None else rowsum.data_ptr()))

    def set_clear_on_forward(self, array):
        """int32 CUDA tensor (or None) that every later forward of this layer clears, ordered after everything in front
        of it in the stream: the row-sum array of another layer of a chain whose consumer has already run."""
        self._clear = array
        check(lib().ltq_layer_set_clear_on_forward(self._h, None if array is None else array.data_ptr(),
                                                   0 if array is None else array.numel()))

    def set_next(self, nxt):
        """Hint for chains at small batch: ``nxt`` (a LayerHandle or None) is the layer whose forward follows this one's
        on the same stream; the weight-streaming kernel then asks the start of its weights into L2 while it finishes.
        Results are unchanged.  Set it again after ``nxt.set_weights``; pass None before ``nxt``'s weights are freed."""
        self._next = nxt  # keeps the weights it points at alive
        check(lib().ltq_layer_set_next(self._h, None if nxt is None else nxt._h))

    def forward_scatter(self, x, dest_ptrs, ld_out, col_offset, out_mode=OUT_U8, flags=0, asum=None, qp_in_dev=None):
        """Like forward, but element (i, j) goes to ``dest_ptrs[d] + (i * ld_out + col_offset + j) * itemsize`` for
        every d.  dest_ptrs are raw device addresses (this GPU's buffer first, then peers' mapped buffers)."""
        assert x.is_cuda and x.dtype == torch.uint8 and x.is_contiguous()
        M = x.numel() // self.K
        arr = (C.c_void_p * len(dest_ptrs))(*dest_ptrs)
        check(lib().ltq_layer_forward_scatter(self._h, x.data_ptr(), None if asum is None else asum.data_ptr(), M,
                                              None if qp_in_dev is None else qp_in_dev.data_ptr(), out_mode, flags, arr,
                                              len(dest_ptrs), ld_out, col_offset, self._stream()))

    def check(self):
        check(lib().ltq_layer_check(self._h, self._stream()))


class FusedMLP:
    """``ltq_mlp``: Quantize(input) and a chain of 2 to 4 quantized linear layers as one kernel launch per batch (clusters
    of 8 CTAs, activations kept in distributed shared memory).  ``layers``: LayerHandles with weights and qparams set,
    layer l+1 consuming layer l's uint8 output.  Raises LtqError(-2) when the chain does not fit one cluster."""

    def __init__(self, layers):
        self.layers = list(layers)           # borrowed by the library: keep them alive
        self._h = C.c_void_p()
        arr = (C.c_void_p * len(self.layers))(*[l._h.value for l in self.layers])
        check(lib().ltq_mlp_create(C.byref(self._h), arr, len(self.layers)))

    def close(self):
        if self._h:
            lib().ltq_mlp_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward(self, x, layer_flags=None, out_mode=OUT_U8, out=None):
        """x: float32 CUDA [M, K0] (contiguous).  Returns [M, N_last] in the dtype of out_mode."""
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
        M = x.shape[0]
        if out is None:
            out = torch.empty((M, self.layers[-1].N), dtype=_OUT_DTYPE[out_mode], device=x.device)
        fl = None if layer_flags is None else (C.c_uint * len(self.layers))(*layer_flags)
        check(lib().ltq_mlp_forward(self._h, x.data_ptr(), M, fl, out_mode, out.data_ptr(),
                                    C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)))
        return out


class FullyConnected_q:
    """Quantized fully-connected layer, same surface as l-ten's (l-ten/layers.h:69-106,
    l-ten/fully_connected.cpp:295-446): uint8 weights ``{1,1,N,K}``, int32 bias ``{N}``, three per-tensor
    QuantizationParams.  Weights are written on the host after ``init()`` (as tests/nn_tests.cpp:818-826 does through
    ``get_all_weights()``), then ``to("cuda", idx)`` moves them and builds the device-side state.

    Differences from the reference, all additive: ``to`` works for CUDA (the reference throws), all leading
    dimensions are folded into M, and ``set_output`` selects float / int32 output and a fused ReLU.  There is no CPU
    compute path in this build: ``forward`` on a CPU tensor raises.
    """

    def __init__(self, input_features, output_features, use_bias=False, data_type=None):
        self.input_features_ = int(input_features)
        self.output_features_ = int(output_features)
        self.use_bias_ = bool(use_bias)
        self.weight_ptr_ = None
        self.bias_ptr_ = None
        self.qparams_in_ = QParams(1.0, 0)
        self.qparams_out_ = QParams(1.0, 0)
        self.qparams_wt_ = QParams(1.0, 0)
        self.is_training_ = True
        self._handle = None
        self._out_mode, self._flags = OUT_U8, 0

    def init(self):
        self.weight_ptr_ = torch.zeros((1, 1, self.output_features_, self.input_features_), dtype=torch.uint8)
        if self.use_bias_:
            self.bias_ptr_ = torch.zeros((self.output_features_,), dtype=torch.int32)
        return True

    def get_weights(self):
        return self.weight_ptr_

    def get_bias(self):
        return self.bias_ptr_

    def get_all_weights(self):
        return [self.weight_ptr_] + ([self.bias_ptr_] if self.use_bias_ else [])

    def is_using_bias(self):
        return self.use_bias_

    def clear_gradients(self):
        pass

    def train(self, is_training):
        self.is_training_ = bool(is_training)

    def set_qparams_in(self, qp):
        self.qparams_in_ = QParams(qp.scale, qp.zero_point)
        self._push_qparams()

    def set_qparams_out(self, qp):
        self.qparams_out_ = QParams(qp.scale, qp.zero_point)
        self._push_qparams()

    def set_qparams_params(self, qparams, count):
        # l-ten/fully_connected.cpp:440-446: only the weight parameters ([0]) are kept
        if qparams and count:
            self.qparams_wt_ = QParams(qparams[0].scale, qparams[0].zero_point)
            self._push_qparams()

    def set_output(self, out_mode=OUT_U8, relu=False, saturate=False):
        self._out_mode = out_mode
        self._flags = (FLAG_RELU if relu else 0) | (FLAG_SATURATE if saturate else 0)

    def _push_qparams(self):
        if self._handle is not None:
            self._handle.set_qparams(self.qparams_in_, self.qparams_wt_, self.qparams_out_)

    def to(self, target_device, target_device_index=0):
        if self.weight_ptr_ is None:
            raise RuntimeError("init() has not been called")
        dev = torch.device(target_device, target_device_index) if str(target_device) != "cpu" else torch.device("cpu")
        self.weight_ptr_ = self.weight_ptr_.to(dev).contiguous()
        if self.bias_ptr_ is not None:
            self.bias_ptr_ = self.bias_ptr_.to(dev).contiguous()
        if self._handle is not None:
            self._handle.close()
            self._handle = None
        if dev.type == "cuda":
            self._handle = LayerHandle(dev.index, self.input_features_, self.output_features_)
            self._handle.set_weights(self.weight_ptr_, self.bias_ptr_)
            self._push_qparams()

    def refresh_weights(self):
        """Call after overwriting the device weight bytes in place (recomputes the cached weight row sums)."""
        self._handle.set_weights(self.weight_ptr_, self.bias_ptr_)

    def forward(self, input, asum=None, qp_in_dev=None):
        # same checks, same messages, same order as l-ten/fully_connected.cpp:330-348
        if input.dim() < 3:
            raise ValueError("FullyConnected_q requires tensors with at least 3 dimensions")
        if (input.device != self.weight_ptr_.device) or (input.dtype != self.weight_ptr_.dtype):
            raise ValueError("Input tensor device type or data type are not the same as this layer's parameters")
        if input.shape[-1] != self.input_features_:
            raise ValueError("Last dimension must be equal to the number of input features")
        if not input.is_cuda:
            raise RuntimeError("FullyConnected_q: this build computes on CUDA devices only; call to('cuda', idx) first")
        x = input.contiguous()
        out = self._handle.forward(x.view(-1, self.input_features_), self._out_mode, self._flags, asum=asum,
                                   qp_in_dev=qp_in_dev)
        return out.view(*input.shape[:-1], self.output_features_)


class ConvHandle:
    """Owns one ``ltq_conv2d`` (device-side derived state of a quantized convolution)."""

    def __init__(self, device_index, channels_in, channels_out, kernel_h, kernel_w, pad_h=0, pad_w=0, stride_h=1,
                 stride_w=1):
        self._h = C.c_void_p()
        self.device_index = device_index
        self.Cin, self.Cout, self.K = channels_in, channels_out, channels_in * kernel_h * kernel_w
        check(lib().ltq_conv2d_create(C.byref(self._h), device_index, channels_in, channels_out, kernel_h, kernel_w,
                                      pad_h, pad_w, stride_h, stride_w))

    def close(self):
        if self._h:
            lib().ltq_conv2d_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device_index).cuda_stream)

    def set_weights(self, w, bias=None):
        assert w.is_cuda and w.dtype == torch.uint8 and w.is_contiguous() and w.numel() == self.Cout * self.K
        if bias is not None:
            assert bias.is_cuda and bias.dtype == torch.int32 and bias.numel() == self.Cout
        self._keep = (w, bias)  # the library borrows these pointers
        check(lib().ltq_conv2d_set_weights(self._h, w.data_ptr(), None if bias is None else bias.data_ptr(),
                                           self._stream()))

    def set_qparams(self, qp_in=None, qp_wt=None, qp_out=None):
        ref = lambda q: None if q is None else C.byref(q)
        check(lib().ltq_conv2d_set_qparams(self._h, ref(qp_in), ref(qp_wt), ref(qp_out)))

    def output_size(self, height_in, width_in):
        ho, wo = C.c_uint64(), C.c_uint64()
        check(lib().ltq_conv2d_output_size(self._h, height_in, width_in, C.byref(ho), C.byref(wo)))
        return ho.value, wo.value

    def forward(self, x, out_mode=OUT_U8, flags=0, out=None):
        """x: uint8 CUDA NCHW (contiguous), or [B, H, W, Cin] with FLAG_NHWC_IN.  Returns [B, Cout, Ho, Wo] - with
        FLAG_NHWC_OUT [B, Ho, Wo, Cout] - in the dtype of out_mode."""
        assert x.is_cuda and x.dtype == torch.uint8 and x.is_contiguous() and x.dim() == 4
        if flags & FLAG_NHWC_IN:
            B, H, W, C = x.shape
        else:
            B, C, H, W = x.shape
        assert C == self.Cin
        ho, wo = self.output_size(H, W)
        if out is None:
            shape = (B, ho, wo, self.Cout) if flags & FLAG_NHWC_OUT else (B, self.Cout, ho, wo)
            out = torch.empty(shape, dtype=_OUT_DTYPE[out_mode], device=x.device)
        check(lib().ltq_conv2d_forward(self._h, x.data_ptr(), B, H, W, out_mode, flags, out.data_ptr(), self._stream()))
        return out


class Conv2d_q:
    """Quantized 2-D convolution with the reference's surface (l-ten/layers.h:453-524, l-ten/conv2d.cpp:238-400):
    uint8 weights ``{Cout, Cin, kh*kw}``, optional int32 bias ``{1, Cout, 1, 1}``, three per-tensor
    QuantizationParams, NCHW uint8 in and out.  The reference computes this layer on the CPU only and its ``to``
    throws; here ``to("cuda", idx)`` builds the device state and ``forward`` runs on the GPU (no CPU compute path).

    ``set_output(bias_per_channel=True)`` adds ``bias[c]`` per output channel; by default the bias is applied the way
    the reference's GEMM applies it, per output position, which is only defined while ``Ho*Wo <= channels_out``.
    """

    def __init__(self, channels_in, channels_out, use_bias, kernel_h, kernel_w, pad_h=0, pad_w=0, stride_h=1, stride_w=1):
        self.channels_in_, self.channels_out_ = int(channels_in), int(channels_out)
        self.kernel_h_, self.kernel_w_ = int(kernel_h), int(kernel_w)
        self.pad_h_, self.pad_w_ = int(pad_h), int(pad_w)
        self.stride_h_, self.stride_w_ = int(stride_h), int(stride_w)
        self.use_bias_ = bool(use_bias)
        self.weight_ptr_ = None
        self.bias_ptr_ = None
        self.qparams_in_ = QParams(1.0, 0)
        self.qparams_out_ = QParams(1.0, 0)
        self.qparams_wt_ = QParams(1.0, 0)
        self._handle = None
        self._out_mode, self._flags = OUT_U8, 0

    def get_channels_out(self):
        return self.channels_out_

    def get_channels_in(self):
        return self.channels_in_

    def get_kernel_h(self):
        return self.kernel_h_

    def get_kernel_w(self):
        return self.kernel_w_

    def get_pad_h(self):
        return self.pad_h_

    def get_pad_w(self):
        return self.pad_w_

    def get_stride_h(self):
        return self.stride_h_

    def get_stride_w(self):
        return self.stride_w_

    def init(self):
        self.weight_ptr_ = torch.zeros((self.channels_out_, self.channels_in_, self.kernel_h_ * self.kernel_w_),
                                       dtype=torch.uint8)
        if self.use_bias_:
            self.bias_ptr_ = torch.zeros((1, self.channels_out_, 1, 1), dtype=torch.int32)
        return True

    def get_weights(self):
        return self.weight_ptr_

    def get_bias(self):
        return self.bias_ptr_

    def get_all_weights(self):
        return [self.weight_ptr_] + ([self.bias_ptr_] if self.use_bias_ else [])

    def clear_gradients(self):
        pass

    def train(self, is_training):
        pass

    def set_qparams_in(self, qp):
        self.qparams_in_ = QParams(qp.scale, qp.zero_point)
        self._push_qparams()

    def set_qparams_out(self, qp):
        self.qparams_out_ = QParams(qp.scale, qp.zero_point)
        self._push_qparams()

    def set_qparams_params(self, qparams, count):
        # l-ten/conv2d.cpp:400-406: only the weight parameters ([0]) are kept
        if qparams and count:
            self.qparams_wt_ = QParams(qparams[0].scale, qparams[0].zero_point)
            self._push_qparams()

    def set_output(self, out_mode=OUT_U8, relu=False, saturate=False, bias_per_channel=False):
        self._out_mode = out_mode
        self._flags = ((self._flags & (FLAG_NHWC_IN | FLAG_NHWC_OUT)) | (FLAG_RELU if relu else 0) |
                       (FLAG_SATURATE if saturate else 0) | (FLAG_BIAS_PER_CHANNEL if bias_per_channel else 0))

    def set_layout(self, channels_last_in=False, channels_last_out=False):
        """Additive: channels-last placement ([N, H, W, C]) of the input and / or the output, for chains of layers that
        are computed from a channels-last copy anyway (stride 1, input channels a multiple of 64, output channels a
        multiple of 16); forward raises for other layers.  The values are those of the NCHW call."""
        self._flags = ((self._flags & ~(FLAG_NHWC_IN | FLAG_NHWC_OUT)) | (FLAG_NHWC_IN if channels_last_in else 0) |
                       (FLAG_NHWC_OUT if channels_last_out else 0))

    def _push_qparams(self):
        if self._handle is not None:
            self._handle.set_qparams(self.qparams_in_, self.qparams_wt_, self.qparams_out_)

    def to(self, target_device, target_device_index=0):
        if self.weight_ptr_ is None:
            raise RuntimeError("init() has not been called")
        dev = torch.device(target_device, target_device_index) if str(target_device) != "cpu" else torch.device("cpu")
        self.weight_ptr_ = self.weight_ptr_.to(dev).contiguous()
        if self.bias_ptr_ is not None:
            self.bias_ptr_ = self.bias_ptr_.to(dev).contiguous()
        if self._handle is not None:
            self._handle.close()
            self._handle = None
        if dev.type == "cuda":
            self._handle = ConvHandle(dev.index, self.channels_in_, self.channels_out_, self.kernel_h_, self.kernel_w_,
                                      self.pad_h_, self.pad_w_, self.stride_h_, self.stride_w_)
            self._handle.set_weights(self.weight_ptr_, self.bias_ptr_)
            self._push_qparams()

    def forward(self, input):
        # same checks, same messages, same order as l-ten/conv2d.cpp:285-301
        if input.dtype != torch.uint8:
            raise ValueError("Conv2d_q is only supported for UINT8 tensors")
        if (input.device != self.weight_ptr_.device) or (input.dtype != self.weight_ptr_.dtype):
            raise ValueError("Input tensor device type or data type are not the same as this layer's parameters")
        if input.dim() != 4:
            raise ValueError("Conv2d_q requires tensors with exactly 4 dimensions (NCHW)")
        if not input.is_cuda:
            raise RuntimeError("Conv2d_q: this build computes on CUDA devices only; call to('cuda', idx) first")
        return self._handle.forward(input.contiguous(), self._out_mode, self._flags)
