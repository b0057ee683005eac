"""``FullyConnected_q`` with the reference's method names (l-ten/layers.h:69-106) driving the CUDA library."""
import ctypes as C

import torch

from ._binding import OUT_F32, OUT_I32, OUT_U8, FLAG_RELU, FLAG_SATURATE, QParams, check, lib

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

    def check(self):
        check(lib().ltq_layer_check(self._h, self._stream()))


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
