"""ltq -- thin Python binding over libltq.so, the sm_100a CUDA library behind include/ltq.h.

Everything here goes through the C ABI with raw device pointers (``torch`` is used only to own device memory and
streams).  There is no fallback: if the shared library is missing or no CUDA device is usable, calls raise.

Names mirror the l-ten reference so that tests read like its own:
``GetMinMax / ComputeQuantizationParams / Quantize / Dequantize`` (l-ten/utils.h:23-27), ``quantized_matmul``
(l-ten/math_fns.h:104), ``FullyConnected_q`` (l-ten/layers.h:69-106) and ``Conv2d_q`` (l-ten/layers.h:453-524).
"""
from ._binding import (LtqError, QParams, lib, lib_path, last_error, last_kernel, kernel_launches, OUT_U8, OUT_F32, OUT_I32,
                       FLAG_RELU, FLAG_SATURATE, FLAG_BIAS_PER_CHANNEL, FLAG_FORCE_SIMT, FLAG_FORCE_TC, FLAG_FORCE_SKINNY, FLAG_FORCE_TC_PAIR, FLAG_FORCE_TC_SINGLE, FLAG_MULTICAST_DEST, FLAG_NHWC_IN, FLAG_NHWC_OUT,
                       DECLARED_SYMBOLS)
from .ops import (GetMinMax, ComputeQuantizationParams, compute_qparams_dev, Quantize, QuantizeInt32, Dequantize,
                  quantize_rows, row_sums, quantized_matmul, quantized_matmul_static, matmul_u8)
from .layer import Conv2d_q, ConvHandle, FullyConnected_q, FusedMLP, LayerHandle
from .calibration import MinMaxObserver, calibrate, quantize_module
from .checkpoint import load_checkpoint, save_checkpoint
from .group import DeviceGroup

__all__ = [
    "LtqError", "QParams", "lib", "lib_path", "last_error", "last_kernel", "kernel_launches", "OUT_U8", "OUT_F32", "OUT_I32",
    "FLAG_RELU", "FLAG_SATURATE", "FLAG_BIAS_PER_CHANNEL", "FLAG_FORCE_SIMT", "FLAG_FORCE_TC", "FLAG_FORCE_SKINNY", "FLAG_FORCE_TC_PAIR", "FLAG_FORCE_TC_SINGLE", "FLAG_MULTICAST_DEST", "FLAG_NHWC_IN", "FLAG_NHWC_OUT", "DECLARED_SYMBOLS",
    "GetMinMax", "ComputeQuantizationParams", "compute_qparams_dev", "Quantize", "QuantizeInt32", "Dequantize",
    "quantize_rows", "row_sums", "quantized_matmul", "quantized_matmul_static", "matmul_u8", "FullyConnected_q", "LayerHandle", "FusedMLP", "Conv2d_q", "ConvHandle", "MinMaxObserver", "calibrate", "quantize_module", "save_checkpoint", "load_checkpoint", "DeviceGroup",
]
