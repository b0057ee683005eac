"""ctypes declarations for every symbol include/ltq.h declares."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG_ROOT = os.path.dirname(os.path.dirname(_HERE))


class LtqError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"ltq status {status}: {message}")
        self.status = status


class QParams(C.Structure):
    """``struct QuantizationParams`` (l-ten/math_fns.h:12-16): real = scale * (q - zero_point)."""
    _fields_ = [("scale", C.c_float), ("zero_point", C.c_uint8)]

    def __repr__(self):
        return f"QParams(scale={self.scale!r}, zero_point={self.zero_point})"


OUT_U8, OUT_F32, OUT_I32 = 0, 1, 2
MAX_DESTS = 8
FLAG_RELU, FLAG_SATURATE, FLAG_BIAS_PER_CHANNEL = 1, 2, 4
FLAG_FORCE_SIMT, FLAG_FORCE_TC, FLAG_FORCE_SKINNY = 0x100, 0x200, 0x400
FLAG_FORCE_TC_PAIR, FLAG_FORCE_TC_SINGLE = 0x800, 0x1000
FLAG_MULTICAST_DEST = 0x2000
FLAG_NHWC_IN, FLAG_NHWC_OUT = 0x4000, 0x8000

_u64, _vp, _int = C.c_uint64, C.c_void_p, C.c_int
_qp = C.POINTER(QParams)

# name -> (restype, argtypes); one entry per declaration in include/ltq.h
_SIGNATURES = {
    "ltq_version": (_int, []),
    "ltq_last_error": (C.c_char_p, []),
    "ltq_kernel_launches": (_u64, []),
    "ltq_last_kernel": (C.c_char_p, []),
    "ltq_get_min_max": (_int, [_vp, _u64, _vp, _int, _vp]),
    "ltq_compute_qparams": (_int, [C.c_float, C.c_float, _qp]),
    "ltq_compute_qparams_dev": (_int, [_vp, _vp, _int, _vp]),
    "ltq_quantize_u8": (_int, [_vp, _vp, _u64, _qp, _int, _vp]),
    "ltq_quantize_i32": (_int, [_vp, _vp, _u64, _qp, _int, _vp]),
    "ltq_dequantize": (_int, [_vp, _vp, _u64, _qp, _int, _vp]),
    "ltq_quantize_rows_u8": (_int, [_vp, _u64, _u64, _qp, _vp, _vp, _vp, _int, _vp]),
    "ltq_row_sums_u8": (_int, [_vp, _u64, _u64, _vp, _int, _vp]),
    "ltq_interleave_column_blocks": (_int, [_vp, _vp, _u64, _u64, _u64, _int, _vp]),
    "ltq_quantized_matmul": (_int, [_int, _int, _u64, _u64, _u64, C.c_uint8, _vp, _vp, C.c_uint8, _vp, _qp, _vp, _vp,
                                    _int, _vp]),
    "ltq_quantized_matmul_ex": (_int, [_int, _int, _u64, _u64, _u64, C.c_uint8, _vp, _vp, C.c_uint8, _vp, _qp, _vp, _vp,
                                       _int, C.c_uint, _int, _vp]),
    "ltq_quantized_matmul_static": (_int, [_int, _int, _u64, _u64, _u64, C.c_uint8, _vp, _vp, C.c_uint8, _vp, _qp, _vp,
                                           _int, _vp]),
    "ltq_static_check": (_int, [_int, _vp]),
    "ltq_selftest_bounded_wait_static": (_int, [_int, C.c_uint32, _vp]),
    "ltq_layer_create": (_int, [C.POINTER(_vp), _int, _u64, _u64]),
    "ltq_layer_destroy": (_int, [_vp]),
    "ltq_layer_set_weights": (_int, [_vp, _vp, _vp, _vp]),
    "ltq_layer_set_qparams": (_int, [_vp, _qp, _qp, _qp]),
    "ltq_layer_forward": (_int, [_vp, _vp, _vp, _u64, _vp, _int, C.c_uint, _vp, _vp]),
    "ltq_layer_check": (_int, [_vp, _vp]),
    "ltq_layer_set_rowsum_output": (_int, [_vp, _vp]),
    "ltq_layer_set_clear_on_forward": (_int, [_vp, _vp, _u64]),
    "ltq_layer_set_next": (_int, [_vp, _vp]),
    "ltq_layer_forward_scatter": (_int, [_vp, _vp, _vp, _u64, _vp, _int, C.c_uint, C.POINTER(_vp), _int, _u64, _u64, _vp]),
    "ltq_peer_alloc": (_int, [C.POINTER(_vp), _u64, _int, C.c_char_p]),
    "ltq_peer_free": (_int, [_vp, _int]),
    "ltq_peer_open": (_int, [C.c_char_p, _int, C.POINTER(_vp)]),
    "ltq_peer_close": (_int, [_vp, _int]),
    "ltq_mlp_create": (_int, [C.POINTER(_vp), C.POINTER(_vp), _int]),
    "ltq_mlp_destroy": (_int, [_vp]),
    "ltq_mlp_forward": (_int, [_vp, _vp, _u64, C.POINTER(C.c_uint), _int, _vp, _vp]),
    "ltq_comm_init_all": (_int, [C.POINTER(_vp), _int, C.POINTER(_int)]),
    "ltq_comm_destroy": (_int, [_vp]),
    "ltq_comm_size": (_int, [_vp]),
    "ltq_comm_device": (_int, [_vp, _int]),
    "ltq_comm_stream": (_vp, [_vp, _int]),
    "ltq_comm_synchronize": (_int, [_vp, C.c_uint32]),
    "ltq_linear_forward_rowsharded": (_int, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_u64),
                                             C.POINTER(_vp), _int, C.c_uint, C.POINTER(_vp)]),
    "ltq_comm_allreduce_minmax": (_int, [_vp, C.POINTER(_vp)]),
    "ltq_linear_forward_colsharded_allgather": (_int, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _u64,
                                                       C.POINTER(_vp), _int, C.c_uint, C.POINTER(_vp), C.POINTER(_vp),
                                                       C.POINTER(_vp)]),
    "ltq_comm_set_backend": (_int, [_vp]),
    "ltq_conv2d_create": (_int, [C.POINTER(_vp), _int] + [_u64] * 8),
    "ltq_conv2d_destroy": (_int, [_vp]),
    "ltq_conv2d_set_weights": (_int, [_vp, _vp, _vp, _vp]),
    "ltq_conv2d_set_qparams": (_int, [_vp, _qp, _qp, _qp]),
    "ltq_conv2d_output_size": (_int, [_vp, _u64, _u64, C.POINTER(_u64), C.POINTER(_u64)]),
    "ltq_conv2d_forward": (_int, [_vp, _vp, _u64, _u64, _u64, _int, C.c_uint, _vp, _vp]),
    "ltq_im2col_t_u8": (_int, [_vp, _u64] + [_u64] * 9 + [_vp, _u64, _int, _vp]),
    "ltq_device_check": (_int, [_int, _vp]),
    "ltq_selftest_bounded_wait": (_int, [_int, C.c_uint32, _vp]),
}
DECLARED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def lib_path():
    return os.environ.get("LTQ_LIBRARY", os.path.join(_PKG_ROOT, "lib", "libltq.so"))


def lib():
    """Loads libltq.so once.  Raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise LtqError(-3, f"{path} not found: build it with `make -C {_PKG_ROOT}` (nvcc, sm_100a); "
                               "there is no CPU fallback")
        L = C.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error():
    return lib().ltq_last_error().decode("utf-8", "replace")


def kernel_launches():
    return int(lib().ltq_kernel_launches())


def last_kernel():
    """Name of the GEMM kernel this thread launched last (what the shape-based dispatch chose)."""
    return lib().ltq_last_kernel().decode("ascii", "replace")


def check(status):
    if status != 0:
        raise LtqError(status, last_error())
