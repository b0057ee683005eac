"""ctypes doors into the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Two libraries live under ``oracle/_ref`` (built by ``oracle/Makefile``):

* ``libltq_oracle.so`` -- ``ltq_oracle.c``, a plain-C restatement of the l-ten
  quantized fully-connected arithmetic (l-ten/math_fns.cpp:1311-1478,
  l-ten/utils.cpp:198-286).  Exposed here as :data:`port`.
* ``liblten_ref.so``   -- the unmodified l-ten reference compiled CPU-only from
  its own sources, behind ``ref_wrapper.cpp``.  Exposed as :data:`ref`
  (``None`` when it was never built).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package; the shipped library never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_OUT = os.path.join(_HERE, "_ref")


class QParams(C.Structure):
    """l-ten/math_fns.h:12-16"""
    _fields_ = [("scale", C.c_float), ("zero_point", C.c_uint8)]

    def __repr__(self):
        return f"QParams(scale={self.scale!r}, zero_point={self.zero_point})"


def qp(scale, zero_point):
    return QParams(np.float32(scale), int(zero_point))


def build(with_ref=None):
    """Compile the oracle libraries (gcc/g++ via oracle/Makefile).

    ``with_ref=None`` builds the reference library only when the reference
    source tree is present on this machine."""
    ref_tree = os.environ.get("LTEN_REFERENCE", "/root/reference")
    if with_ref is None:
        with_ref = os.path.isdir(os.path.join(ref_tree, "l-ten"))
    targets = ["oracle"] + (["ref"] if with_ref else [])
    subprocess.run(["make", "-s", "-j8", "-C", _HERE, f"REF={ref_tree}"] + targets, check=True)


def _ptr(a, ct):
    return a.ctypes.data_as(C.POINTER(ct))


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


class _Port:
    """Plain-C restatement (``kind: "port"``)."""

    def __init__(self, path):
        self.lib = C.CDLL(path)
        L = self.lib
        u64, vp = C.c_uint64, C.c_void_p
        L.oracle_get_min_max.argtypes = [vp, u64, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.oracle_compute_qparams.argtypes = [C.c_float, C.c_float, C.POINTER(QParams)]
        L.oracle_quantize_u8.argtypes = [vp, vp, u64, C.POINTER(QParams)]
        L.oracle_quantize_i32.argtypes = [vp, vp, u64, C.POINTER(QParams)]
        L.oracle_dequantize.argtypes = [vp, vp, u64, C.POINTER(QParams)]
        L.oracle_operand_sums.argtypes = [C.c_int, C.c_int, u64, u64, u64, vp, vp, vp, vp]
        L.oracle_acc_i32.argtypes = [C.c_int, C.c_int, u64, u64, u64, vp, vp, C.c_int, C.c_int, vp, vp]
        L.oracle_real_multiplier.argtypes = [C.c_float] * 3
        L.oracle_real_multiplier.restype = C.c_float
        L.oracle_epilogue_u8.argtypes = [vp, u64, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int, C.c_int, vp]
        L.oracle_epilogue_f32.argtypes = [vp, u64, C.c_float, C.c_float, C.c_int, vp]
        L.oracle_quantized_matmul.argtypes = [C.c_int, C.c_int, u64, u64, u64, C.c_uint8, vp, vp, C.c_uint8, vp,
                                              C.POINTER(QParams), vp, vp]
        L.oracle_quantized_matmul.restype = C.c_int
        L.oracle_im2col.argtypes = [vp] + [u64] * 9 + [vp]
        L.oracle_conv2d_q.argtypes = [vp, u64, u64, u64, u64, vp, vp, C.c_int] + [u64] * 7 + [C.POINTER(QParams)] * 3 + [vp]
        L.oracle_conv2d_q.restype = C.c_int

    def get_min_max(self, x):
        x = _c(x, np.float32)
        mn, mx = C.c_float(), C.c_float()
        self.lib.oracle_get_min_max(x.ctypes.data, x.size, C.byref(mn), C.byref(mx))
        return np.float32(mn.value), np.float32(mx.value)

    def compute_qparams(self, mn, mx):
        out = QParams()
        self.lib.oracle_compute_qparams(np.float32(mn), np.float32(mx), C.byref(out))
        return out

    def quantize_u8(self, x, q):
        x = _c(x, np.float32)
        out = np.empty(x.shape, np.uint8)
        self.lib.oracle_quantize_u8(x.ctypes.data, out.ctypes.data, x.size, C.byref(q))
        return out

    def quantize_i32(self, x, q):
        x = _c(x, np.float32)
        out = np.empty(x.shape, np.int32)
        self.lib.oracle_quantize_i32(x.ctypes.data, out.ctypes.data, x.size, C.byref(q))
        return out

    def dequantize(self, qv, q):
        qv = _c(qv, np.uint8)
        out = np.empty(qv.shape, np.float32)
        self.lib.oracle_dequantize(out.ctypes.data, qv.ctypes.data, qv.size, C.byref(q))
        return out

    def operand_sums(self, A, B, M, N, K, tA=False, tB=True):
        A, B = _c(A, np.uint8), _c(B, np.uint8)
        bsum, asum = np.empty(N, np.int32), np.empty(M, np.int32)
        self.lib.oracle_operand_sums(int(tA), int(tB), M, N, K, A.ctypes.data, B.ctypes.data, bsum.ctypes.data,
                                     asum.ctypes.data)
        return bsum, asum

    def acc_i32(self, A, B, M, N, K, zA, zB, bias=None, tA=False, tB=True):
        """int32 value before scaling (l-ten/math_fns.cpp:1433-1473)."""
        A, B = _c(A, np.uint8), _c(B, np.uint8)
        assert A.size == M * K and B.size == N * K
        acc = np.empty((M, N), np.int32)
        b = None if bias is None else _c(bias, np.int32)
        self.lib.oracle_acc_i32(int(tA), int(tB), M, N, K, A.ctypes.data, B.ctypes.data, int(zA), int(zB),
                                None if b is None else b.ctypes.data, acc.ctypes.data)
        return acc

    def real_multiplier(self, sA, sB, sC):
        return np.float32(self.lib.oracle_real_multiplier(np.float32(sA), np.float32(sB), np.float32(sC)))

    def epilogue_u8(self, acc, sA, sB, sC, zC, relu=False, saturate=False):
        acc = _c(acc, np.int32)
        out = np.empty(acc.shape, np.uint8)
        self.lib.oracle_epilogue_u8(acc.ctypes.data, acc.size, np.float32(sA), np.float32(sB), np.float32(sC),
                                    int(zC), int(relu), int(saturate), out.ctypes.data)
        return out

    def epilogue_f32(self, acc, sA, sB, relu=False):
        acc = _c(acc, np.int32)
        out = np.empty(acc.shape, np.float32)
        self.lib.oracle_epilogue_f32(acc.ctypes.data, acc.size, np.float32(sA), np.float32(sB), int(relu),
                                     out.ctypes.data)
        return out

    def quantized_matmul(self, A, B, M, N, K, qps, bias=None, tA=False, tB=True, alpha=1, beta=0):
        """Whole reference call; returns (C u8 [M,N], workspace int32 [N+M]) or raises on alpha/beta."""
        A, B = _c(A, np.uint8), _c(B, np.uint8)
        Cm = np.empty((M, N), np.uint8)
        ws = np.empty(M + N, np.int32)
        b = None if bias is None else _c(bias, np.int32)
        arr = (QParams * 3)(*qps)
        rc = self.lib.oracle_quantized_matmul(int(tA), int(tB), M, N, K, alpha, A.ctypes.data, B.ctypes.data, beta,
                                              Cm.ctypes.data, arr, None if b is None else b.ctypes.data,
                                              ws.ctypes.data)
        if rc != 0:
            raise ValueError("Support for alpha != 1 and beta != 0 not implemented")
        return Cm, ws


    def im2col(self, im, kh, kw, ph=0, pw=0, sh=1, sw=1):
        """im u8 [C,H,W] -> col u8 [C*kh*kw, Ho*Wo] (the reference's layout)."""
        im = _c(im, np.uint8)
        Cn, H, W = im.shape
        ho, wo = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        col = np.empty((Cn * kh * kw, ho * wo), np.uint8)
        self.lib.oracle_im2col(im.ctypes.data, Cn, H, W, kh, kw, ph, pw, sh, sw, col.ctypes.data)
        return col

    def conv2d_q(self, x, w, cout, kh, kw, qp_in, qp_wt, qp_out, bias=None, ph=0, pw=0, sh=1, sw=1,
                 bias_per_channel=False):
        """x u8 [B,Cin,H,W], w u8 [Cout, Cin*kh*kw] -> out u8 [B,Cout,Ho,Wo]."""
        x, w = _c(x, np.uint8), _c(w, np.uint8)
        B, Cin, H, W = x.shape
        ho, wo = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        out = np.empty((B, cout, ho, wo), np.uint8)
        b = None if bias is None else _c(bias, np.int32)
        rc = self.lib.oracle_conv2d_q(x.ctypes.data, B, Cin, H, W, w.ctypes.data, None if b is None else b.ctypes.data,
                                      int(bias_per_channel), cout, kh, kw, ph, pw, sh, sw, C.byref(qp_in),
                                      C.byref(qp_wt), C.byref(qp_out), out.ctypes.data)
        if rc != 0:
            raise MemoryError("oracle_conv2d_q")
        return out


class _Ref:
    """The unmodified reference (``kind: "reference"``)."""

    def __init__(self, path):
        self.lib = C.CDLL(path)
        L = self.lib
        u64, vp = C.c_uint64, C.c_void_p
        L.ref_get_min_max.argtypes = [vp, u64, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.ref_compute_qparams.argtypes = [C.c_float, C.c_float, C.POINTER(QParams)]
        L.ref_quantize_u8.argtypes = [vp, vp, u64, C.POINTER(QParams)]
        L.ref_quantize_i32.argtypes = [vp, vp, u64, C.POINTER(QParams)]
        L.ref_dequantize.argtypes = [vp, vp, u64, C.POINTER(QParams)]
        L.ref_quantized_matmul.argtypes = [C.c_int, C.c_int, u64, u64, u64, C.c_uint8, vp, vp, C.c_uint8, vp,
                                           C.POINTER(QParams), vp, vp]
        L.ref_quantized_matmul.restype = C.c_int
        L.ref_fc_q_forward.argtypes = [u64, u64, u64, vp, vp, vp, C.POINTER(QParams), C.POINTER(QParams),
                                       C.POINTER(QParams), vp, C.c_int]
        L.ref_fc_q_forward.restype = C.c_double
        if hasattr(L, "ref_conv2d_q_forward"):
            L.ref_im2col.argtypes = [vp] + [u64] * 9 + [vp]
            L.ref_conv2d_q_forward.argtypes = [u64] * 5 + [C.c_int] * 6 + [vp, vp, vp] + [C.POINTER(QParams)] * 3 + [vp]
            L.ref_conv2d_q_forward.restype = C.c_int

    def get_min_max(self, x):
        x = _c(x, np.float32)
        mn, mx = C.c_float(), C.c_float()
        self.lib.ref_get_min_max(x.ctypes.data, x.size, C.byref(mn), C.byref(mx))
        return np.float32(mn.value), np.float32(mx.value)

    def compute_qparams(self, mn, mx):
        out = QParams()
        self.lib.ref_compute_qparams(np.float32(mn), np.float32(mx), C.byref(out))
        return out

    def quantize_u8(self, x, q):
        x = _c(x, np.float32)
        out = np.empty(x.shape, np.uint8)
        self.lib.ref_quantize_u8(x.ctypes.data, out.ctypes.data, x.size, C.byref(q))
        return out

    def quantize_i32(self, x, q):
        x = _c(x, np.float32)
        out = np.empty(x.shape, np.int32)
        self.lib.ref_quantize_i32(x.ctypes.data, out.ctypes.data, x.size, C.byref(q))
        return out

    def dequantize(self, qv, q):
        qv = _c(qv, np.uint8)
        out = np.empty(qv.shape, np.float32)
        self.lib.ref_dequantize(out.ctypes.data, qv.ctypes.data, qv.size, C.byref(q))
        return out

    def quantized_matmul(self, A, B, M, N, K, qps, bias=None, tA=False, tB=True, alpha=1, beta=0):
        A, B = _c(A, np.uint8), _c(B, np.uint8)
        Cm = np.empty((M, N), np.uint8)
        ws = np.empty(M + N, np.int32)
        b = None if bias is None else _c(bias, np.int32)
        arr = (QParams * 3)(*qps)
        rc = self.lib.ref_quantized_matmul(int(tA), int(tB), M, N, K, alpha, A.ctypes.data, B.ctypes.data, beta,
                                           Cm.ctypes.data, arr, None if b is None else b.ctypes.data, ws.ctypes.data)
        if rc != 0:
            raise ValueError("reference raised")
        return Cm, ws

    def fc_q_forward(self, x, w, M, N, K, qp_in, qp_wt, qp_out, bias=None, repeats=1):
        """FullyConnected_q::forward on a {1,M,K} tensor; returns (out u8 [M,N], best seconds)."""
        x, w = _c(x, np.uint8), _c(w, np.uint8)
        out = np.empty((M, N), np.uint8)
        b = None if bias is None else _c(bias, np.int32)
        secs = self.lib.ref_fc_q_forward(M, N, K, x.ctypes.data, w.ctypes.data, None if b is None else b.ctypes.data,
                                         C.byref(qp_in), C.byref(qp_wt), C.byref(qp_out), out.ctypes.data, repeats)
        if secs < 0:
            raise RuntimeError("reference raised")
        return out, secs


    def im2col(self, im, kh, kw, ph=0, pw=0, sh=1, sw=1):
        im = _c(im, np.uint8)
        Cn, H, W = im.shape
        ho, wo = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        col = np.empty((Cn * kh * kw, ho * wo), np.uint8)
        self.lib.ref_im2col(im.ctypes.data, Cn, H, W, kh, kw, ph, pw, sh, sw, col.ctypes.data)
        return col

    def conv2d_q(self, x, w, cout, kh, kw, qp_in, qp_wt, qp_out, bias=None, ph=0, pw=0, sh=1, sw=1):
        """Conv2d_q::forward; only call with a bias while Ho*Wo <= cout (beyond that the reference reads out of bounds)."""
        x, w = _c(x, np.uint8), _c(w, np.uint8)
        B, Cin, H, W = x.shape
        ho, wo = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        if bias is not None and ho * wo > cout:
            raise ValueError("the reference would read past its bias tensor")
        out = np.empty((B, cout, ho, wo), np.uint8)
        b = None if bias is None else _c(bias, np.int32)
        rc = self.lib.ref_conv2d_q_forward(B, Cin, H, W, cout, kh, kw, ph, pw, sh, sw, x.ctypes.data, w.ctypes.data,
                                           None if b is None else b.ctypes.data, C.byref(qp_in), C.byref(qp_wt),
                                           C.byref(qp_out), out.ctypes.data)
        if rc != 0:
            raise RuntimeError("reference raised")
        return out


def _load():
    p = os.path.join(_OUT, "libltq_oracle.so")
    r = os.path.join(_OUT, "liblten_ref.so")
    if not os.path.exists(p):
        build()
    port_ = _Port(p)
    ref_ = _Ref(r) if os.path.exists(r) else None
    return port_, ref_


port, ref = _load()
