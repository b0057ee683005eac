"""Function-level mirror of the reference's free functions, on device tensors, through the C ABI."""
import ctypes as C

import torch

from ._binding import OUT_F32, OUT_I32, OUT_U8, QParams, check, lib


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _dev(t):
    if not t.is_cuda:
        raise ValueError("ltq operates on CUDA tensors only (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def GetMinMax(data, out=None):
    """l-ten/utils.cpp:198-226 on a float32 CUDA tensor.  Returns a 2-element float32 CUDA tensor {min, max} (`out` if
    given: a loop that must not allocate passes its own)."""
    assert data.dtype == torch.float32
    d = _dev(data)
    if out is None:
        out = torch.empty(2, dtype=torch.float32, device=data.device)
    check(lib().ltq_get_min_max(data.data_ptr(), data.numel(), out.data_ptr(), d, _stream(data)))
    return out


def ComputeQuantizationParams(min_val, max_val):
    """l-ten/utils.cpp:266-286 (host scalars)."""
    qp = QParams()
    check(lib().ltq_compute_qparams(float(min_val), float(max_val), C.byref(qp)))
    return qp


def compute_qparams_dev(minmax, out=None):
    """Same rule evaluated on the device: returns an 8-byte CUDA buffer laid out as QParams (`out` if given; its padding
    bytes are left as they are)."""
    d = _dev(minmax)
    if out is None:
        out = torch.zeros(8, dtype=torch.uint8, device=minmax.device)
    check(lib().ltq_compute_qparams_dev(minmax.data_ptr(), out.data_ptr(), d, _stream(minmax)))
    return out


def qparams_from_dev(buf):
    """Copies a device QParams buffer back to the host (synchronises)."""
    raw = bytes(buf.cpu().numpy().tobytes())
    return QParams.from_buffer_copy(raw)


def Quantize(data, qp, out=None):
    """Quantize(float*, uint8_t*, len, qp), l-ten/utils.cpp:243-254."""
    assert data.dtype == torch.float32
    d = _dev(data)
    if out is None:
        out = torch.empty(data.shape, dtype=torch.uint8, device=data.device)
    check(lib().ltq_quantize_u8(data.data_ptr(), out.data_ptr(), data.numel(), C.byref(qp), d, _stream(data)))
    return out


def QuantizeInt32(data, qp, out=None):
    """Quantize(float*, int*, len, qp), l-ten/utils.cpp:228-241 (bias)."""
    assert data.dtype == torch.float32
    d = _dev(data)
    if out is None:
        out = torch.empty(data.shape, dtype=torch.int32, device=data.device)
    check(lib().ltq_quantize_i32(data.data_ptr(), out.data_ptr(), data.numel(), C.byref(qp), d, _stream(data)))
    return out


def Dequantize(q, qp, out=None):
    """Dequantize, l-ten/utils.cpp:256-264."""
    assert q.dtype == torch.uint8
    d = _dev(q)
    if out is None:
        out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    check(lib().ltq_dequantize(out.data_ptr(), q.data_ptr(), q.numel(), C.byref(qp), d, _stream(q)))
    return out


def quantize_rows(x, qp=None, qp_dev=None, q=None, asum=None):
    """Activation quantise fused with the row sums the GEMM epilogue needs.  x: float32 [M,K]."""
    assert x.dtype == torch.float32 and x.dim() == 2
    d = _dev(x)
    M, K = x.shape
    if q is None:
        q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    if asum is None:
        asum = torch.empty(M, dtype=torch.int32, device=x.device)
    check(lib().ltq_quantize_rows_u8(x.data_ptr(), M, K, None if qp is None else C.byref(qp),
                                     None if qp_dev is None else qp_dev.data_ptr(), q.data_ptr(), asum.data_ptr(), d,
                                     _stream(x)))
    return q, asum


def row_sums(m):
    assert m.dtype == torch.uint8 and m.dim() == 2
    d = _dev(m)
    out = torch.empty(m.shape[0], dtype=torch.int32, device=m.device)
    check(lib().ltq_row_sums_u8(m.data_ptr(), m.shape[0], m.shape[1], out.data_ptr(), d, _stream(m)))
    return out


def quantized_matmul(transpose_A, transpose_B, M, N, K, alpha, A, B, beta, C_out, qparams, bias, workspace):
    """quantized_matmul (l-ten/math_fns.h:104), same argument order; tensors are CUDA tensors.

    ``workspace``: int32 CUDA tensor with at least M + N elements."""
    d = _dev(A)
    assert A.dtype == torch.uint8 and B.dtype == torch.uint8 and C_out.dtype == torch.uint8
    assert workspace.dtype == torch.int32 and workspace.numel() >= M + N
    arr = (QParams * 3)(*qparams)
    check(lib().ltq_quantized_matmul(int(transpose_A), int(transpose_B), M, N, K, alpha, A.data_ptr(), B.data_ptr(),
                                     beta, C_out.data_ptr(), arr, None if bias is None else bias.data_ptr(),
                                     workspace.data_ptr(), d, _stream(A)))
    return C_out


def matmul_u8(A, B, transpose_A=False, transpose_B=False, qparams=None, bias=None, out_mode=OUT_I32, flags=0):
    """uint8 x uint8 matrix product on CUDA tensors (2-D, contiguous) with the transpose conventions of
    quantized_matmul: A is [M,K] ([K,M] transposed), B is [K,N] ([N,K] transposed).  Default: the plain int32 product
    (zero points 0) -- what ``Tensor::matmul`` has no implementation for with UINT8 tensors (l-ten/math_fns.cpp:1295-1305).
    With ``qparams`` (three QuantizationParams) the zero-point-corrected product in the chosen output mode."""
    assert A.dtype == torch.uint8 and B.dtype == torch.uint8 and A.dim() == 2 and B.dim() == 2
    M, K = (A.shape[1], A.shape[0]) if transpose_A else A.shape
    N = B.shape[0] if transpose_B else B.shape[1]
    assert (B.shape[1] if transpose_B else B.shape[0]) == K, "inner dimensions differ"
    d = _dev(A)
    arr = (QParams * 3)(*(qparams or [QParams(1.0, 0)] * 3))
    out = torch.empty((M, N), dtype={OUT_U8: torch.uint8, OUT_F32: torch.float32, OUT_I32: torch.int32}[out_mode],
                      device=A.device)
    ws = torch.empty(M + N, dtype=torch.int32, device=A.device)
    check(lib().ltq_quantized_matmul_ex(int(transpose_A), int(transpose_B), M, N, K, 1, A.data_ptr(), B.data_ptr(), 0,
                                        out.data_ptr(), arr, None if bias is None else bias.data_ptr(), ws.data_ptr(),
                                        out_mode, flags, d, _stream(A)))
    return out


def quantized_matmul_static(transpose_A, transpose_B, M, N, K, alpha, A, B, beta, C_out, qparams, bias):
    """``quantized_matmul`` without a caller workspace and without any device allocation: for callers that are not
    allowed to allocate (they run inside a host framework's planned memory, or must stay clear of the allocator's lock).
    The operand sums go to a fixed scratch array inside the library; M + N is limited to 262144 and calls that overlap
    on the GPU must be ordered by the caller."""
    d = _dev(A)
    assert A.dtype == torch.uint8 and B.dtype == torch.uint8 and C_out.dtype == torch.uint8
    arr = (QParams * 3)(*qparams)
    check(lib().ltq_quantized_matmul_static(int(transpose_A), int(transpose_B), M, N, K, alpha, A.data_ptr(),
                                            B.data_ptr(), beta, C_out.data_ptr(), arr,
                                            None if bias is None else bias.data_ptr(), d, _stream(A)))
    return C_out
