"""CPU: the C-ABI library loads, exports every symbol include/ltq.h declares, and its host-only logic behaves.
No compute call is made here (there is no GPU); calls that would need one must fail with a CUDA status, never fall
back to the host."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "ltq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ltq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import ltq
    L = ltq.lib()
    names = header_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/ltq.h but not exported by libltq.so"
    assert sorted(ltq.DECLARED_SYMBOLS) == names, "python binding and header disagree"
    assert L.ltq_version() == 1


def test_qparams_layout_matches_reference_struct():
    import ltq
    assert C.sizeof(ltq.QParams) == 8
    assert ltq.QParams.scale.offset == 0 and ltq.QParams.zero_point.offset == 4


def test_compute_qparams_matches_oracle(oracle):
    import ltq
    rng = np.random.default_rng(3)
    for _ in range(200):
        lo, hi = sorted(np.float32(v) for v in rng.normal(0, 3, 2))
        if rng.integers(0, 4) == 0:
            lo = np.float32(abs(lo))
            hi = np.float32(lo + abs(hi))
        a = ltq.ComputeQuantizationParams(lo, hi)
        b = oracle.port.compute_qparams(lo, hi)
        assert (np.float32(a.scale), a.zero_point) == (np.float32(b.scale), b.zero_point)


def test_compute_qparams_rejects_empty_range():
    import ltq
    with pytest.raises(ltq.LtqError) as e:
        ltq.ComputeQuantizationParams(0.0, 0.0)
    assert e.value.status == -1


def test_argument_errors_are_status_codes():
    import ltq
    L = ltq.lib()
    qp = (ltq.QParams * 3)(ltq.QParams(1, 0), ltq.QParams(1, 0), ltq.QParams(1, 0))
    # alpha != 1 / beta != 0 -> unsupported, with the reference's message (l-ten/math_fns.cpp:1331-1334)
    assert L.ltq_quantized_matmul(0, 1, 4, 4, 4, 2, 16, 16, 0, 16, qp, None, 16, 0, None) == -2
    assert "alpha != 1" in ltq.last_error()
    assert L.ltq_quantized_matmul(0, 1, 4, 4, 4, 1, 16, 16, 1, 16, qp, None, 16, 0, None) == -2
    # null pointers
    assert L.ltq_quantized_matmul(0, 1, 4, 4, 4, 1, None, 16, 0, 16, qp, None, 16, 0, None) == -1
    assert L.ltq_get_min_max(None, 10, None, 0, None) == -1
    assert L.ltq_layer_forward(None, None, None, 1, None, 0, 0, None, None) == -1
    # K * zA * zB must fit an int (l-ten/math_fns.cpp:1433-1434)
    big = (ltq.QParams * 3)(ltq.QParams(1, 255), ltq.QParams(1, 255), ltq.QParams(1, 0))
    assert L.ltq_quantized_matmul(0, 1, 4, 4, 40000, 1, 16, 16, 0, 16, big, None, 16, 0, None) == -2


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import ltq
    L = ltq.lib()
    h = C.c_void_p()
    rc = L.ltq_layer_create(C.byref(h), 0, 64, 16)
    assert rc == -3 and not h.value, "without a device the library must fail with LTQ_ERR_CUDA"
    x = np.zeros(16, np.float32)
    q = np.zeros(16, np.uint8)
    qp = ltq.QParams(1, 0)
    assert L.ltq_quantize_u8(x.ctypes.data, q.ctypes.data, 16, C.byref(qp), 0, None) == -3


def test_python_layer_mirror_checks():
    import torch
    import ltq
    fc = ltq.FullyConnected_q(8, 4, True)
    assert fc.init()
    ws = fc.get_all_weights()
    assert tuple(ws[0].shape) == (1, 1, 4, 8) and ws[0].dtype == torch.uint8
    assert tuple(ws[1].shape) == (4,) and ws[1].dtype == torch.int32
    assert fc.is_using_bias()
    with pytest.raises(ValueError, match="at least 3 dimensions"):
        fc.forward(torch.zeros((2, 8), dtype=torch.uint8))
    with pytest.raises(ValueError, match="not the same as this layer's parameters"):
        fc.forward(torch.zeros((1, 2, 8), dtype=torch.float32))
    with pytest.raises(ValueError, match="Last dimension"):
        fc.forward(torch.zeros((1, 2, 9), dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        fc.forward(torch.zeros((1, 2, 8), dtype=torch.uint8))
    qs = [ltq.QParams(0.5, 3), ltq.QParams(0.25, 9)]
    fc.set_qparams_params(qs, 2)
    assert fc.qparams_wt_.zero_point == 3  # only [0] is kept (l-ten/fully_connected.cpp:440-446)
