"""GPU: the allocation-free entry point ``ltq_quantized_matmul_static`` against the ordinary ``ltq_quantized_matmul``
and against the CPU oracle.

Some callers cannot give the library a workspace because they cannot allocate device memory at all: they run inside a
host framework that planned every byte beforehand, or in a loop that must never touch the allocator.  For them the
operand sums live in a fixed array inside the library.  That array is shared between calls and keeps what the last call
wrote, so the test makes two calls in a row with different operands and shapes (the second smaller, so stale sums sit
right behind its own) and expects byte-identical output to the workspace-taking entry point each time -- the same
tolerance (none) the other uint8 parity tests use.  Kept in a file that sorts last so that a stop-at-first-failure run
has already been through every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _pair(cuda, ltq, oracle, rng, M, N, K, tA, tB):
    A_h = rng.integers(0, 256, M * K, dtype=np.uint8)
    B_h = rng.integers(0, 256, N * K, dtype=np.uint8)
    bias_h = rng.integers(-30000, 30000, N, dtype=np.int32)
    A, B, bias = cuda.from_numpy(A_h).cuda(), cuda.from_numpy(B_h).cuda(), cuda.from_numpy(bias_h).cuda()
    rows = [(0.02, int(rng.integers(0, 256))), (0.005, int(rng.integers(0, 256))), (float(K) * 0.05, int(rng.integers(0, 256)))]
    qps = [ltq.QParams(s, z) for s, z in rows]
    want = cuda.full((M, N), 0x5A, dtype=cuda.uint8, device="cuda")
    ws = cuda.empty(M + N, dtype=cuda.int32, device="cuda")
    ltq.quantized_matmul(tA, tB, M, N, K, 1, A, B, 0, want, qps, bias, ws)
    got = cuda.full((M, N), 0xA5, dtype=cuda.uint8, device="cuda")
    ltq.quantized_matmul_static(tA, tB, M, N, K, 1, A, B, 0, got, qps, bias)
    cuda.cuda.synchronize()
    assert ltq.lib().ltq_static_check(0, None) == 0
    # the CPU oracle on the same bytes (A is [M,K] or [K,M], B is [K,N] or [N,K], as quantized_matmul reads them)
    ref, _ = oracle.port.quantized_matmul(A_h.reshape((K, M) if tA else (M, K)), B_h.reshape((N, K) if tB else (K, N)),
                                          M, N, K, [oracle.qp(np.float32(s), z) for s, z in rows], bias=bias_h, tA=tA, tB=tB)
    return got, want, ref


@pytest.mark.parametrize("variant", [(False, True), (False, False), (True, True), (True, False)])
def test_two_calls_in_a_row_match_the_workspace_entry_point(cuda, oracle, variant):
    import ltq
    rng = np.random.default_rng(42)
    tA, tB = variant
    # first call: tensor-core sized for the FC layout; second: smaller and ragged, reusing the same scratch
    for (M, N, K) in ((384, 640, 1024), (37, 90, 200)):
        got, want, ref = _pair(cuda, ltq, oracle, rng, M, N, K, tA, tB)
        assert cuda.equal(got, want), f"M={M} N={N} K={K} tA={tA} tB={tB}"
        np.testing.assert_array_equal(got.cpu().numpy(), ref)


def test_skinny_shape_twice(cuda, oracle):
    import ltq
    rng = np.random.default_rng(43)
    for (M, N, K) in ((16, 1000, 4096), (3, 1000, 4096)):
        got, want, ref = _pair(cuda, ltq, oracle, rng, M, N, K, False, True)
        assert cuda.equal(got, want)
        np.testing.assert_array_equal(got.cpu().numpy(), ref)
        assert ltq.last_kernel().startswith("gemv_kernel")


def test_no_device_memory_is_allocated(cuda):
    """The property in the name: once the operands exist, calls of any shape (skinny, single-CTA and CTA-pair tensor-core
    kernels, the generic kernel) leave the device's free memory exactly where it was."""
    import ltq
    rng = np.random.default_rng(44)
    shapes = [((8, 520, 1024), False, True, "gemv_kernel"), ((384, 640, 1024), False, True, "gemm_tc_kernel"),
              ((2048, 2304, 256), False, True, "gemm_tc_pair_kernel"), ((90, 70, 100), True, False, "gemm_simt_kernel")]
    ops = []
    for (M, N, K), tA, tB, _ in shapes:
        ops.append((cuda.from_numpy(rng.integers(0, 256, M * K, dtype=np.uint8)).cuda(),
                    cuda.from_numpy(rng.integers(0, 256, N * K, dtype=np.uint8)).cuda(),
                    cuda.empty((M, N), dtype=cuda.uint8, device="cuda"), cuda.empty((M, N), dtype=cuda.uint8, device="cuda"),
                    cuda.empty(M + N, dtype=cuda.int32, device="cuda")))
    qps = [ltq.QParams(0.02, 7), ltq.QParams(0.005, 9), ltq.QParams(40.0, 100)]

    def run_all():
        for ((M, N, K), tA, tB, kern), (A, B, C, _, _) in zip(shapes, ops):
            ltq.quantized_matmul_static(tA, tB, M, N, K, 1, A, B, 0, C, qps, None)
            assert ltq.last_kernel().startswith(kern), (ltq.last_kernel(), kern)
        cuda.cuda.synchronize()

    run_all()                                   # first use of each kernel: module loading, function attributes
    free0 = cuda.cuda.mem_get_info()[0]
    for _ in range(3):
        run_all()
    assert ltq.lib().ltq_static_check(0, None) == 0
    assert cuda.cuda.mem_get_info()[0] == free0, "device memory was allocated by an allocation-free call"
    for ((M, N, K), tA, tB, _), (A, B, C, want, ws) in zip(shapes, ops):
        ltq.quantized_matmul(tA, tB, M, N, K, 1, A, B, 0, want, qps, None, ws)
        assert cuda.equal(C, want)


def test_static_status_word_is_reported_by_the_allocation_free_check(cuda):
    """A bounded wait that runs out inside an allocation-free call lands in the library's built-in status word:
    ltq_static_check reports it once and clears it; ltq_device_check (the allocated word) never sees it."""
    import ltq
    L = ltq.lib()
    assert L.ltq_static_check(0, None) == 0
    assert L.ltq_selftest_bounded_wait_static(0, 5000, None) == 0       # 5 ms limit, nothing hangs or faults
    assert L.ltq_device_check(0, None) == 0
    assert L.ltq_static_check(0, None) == -4
    assert "0x900" in ltq.last_error()
    assert L.ltq_static_check(0, None) == 0
    a = cuda.zeros((64, 64), dtype=cuda.uint8, device="cuda")
    c = cuda.empty((64, 64), dtype=cuda.uint8, device="cuda")
    ltq.quantized_matmul_static(False, True, 64, 64, 64, 1, a, a, 0, c, [ltq.QParams(1, 0)] * 3, None)
    assert L.ltq_static_check(0, None) == 0


def test_rejects_sizes_beyond_the_built_in_scratch(cuda):
    import ltq
    a = cuda.zeros(16, dtype=cuda.uint8, device="cuda")
    with pytest.raises(ltq.LtqError) as e:
        ltq.quantized_matmul_static(False, True, 200000, 70000, 16, 1, a, a, 0, a, [ltq.QParams(1, 0)] * 3, None)
    assert e.value.status == -6 and "262144" in str(e.value)
