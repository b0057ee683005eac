"""GPU: the allocation-free entry point ``ltq_quantized_matmul_static`` against the ordinary ``ltq_quantized_matmul``.

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


def _pair(cuda, ltq, rng, M, N, K, tA, tB):
    A = cuda.from_numpy(rng.integers(0, 256, M * K, dtype=np.uint8)).cuda()
    B = cuda.from_numpy(rng.integers(0, 256, N * K, dtype=np.uint8)).cuda()
    bias = cuda.from_numpy(rng.integers(-30000, 30000, N, dtype=np.int32)).cuda()
    qps = [ltq.QParams(0.02, int(rng.integers(0, 256))), ltq.QParams(0.005, int(rng.integers(0, 256))),
           ltq.QParams(float(K) * 0.05, int(rng.integers(0, 256)))]
    want = cuda.full((M, N), 0x5A, dtype=cuda.uint8, device="cuda")
    ws = cuda.empty(M + N, dtype=cuda.int32, device="cuda")
    ltq.quantized_matmul(tA, tB, M, N, K, 1, A, B, 0, want, qps, bias, ws)
    got = cuda.full((M, N), 0xA5, dtype=cuda.uint8, device="cuda")
    ltq.quantized_matmul_static(tA, tB, M, N, K, 1, A, B, 0, got, qps, bias)
    cuda.cuda.synchronize()
    return got, want


@pytest.mark.parametrize("variant", [(False, True), (False, False), (True, True), (True, False)])
def test_two_calls_in_a_row_match_the_workspace_entry_point(cuda, variant):
    import ltq
    rng = np.random.default_rng(42)
    tA, tB = variant
    # first call: tensor-core sized for the FC layout; second: smaller and ragged, reusing the same scratch
    for (M, N, K) in ((384, 640, 1024), (37, 90, 200)):
        got, want = _pair(cuda, ltq, rng, M, N, K, tA, tB)
        assert cuda.equal(got, want), f"M={M} N={N} K={K} tA={tA} tB={tB}"


def test_skinny_shape_twice(cuda):
    import ltq
    rng = np.random.default_rng(43)
    for (M, N, K) in ((16, 1000, 4096), (3, 1000, 4096)):
        got, want = _pair(cuda, ltq, rng, M, N, K, False, True)
        assert cuda.equal(got, want)


def test_rejects_sizes_beyond_the_built_in_scratch(cuda):
    import ltq
    a = cuda.zeros(16, dtype=cuda.uint8, device="cuda")
    with pytest.raises(ltq.LtqError) as e:
        ltq.quantized_matmul_static(False, True, 200000, 70000, 16, 1, a, a, 0, a, [ltq.QParams(1, 0)] * 3, None)
    assert e.value.status == -6 and "262144" in str(e.value)
