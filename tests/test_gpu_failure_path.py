"""GPU: the device-side failure path, exercised without hanging or faulting anything.  A probe kernel waits on a barrier
that nothing ever signals; its bounded wait gives up after a few milliseconds, records a code in the device status word
and returns.  The host then sees LTQ_ERR_DEVICE_TIMEOUT once, the word is cleared, and the context keeps working."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_is_reported_once(cuda, oracle):
    import ltq
    L = ltq.lib()
    assert L.ltq_device_check(0, None) == 0
    t0 = time.time()
    assert L.ltq_selftest_bounded_wait(0, 5000, None) == 0          # 5 ms limit
    rc = L.ltq_device_check(0, None)                                # synchronises
    elapsed = time.time() - t0
    assert rc == -4, "expected LTQ_ERR_DEVICE_TIMEOUT"
    assert "0x900" in ltq.last_error()
    assert 0.004 < elapsed < 2.0, f"the wait should give up after ~5 ms, took {elapsed:.3f} s"
    assert L.ltq_device_check(0, None) == 0, "the status word is cleared after it has been reported"
    # the context is still usable: a tensor-core GEMM right after, checked against the oracle
    rng = np.random.default_rng(1)
    M, N, K = 256, 256, 512
    a = rng.integers(0, 256, (M, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    h = ltq.LayerHandle(0, K, N)
    h.set_weights(cuda.from_numpy(w).cuda(), None)
    h.set_qparams(ltq.QParams(0.1, 3), ltq.QParams(0.1, 200), ltq.QParams(1.0, 0))
    got = h.forward(cuda.from_numpy(a).cuda(), ltq.OUT_I32, ltq.FLAG_FORCE_TC).cpu().numpy()
    h.check()
    np.testing.assert_array_equal(got, oracle.port.acc_i32(a, w, M, N, K, 3, 200))


def test_selftest_rejects_silly_limits(cuda):
    import ltq
    assert ltq.lib().ltq_selftest_bounded_wait(0, 0, None) == -1
    assert ltq.lib().ltq_selftest_bounded_wait(0, 5_000_000, None) == -1
