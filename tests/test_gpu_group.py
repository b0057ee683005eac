"""GPU: the single-process multi-device entry points (ltq_comm_*, ltq_linear_forward_rowsharded,
ltq_linear_forward_colsharded_allgather) through ``ltq.DeviceGroup``, against the CPU oracle.  Runs with as many devices
as the box has, up to 4 (one device exercises the same code with a group of one; the NCCL all-gather and the relayout
need two or more)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _devices(cuda):
    return list(range(min(cuda.cuda.device_count(), 4)))


def test_row_sharded_group_matches_the_oracle(cuda, oracle):
    import ltq
    devs = _devices(cuda)
    rng = np.random.default_rng(3)
    M, K, N = 600, 512, 384
    a = rng.integers(0, 256, (M, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    bias = rng.integers(-9000, 9000, N, dtype=np.int32)
    qps = (ltq.QParams(0.02, 101), ltq.QParams(0.004, 140), ltq.QParams(0.7, 31))
    want, _ = oracle.port.quantized_matmul(a, w, M, N, K, [oracle.qp(q.scale, q.zero_point) for q in qps], bias=bias)
    grp = ltq.DeviceGroup(devs)
    layers, xs, keep = [], [], []
    bounds = [M * i // len(devs) for i in range(len(devs) + 1)]
    for i, d in enumerate(devs):
        wd, bd = cuda.from_numpy(w).to(f"cuda:{d}"), cuda.from_numpy(bias).to(f"cuda:{d}")
        h = ltq.LayerHandle(d, K, N)
        h.set_weights(wd, bd)
        h.set_qparams(*qps)
        layers.append(h)
        xs.append(cuda.from_numpy(a[bounds[i]:bounds[i + 1]]).to(f"cuda:{d}"))
    for d in devs:
        cuda.cuda.synchronize(d)
    outs = grp.forward_rowsharded(layers, xs)
    grp.synchronize(timeout_ms=20000)
    got = np.concatenate([o.cpu().numpy() for o in outs])
    np.testing.assert_array_equal(got, want)
    # dynamic quantisation: the global min / max over every device's rows
    x32 = rng.normal(0, 2, (M, 64)).astype(np.float32)
    mms = []
    for i, d in enumerate(devs):
        part = cuda.from_numpy(x32[bounds[i]:bounds[i + 1]]).to(f"cuda:{d}")
        with cuda.cuda.device(d), cuda.cuda.stream(grp.streams[i]):
            mms.append(ltq.GetMinMax(part))
    grp.allreduce_minmax(mms)
    grp.synchronize(timeout_ms=20000)
    for mm in mms:
        np.testing.assert_array_equal(mm.cpu().numpy(), np.array([x32.min(), x32.max()], dtype=np.float32))
    grp.close()


@pytest.mark.parametrize("out_mode", ["u8", "f32"])
def test_column_sharded_group_matches_the_oracle(cuda, oracle, out_mode):
    import ltq
    devs = _devices(cuda)
    n = len(devs)
    rng = np.random.default_rng(4)
    M, K, N = 300, 256, 96 * n
    a = rng.integers(0, 256, (M, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    bias = rng.integers(-9000, 9000, N, dtype=np.int32)
    qps = (ltq.QParams(0.02, 101), ltq.QParams(0.004, 140), ltq.QParams(0.4, 31))
    acc = oracle.port.acc_i32(a, w, M, N, K, 101, 140, bias=bias)
    mode = ltq.OUT_U8 if out_mode == "u8" else ltq.OUT_F32
    want = oracle.port.epilogue_u8(acc, 0.02, 0.004, 0.4, 31) if out_mode == "u8" else oracle.port.epilogue_f32(acc, 0.02, 0.004)
    grp = ltq.DeviceGroup(devs)
    layers, xs = [], []
    nloc = N // n
    for i, d in enumerate(devs):
        wd = cuda.from_numpy(w[i * nloc:(i + 1) * nloc].copy()).to(f"cuda:{d}")
        bd = cuda.from_numpy(bias[i * nloc:(i + 1) * nloc].copy()).to(f"cuda:{d}")
        h = ltq.LayerHandle(d, K, nloc)
        h.set_weights(wd, bd)
        h.set_qparams(*qps)
        layers.append(h)
        xs.append(cuda.from_numpy(a).to(f"cuda:{d}"))
    for d in devs:
        cuda.cuda.synchronize(d)
    for _ in range(2):      # twice: buffers and communicators are reusable
        outs = grp.forward_colsharded(layers, xs, mode)
        grp.synchronize(timeout_ms=20000)
        for o in outs:
            got = o.cpu().numpy()
            np.testing.assert_array_equal(got.view(np.uint32) if out_mode == "f32" else got,
                                          want.view(np.uint32) if out_mode == "f32" else want)
    grp.close()
