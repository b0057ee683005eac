"""GPU: the reference-shaped quantized_matmul entry point and every GEMM kernel against golden vectors and the CPU
oracle.  int32 and uint8 results are compared bit for bit; float results bit for bit as well (tolerance 0), which is
inside the 1e-5 relative bound the path is specified to."""
import numpy as np
import pytest

from helpers import iter_qmm_cases, ltq_qp, qp_of

pytestmark = pytest.mark.gpu


def test_quantized_matmul_small_matches_golden(cuda, golden):
    import ltq
    g = golden("qmm_small.npz")
    n = 0
    for c in iter_qmm_cases(g):
        M, N, K = c["M"], c["N"], c["K"]
        A = cuda.from_numpy(c["A"]).cuda()
        B = cuda.from_numpy(c["B"]).cuda()
        bias = None if c["bias"] is None else cuda.from_numpy(c["bias"]).cuda()
        Cd = cuda.full((M, N), 0xAB, dtype=cuda.uint8, device="cuda")
        ws = cuda.zeros(M + N, dtype=cuda.int32, device="cuda")
        ltq.quantized_matmul(c["tA"], c["tB"], M, N, K, 1, A, B, 0, Cd, [ltq_qp(r) for r in c["qp"]], bias, ws)
        np.testing.assert_array_equal(Cd.cpu().numpy(), c["C"], err_msg=c["key"])
        np.testing.assert_array_equal(ws.cpu().numpy(), c["ws"], err_msg=c["key"])
        n += 1
    assert n >= 100


def _run_layer(cuda, ltq, a, w, bias, qps, out_mode, flags, asum=None):
    N, K = w.shape
    h = ltq.LayerHandle(0, K, N)
    wd = cuda.from_numpy(w).cuda()
    bd = None if bias is None else cuda.from_numpy(bias).cuda()
    h.set_weights(wd, bd)
    h.set_qparams(*qps)
    out = h.forward(cuda.from_numpy(a).cuda(), out_mode, flags, asum=asum)
    h.check()
    res = out.cpu().numpy()
    h.close()
    return res


SHAPES = [
    # (M, N, K)
    (1, 8, 16), (1, 11008 // 8, 4096), (4, 100, 4096), (16, 264, 1040), (9, 72, 48), (16, 8, 8192), (5, 40, 6144), (3, 24, 16384), (4, 16, 32768),
    (16, 333, 384), (3, 7, 128), (12, 1001, 1152), (8, 596, 2048),
    (17, 10, 784), (64, 512, 784), (64, 10, 512), (128, 256, 128), (130, 300, 400), (256, 512, 1024),
    (300, 129, 2064), (128, 64, 16), (1, 1, 16), (77, 333, 112), (600, 520, 1152), (1024, 768, 512),
]


@pytest.mark.parametrize("path", ["simt", "tc", "tcpair", "skinny", "auto"])
@pytest.mark.parametrize("shape", SHAPES)
def test_kernels_vs_oracle_all_modes(cuda, oracle, shape, path):
    import ltq
    M, N, K = shape
    if path == "skinny" and (M > 16 or K % 128):
        pytest.skip("skinny kernel takes M <= 16, K % 128 == 0")
    force = {"simt": ltq.FLAG_FORCE_SIMT, "tc": ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_SINGLE,
             "tcpair": ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR, "skinny": ltq.FLAG_FORCE_SKINNY, "auto": 0}[path]
    rng = np.random.default_rng(M * 7919 + N * 31 + K)
    a = rng.integers(0, 256, (M, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    bias = rng.integers(-50000, 50000, N, dtype=np.int32)
    za, zw, zc = int(rng.integers(0, 256)), int(rng.integers(0, 256)), int(rng.integers(0, 256))
    sa, sw = np.float32(0.02), np.float32(0.005)
    acc = oracle.port.acc_i32(a, w, M, N, K, za, zw, bias=bias)
    # output scale such that results spread over (and beyond) the uint8 range
    sc = np.float32(max(1e-6, np.abs(acc).max() * float(sa * sw) / 150.0))
    qps = (ltq.QParams(sa, za), ltq.QParams(sw, zw), ltq.QParams(sc, zc))

    got = _run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_I32, force)
    np.testing.assert_array_equal(got, acc)
    got = _run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_I32, force | ltq.FLAG_RELU)
    np.testing.assert_array_equal(got, np.maximum(acc, 0))
    for relu in (False, True):
        for sat in (False, True):
            fl = force | (ltq.FLAG_RELU if relu else 0) | (ltq.FLAG_SATURATE if sat else 0)
            got = _run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_U8, fl)
            want = oracle.port.epilogue_u8(acc, sa, sw, sc, zc, relu=relu, saturate=sat)
            np.testing.assert_array_equal(got, want)
        got = _run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_F32, force | (ltq.FLAG_RELU if relu else 0))
        want = oracle.port.epilogue_f32(acc, sa, sw, relu=relu)
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))  # tolerance: 0 ulp
    # no bias, caller-provided activation sums
    asum = cuda.from_numpy(a.astype(np.int64).sum(1).astype(np.int32)).cuda()
    got = _run_layer(cuda, ltq, a, w, None, qps, ltq.OUT_I32, force, asum=asum)
    np.testing.assert_array_equal(got, oracle.port.acc_i32(a, w, M, N, K, za, zw))


@pytest.mark.parametrize("zs", [(0, 0), (255, 255), (0, 255), (255, 0)])
def test_extreme_zero_points_and_saturated_inputs(cuda, oracle, zs):
    import ltq
    M, N, K = 128, 256, 2048
    for fill in (0, 255):
        a = np.full((M, K), fill, np.uint8)
        w = np.full((N, K), 255 - fill if zs[0] else fill, np.uint8)
        qps = (ltq.QParams(0.01, zs[0]), ltq.QParams(0.01, zs[1]), ltq.QParams(1.0, 0))
        for force in (ltq.FLAG_FORCE_SIMT, ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_SINGLE,
                      ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR):
            got = _run_layer(cuda, ltq, a, w, None, qps, ltq.OUT_I32, force)
            np.testing.assert_array_equal(got, oracle.port.acc_i32(a, w, M, N, K, zs[0], zs[1]))


def test_int32_wraps_like_the_reference_beyond_k_33025(cuda, oracle):
    """K * 255^2 exceeds int32 for K > 33025: raw sums wrap mod 2^32 on both sides (no saturation in the MMA)."""
    import ltq
    M, N, K = 128, 64, 34048
    a = np.full((M, K), 255, np.uint8)
    w = np.full((N, K), 255, np.uint8)
    a[::3, ::5] = 7
    qps = (ltq.QParams(0.01, 0), ltq.QParams(0.01, 0), ltq.QParams(1.0, 0))
    want = oracle.port.acc_i32(a, w, M, N, K, 0, 0)
    assert (want < 0).any()
    for force in (ltq.FLAG_FORCE_SIMT, ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_SINGLE,
                  ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR):
        np.testing.assert_array_equal(_run_layer(cuda, ltq, a, w, None, qps, ltq.OUT_I32, force), want)


@pytest.mark.parametrize("shape", [(9472, 448, 256), (9472, 384, 128), (2048, 4096, 128), (9472, 512, 128)])
def test_pair_kernel_tile_widths(cuda, oracle, shape):
    """Shapes for which the CTA-pair kernel picks 224-, 192-, 240- and 256-column tiles (fullest last wave)."""
    import ltq
    M, N, K = shape
    rng = np.random.default_rng(N)
    a = rng.integers(0, 256, (M, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    bias = rng.integers(-50000, 50000, N, dtype=np.int32)
    qps = (ltq.QParams(0.02, 77), ltq.QParams(0.005, 131), ltq.QParams(0.9, 100))
    acc = oracle.port.acc_i32(a, w, M, N, K, 77, 131, bias=bias)
    force = ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR
    np.testing.assert_array_equal(_run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_I32, force), acc)
    np.testing.assert_array_equal(_run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_U8, force),
                                  oracle.port.epilogue_u8(acc, 0.02, 0.005, 0.9, 100))
    got = _run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_F32, force | ltq.FLAG_RELU)
    want = oracle.port.epilogue_f32(acc, 0.02, 0.005, relu=True)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("shape", [(2500, 2000, 192), (2560, 2048, 64), (4096, 4096, 128)])
def test_pair_kernel_ragged_tile_widths(cuda, oracle, shape):
    """Shapes whose 256-wide tiles would leave a short remainder behind the last whole round of CTA pairs: the pair
    kernel cuts every band into tiles of up to four different widths instead (ragged last rows and columns included).
    All output modes against the oracle."""
    import ltq
    M, N, K = shape
    rng = np.random.default_rng(M + N)
    a = rng.integers(0, 256, (M, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    bias = rng.integers(-50000, 50000, N, dtype=np.int32)
    qps = (ltq.QParams(0.02, 77), ltq.QParams(0.005, 131), ltq.QParams(0.9, 100))
    acc = oracle.port.acc_i32(a, w, M, N, K, 77, 131, bias=bias)
    force = ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR
    np.testing.assert_array_equal(_run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_I32, force), acc)
    assert "tiles of" in ltq.last_kernel(), ltq.last_kernel()
    for fl in (0, ltq.FLAG_RELU, ltq.FLAG_SATURATE):
        np.testing.assert_array_equal(_run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_U8, force | fl),
                                      oracle.port.epilogue_u8(acc, 0.02, 0.005, 0.9, 100, relu=bool(fl & ltq.FLAG_RELU),
                                                              saturate=bool(fl & ltq.FLAG_SATURATE)))
    got = _run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_F32, force | ltq.FLAG_RELU)
    want = oracle.port.epilogue_f32(acc, 0.02, 0.005, relu=True)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    # a large real multiplier (rm > 0.5) takes the general cast, where t can pass 2^31
    big = (ltq.QParams(300.0, 77), ltq.QParams(200.0, 131), ltq.QParams(0.01, 100))
    np.testing.assert_array_equal(_run_layer(cuda, ltq, a, w, bias, big, ltq.OUT_U8, force),
                                  oracle.port.epilogue_u8(acc, 300.0, 200.0, 0.01, 100))


@pytest.mark.parametrize("tA,tB", [(False, False), (False, True), (True, False), (True, True)])
def test_matmul_u8_plain_int32_product_and_modes(cuda, oracle, tA, tB):
    """The generic uint8 matrix product (every transpose variant): plain int32 product with zero points 0, and the
    corrected product in int32 / float / uint8 with qparams, against the oracle."""
    import ltq
    rng = np.random.default_rng(40 + 2 * tA + tB)
    M, N, K = 70, 52, 96
    A = rng.integers(0, 256, (K, M) if tA else (M, K), dtype=np.uint8)
    B = rng.integers(0, 256, (N, K) if tB else (K, N), dtype=np.uint8)
    Ad, Bd = cuda.from_numpy(A).cuda(), cuda.from_numpy(B).cuda()
    plain = ltq.matmul_u8(Ad, Bd, tA, tB).cpu().numpy()
    a2 = (A.T if tA else A).astype(np.int64)
    b2 = (B if tB else B.T).astype(np.int64)
    np.testing.assert_array_equal(plain, (a2 @ b2.T).astype(np.int32))
    rows = [(0.02, 128), (0.005, 127), (0.9, 3)]
    qps = [ltq.QParams(float(np.float32(s)), z) for s, z in rows]
    bias = rng.integers(-9000, 9000, N, dtype=np.int32)
    acc = oracle.port.acc_i32(A, B, M, N, K, 128, 127, bias=bias, tA=tA, tB=tB)
    bd = cuda.from_numpy(bias).cuda()
    np.testing.assert_array_equal(ltq.matmul_u8(Ad, Bd, tA, tB, qps, bd, ltq.OUT_I32).cpu().numpy(), acc)
    np.testing.assert_array_equal(ltq.matmul_u8(Ad, Bd, tA, tB, qps, bd, ltq.OUT_F32, ltq.FLAG_RELU).cpu().numpy(),
                                  oracle.port.epilogue_f32(acc, 0.02, 0.005, relu=True))
    np.testing.assert_array_equal(ltq.matmul_u8(Ad, Bd, tA, tB, qps, bd, ltq.OUT_U8).cpu().numpy(),
                                  oracle.port.epilogue_u8(acc, 0.02, 0.005, 0.9, 3))


@pytest.mark.parametrize("path", ["tc", "tcpair"])
@pytest.mark.parametrize("rm_case", ["small", "medium", "large"])
def test_epilogue_conversion_free_path_boundaries(cuda, oracle, path, rm_case):
    """The tensor-core epilogues convert without I2F / F2I while the accumulator is inside a range derived from the real
    multiplier and the output zero point, and fall back to the general conversion outside it.  Accumulators are steered
    through the bias (activations all equal to their zero point, so acc[i, j] = bias[j]) across every boundary of that
    range: around 0, around -zC/rm and 2^23/rm, around +-2^22, and the int32 extremes."""
    import ltq
    M, K = (256, 64) if path == "tc" else (512, 64)
    sa, sw = np.float32(0.02), np.float32(0.005)
    sc = {"small": np.float32(0.37), "medium": np.float32(1e-4), "large": np.float32(1e-7)}[rm_case]
    zc = 37
    rm = float(np.float32(sa * sw) / sc)
    pts = [0, 1, -1, 255, -255, 2 ** 22, -2 ** 22, 2 ** 23, -2 ** 23, 2 ** 24 + 3, -2 ** 24 - 3, 2 ** 31 - 1, -2 ** 31,
           int(-zc / rm), int((2 ** 23 - 512 - zc) / rm), int((2 ** 23 - zc) / rm), int(2 ** 31 / rm), int(-2 ** 31 / rm)]
    vals = []
    for p in pts:
        for d in range(-40, 41):
            for scale in (1, 1000):
                vals.append(min(2 ** 31 - 1, max(-2 ** 31, p + d * scale)))
    rng = np.random.default_rng(9)
    vals += list(rng.integers(-2 ** 22, 2 ** 22, 700)) + list(rng.integers(-2 ** 31, 2 ** 31, 300))
    N = (len(vals) + 255) // 256 * 256
    bias = np.zeros(N, dtype=np.int32)
    bias[:len(vals)] = np.array(vals, dtype=np.int64).astype(np.int32)
    a = np.full((M, K), 9, dtype=np.uint8)           # equal to its zero point: contributes nothing
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    qps = (ltq.QParams(sa, 9), ltq.QParams(sw, 131), ltq.QParams(sc, zc))
    acc = oracle.port.acc_i32(a, w, M, N, K, 9, 131, bias=bias)
    assert np.array_equal(acc[0], bias)
    force = ltq.FLAG_FORCE_TC | (ltq.FLAG_FORCE_TC_SINGLE if path == "tc" else ltq.FLAG_FORCE_TC_PAIR)
    for relu in (False, True):
        fl = force | (ltq.FLAG_RELU if relu else 0)
        np.testing.assert_array_equal(_run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_U8, fl),
                                      oracle.port.epilogue_u8(acc, sa, sw, sc, zc, relu=relu))
        got = _run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_F32, fl)
        np.testing.assert_array_equal(got.view(np.uint32), oracle.port.epilogue_f32(acc, sa, sw, relu=relu).view(np.uint32))
    np.testing.assert_array_equal(_run_layer(cuda, ltq, a, w, bias, qps, ltq.OUT_U8, force | ltq.FLAG_SATURATE),
                                  oracle.port.epilogue_u8(acc, sa, sw, sc, zc, saturate=True))
