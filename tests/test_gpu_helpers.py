"""GPU: quantisation helper kernels against the golden fixtures and the CPU oracle (bit-exact)."""
import numpy as np
import pytest

from helpers import ltq_qp, qp_of

pytestmark = pytest.mark.gpu

CASES = ["normal", "uniform01", "negative_only", "positive_offset", "wide", "tiny", "single", "ties"]


@pytest.mark.parametrize("name", CASES)
def test_helpers_match_golden(cuda, golden, name):
    import ltq
    g = golden("helpers.npz")
    x = cuda.from_numpy(g[f"{name}.x"]).cuda()
    mm = ltq.GetMinMax(x).cpu().numpy()
    np.testing.assert_array_equal(mm, g[f"{name}.minmax"])
    qp = ltq.ComputeQuantizationParams(mm[0], mm[1])
    assert (np.float32(qp.scale), qp.zero_point) == (np.float32(g[f"{name}.qp"][0]), int(g[f"{name}.qp"][1]))
    qpd = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(x)))
    assert (np.float32(qpd.scale), qpd.zero_point) == (np.float32(qp.scale), qp.zero_point)
    q = ltq.Quantize(x, qp)
    np.testing.assert_array_equal(q.cpu().numpy(), g[f"{name}.q"])
    np.testing.assert_array_equal(ltq.Dequantize(q, qp).cpu().numpy(), g[f"{name}.dq"])


def test_explicit_and_bias_quantize(cuda, golden):
    import ltq
    g = golden("helpers.npz")
    q = ltq.Quantize(cuda.from_numpy(g["explicit.x"]).cuda(), ltq_qp(g["explicit.qp"]))
    np.testing.assert_array_equal(q.cpu().numpy(), g["explicit.q"])
    b = ltq.QuantizeInt32(cuda.from_numpy(g["bias.x"]).cuda(), ltq_qp(g["bias.qp"]))
    np.testing.assert_array_equal(b.cpu().numpy(), g["bias.q"])


@pytest.mark.parametrize("shape", [(1, 1), (1, 4096), (3, 17), (16, 4096), (64, 784), (257, 2050), (5, 33000),
                                   (1000, 48), (601, 4096), (1000, 4100), (593, 2049)])   # the last three: two warps per row when the parameters are on the device
def test_quantize_rows_and_sums_vs_oracle(cuda, oracle, shape):
    import ltq
    rng = np.random.default_rng(shape[0] * 1000 + shape[1])
    x = (rng.standard_normal(shape) * 2.5).astype(np.float32)
    mn, mx = oracle.port.get_min_max(x)
    oq = oracle.port.compute_qparams(mn, mx)
    want = oracle.port.quantize_u8(x, oq)
    xd = cuda.from_numpy(x).cuda()
    # static (host qparams) and dynamic (device qparams, no host round trip) give the same bytes
    q1, s1 = ltq.quantize_rows(xd, qp=ltq.QParams(oq.scale, oq.zero_point))
    qp_dev = ltq.compute_qparams_dev(ltq.GetMinMax(xd))
    q2, s2 = ltq.quantize_rows(xd, qp_dev=qp_dev)
    for q, s in ((q1, s1), (q2, s2)):
        np.testing.assert_array_equal(q.cpu().numpy(), want)
        np.testing.assert_array_equal(s.cpu().numpy(), want.astype(np.int64).sum(1).astype(np.int32))
    np.testing.assert_array_equal(ltq.row_sums(q1).cpu().numpy(), want.astype(np.int64).sum(1).astype(np.int32))


def test_unaligned_views(cuda, oracle):
    """Pointers that are not 16-byte aligned take the scalar head/tail paths."""
    import ltq
    rng = np.random.default_rng(5)
    base = (rng.standard_normal(5003) * 4).astype(np.float32)
    xd = cuda.from_numpy(base).cuda()
    for off in (1, 2, 3):
        v = xd[off:off + 4001]
        mm = ltq.GetMinMax(v).cpu().numpy()
        assert tuple(mm) == oracle.port.get_min_max(base[off:off + 4001])
        oq = oracle.port.compute_qparams(*mm)
        q = ltq.Quantize(v, ltq.QParams(oq.scale, oq.zero_point))
        np.testing.assert_array_equal(q.cpu().numpy(), oracle.port.quantize_u8(base[off:off + 4001], oq))
    m = cuda.from_numpy(rng.integers(0, 256, (7, 1001), dtype=np.uint8)).cuda()
    np.testing.assert_array_equal(ltq.row_sums(m).cpu().numpy(), m.cpu().numpy().astype(np.int64).sum(1))


def test_quantize_at_the_rounding_boundaries(cuda, oracle):
    """The device kernels screen with a multiplication and fall back to the reference's division only near a rounding
    boundary.  Inputs that sit on, and a few float steps either side of, every boundary k + 0.5 (and the clamp edges)
    for many scales and zero points must give the reference's bytes (l-ten/utils.cpp:243-254)."""
    import ltq
    rng = np.random.default_rng(2024)
    scales = np.concatenate([rng.uniform(1e-3, 0.3, 40), 10.0 ** rng.uniform(-6, 3, 40), [0.1, 0.25, 1.0, 3.0, 1 / 3]]).astype(np.float32)
    ks = np.arange(-2, 258, dtype=np.float32) + np.float32(0.5)                   # every boundary, and beyond both clamp edges
    steps = np.arange(-6, 7)
    for scale in scales:
        zp = int(rng.integers(0, 256))
        x0 = ((ks - np.float32(zp)) * scale).astype(np.float32)
        xs = [x0]
        up, down = x0.copy(), x0.copy()
        for _ in range(6):
            up = np.nextafter(up, np.float32(np.inf)).astype(np.float32)
            down = np.nextafter(down, np.float32(-np.inf)).astype(np.float32)
            xs += [up.copy(), down.copy()]
        x = np.concatenate(xs + [np.float32([0.0, -0.0, 1e30, -1e30])])
        x = np.resize(x, (x.size + 127) // 128 * 128).reshape(-1, 128).copy()    # rows of 128 for quantize_rows
        oq = oracle.qp(scale, zp)
        want = oracle.port.quantize_u8(x, oq)
        xd = cuda.from_numpy(x).cuda()
        qp = ltq.QParams(float(scale), zp)
        np.testing.assert_array_equal(ltq.Quantize(xd, qp).cpu().numpy(), want, err_msg=f"scale {scale} zp {zp}")
        np.testing.assert_array_equal(ltq.Quantize(xd.view(-1)[1:], qp).cpu().numpy(), want.ravel()[1:])   # scalar path
        q, s = ltq.quantize_rows(xd, qp=qp)
        np.testing.assert_array_equal(q.cpu().numpy(), want)
        np.testing.assert_array_equal(s.cpu().numpy(), want.astype(np.int64).sum(1).astype(np.int32))
        wide = xd.view(1, -1) if xd.numel() > 2048 else None                       # one long row: the whole-CTA-per-row form
        if wide is not None:
            q2, _ = ltq.quantize_rows(wide.contiguous(), qp=qp)
            np.testing.assert_array_equal(q2.cpu().numpy().ravel(), want.ravel())


def test_min_max_with_nans_follows_the_reference_loop(cuda, oracle):
    """The reference seeds min and max with data[0] and replaces them when a comparison is true (l-ten/utils.cpp:209-223):
    NaNs after the first element are skipped, a NaN in the first element stays in both results."""
    import ltq
    rng = np.random.default_rng(77)
    base = (rng.standard_normal(9000) * 3).astype(np.float32)
    cases = []
    a = base.copy(); a[[5, 4000, 8999]] = np.nan; cases.append(a)          # NaNs in the middle and at the end
    b = base.copy(); b[0] = np.nan; cases.append(b)                         # NaN seed
    cases.append(np.full(300, np.nan, np.float32))                          # nothing comparable
    c = base.copy(); c[1:] = np.nan; cases.append(c)                        # only the seed is a number
    for x in cases:
        got = ltq.GetMinMax(cuda.from_numpy(x).cuda()).cpu().numpy()
        want = np.array(oracle.port.get_min_max(x), np.float32)
        np.testing.assert_array_equal(got, want)                            # NaN == NaN for this comparison


def test_large_tensor_properties(cuda):
    """Full-size activation block of the 4096^3 configuration: dequantize(quantize(x)) stays within half a step and
    the fused row sums equal the sums of the bytes written."""
    import ltq
    g = cuda.Generator(device="cuda").manual_seed(1)
    x = cuda.randn((4096, 4096), generator=g, device="cuda")
    mm = ltq.GetMinMax(x)
    assert float(mm[0]) == float(x.min()) and float(mm[1]) == float(x.max())
    qp = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(mm))
    q, s = ltq.quantize_rows(x, qp=qp)
    assert cuda.equal(s, q.to(cuda.int32).sum(1).to(cuda.int32))
    err = (ltq.Dequantize(q, qp) - x).abs().max().item()
    assert err <= 0.5 * qp.scale * 1.0001
