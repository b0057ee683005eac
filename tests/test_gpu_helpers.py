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
                                   (1000, 48)])
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
