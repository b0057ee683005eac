"""CPU: a numpy model of the screening step the device kernels use in Quantize (float -> uint8) against the oracle.

The kernels (csrc/ltq_quant.cuh) compute v = fma(x, 1 / scale, zp), clamp it to [0, 255] and take the nearest integer;
only when v lies within 1.2e-4 of a half-integer do they repeat the element with the reference's own sequence
(IEEE division, add, clamp, round half away from zero; l-ten/utils.cpp:243-254).  This test checks the claim that makes
the shortcut legal - every element the screen calls "far from a rounding boundary" already has the reference's byte -
on inputs placed on and around every boundary, for many scales and zero points, and that few elements are "near"."""
import numpy as np

F = np.float32
MARGIN = F(1.2e-4)


def screened(x, scale, zp):
    inv = F(1) / F(scale)
    v = (x.astype(np.float64) * np.float64(inv) + np.float64(zp)).astype(F)     # the fused multiply-add, to float32
    v = np.maximum(F(0), np.minimum(F(255), v))
    big = (v + F(8388608)).astype(F)                                            # nearest integer in the low mantissa bits
    r = (big - F(8388608)).astype(F)
    far = np.abs((v - r).astype(F)) <= F(0.5) - MARGIN
    return (big.view(np.uint32) & 0xFF).astype(np.uint8), far


def test_far_elements_already_have_the_reference_byte(oracle):
    rng = np.random.default_rng(11)
    ks = np.arange(-2, 258, dtype=F) + F(0.5)
    total = near_random = n_random = 0
    for _ in range(150):
        scale = F(10.0 ** rng.uniform(-6, 3))
        zp = int(rng.integers(0, 256))
        x0 = ((ks - F(zp)) * scale).astype(F)
        xs, up, dn = [x0], x0.copy(), x0.copy()
        for _ in range(24):
            up = np.nextafter(up, F(np.inf))
            dn = np.nextafter(dn, F(-np.inf))
            xs += [up.copy(), dn.copy()]
        rnd = (rng.standard_normal(8000) * 60).astype(F) * scale
        x = np.concatenate(xs + [rnd])
        want = oracle.port.quantize_u8(x, oracle.qp(scale, zp))
        got, far = screened(x, scale, zp)
        bad = (got != want) & far
        assert not bad.any(), (scale, zp, x[bad][:4], got[bad][:4], want[bad][:4])
        total += x.size
        near_random += int((~far[-8000:]).sum())
        n_random += 8000
    assert total > 3_000_000
    assert near_random / n_random < 1e-3          # a few in ten thousand take the division
