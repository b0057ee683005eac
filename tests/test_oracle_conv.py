"""CPU: the C restatement of Conv2d_q::forward / im2col_cpu against the fixtures generated from the reference build, and
against the reference library itself where it is present."""
import numpy as np
import pytest

from helpers import iter_conv_cases, qp_of


def test_im2col_and_conv_match_golden(oracle, golden):
    g = golden("conv2d.npz")
    n = 0
    for c in iter_conv_cases(g):
        col = oracle.port.im2col(c["x"][0], c["kh"], c["kw"], c["ph"], c["pw"], c["sh"], c["sw"])
        np.testing.assert_array_equal(col, c["col0"], err_msg=c["key"])
        qi, qw, qo = [qp_of(oracle, r) for r in c["qp"]]
        y = oracle.port.conv2d_q(c["x"], c["w"], c["Cout"], c["kh"], c["kw"], qi, qw, qo, bias=c["bias"], ph=c["ph"],
                                 pw=c["pw"], sh=c["sh"], sw=c["sw"])
        np.testing.assert_array_equal(y, c["y"], err_msg=c["key"])
        n += 1
    assert n == 9


def test_conv_is_the_matmul_of_its_patches(oracle):
    """Conv2d_q::forward is quantized_matmul(false, false, Cout, Ho*Wo, K, weights, im2col(image)) with qparams
    {weights, input, output} (l-ten/conv2d.cpp:340-367)."""
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, (2, 3, 9, 8), dtype=np.uint8)
    w = rng.integers(0, 256, (6, 3 * 3 * 2), dtype=np.uint8)
    qi, qw, qo = oracle.qp(0.02, 120), oracle.qp(0.004, 90), oracle.qp(0.07, 11)
    y = oracle.port.conv2d_q(x, w, 6, 3, 2, qi, qw, qo, ph=1, pw=0, sh=2, sw=1)
    for b in range(2):
        col = oracle.port.im2col(x[b], 3, 2, 1, 0, 2, 1)
        K, N = col.shape
        Cm, _ = oracle.port.quantized_matmul(w, col, 6, N, K, [qw, qi, qo], tA=False, tB=False)
        np.testing.assert_array_equal(y[b].reshape(6, N), Cm)


def test_bias_per_channel_differs_from_reference_indexing_only_in_the_bias(oracle):
    rng = np.random.default_rng(6)
    x = rng.integers(0, 256, (1, 2, 6, 6), dtype=np.uint8)
    w = rng.integers(0, 256, (20, 2 * 9), dtype=np.uint8)
    qi, qw, qo = oracle.qp(1.0, 0), oracle.qp(1.0, 0), oracle.qp(1.0, 0)   # rm = 1, z = 0: output = low byte of acc
    y0 = oracle.port.conv2d_q(x, w, 20, 3, 3, qi, qw, qo)
    bias = rng.integers(0, 100, 20, dtype=np.int32)
    y_pos = oracle.port.conv2d_q(x, w, 20, 3, 3, qi, qw, qo, bias=bias)                       # 16 positions <= 20
    y_ch = oracle.port.conv2d_q(x, w, 20, 3, 3, qi, qw, qo, bias=bias, bias_per_channel=True)
    d_pos = (y_pos.astype(np.int32) - y0).reshape(20, 16) % 256
    d_ch = (y_ch.astype(np.int32) - y0).reshape(20, 16) % 256
    np.testing.assert_array_equal(d_pos, np.broadcast_to(bias[:16] % 256, (20, 16)))
    np.testing.assert_array_equal(d_ch, np.broadcast_to((bias % 256)[:, None], (20, 16)))


def test_port_matches_reference_library_on_random_conv(oracle):
    if oracle.ref is None or not hasattr(oracle.ref.lib, "ref_conv2d_q_forward"):
        pytest.skip("reference library not built here")
    rng = np.random.default_rng(7)
    for _ in range(12):
        B, Cin, Cout = int(rng.integers(1, 4)), int(rng.integers(1, 9)), int(rng.integers(1, 20))
        kh, kw = int(rng.integers(1, 5)), int(rng.integers(1, 5))
        ph, pw, sh, sw = int(rng.integers(0, 3)), int(rng.integers(0, 3)), int(rng.integers(1, 4)), int(rng.integers(1, 4))
        H, W = int(rng.integers(kh, 15)), int(rng.integers(kw, 15))
        x = rng.integers(0, 256, (B, Cin, H, W), dtype=np.uint8)
        w = rng.integers(0, 256, (Cout, Cin * kh * kw), dtype=np.uint8)
        qs = [oracle.qp(float(rng.uniform(0.001, 0.1)), int(rng.integers(0, 256))) for _ in range(2)]
        qo = oracle.qp(float(rng.uniform(0.01, 2.0)), int(rng.integers(0, 256)))
        a = oracle.port.conv2d_q(x, w, Cout, kh, kw, qs[0], qs[1], qo, ph=ph, pw=pw, sh=sh, sw=sw)
        b = oracle.ref.conv2d_q(x, w, Cout, kh, kw, qs[0], qs[1], qo, ph=ph, pw=pw, sh=sh, sw=sw)
        np.testing.assert_array_equal(a, b)
