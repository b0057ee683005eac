"""GPU: the calibration / quantisation set-up helper against the oracle's restatement of the reference recipe
(tests/nn_tests.cpp:538-608, 786-884): running min/max over batches, weight and bias quantisation written through
get_all_weights(), and the resulting quantized conv -> fc network against the oracle end to end."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_observer_and_module_setup_match_the_reference_recipe(cuda, oracle):
    import ltq
    rng = np.random.default_rng(31)
    B, Cin, H, W, Cout, k, hid = 6, 2, 12, 12, 5, 3, 7
    flat = Cout * (H - k + 1) * (W - k + 1)
    wc = rng.normal(0, 0.3, (Cout, Cin, k, k)).astype(np.float32)
    w1 = rng.normal(0, 0.05, (hid, flat)).astype(np.float32)
    b1 = rng.normal(0, 0.02, hid).astype(np.float32)
    batches = [rng.random((B, Cin, H, W), dtype=np.float32) for _ in range(3)]
    wc_d, w1_d, b1_d = [cuda.from_numpy(a).cuda() for a in (wc, w1, b1)]

    def net(x):   # float32 network with taps: input, conv output, fc output
        cols = cuda.nn.functional.unfold(x, k)                                  # [B, Cin*k*k, Ho*Wo]
        a1 = (wc_d.reshape(Cout, -1) @ cols).reshape(x.shape[0], Cout, H - k + 1, W - k + 1)
        a2 = a1.reshape(x.shape[0], -1) @ w1_d.t() + b1_d
        return [x, a1, a2]

    qps = ltq.calibrate(net, [cuda.from_numpy(b).cuda() for b in batches])
    # the oracle's min/max over everything seen (seeded as the reference seeds blob_statistics)
    taps = [[t.cpu().numpy() for t in net(cuda.from_numpy(b).cuda())] for b in batches]
    for i, q in enumerate(qps):
        allv = np.concatenate([t[i].ravel() for t in taps])
        want = oracle.port.compute_qparams(*oracle.port.get_min_max(allv))
        assert (np.float32(q.scale), q.zero_point) == (np.float32(want.scale), want.zero_point), f"tap {i}"

    conv = ltq.Conv2d_q(Cin, Cout, False, k, k)
    conv.init()
    fc = ltq.FullyConnected_q(flat, hid, True)
    fc.init()
    q_wc = ltq.quantize_module(conv, wc_d, None, qps[0], qps[1])
    q_w1 = ltq.quantize_module(fc, w1_d, b1_d, qps[1], qps[2])
    # bytes written through get_all_weights() are the oracle's
    o_wc = oracle.port.compute_qparams(*oracle.port.get_min_max(wc.ravel()))
    o_w1 = oracle.port.compute_qparams(*oracle.port.get_min_max(w1.ravel()))
    assert (np.float32(q_wc.scale), q_wc.zero_point) == (np.float32(o_wc.scale), o_wc.zero_point)
    np.testing.assert_array_equal(conv.get_weights().numpy().ravel(), oracle.port.quantize_u8(wc.ravel(), o_wc))
    np.testing.assert_array_equal(fc.get_weights().numpy().ravel(), oracle.port.quantize_u8(w1.ravel(), o_w1))
    o_b = oracle.qp(np.float32(qps[1].scale) * np.float32(o_w1.scale), 0)
    np.testing.assert_array_equal(fc.get_bias().numpy().ravel(), oracle.port.quantize_i32(b1, o_b))

    # inference: Quantize -> Conv2d_q -> reshape -> FullyConnected_q, against the oracle
    conv.to("cuda", 0)
    fc.to("cuda", 0)
    x = batches[1]
    o_q = [oracle.qp(np.float32(q.scale), q.zero_point) for q in qps]
    xq = ltq.Quantize(cuda.from_numpy(x).cuda(), qps[0])
    y1 = conv.forward(xq)
    y2 = fc.forward(y1.reshape(B, 1, flat))
    xq_o = oracle.port.quantize_u8(x, o_q[0])
    np.testing.assert_array_equal(xq.cpu().numpy(), xq_o)
    y1_o = oracle.port.conv2d_q(xq_o, conv.get_weights().cpu().numpy().reshape(Cout, -1), Cout, k, k, o_q[0], o_wc, o_q[1])
    np.testing.assert_array_equal(y1.cpu().numpy(), y1_o)
    y2_o, _ = oracle.port.quantized_matmul(y1_o.reshape(B, flat), fc.get_weights().cpu().numpy().reshape(hid, flat), B, hid,
                                           flat, [o_q[1], o_w1, o_q[2]], bias=fc.get_bias().cpu().numpy().ravel())
    np.testing.assert_array_equal(y2.cpu().numpy().reshape(B, hid), y2_o)
    # and the quantized network tracks the float one
    got = ltq.Dequantize(y2, qps[2]).cpu().numpy().reshape(B, hid)
    ref = taps[1][2]
    # (loose: the reference requantises by truncation, half an LSB of bias per layer, and this network is tiny)
    assert np.abs(got - ref).mean() / np.abs(ref).mean() < 0.35


def test_observer_without_data_raises():
    import ltq
    with pytest.raises(ValueError):
        ltq.MinMaxObserver().qparams()
