"""GPU: layer-level parity on the benchmark configurations -- golden fixtures for the MNIST-shaped MLP and the 1024^3
linear, the CPU oracle on sampled rows plus cross-kernel agreement at 4096^3, the skinny sweep in full."""
import hashlib

import numpy as np
import pytest

from helpers import ltq_qp, qp_of

pytestmark = pytest.mark.gpu


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_mlp_chain_matches_golden(cuda, golden):
    """784-512-512-10, batch 64: FullyConnected_q with the reference's method names, chained uint8 -> uint8, then
    Dequantize, as tests/nn_tests.cpp:930-963 drives it."""
    import ltq
    from ltq import workloads
    g = golden("fc_mlp.npz")
    x, layers = workloads.mlp_mnist(seed=0, batch=64)
    qp_in = ltq_qp(g["l0.qp"][0])
    xq = ltq.Quantize(cuda.from_numpy(x).cuda(), qp_in)
    np.testing.assert_array_equal(xq.cpu().numpy(), g["x_q"])
    h = xq.view(1, 64, 784)
    for li, (w, b) in enumerate(layers):
        N, K = w.shape
        qps = [ltq_qp(r) for r in g[f"l{li}.qp"]]
        fc = ltq.FullyConnected_q(K, N, True)
        fc.init()
        # quantisation set-up on the device, then written through get_all_weights() like tests/nn_tests.cpp:818-826
        wq = ltq.Quantize(cuda.from_numpy(w).cuda(), qps[1])
        bq = ltq.QuantizeInt32(cuda.from_numpy(b).cuda(), ltq.QParams(np.float32(qps[0].scale) * np.float32(qps[1].scale), 0))
        np.testing.assert_array_equal(wq.cpu().numpy(), g[f"l{li}.w_q"])
        np.testing.assert_array_equal(bq.cpu().numpy(), g[f"l{li}.b_q"])
        ws = fc.get_all_weights()
        ws[0].copy_(wq.cpu().view(1, 1, N, K))
        ws[1].copy_(bq.cpu())
        fc.set_qparams_in(qps[0])
        fc.set_qparams_out(qps[2])
        fc.set_qparams_params([qps[1]], 1)
        fc.to("cuda", 0)
        h = fc.forward(h)
        assert tuple(h.shape) == (1, 64, N) and h.dtype == cuda.uint8
        np.testing.assert_array_equal(h.cpu().numpy().reshape(64, N), g[f"l{li}.y"])
    logits = ltq.Dequantize(h, qps[2])
    np.testing.assert_array_equal(logits.cpu().numpy().reshape(64, 10), g["logits"])


def test_leading_dims_fold_into_m(cuda, oracle):
    import ltq
    rng = np.random.default_rng(11)
    K, N = 64, 48
    x = rng.integers(0, 256, (3, 5, 7, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    fc = ltq.FullyConnected_q(K, N)
    fc.init()
    fc.get_all_weights()[0].copy_(cuda.from_numpy(w).view(1, 1, N, K))
    qps = (ltq.QParams(0.1, 5), ltq.QParams(0.2, 9), ltq.QParams(90.0, 100))
    fc.set_qparams_in(qps[0]); fc.set_qparams_out(qps[2]); fc.set_qparams_params([qps[1]], 1)
    fc.to("cuda", 0)
    y = fc.forward(cuda.from_numpy(x).cuda())
    assert tuple(y.shape) == (3, 5, 7, N)
    want, _ = oracle.port.quantized_matmul(x.reshape(-1, K), w, 105, N, K,
                                           [oracle.qp(q.scale, q.zero_point) for q in qps])
    np.testing.assert_array_equal(y.cpu().numpy().reshape(105, N), want)


@pytest.mark.parametrize("path", ["auto", "simt"])
def test_linear_1024_matches_golden(cuda, golden, path):
    import ltq
    from ltq import workloads
    g = golden("linear_1024.npz")
    wl = workloads.linear_u8(seed=2)
    qa, qw = ltq.QParams(*wl["qp_a"]), ltq.QParams(*wl["qp_w"])
    bq = ltq.QuantizeInt32(cuda.from_numpy(wl["bias"]).cuda(), ltq.QParams(np.float32(qa.scale) * np.float32(qw.scale), 0))
    np.testing.assert_array_equal(bq.cpu().numpy(), g["bias_q"])
    force = ltq.FLAG_FORCE_SIMT if path == "simt" else 0
    h = ltq.LayerHandle(0, 1024, 1024)
    wd, ad = cuda.from_numpy(wl["w"]).cuda(), cuda.from_numpy(wl["a"]).cuda()
    h.set_weights(wd, bq)
    for i in range(4):
        sc, zc = g[f"o{i}.qp"]
        h.set_qparams(qa, qw, ltq.QParams(np.float32(sc), int(zc)))
        C = h.forward(ad, ltq.OUT_U8, force).cpu().numpy()
        np.testing.assert_array_equal(C[::64], g[f"o{i}.rows"])
        assert sha(C) == str(g[f"o{i}.sha"])
    # same through the reference-shaped stateless call
    Cd = cuda.empty((1024, 1024), dtype=cuda.uint8, device="cuda")
    ws = cuda.empty(2048, dtype=cuda.int32, device="cuda")
    sc, zc = g["o0.qp"]
    ltq.quantized_matmul(False, True, 1024, 1024, 1024, 1, ad, wd, 0, Cd, [qa, qw, ltq.QParams(np.float32(sc), int(zc))], bq, ws)
    assert sha(Cd.cpu().numpy()) == str(g["o0.sha"])
    h.check()


def test_linear_1024_f32_relu_and_int32_vs_oracle(cuda, oracle):
    """fp32 dequantized output with fused ReLU, and the bit-exact int32 accumulator check."""
    import ltq
    from ltq import workloads
    wl = workloads.linear_u8(seed=2)
    qa, qw = oracle.qp(*wl["qp_a"]), oracle.qp(*wl["qp_w"])
    bias_q = oracle.port.quantize_i32(wl["bias"], oracle.qp(np.float32(qa.scale) * np.float32(qw.scale), 0))
    acc = oracle.port.acc_i32(wl["a"], wl["w"], 1024, 1024, 1024, qa.zero_point, qw.zero_point, bias=bias_q)
    h = ltq.LayerHandle(0, 1024, 1024)
    wd, ad = cuda.from_numpy(wl["w"]).cuda(), cuda.from_numpy(wl["a"]).cuda()
    h.set_weights(wd, cuda.from_numpy(bias_q).cuda())
    h.set_qparams(ltq.QParams(qa.scale, qa.zero_point), ltq.QParams(qw.scale, qw.zero_point), ltq.QParams(1.0, 0))
    np.testing.assert_array_equal(h.forward(ad, ltq.OUT_I32).cpu().numpy(), acc)
    got = h.forward(ad, ltq.OUT_F32, ltq.FLAG_RELU).cpu().numpy()
    want = oracle.port.epilogue_f32(acc, qa.scale, qw.scale, relu=True)
    rel = np.abs(got - want) / np.maximum(np.abs(want), 1e-30)
    assert rel.max() <= 1e-5  # specified tolerance; the kernels in fact match bit for bit:
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    h.check()


def test_square_4096_requant(cuda, oracle):
    """4096^3, activations and weights quantized per tensor by min/max on the device, output requantized to uint8 with
    qparams from the fp32 product's min/max.  Checks: (1) 96 sampled rows against the CPU oracle, bit for bit;
    (2) both tcgen05 kernels (CTA pair and single CTA) and the dp4a kernel agree on the whole 16 Mi-element output; (3) linearity-free integer
    identity: the int32 outputs summed per row equal what the operand sums predict."""
    import ltq
    from ltq import workloads
    x, w = workloads.square_4096(seed=3)
    xd, wd = cuda.from_numpy(x).cuda(), cuda.from_numpy(w).cuda()
    qx = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(xd)))
    qw = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(wd)))
    xq, asum = ltq.quantize_rows(xd, qp=qx)
    wq = ltq.Quantize(wd, qw)
    ref32 = xd @ wd.t()
    qo = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(ref32)))
    del ref32
    h = ltq.LayerHandle(0, 4096, 4096)
    h.set_weights(wq, None)
    h.set_qparams(qx, qw, qo)
    out_tc = h.forward(xq, ltq.OUT_U8, ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR, asum=asum)
    out_single = h.forward(xq, ltq.OUT_U8, ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_SINGLE, asum=asum)
    out_simt = h.forward(xq, ltq.OUT_U8, ltq.FLAG_FORCE_SIMT, asum=asum)
    h.check()
    assert cuda.equal(out_tc, out_simt) and cuda.equal(out_single, out_simt)
    rows = np.sort(np.random.default_rng(0).choice(4096, 96, replace=False))
    xq_h, wq_h = xq.cpu().numpy(), wq.cpu().numpy()
    acc = oracle.port.acc_i32(xq_h[rows], wq_h, len(rows), 4096, 4096, qx.zero_point, qw.zero_point)
    want = oracle.port.epilogue_u8(acc, qx.scale, qw.scale, qo.scale, qo.zero_point)
    np.testing.assert_array_equal(out_tc.cpu().numpy()[rows], want)
    # the quantized result tracks the fp32 product to within one output step (what requantisation promises)
    deq = ltq.Dequantize(out_tc, qo)
    assert (deq - xd @ wd.t()).abs().max().item() < 6 * qo.scale
    # integer identity at full size: sum_j acc[i,j] = sum_k (a[i,k]-za) * (colsum_w[k] - N*zw)
    acc_full = h.forward(xq, ltq.OUT_I32, ltq.FLAG_FORCE_TC, asum=asum).to(cuda.int64).sum(1)
    colw = wq.to(cuda.int64).sum(0) - 4096 * qw.zero_point
    pred = ((xq.to(cuda.int64) - qx.zero_point) * colw[None, :]).sum(1)
    assert cuda.equal(acc_full, pred)


@pytest.mark.parametrize("M", [1, 4, 16])
def test_skinny_sweep_full_vs_oracle(cuda, oracle, M):
    """M in {1,4,16}, K=4096, N=11008: weights quantized once, activations quantized per call (dynamic min/max on the
    device, qparams never leave it), fp32 out.  Entire output compared with the CPU oracle."""
    import ltq
    from ltq import workloads
    x, w = workloads.skinny(seed=4, M=M)
    xd, wd = cuda.from_numpy(x).cuda(), cuda.from_numpy(w).cuda()
    qw = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(wd)))
    wq = ltq.Quantize(wd, qw)
    qx_dev = ltq.compute_qparams_dev(ltq.GetMinMax(xd))
    xq, asum = ltq.quantize_rows(xd, qp_dev=qx_dev)
    h = ltq.LayerHandle(0, 4096, 11008)
    h.set_weights(wq, None)
    h.set_qparams(None, qw, None)
    out = h.forward(xq, ltq.OUT_F32, 0, asum=asum, qp_in_dev=qx_dev).cpu().numpy()
    h.check()
    # oracle side
    oqx = oracle.port.compute_qparams(*oracle.port.get_min_max(x))
    oqw = oracle.port.compute_qparams(*oracle.port.get_min_max(w))
    xq_o, wq_o = oracle.port.quantize_u8(x, oqx), oracle.port.quantize_u8(w, oqw)
    np.testing.assert_array_equal(xq.cpu().numpy(), xq_o)
    np.testing.assert_array_equal(wq.cpu().numpy(), wq_o)
    acc = oracle.port.acc_i32(xq_o, wq_o, M, 11008, 4096, oqx.zero_point, oqw.zero_point)
    want = oracle.port.epilogue_f32(acc, oqx.scale, oqw.scale)
    rel = np.abs(out - want) / np.maximum(np.abs(want), 1e-30)
    assert rel.max() <= 1e-5
    np.testing.assert_array_equal(out.view(np.uint32), want.view(np.uint32))


def test_back_to_back_skinny_launches_respect_their_inputs(cuda, oracle):
    """The skinny kernel starts streaming weights before the kernel in front of it has finished.  Everything else it
    reads must wait: here each call's activations and row sums are written by the kernel launched just before it (the
    same buffers every time), and a second layer consumes the first layer's output directly."""
    import ltq
    rng = np.random.default_rng(21)
    K, N1, N2, M, reps = 1024, 2048, 512, 4, 12
    w1 = rng.integers(0, 256, (N1, K), dtype=np.uint8)
    w2 = rng.integers(0, 256, (N2, N1), dtype=np.uint8)
    b1 = rng.integers(-5000, 5000, N1, dtype=np.int32)
    rows = [(0.02, 128), (0.005, 127), (3.0, 7), (0.004, 120), (40.0, 100)]   # in, w1, mid, w2, out
    q_in, q_w1, q_mid, q_w2, q_out = [ltq_qp(r) for r in rows]
    l1 = ltq.LayerHandle(0, K, N1)
    l1.set_weights(cuda.from_numpy(w1).cuda(), cuda.from_numpy(b1).cuda())
    l1.set_qparams(q_in, q_w1, q_mid)
    l2 = ltq.LayerHandle(0, N1, N2)
    l2.set_weights(cuda.from_numpy(w2).cuda())
    l2.set_qparams(q_mid, q_w2, q_out)
    xs = [rng.normal(0, 0.8, (M, K)).astype(np.float32) for _ in range(reps)]
    xs_dev = [cuda.from_numpy(x).cuda() for x in xs]
    xq = cuda.empty((M, K), dtype=cuda.uint8, device="cuda")
    asum = cuda.empty(M, dtype=cuda.int32, device="cuda")
    mids = [cuda.empty((M, N1), dtype=cuda.uint8, device="cuda") for _ in range(reps)]
    outs = [cuda.empty((M, N2), dtype=cuda.uint8, device="cuda") for _ in range(reps)]
    cuda.cuda.synchronize()
    for i in range(reps):   # no synchronisation inside the loop: 3 dependent kernels per iteration, back to back
        ltq.quantize_rows(xs_dev[i], qp=q_in, q=xq, asum=asum)
        l1.forward(xq, ltq.OUT_U8, ltq.FLAG_FORCE_SKINNY, asum=asum, out=mids[i])
        l2.forward(mids[i], ltq.OUT_U8, ltq.FLAG_FORCE_SKINNY, out=outs[i])
    cuda.cuda.synchronize()
    o_in, o_w1, o_mid, o_w2, o_out = [qp_of(oracle, r) for r in rows]
    for i in range(reps):
        xq_ref = oracle.port.quantize_u8(xs[i], o_in)
        mid_ref, _ = oracle.port.quantized_matmul(xq_ref, w1, M, N1, K, [o_in, o_w1, o_mid], bias=b1)
        out_ref, _ = oracle.port.quantized_matmul(mid_ref, w2, M, N2, N1, [o_mid, o_w2, o_out])
        np.testing.assert_array_equal(mids[i].cpu().numpy(), mid_ref, err_msg=f"layer 1, iteration {i}")
        np.testing.assert_array_equal(outs[i].cpu().numpy(), out_ref, err_msg=f"layer 2, iteration {i}")
    l1.check()


@pytest.mark.parametrize("M", [1, 9, 16])
def test_next_layer_hint_leaves_results_unchanged(cuda, oracle, M):
    """ltq_layer_set_next: a layer that names its successor asks the start of the successor's weights into L2 from
    inside its own weight-streaming kernel.  A chain l1 -> l2 -> l3 -> l1 ... with every hint set (same split over the
    SMs for l1 / l2, a different one for l3, which the hint must survive), run back to back, against the oracle; then
    with the hints cleared; a layer without weights is refused as a successor."""
    import ltq
    rng = np.random.default_rng(400 + M)
    K, N1, N2, N3, reps = 1024, 2048, 1536, 512, 6
    w1 = rng.integers(0, 256, (N1, K), dtype=np.uint8)
    w2 = rng.integers(0, 256, (N2, N1), dtype=np.uint8)
    w3 = rng.integers(0, 256, (N3, N2), dtype=np.uint8)
    rows = [(0.02, 128), (0.005, 127), (3.0, 7), (0.004, 120), (40.0, 100), (0.003, 131), (500.0, 90)]
    q_in, q_w1, q_a, q_w2, q_b, q_w3, q_out = [ltq_qp(r) for r in rows]
    ls = [ltq.LayerHandle(0, K, N1), ltq.LayerHandle(0, N1, N2), ltq.LayerHandle(0, N2, N3)]
    for l, w, qs in zip(ls, (w1, w2, w3), ((q_in, q_w1, q_a), (q_a, q_w2, q_b), (q_b, q_w3, q_out))):
        l.set_weights(cuda.from_numpy(w).cuda())
        l.set_qparams(*qs)
    empty = ltq.LayerHandle(0, K, N1)
    with pytest.raises(ltq.LtqError):
        ls[0].set_next(empty)
    xq = [rng.integers(0, 256, (M, K), dtype=np.uint8) for _ in range(reps)]
    xq_dev = [cuda.from_numpy(x).cuda() for x in xq]
    o = [qp_of(oracle, r) for r in rows]
    want = []
    for i in range(reps):
        a, _ = oracle.port.quantized_matmul(xq[i], w1, M, N1, K, [o[0], o[1], o[2]])
        b, _ = oracle.port.quantized_matmul(a, w2, M, N2, N1, [o[2], o[3], o[4]])
        c, _ = oracle.port.quantized_matmul(b, w3, M, N3, N2, [o[4], o[5], o[6]])
        want.append(c)
    for hinted in (True, False):
        for i, l in enumerate(ls):
            l.set_next(ls[(i + 1) % 3] if hinted else None)
        outs = []
        cuda.cuda.synchronize()
        for i in range(reps):   # 3 dependent weight-streaming launches per iteration, nothing in between
            a = ls[0].forward(xq_dev[i], ltq.OUT_U8, ltq.FLAG_FORCE_SKINNY)
            b = ls[1].forward(a, ltq.OUT_U8, ltq.FLAG_FORCE_SKINNY)
            outs.append(ls[2].forward(b, ltq.OUT_U8, ltq.FLAG_FORCE_SKINNY))
            assert ltq.last_kernel().startswith("gemv_kernel")
        cuda.cuda.synchronize()
        for i in range(reps):
            np.testing.assert_array_equal(outs[i].cpu().numpy(), want[i], err_msg=f"hinted={hinted}, iteration {i}")
        for l in ls:
            l.check()
    for l in ls:
        l.set_next(None)


@pytest.mark.parametrize("M", [64, 300])
def test_back_to_back_tensor_core_layers_respect_their_inputs(cuda, oracle, M):
    """quantize_rows, the row-sum kernel and the tensor-core GEMMs are launched as programmatic dependents of the kernel
    in front of them (their set-up overlaps its tail).  A three-layer chain, run many times without any synchronisation
    and with every intermediate buffer reused, must still give the oracle's result each time."""
    import ltq
    rng = np.random.default_rng(23 + M)
    dims = [784, 512, 256, 48]
    ws = [rng.integers(0, 256, (dims[i + 1], dims[i]), dtype=np.uint8) for i in range(3)]
    bs = [rng.integers(-4000, 4000, dims[i + 1], dtype=np.int32) for i in range(3)]
    rows = [(0.02, 128), (0.004, 127), (2.5, 9), (0.003, 130), (30.0, 60), (0.005, 100), (300.0, 128)]
    q_act = [ltq_qp(rows[0]), ltq_qp(rows[2]), ltq_qp(rows[4]), ltq_qp(rows[6])]
    q_w = [ltq_qp(rows[1]), ltq_qp(rows[3]), ltq_qp(rows[5])]
    layers = []
    for i in range(3):
        h = ltq.LayerHandle(0, dims[i], dims[i + 1])
        h.set_weights(cuda.from_numpy(ws[i]).cuda(), cuda.from_numpy(bs[i]).cuda())
        h.set_qparams(q_act[i], q_w[i], q_act[i + 1])
        layers.append(h)
    reps = 10
    xs = [rng.normal(0, 0.8, (M, dims[0])).astype(np.float32) for _ in range(reps)]
    xs_dev = [cuda.from_numpy(x).cuda() for x in xs]
    xq = cuda.empty((M, dims[0]), dtype=cuda.uint8, device="cuda")
    asum = cuda.empty(M, dtype=cuda.int32, device="cuda")
    h1 = cuda.empty((M, dims[1]), dtype=cuda.uint8, device="cuda")       # reused by every iteration
    h2 = cuda.empty((M, dims[2]), dtype=cuda.uint8, device="cuda")
    outs = [cuda.empty((M, dims[3]), dtype=cuda.uint8, device="cuda") for _ in range(reps)]
    cuda.cuda.synchronize()
    for i in range(reps):
        ltq.quantize_rows(xs_dev[i], qp=q_act[0], q=xq, asum=asum)
        layers[0].forward(xq, ltq.OUT_U8, ltq.FLAG_RELU, asum=asum, out=h1)
        layers[1].forward(h1, ltq.OUT_U8, ltq.FLAG_RELU, out=h2)           # row sums computed by a kernel in between
        layers[2].forward(h2, ltq.OUT_U8, 0, out=outs[i])
    cuda.cuda.synchronize()
    o_act = [qp_of(oracle, rows[0]), qp_of(oracle, rows[2]), qp_of(oracle, rows[4]), qp_of(oracle, rows[6])]
    o_w = [qp_of(oracle, rows[1]), qp_of(oracle, rows[3]), qp_of(oracle, rows[5])]
    for i in range(reps):
        a = oracle.port.quantize_u8(xs[i], o_act[0])
        for li in range(3):
            acc = oracle.port.acc_i32(a, ws[li], M, dims[li + 1], dims[li], o_act[li].zero_point, o_w[li].zero_point, bias=bs[li])
            a = oracle.port.epilogue_u8(acc, o_act[li].scale, o_w[li].scale, o_act[li + 1].scale, o_act[li + 1].zero_point,
                                        relu=(li < 2))
        np.testing.assert_array_equal(outs[i].cpu().numpy(), a, err_msg=f"iteration {i}")
    layers[0].check()


@pytest.mark.parametrize("path,shape", [
    ("simt", (33, 48, 100)), ("tc", (200, 272, 256)), ("tc", (64, 512, 784)), ("tcpair", (300, 720, 128)),
    ("tcpair", (2000, 2160, 64)), ("skinny", (5, 160, 256)), ("skinny", (16, 1000, 1024)),
])
def test_rowsum_output_equals_the_row_sums_of_the_uint8_result(cuda, path, shape):
    """ltq_layer_set_rowsum_output: the epilogue adds each output row's byte sum to a caller-cleared array, on every
    kernel path; float output leaves the array alone; a chain that uses it instead of the row-sum pass gives the same
    bytes."""
    import ltq
    M, N, K = shape
    force = {"simt": ltq.FLAG_FORCE_SIMT, "tc": ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_SINGLE,
             "tcpair": ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR, "skinny": ltq.FLAG_FORCE_SKINNY}[path]
    g = cuda.Generator(device="cuda").manual_seed(M + N + K)
    x = cuda.randint(0, 256, (M, K), dtype=cuda.uint8, device="cuda", generator=g)
    w = cuda.randint(0, 256, (N, K), dtype=cuda.uint8, device="cuda", generator=g)
    h = ltq.LayerHandle(0, K, N)
    h.set_weights(w)
    h.set_qparams(ltq.QParams(0.02, 128), ltq.QParams(0.005, 127), ltq.QParams(0.5, 20))
    sums = cuda.zeros(M, dtype=cuda.int32, device="cuda")
    plain = h.forward(x, ltq.OUT_U8, force | ltq.FLAG_RELU)
    h.set_rowsum_output(sums)
    y = h.forward(x, ltq.OUT_U8, force | ltq.FLAG_RELU)
    assert cuda.equal(y, plain)
    assert cuda.equal(sums, y.to(cuda.int32).sum(1).to(cuda.int32))
    h.forward(x, ltq.OUT_U8, force | ltq.FLAG_RELU)                       # accumulates: the caller clears
    assert cuda.equal(sums, 2 * y.to(cuda.int32).sum(1).to(cuda.int32))
    sums.zero_()
    h.forward(x, ltq.OUT_F32, force)                                      # other output modes leave it alone
    assert int(sums.abs().sum()) == 0
    h.set_rowsum_output(None)
    h.forward(x, ltq.OUT_U8, force)
    assert int(sums.abs().sum()) == 0
    # a second layer fed with (y, sums) equals the same layer computing the sums itself
    h.set_rowsum_output(sums)
    y = h.forward(x, ltq.OUT_U8, force | ltq.FLAG_RELU)
    w2 = cuda.randint(0, 256, (64, N), dtype=cuda.uint8, device="cuda", generator=g)
    h2 = ltq.LayerHandle(0, N, 64)
    h2.set_weights(w2)
    h2.set_qparams(ltq.QParams(0.5, 20), ltq.QParams(0.01, 100), ltq.QParams(1.0, 0))
    assert cuda.equal(h2.forward(y, ltq.OUT_I32, 0, asum=sums), h2.forward(y, ltq.OUT_I32, 0))


@pytest.mark.parametrize("M", [64, 12])
def test_chain_with_epilogue_row_sums_and_clear_hooks(cuda, oracle, M):
    """Three layers chained without any sum pass or clearing launch in between: layers 1 and 2 emit the row sums of their
    outputs, layer 3 clears the first array and layer 1 (of the next batch) the second.  Several batches back to back
    without synchronisation must each give the oracle's bytes."""
    import ltq
    rng = np.random.default_rng(77 + M)
    dims = [256, 512, 384, 40]
    ws = [rng.integers(0, 256, (dims[i + 1], dims[i]), dtype=np.uint8) for i in range(3)]
    rows = [(0.02, 128), (0.004, 127), (2.5, 9), (0.003, 130), (30.0, 60), (0.005, 100), (300.0, 128)]
    q_act = [ltq_qp(rows[0]), ltq_qp(rows[2]), ltq_qp(rows[4]), ltq_qp(rows[6])]
    q_w = [ltq_qp(rows[1]), ltq_qp(rows[3]), ltq_qp(rows[5])]
    layers = []
    for i in range(3):
        h = ltq.LayerHandle(0, dims[i], dims[i + 1])
        h.set_weights(cuda.from_numpy(ws[i]).cuda())
        h.set_qparams(q_act[i], q_w[i], q_act[i + 1])
        layers.append(h)
    sums = cuda.zeros((2, M), dtype=cuda.int32, device="cuda")
    layers[0].set_rowsum_output(sums[0])
    layers[1].set_rowsum_output(sums[1])
    layers[2].set_clear_on_forward(sums[0])
    layers[0].set_clear_on_forward(sums[1])
    reps = 6
    xs = [rng.integers(0, 256, (M, dims[0]), dtype=np.uint8) for _ in range(reps)]
    xs_dev = [cuda.from_numpy(x).cuda() for x in xs]
    h1 = cuda.empty((M, dims[1]), dtype=cuda.uint8, device="cuda")
    h2 = cuda.empty((M, dims[2]), dtype=cuda.uint8, device="cuda")
    outs = [cuda.empty((M, dims[3]), dtype=cuda.uint8, device="cuda") for _ in range(reps)]
    cuda.cuda.synchronize()
    for i in range(reps):
        layers[0].forward(xs_dev[i], ltq.OUT_U8, ltq.FLAG_RELU, out=h1)
        layers[1].forward(h1, ltq.OUT_U8, ltq.FLAG_RELU, asum=sums[0], out=h2)
        layers[2].forward(h2, ltq.OUT_U8, 0, asum=sums[1], out=outs[i])
    cuda.cuda.synchronize()
    o_act = [qp_of(oracle, rows[0]), qp_of(oracle, rows[2]), qp_of(oracle, rows[4]), qp_of(oracle, rows[6])]
    o_w = [qp_of(oracle, rows[1]), qp_of(oracle, rows[3]), qp_of(oracle, rows[5])]
    for i in range(reps):
        a = xs[i]
        for li in range(3):
            acc = oracle.port.acc_i32(a, ws[li], M, dims[li + 1], dims[li], o_act[li].zero_point, o_w[li].zero_point)
            a = oracle.port.epilogue_u8(acc, o_act[li].scale, o_w[li].scale, o_act[li + 1].scale, o_act[li + 1].zero_point,
                                        relu=(li < 2))
        np.testing.assert_array_equal(outs[i].cpu().numpy(), a, err_msg=f"batch {i}")
    with pytest.raises(ltq.LtqError):
        layers[0].set_clear_on_forward(sums[0])      # its own accumulation target


def test_mlp_block_shapes_sampled_rows(cuda, oracle):
    """The 8192 -> 32768 -> 8192 block at its real widths (512 tokens): layer 1 uint8 + ReLU leaving the row sums of its
    output behind, layer 2 fp32 fed with those sums, both on the kernel the dispatcher picks by shape (the CTA-pair
    kernel).  64 random rows are pushed through both layers by the CPU oracle and compared bit for bit; the whole tensors
    are compared with the dp4a kernel; and layer 2's K = 32768 is run once more with both zero points at 255, where
    K*zA*zB sits 0.8 % under the int32 limit (l-ten/math_fns.cpp:1433-1434)."""
    import ltq
    M, K1, N1, N2 = 512, 8192, 32768, 8192
    g = cuda.Generator(device="cuda").manual_seed(5)
    x = cuda.randn((M, K1), generator=g, device="cuda")
    w1 = cuda.randn((N1, K1), generator=g, device="cuda") * 0.01
    w2 = cuda.randn((N2, N1), generator=g, device="cuda") * 0.01
    b1 = cuda.randn(N1, generator=g, device="cuda") * 0.05
    qx = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(x)))
    qw1 = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(w1)))
    qw2 = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(w2)))
    qh = ltq.ops.qparams_from_dev(ltq.compute_qparams_dev(ltq.GetMinMax(cuda.relu(x[:128] @ w1.t() + b1))))
    xq, asum = ltq.quantize_rows(x, qp=qx)
    w1q, w2q = ltq.Quantize(w1, qw1), ltq.Quantize(w2, qw2)
    b1q = ltq.QuantizeInt32(b1, ltq.QParams(np.float32(qx.scale) * np.float32(qw1.scale), 0))
    del x, w1, w2
    l1 = ltq.LayerHandle(0, K1, N1)
    l1.set_weights(w1q, b1q)
    l1.set_qparams(qx, qw1, qh)
    l2 = ltq.LayerHandle(0, N1, N2)
    l2.set_weights(w2q, None)
    l2.set_qparams(qh, qw2, ltq.QParams(1.0, 0))
    hsum = cuda.zeros(M, dtype=cuda.int32, device="cuda")
    l1.set_rowsum_output(hsum)
    hq = l1.forward(xq, ltq.OUT_U8, ltq.FLAG_RELU, asum=asum)
    assert ltq.last_kernel().startswith("gemm_tc_pair_kernel<"), ltq.last_kernel()
    y = l2.forward(hq, ltq.OUT_F32, 0, asum=hsum)
    assert ltq.last_kernel().startswith("gemm_tc_pair_kernel<"), ltq.last_kernel()
    l2.check()
    assert cuda.equal(hsum, hq.to(cuda.int32).sum(1).to(cuda.int32))
    # whole tensors against the dp4a kernel (which computes its own row sums for layer 2)
    l1.set_rowsum_output(None)
    assert cuda.equal(hq, l1.forward(xq, ltq.OUT_U8, ltq.FLAG_RELU | ltq.FLAG_FORCE_SIMT, asum=asum))
    assert cuda.equal(y, l2.forward(hq, ltq.OUT_F32, ltq.FLAG_FORCE_SIMT))
    # 64 random rows through both layers on the CPU
    rows = np.sort(np.random.default_rng(5).choice(M, 64, replace=False))
    oqx, oqw1, oqw2, oqh = [oracle.qp(q.scale, q.zero_point) for q in (qx, qw1, qw2, qh)]
    xq_h, w1_h, w2_h, b1_h = xq.cpu().numpy()[rows], w1q.cpu().numpy(), w2q.cpu().numpy(), b1q.cpu().numpy()
    acc1 = oracle.port.acc_i32(xq_h, w1_h, 64, N1, K1, oqx.zero_point, oqw1.zero_point, bias=b1_h)
    h_ref = oracle.port.epilogue_u8(acc1, oqx.scale, oqw1.scale, oqh.scale, oqh.zero_point, relu=True)
    np.testing.assert_array_equal(hq.cpu().numpy()[rows], h_ref)
    acc2 = oracle.port.acc_i32(h_ref, w2_h, 64, N2, N1, oqh.zero_point, oqw2.zero_point)
    y_ref = oracle.port.epilogue_f32(acc2, oqh.scale, oqw2.scale)
    np.testing.assert_array_equal(y.cpu().numpy()[rows].view(np.uint32), y_ref.view(np.uint32))
    # K = 32768 with zA = zB = 255: K*zA*zB = 2 130 739 200 < 2^31 - 1; random bytes so that raw sums are large too
    hr = cuda.randint(0, 256, (M, N1), dtype=cuda.uint8, device="cuda", generator=g)
    l2.set_qparams(ltq.QParams(0.03, 255), ltq.QParams(0.002, 255), ltq.QParams(1.0, 0))
    acc_dev = l2.forward(hr, ltq.OUT_I32, 0)
    assert ltq.last_kernel().startswith("gemm_tc_pair_kernel<"), ltq.last_kernel()
    assert cuda.equal(acc_dev, l2.forward(hr, ltq.OUT_I32, ltq.FLAG_FORCE_SIMT))
    want = oracle.port.acc_i32(hr.cpu().numpy()[rows], w2_h, 64, N2, N1, 255, 255)
    np.testing.assert_array_equal(acc_dev.cpu().numpy()[rows], want)
    l2.check()
