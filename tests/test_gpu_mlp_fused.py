"""GPU: the fused chain (Quantize + 2..4 FullyConnected_q layers in one launch, ltq_mlp_*) against the golden MLP fixture
from the reference, the CPU oracle, and the layer-by-layer path on the same device.  Everything is compared bit for bit."""
import numpy as np
import pytest

from helpers import ltq_qp, qp_of

pytestmark = pytest.mark.gpu


def _build(cuda, ltq, rng, dims, batch):
    """Random chain: returns (layers, host weights / biases, qparams rows, x)."""
    L = len(dims) - 1
    ws = [rng.integers(0, 256, (dims[i + 1], dims[i]), dtype=np.uint8) for i in range(L)]
    bs = [rng.integers(-4000, 4000, dims[i + 1], dtype=np.int32) for i in range(L)]
    acts = [(0.02, 128)] + [(float(2.0 + i), 5 + 3 * i) for i in range(L)]       # activation qparams: input, h1, h2, ..., out
    wqp = [(0.003 + 0.001 * i, 120 + 5 * i) for i in range(L)]
    layers = []
    for i in range(L):
        h = ltq.LayerHandle(0, dims[i], dims[i + 1])
        h.set_weights(cuda.from_numpy(ws[i]).cuda(), cuda.from_numpy(bs[i]).cuda())
        h.set_qparams(ltq_qp(acts[i]), ltq_qp(wqp[i]), ltq_qp(acts[i + 1]))
        layers.append(h)
    x = rng.normal(0, 0.9, (batch, dims[0])).astype(np.float32)
    return layers, ws, bs, acts, wqp, x


def _oracle_chain(oracle, ws, bs, acts, wqp, x, relu, last_mode):
    a = oracle.port.quantize_u8(x, qp_of(oracle, acts[0]))
    L = len(ws)
    for i in range(L):
        N, K = ws[i].shape
        acc = oracle.port.acc_i32(a, ws[i], a.shape[0], N, K, acts[i][1], wqp[i][1], bias=bs[i])
        if i < L - 1:
            a = oracle.port.epilogue_u8(acc, np.float32(acts[i][0]), np.float32(wqp[i][0]), np.float32(acts[i + 1][0]), acts[i + 1][1],
                                        relu=relu[i])
        elif last_mode == "u8":
            return oracle.port.epilogue_u8(acc, np.float32(acts[i][0]), np.float32(wqp[i][0]), np.float32(acts[i + 1][0]), acts[i + 1][1],
                                           relu=relu[i])
        elif last_mode == "f32":
            return oracle.port.epilogue_f32(acc, np.float32(acts[i][0]), np.float32(wqp[i][0]), relu=relu[i])
        else:
            return np.maximum(acc, 0) if relu[i] else acc


@pytest.mark.parametrize("dims,batch", [((784, 512, 512, 10), 64), ((784, 512, 512, 10), 37), ((256, 384, 48), 200),
                                        ((128, 1024, 256, 128, 16), 64), ((1024, 640, 24), 5)])
@pytest.mark.parametrize("last_mode", ["u8", "f32", "i32"])
def test_fused_chain_vs_oracle_and_layer_by_layer(cuda, oracle, dims, batch, last_mode):
    import ltq
    rng = np.random.default_rng(sum(dims) + batch)
    layers, ws, bs, acts, wqp, x = _build(cuda, ltq, rng, dims, batch)
    L = len(ws)
    relu = [True] * (L - 1) + [last_mode == "i32"]
    flags = [ltq.FLAG_RELU if r else 0 for r in relu]
    mode = {"u8": ltq.OUT_U8, "f32": ltq.OUT_F32, "i32": ltq.OUT_I32}[last_mode]
    mlp = ltq.FusedMLP(layers)
    xd = cuda.from_numpy(x).cuda()
    got = mlp.forward(xd, flags, mode)
    assert ltq.last_kernel().startswith("mlp_fused_kernel<"), ltq.last_kernel()
    layers[0].check()
    # layer by layer on the device
    a, asum = ltq.quantize_rows(xd, qp=ltq_qp(acts[0]))
    for i in range(L - 1):
        a = layers[i].forward(a, ltq.OUT_U8, flags[i], asum=asum if i == 0 else None)
    ref_dev = layers[-1].forward(a, mode, flags[-1])
    assert cuda.equal(got, ref_dev)
    want = _oracle_chain(oracle, ws, bs, acts, wqp, x, relu, last_mode)
    g = got.cpu().numpy()
    np.testing.assert_array_equal(g.view(np.uint32) if last_mode == "f32" else g, want.view(np.uint32) if last_mode == "f32" else want)
    # again, back to back without synchronisation, into the same output
    outs = [mlp.forward(xd, flags, mode) for _ in range(5)]
    for o in outs:
        assert cuda.equal(o, got)
    mlp.close()


@pytest.mark.parametrize("relu", [True, False])
@pytest.mark.parametrize("batch", [64, 9, 300])
def test_fused_chain_hidden_epilogue_across_the_accumulator_range(cuda, oracle, relu, batch):
    """The hidden layers' uint8 conversion takes a shortcut that is exact only for accumulators within +-2^22 and
    non-negative results, and must fall back to the reference sequence elsewhere.  Biases steer whole columns to both
    sides of every boundary (around +-2^22, far beyond it, results that wrap below 0 or above 255), with and without
    ReLU; every layer's bytes feed the next, so one wrong byte changes the output."""
    import ltq
    rng = np.random.default_rng(77 + batch + int(relu))
    dims = (256, 512, 256, 64)
    L = len(dims) - 1
    ws = [rng.integers(0, 256, (dims[i + 1], dims[i]), dtype=np.uint8) for i in range(L)]
    edges = np.array([0, 1, -1, (1 << 22) - 3, 1 << 22, (1 << 22) + 5, -(1 << 22) + 2, -(1 << 22) - 1, 1 << 23, -(1 << 23),
                      1 << 26, -(1 << 26), (1 << 31) - 1 - (1 << 24), -(1 << 31) + (1 << 24), 3000, -3000], dtype=np.int64)
    bs = []
    for i in range(L):
        b = rng.integers(-60000, 60000, dims[i + 1]).astype(np.int64)
        pick = rng.choice(dims[i + 1], size=len(edges) * 4, replace=False)
        b[pick] = np.repeat(edges, 4) + rng.integers(-40, 40, len(pick))
        bs.append(b.astype(np.int32))
    # output scales that make rm = sA * sB / sC 0.3 .. 0.4: the shortcut applies (rm <= 0.5) and results spread over many
    # multiples of 256, so the wrapped bytes carry every accumulator's low bits into the next layer
    acts = [(0.02, 128), (0.0002, 3), (2e-6, 200), (3e-8, 17)]
    wqp = [(0.004, 117), (0.003, 131), (0.005, 125)]
    layers = []
    for i in range(L):
        h = ltq.LayerHandle(0, dims[i], dims[i + 1])
        h.set_weights(cuda.from_numpy(ws[i]).cuda(), cuda.from_numpy(bs[i]).cuda())
        h.set_qparams(ltq_qp(acts[i]), ltq_qp(wqp[i]), ltq_qp(acts[i + 1]))
        layers.append(h)
    x = rng.normal(0, 0.9, (batch, dims[0])).astype(np.float32)
    relus = [relu] * (L - 1) + [False]
    flags = [ltq.FLAG_RELU if r else 0 for r in relus]
    mlp = ltq.FusedMLP(layers)
    got = mlp.forward(cuda.from_numpy(x).cuda(), flags, ltq.OUT_I32).cpu().numpy()
    layers[0].check()
    want = _oracle_chain(oracle, ws, bs, acts, wqp, x, relus, "i32")
    np.testing.assert_array_equal(got, want)
    mlp.close()


def test_fused_chain_matches_the_reference_fixture(cuda, golden):
    """784-512-512-10, batch 64: the bytes FullyConnected_q::forward of the reference produced, layer after layer."""
    import ltq
    from ltq import workloads
    g = golden("fc_mlp.npz")
    x, wl = workloads.mlp_mnist(seed=0, batch=64)
    layers = []
    for li, (w, b) in enumerate(wl):
        N, K = w.shape
        qps = [ltq_qp(r) for r in g[f"l{li}.qp"]]
        h = ltq.LayerHandle(0, K, N)
        h.set_weights(cuda.from_numpy(g[f"l{li}.w_q"]).cuda(), cuda.from_numpy(g[f"l{li}.b_q"]).cuda())
        h.set_qparams(*qps)
        layers.append(h)
    mlp = ltq.FusedMLP(layers)
    y = mlp.forward(cuda.from_numpy(x).cuda(), None, ltq.OUT_U8)      # the reference's QNet has no activation function
    np.testing.assert_array_equal(y.cpu().numpy(), g["l2.y"])
    logits = ltq.Dequantize(y, ltq_qp(g["l2.qp"][2]))
    np.testing.assert_array_equal(logits.cpu().numpy(), g["logits"])
    layers[0].check()


def test_chains_that_do_not_fit_are_refused(cuda):
    import ltq
    def layer(K, N):
        h = ltq.LayerHandle(0, K, N)
        h.set_weights(cuda.zeros((N, K), dtype=cuda.uint8, device="cuda"))
        return h
    with pytest.raises(ltq.LtqError) as e:
        ltq.FusedMLP([layer(4096, 4096), layer(4096, 512)])          # far beyond one cluster's shared memory
    assert e.value.status == -2
    with pytest.raises(ltq.LtqError):
        ltq.FusedMLP([layer(64, 32), layer(48, 16)])                  # widths do not chain
    with pytest.raises(ltq.LtqError):
        ltq.FusedMLP([layer(64, 32)])                                  # a chain has at least two layers
