"""Shared helpers for the parity tests."""
import numpy as np


def qp_of(oracle, row):
    return oracle.qp(np.float32(row[0]), int(row[1]))


def ltq_qp(row):
    import ltq
    return ltq.QParams(float(np.float32(row[0])), int(row[1]))


def iter_qmm_cases(g):
    n = int(g["count"][0])
    for i in range(n):
        key = f"c{i}"
        if key + ".meta" not in g:
            continue
        M, N, K, tA, tB, use_bias, qi = [int(v) for v in g[key + ".meta"]]
        yield dict(key=key, M=M, N=N, K=K, tA=tA, tB=tB, qp=g[key + ".qp"], A=g[key + ".A"], B=g[key + ".B"],
                   bias=g[key + ".bias"] if use_bias else None, C=g[key + ".C"], ws=g[key + ".ws"])


def iter_conv_cases(g):
    for i, row in enumerate(g["cases"]):
        B, Cin, H, W, Cout, kh, kw, ph, pw, sh, sw, use_bias = [int(v) for v in row]
        key = f"v{i}"
        yield dict(key=key, B=B, Cin=Cin, H=H, W=W, Cout=Cout, kh=kh, kw=kw, ph=ph, pw=pw, sh=sh, sw=sw, qp=g[key + ".qp"],
                   x=g[key + ".x"], w=g[key + ".w"], bias=g[key + ".bias"] if use_bias else None, y=g[key + ".y"],
                   col0=g[key + ".col0"])


# ---- stand-in for the reference's quantized classification replay (tests/nn_tests.cpp:536-974) ----
# The reference trains a float32 network (5 x 5 convolution 1 -> 10 without bias, 5760 -> 50, 50 -> 10, no activation
# function) on 28 x 28 digit images for 1000 iterations of 32 images with SGD (lr 0.001), records the range of the input
# and of every layer output while training, quantises the network from those ranges and passes if the uint8 network
# keeps more than 95 % of the float32 accuracy on the test images.  The digit files are not available, so seeded
# synthetic ten-class images of the same shape and value range (8-bit pixels / 255, dark background, bright strokes)
# take their place.

def synthetic_digits(seed, n):
    """n images [n, 1, 28, 28] float32 in [0, 1] and their labels: ten fixed stroke templates, shifted by up to 3
    pixels, dimmed and covered in noise."""
    yy, xx = np.mgrid[0:28, 0:28].astype(np.float32)
    trng = np.random.default_rng(1234)          # the ten classes are the same for every split
    tmpl = np.zeros((10, 28, 28), np.float32)
    for c in range(10):
        for _ in range(3):
            p0, p1 = trng.uniform(5, 23, 2), trng.uniform(5, 23, 2)
            for t in np.linspace(0, 1, 60):
                y, x = p0 + t * (p1 - p0)
                tmpl[c] = np.maximum(tmpl[c], np.exp(-((yy - y) ** 2 + (xx - x) ** 2) / 1.6))
    rng = np.random.default_rng(seed)
    labels = rng.integers(0, 10, n)
    imgs = np.empty((n, 1, 28, 28), np.float32)
    for i, c in enumerate(labels):
        dy, dx = rng.integers(-3, 4, 2)
        im = np.roll(np.roll(tmpl[c], dy, 0), dx, 1) * rng.uniform(0.6, 1.0) + rng.normal(0, 0.25, (28, 28))
        imgs[i, 0] = np.round(np.clip(im, 0, 1) * 255) / 255
    return imgs, labels.astype(np.int64)


def train_float_digit_net(images, labels, iterations=1000, batch=32, lr=0.001, observe=None):
    """The float32 side of the replay, on the CPU with torch: returns the three weight arrays (convolution [10, 25],
    [50, 5760], [10, 50]) and a predict(images) function.  `observe(taps)` is called on every training batch with
    [input, conv output, fc1 output, fc2 output], the four tensors whose ranges the reference records."""
    import torch
    torch.manual_seed(0)
    conv = torch.nn.Conv2d(1, 10, 5, bias=False)
    fc1 = torch.nn.Linear(5760, 50, bias=False)
    fc2 = torch.nn.Linear(50, 10, bias=False)
    opt = torch.optim.SGD([*conv.parameters(), *fc1.parameters(), *fc2.parameters()], lr=lr)
    for it in range(iterations):
        idx = (it * batch + np.arange(batch)) % len(images)
        xb, yb = torch.from_numpy(images[idx]), torch.from_numpy(labels[idx])
        a1 = conv(xb)
        a2 = fc1(a1.reshape(batch, -1))
        a3 = fc2(a2)
        if observe is not None:
            observe([t.detach() for t in (xb, a1, a2, a3)])
        loss = torch.nn.functional.nll_loss(torch.log_softmax(a3, 1), yb, reduction="sum")
        opt.zero_grad()
        loss.backward()
        opt.step()

    def predict(x):
        with torch.no_grad():
            return fc2(fc1(conv(torch.from_numpy(x)).reshape(len(x), -1))).argmax(1).numpy()

    weights = [conv.weight.detach().numpy().reshape(10, 25).copy(), fc1.weight.detach().numpy().copy(),
               fc2.weight.detach().numpy().copy()]
    return weights, predict


def oracle_digit_replay(oracle, images, weights, ranges):
    """The uint8 side through the oracle: ranges = four (min, max) pairs -> ComputeQuantizationParams; weights quantised
    from their own min / max; Quantize -> Conv2d_q -> reshape -> FullyConnected_q x 2 -> Dequantize.  Returns the uint8
    outputs of the three layers and the float logits."""
    P = oracle.port
    qps = [P.compute_qparams(np.float32(lo), np.float32(hi)) for lo, hi in ranges]
    qw = [P.compute_qparams(*P.get_min_max(w.ravel())) for w in weights]
    wq = [P.quantize_u8(w.ravel(), q).reshape(w.shape) for w, q in zip(weights, qw)]
    n = len(images)
    xq = P.quantize_u8(images, qps[0])
    y1 = P.conv2d_q(xq, wq[0], 10, 5, 5, qps[0], qw[0], qps[1])
    y2, _ = P.quantized_matmul(y1.reshape(n, 5760), wq[1], n, 50, 5760, [qps[1], qw[1], qps[2]])
    y3, _ = P.quantized_matmul(y2, wq[2], n, 10, 50, [qps[2], qw[2], qps[3]])
    return (y1, y2, y3), P.dequantize(y3, qps[3])
