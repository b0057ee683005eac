"""Generates the golden fixtures in this directory by running the UNMODIFIED l-ten reference
(oracle/_ref/liblten_ref.so, built from the reference sources by oracle/Makefile) on seeded inputs.

    python tests/golden/make_golden.py

The reference's own tests hold no known-answer vector for its quantized path (its only check is an accuracy ratio on
MNIST), so these files are the pin: the C restatement in oracle/ltq_oracle.c and the CUDA library are both tested
against them.  Needs the reference source tree at build time only; the fixtures are committed.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "light-tensor_b200", "python"))

import oracle  # noqa: E402
from ltq import workloads  # noqa: E402

ref = oracle.ref
if ref is None:
    oracle.build(with_ref=True)
    ref = oracle._Ref(os.path.join(ROOT, "oracle", "_ref", "liblten_ref.so"))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def helpers():
    """GetMinMax / ComputeQuantizationParams / Quantize (u8 and int32) / Dequantize."""
    rng = np.random.default_rng(100)
    out = {}
    cases = {
        "normal": rng.standard_normal(4099).astype(np.float32),
        "uniform01": rng.random(1000, dtype=np.float32),
        "negative_only": -rng.random(513, dtype=np.float32) * 3,
        "positive_offset": rng.random(777, dtype=np.float32) * 5 + 2,
        "wide": (rng.standard_normal(2048) * 1000).astype(np.float32),
        "tiny": (rng.standard_normal(300) * 1e-6).astype(np.float32),
        "single": np.array([0.75], np.float32),
    }
    # exact .5 ties after division, to pin round-half-away-from-zero
    ties = np.arange(-40, 40, dtype=np.float32) * 0.5
    cases["ties"] = ties
    for name, x in cases.items():
        mn, mx = ref.get_min_max(x)
        qp = ref.compute_qparams(mn, mx)
        q = ref.quantize_u8(x, qp)
        dq = ref.dequantize(q, qp)
        out[f"{name}.x"] = x
        out[f"{name}.minmax"] = np.array([mn, mx], np.float32)
        out[f"{name}.qp"] = np.array([qp.scale, qp.zero_point], np.float64)
        out[f"{name}.q"] = q
        out[f"{name}.dq"] = dq
    # explicit qparams (power-of-two scale makes the ties exact); includes values clamped at both ends
    qp = oracle.qp(0.5, 7)
    x = np.concatenate([ties, np.array([1e9, -1e9, 123.75, 124.0, 124.25, -3.5, -3.75], np.float32)])
    out["explicit.x"] = x
    out["explicit.qp"] = np.array([0.5, 7], np.float64)
    out["explicit.q"] = ref.quantize_u8(x, qp)
    # bias quantisation to int32: scale = s_in * s_wt, zero point 0 (tests/nn_tests.cpp:824-826)
    b = np.concatenate([rng.normal(0, 0.1, 600).astype(np.float32),
                        np.array([0.0, 1e-4 * 0.5, -1e-4 * 0.5, 1e-4 * 1.5, 3e5, -3e5, 1e12, -1e12], np.float32)])
    qpb = oracle.qp(np.float32(0.02) * np.float32(0.005), 0)
    out["bias.x"] = b
    out["bias.qp"] = np.array([qpb.scale, 0], np.float64)
    out["bias.q"] = ref.quantize_i32(b, qpb)
    np.savez_compressed(os.path.join(HERE, "helpers.npz"), **out)
    print("helpers.npz:", len(cases) + 2, "cases")


def qmm_small():
    """quantized_matmul on small hand-checkable shapes: all transpose variants, ragged K/N/M, extreme zero points,
    outputs that leave [0,255] (the reference build wraps them), with and without bias."""
    rng = np.random.default_rng(200)
    shapes = [(1, 1, 1), (1, 10, 33), (3, 5, 7), (8, 16, 64), (17, 10, 784 // 8), (5, 24, 31), (16, 8, 128),
              (33, 65, 100), (2, 3, 300)]
    qsets = [
        ((0.02, 128), (0.005, 127), (0.05, 3)),
        ((0.1, 0), (0.1, 255), (0.5, 200)),
        ((0.1, 255), (0.1, 0), (0.01, 128)),     # small output scale: many values wrap
        ((1.0, 0), (1.0, 0), (1.0, 0)),          # rm = 1, z = 0: low byte of acc
        ((0.03, 17), (0.007, 201), (2.0, 250)),
    ]
    out = {}
    n = 0
    for (M, N, K) in shapes:
        for qi, qs in enumerate(qsets):
            for tA in (0, 1):
                for tB in (0, 1):
                    for use_bias in (0, 1):
                        if (n % 3) and not (tA == 0 and tB == 1):
                            n += 1
                            continue  # thin out the non-FC variants
                        A = rng.integers(0, 256, M * K, dtype=np.uint8)
                        B = rng.integers(0, 256, N * K, dtype=np.uint8)
                        bias = rng.integers(-20000, 20000, N, dtype=np.int32) if use_bias else None
                        qps = [oracle.qp(*q) for q in qs]
                        C, ws = ref.quantized_matmul(A, B, M, N, K, qps, bias=bias, tA=bool(tA), tB=bool(tB))
                        key = f"c{n}"
                        out[key + ".meta"] = np.array([M, N, K, tA, tB, use_bias, qi], np.int64)
                        out[key + ".qp"] = np.array([[q[0], q[1]] for q in qs], np.float64)
                        out[key + ".A"] = A
                        out[key + ".B"] = B
                        if use_bias:
                            out[key + ".bias"] = bias
                        out[key + ".C"] = C
                        out[key + ".ws"] = ws
                        n += 1
    out["count"] = np.array([n], np.int64)
    np.savez_compressed(os.path.join(HERE, "qmm_small.npz"), **out)
    print("qmm_small.npz:", sum(1 for k in out if k.endswith(".meta")), "cases")


def fc_mlp():
    """The MNIST-shaped 784-512-512-10 MLP, batch 64, seed 0, pushed through the reference exactly as its quantized test
    does (tests/nn_tests.cpp:786-884, 940-942): calibrate each activation tensor from an fp32 run, quantize weights by
    min/max and biases to int32 with scale s_in*s_wt, chain FullyConnected_q::forward (uint8 in, uint8 out, no
    activation function in between -- the reference has none)."""
    x, layers = workloads.mlp_mnist(seed=0, batch=64)
    acts = [x]
    h = x
    for (w, b) in layers:
        h = (h @ w.T + b).astype(np.float32)
        acts.append(h)
    qp_act = [ref.compute_qparams(*ref.get_min_max(a)) for a in acts]
    out = {"x_sha": np.array(sha(x)), "w_sha": np.array([sha(w) for w, _ in layers])}
    q = ref.quantize_u8(x, qp_act[0])
    out["x_q"] = q
    for li, (w, b) in enumerate(layers):
        N, K = w.shape
        qp_w = ref.compute_qparams(*ref.get_min_max(w))
        w_q = ref.quantize_u8(w, qp_w)
        b_q = ref.quantize_i32(b, oracle.qp(np.float32(qp_act[li].scale) * np.float32(qp_w.scale), 0))
        y, _ = ref.fc_q_forward(q, w_q, 64, N, K, qp_act[li], qp_w, qp_act[li + 1], bias=b_q)
        out[f"l{li}.qp"] = np.array([[qp_act[li].scale, qp_act[li].zero_point], [qp_w.scale, qp_w.zero_point],
                                     [qp_act[li + 1].scale, qp_act[li + 1].zero_point]], np.float64)
        out[f"l{li}.w_q"] = w_q
        out[f"l{li}.b_q"] = b_q
        out[f"l{li}.y"] = y
        q = y
    out["logits"] = ref.dequantize(q, qp_act[-1])
    np.savez_compressed(os.path.join(HERE, "fc_mlp.npz"), **out)
    print("fc_mlp.npz: 3 layers")


def linear_1024():
    """Single 1024^3 quantized linear (A z=128 s=0.02, W z=127 s=0.005, bias N(0,0.1) -> int32 with scale 1e-4).
    The reference only emits uint8, so the int32 accumulator is pinned through byte planes: with rm = 2^-8s and
    z_out = 0 its wrapping cast returns byte s of trunc(acc / 2^8s).  Inputs are regenerated from the seed by the tests;
    hashes of inputs and outputs plus every 64th output row are stored."""
    wl = workloads.linear_u8(seed=2)
    M = N = K = 1024
    qa, qw = oracle.qp(*wl["qp_a"]), oracle.qp(*wl["qp_w"])
    bias_q = ref.quantize_i32(wl["bias"], oracle.qp(np.float32(qa.scale) * np.float32(qw.scale), 0))
    out = {"a_sha": np.array(sha(wl["a"])), "w_sha": np.array(sha(wl["w"])), "bias_q": bias_q}
    # (scale_out, z_out): a realistic requant + three byte planes (s_out = s_a*s_w * 2^(8s) makes rm = 2^-8s exactly)
    sab = np.float32(qa.scale) * np.float32(qw.scale)
    outs = [(np.float32(0.35), 131)] + [(np.float32(sab * np.float32(2.0 ** (8 * s))), 0) for s in range(3)]
    for i, (sc, zc) in enumerate(outs):
        C, _ = ref.quantized_matmul(wl["a"], wl["w"], M, N, K, [qa, qw, oracle.qp(sc, zc)], bias=bias_q)
        out[f"o{i}.qp"] = np.array([sc, zc], np.float64)
        out[f"o{i}.sha"] = np.array(sha(C))
        out[f"o{i}.rows"] = C[::64].copy()
    np.savez_compressed(os.path.join(HERE, "linear_1024.npz"), **out)
    print("linear_1024.npz:", len(outs), "output settings")


CONV_CASES = [
    # batches, Cin, H, W, Cout, kh, kw, ph, pw, sh, sw, bias
    (4, 1, 28, 28, 10, 5, 5, 0, 0, 1, 1, 0),     # the reference's quantized conv test net (tests/nn_tests.cpp:620-627)
    (2, 3, 17, 13, 8, 3, 3, 1, 1, 1, 1, 0),      # padding, K = 27
    (2, 16, 12, 12, 24, 3, 3, 1, 1, 2, 2, 0),    # stride 2, K = 144 (multiple of 16)
    (1, 64, 14, 14, 32, 3, 3, 1, 1, 1, 1, 0),    # K = 576
    (3, 5, 9, 11, 7, 2, 4, 0, 2, 1, 3, 0),       # rectangular kernel, pad and stride differ per axis
    (2, 32, 6, 6, 16, 1, 1, 0, 0, 1, 1, 0),      # 1 x 1 kernel
    (2, 4, 8, 8, 32, 5, 5, 0, 0, 1, 1, 1),       # bias: Ho*Wo = 16 <= Cout = 32, the only range where the reference's
    (1, 8, 5, 5, 48, 3, 3, 1, 1, 2, 2, 1),       # per-position bias indexing stays inside its tensor (9 <= 48)
    (2, 2, 7, 7, 3, 7, 7, 3, 3, 1, 1, 0),        # kernel as large as the image, heavy padding
]


def conv2d():
    """Conv2d_q::forward (l-ten/conv2d.cpp:266-379) and im2col_cpu (l-ten/im_col.h:5-33) on seeded inputs."""
    rng = np.random.default_rng(300)
    qsets = [((0.02, 128), (0.005, 127), (0.05, 3)), ((0.1, 7), (0.03, 250), (0.9, 100)), ((0.05, 0), (0.01, 131), (0.02, 64))]
    out = {"cases": np.array(CONV_CASES, np.int64)}
    for ci, (B, Cin, H, W, Cout, kh, kw, ph, pw, sh, sw, use_bias) in enumerate(CONV_CASES):
        x = rng.integers(0, 256, (B, Cin, H, W), dtype=np.uint8)
        w = rng.integers(0, 256, (Cout, Cin * kh * kw), dtype=np.uint8)
        bias = rng.integers(-20000, 20000, Cout, dtype=np.int32) if use_bias else None
        q_in, q_wt, q_out = [oracle.qp(*q) for q in qsets[ci % len(qsets)]]
        y = ref.conv2d_q(x, w, Cout, kh, kw, q_in, q_wt, q_out, bias=bias, ph=ph, pw=pw, sh=sh, sw=sw)
        key = f"v{ci}"
        out[key + ".qp"] = np.array([[q.scale, q.zero_point] for q in (q_in, q_wt, q_out)], np.float64)
        out[key + ".x"] = x
        out[key + ".w"] = w
        if use_bias:
            out[key + ".bias"] = bias
        out[key + ".y"] = y
        out[key + ".col0"] = ref.im2col(x[0], kh, kw, ph, pw, sh, sw)
    np.savez_compressed(os.path.join(HERE, "conv2d.npz"), **out)
    print("conv2d.npz:", len(CONV_CASES), "cases")


if __name__ == "__main__":
    conv2d()
    helpers()
    qmm_small()
    fc_mlp()
    linear_1024()
