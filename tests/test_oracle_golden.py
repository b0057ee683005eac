"""CPU: the C restatement (oracle/ltq_oracle.c) against the fixtures generated from the unmodified reference, and
against the reference library itself when it has been built on this machine."""
import hashlib

import numpy as np
import pytest

from helpers import iter_qmm_cases, qp_of

HELPER_CASES = ["normal", "uniform01", "negative_only", "positive_offset", "wide", "tiny", "single", "ties"]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("name", HELPER_CASES)
def test_helpers_match_golden(oracle, golden, name):
    g = golden("helpers.npz")
    x = g[f"{name}.x"]
    mn, mx = oracle.port.get_min_max(x)
    assert [mn, mx] == list(g[f"{name}.minmax"])
    qp = oracle.port.compute_qparams(mn, mx)
    assert np.float32(qp.scale) == np.float32(g[f"{name}.qp"][0]) and qp.zero_point == int(g[f"{name}.qp"][1])
    q = oracle.port.quantize_u8(x, qp)
    np.testing.assert_array_equal(q, g[f"{name}.q"])
    np.testing.assert_array_equal(oracle.port.dequantize(q, qp), g[f"{name}.dq"])


def test_explicit_and_bias_quantize_match_golden(oracle, golden):
    g = golden("helpers.npz")
    qp = qp_of(oracle, g["explicit.qp"])
    np.testing.assert_array_equal(oracle.port.quantize_u8(g["explicit.x"], qp), g["explicit.q"])
    qpb = qp_of(oracle, g["bias.qp"])
    np.testing.assert_array_equal(oracle.port.quantize_i32(g["bias.x"], qpb), g["bias.q"])


def test_quantized_matmul_small_matches_golden(oracle, golden):
    g = golden("qmm_small.npz")
    n = 0
    for c in iter_qmm_cases(g):
        qps = [qp_of(oracle, r) for r in c["qp"]]
        C, ws = oracle.port.quantized_matmul(c["A"], c["B"], c["M"], c["N"], c["K"], qps, bias=c["bias"],
                                             tA=bool(c["tA"]), tB=bool(c["tB"]))
        np.testing.assert_array_equal(C, c["C"], err_msg=c["key"])
        np.testing.assert_array_equal(ws, c["ws"], err_msg=c["key"])
        # the factored form (acc + epilogue) used for the GPU parity checks gives the same bytes
        acc = oracle.port.acc_i32(c["A"], c["B"], c["M"], c["N"], c["K"], qps[0].zero_point, qps[1].zero_point,
                                  bias=c["bias"], tA=bool(c["tA"]), tB=bool(c["tB"]))
        C2 = oracle.port.epilogue_u8(acc, qps[0].scale, qps[1].scale, qps[2].scale, qps[2].zero_point)
        np.testing.assert_array_equal(C2, c["C"], err_msg=c["key"])
        n += 1
    assert n >= 100


def test_alpha_beta_rejected(oracle):
    A = np.zeros(4, np.uint8)
    qps = [oracle.qp(1, 0)] * 3
    with pytest.raises(ValueError):
        oracle.port.quantized_matmul(A, A, 2, 2, 2, qps, alpha=2)
    with pytest.raises(ValueError):
        oracle.port.quantized_matmul(A, A, 2, 2, 2, qps, beta=1)


def test_fc_mlp_matches_golden(oracle, golden):
    from ltq import workloads
    g = golden("fc_mlp.npz")
    x, layers = workloads.mlp_mnist(seed=0, batch=64)
    assert sha(x) == str(g["x_sha"]), "synthetic generator drifted from the committed fixture"
    q = g["x_q"]
    for li in range(3):
        qps = [qp_of(oracle, r) for r in g[f"l{li}.qp"]]
        w_q, b_q = g[f"l{li}.w_q"], g[f"l{li}.b_q"]
        N, K = w_q.shape
        # weights / bias quantisation restated from the fp32 tensors
        w, b = layers[li]
        np.testing.assert_array_equal(oracle.port.quantize_u8(w, qps[1]), w_q)
        np.testing.assert_array_equal(
            oracle.port.quantize_i32(b, oracle.qp(np.float32(qps[0].scale) * np.float32(qps[1].scale), 0)), b_q)
        y, _ = oracle.port.quantized_matmul(q, w_q, 64, N, K, qps, bias=b_q)
        np.testing.assert_array_equal(y, g[f"l{li}.y"])
        q = y
    np.testing.assert_array_equal(oracle.port.dequantize(q, qps[2]), g["logits"])


def test_linear_1024_matches_golden(oracle, golden):
    from ltq import workloads
    g = golden("linear_1024.npz")
    wl = workloads.linear_u8(seed=2)
    assert sha(wl["a"]) == str(g["a_sha"]) and sha(wl["w"]) == str(g["w_sha"])
    qa, qw = oracle.qp(*wl["qp_a"]), oracle.qp(*wl["qp_w"])
    bias_q = oracle.port.quantize_i32(wl["bias"], oracle.qp(np.float32(qa.scale) * np.float32(qw.scale), 0))
    np.testing.assert_array_equal(bias_q, g["bias_q"])
    acc = oracle.port.acc_i32(wl["a"], wl["w"], 1024, 1024, 1024, qa.zero_point, qw.zero_point, bias=bias_q)
    for i in range(4):
        sc, zc = g[f"o{i}.qp"]
        C = oracle.port.epilogue_u8(acc, qa.scale, qw.scale, np.float32(sc), int(zc))
        np.testing.assert_array_equal(C[::64], g[f"o{i}.rows"])
        assert sha(C) == str(g[f"o{i}.sha"])
    # the three byte planes stored by the reference reassemble the accumulator wherever it is non-negative
    planes = [oracle.port.epilogue_u8(acc, qa.scale, qw.scale, np.float32(g[f"o{i}.qp"][0]), 0).astype(np.int64)
              for i in (1, 2, 3)]
    pos = acc >= 0
    rebuilt = planes[0] + (planes[1] << 8) + (planes[2] << 16)
    np.testing.assert_array_equal(rebuilt[pos], acc[pos].astype(np.int64) & 0xFFFFFF)


def test_port_matches_reference_library_on_random_cases(oracle):
    """Direct port-vs-reference comparison; only where the reference library exists (it cannot travel without the
    reference sources having been compiled on this machine)."""
    if oracle.ref is None:
        pytest.skip("oracle/_ref/liblten_ref.so not built here")
    rng = np.random.default_rng(7)
    for _ in range(40):
        M, N, K = (int(v) for v in rng.integers(1, 70, 3))
        tA, tB = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        A = rng.integers(0, 256, M * K, dtype=np.uint8)
        B = rng.integers(0, 256, N * K, dtype=np.uint8)
        bias = rng.integers(-100000, 100000, N, dtype=np.int32) if rng.integers(0, 2) else None
        qps = [oracle.qp(np.float32(rng.uniform(0.001, 0.2)), int(rng.integers(0, 256))) for _ in range(3)]
        C1, w1 = oracle.port.quantized_matmul(A, B, M, N, K, qps, bias=bias, tA=tA, tB=tB)
        C2, w2 = oracle.ref.quantized_matmul(A, B, M, N, K, qps, bias=bias, tA=tA, tB=tB)
        np.testing.assert_array_equal(C1, C2)
        np.testing.assert_array_equal(w1, w2)
    x = (rng.standard_normal(5000) * 3).astype(np.float32)
    assert oracle.port.get_min_max(x) == oracle.ref.get_min_max(x)
    qp = oracle.ref.compute_qparams(*oracle.ref.get_min_max(x))
    qp2 = oracle.port.compute_qparams(*oracle.port.get_min_max(x))
    assert (qp.scale, qp.zero_point) == (qp2.scale, qp2.zero_point)
    np.testing.assert_array_equal(oracle.port.quantize_u8(x, qp), oracle.ref.quantize_u8(x, qp))
    np.testing.assert_array_equal(oracle.port.quantize_i32(x * 1e4, qp), oracle.ref.quantize_i32(x * 1e4, qp))


def test_saturate_and_relu_epilogues(oracle):
    acc = np.array([-1000, -1, 0, 1, 50, 255, 256, 1000, 2**31 - 1, -2**31], np.int32)
    wrap = oracle.port.epilogue_u8(acc, 1.0, 1.0, 1.0, 0)
    sat = oracle.port.epilogue_u8(acc, 1.0, 1.0, 1.0, 0, saturate=True)
    assert list(wrap[:8]) == [(-1000) & 255, 255, 0, 1, 50, 255, 0, 1000 & 255]
    assert list(sat[:8]) == [0, 0, 0, 1, 50, 255, 255, 255]
    assert wrap[8] == 0 and wrap[9] == 0  # |t| >= 2^31: the x86 conversion yields 0x80000000, low byte 0
    relu = oracle.port.epilogue_f32(acc, 0.5, 0.5, relu=True)
    assert relu[0] == 0 and relu[1] == 0 and relu[4] == np.float32(0.25) * np.float32(50)
