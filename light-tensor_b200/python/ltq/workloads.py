"""Seeded synthetic inputs for the benchmark configurations of the quantized fully-connected path.

Generator convention: ``numpy.random.default_rng(seed)`` (PCG64); draw order activations, then per layer weights and
bias; "N(mu, sigma)" takes the standard deviation.  Only float32 / uint8 host arrays are produced here; whoever needs
quantized bytes quantizes them with the implementation under test (or, in the tests, with the oracle).
"""
import numpy as np


def mlp_mnist(seed=0, batch=64, dims=(784, 512, 512, 10)):
    """MNIST-shaped MLP: x U[0,1) [batch,784]; W_l N(0,0.05) [out,in]; b_l N(0,0.01)."""
    rng = np.random.default_rng(seed)
    x = rng.random((batch, dims[0]), dtype=np.float32)
    layers = []
    for i in range(len(dims) - 1):
        w = rng.normal(0.0, 0.05, (dims[i + 1], dims[i])).astype(np.float32)
        b = rng.normal(0.0, 0.01, (dims[i + 1],)).astype(np.float32)
        layers.append((w, b))
    return x, layers


def linear_u8(seed=2, M=1024, K=1024, N=1024):
    """Single quantized linear given directly in uint8: A U{0..255} z=128 s=0.02; W U{0..255} z=127 s=0.005;
    bias N(0,0.1) fp32."""
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 256, (M, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    b = rng.normal(0.0, 0.1, (N,)).astype(np.float32)
    return dict(a=a, w=w, bias=b, qp_a=(np.float32(0.02), 128), qp_w=(np.float32(0.005), 127))


def linear_f32(seed, M, K, N, w_std):
    """Activations N(0,1) fp32 [M,K], weights N(0,w_std) fp32 [N,K] (to be quantized per tensor by min/max)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(w_std)).astype(np.float32)
    return x, w


def square_4096(seed=3):
    return linear_f32(seed, 4096, 4096, 4096, 0.02)


def skinny(seed=4, M=16, K=4096, N=11008):
    return linear_f32(seed, M, K, N, 0.02)
