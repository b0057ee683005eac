"""GPU: the C++ host side (light-tensor_b200/host: lten::Tensor subset, lten::FullyConnected_q, lten::Conv2d_q, the free quantisation
functions) driving libltq.  The test program is C++ and reads like l-ten's own quantized test; it compares every layer
output with the CPU oracle and exercises the layer's argument checks."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "light-tensor_b200", "host", "build", "test_fc_q")
BIN_CONV = os.path.join(ROOT, "light-tensor_b200", "host", "build", "test_conv_q")


def test_host_library_and_test_program_are_built():
    assert os.path.exists(os.path.join(ROOT, "light-tensor_b200", "host", "build", "liblten_q.so")), \
        "build with `make -C light-tensor_b200/host` (done by __graft_entry__.build())"
    assert os.path.exists(BIN) and os.path.exists(BIN_CONV)


@pytest.mark.gpu
def test_cpp_quantized_mlp_matches_oracle(cuda):
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "PASS" in r.stdout


@pytest.mark.gpu
def test_cpp_quantized_conv_net_matches_oracle(cuda):
    """Conv2d_q(1 -> 10, 5 x 5) + two FullyConnected_q, the network of the reference's quantized convolution test."""
    r = subprocess.run([BIN_CONV], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "PASS" in r.stdout
