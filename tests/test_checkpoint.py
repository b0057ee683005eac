"""CPU: quantized checkpoint I/O (weights uint8, bias int32, three QuantizationParams per module) through the Python
mirror, and agreement with the file the C++ host side writes."""
import os
import subprocess

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP_WRITER = os.path.join(ROOT, "light-tensor_b200", "host", "build", "test_checkpoint")


def _modules(seed, fill=True):
    import ltq
    rng = np.random.default_rng(seed)
    conv = ltq.Conv2d_q(2, 5, True, 3, 3, 1, 1)
    fc = ltq.FullyConnected_q(20, 7, True)
    fc2 = ltq.FullyConnected_q(7, 3, False)
    mods = [conv, fc, fc2]
    for m in mods:
        m.init()
        if fill:
            for t in m.get_all_weights():
                if t.dtype == torch.uint8:
                    t.copy_(torch.from_numpy(rng.integers(0, 256, tuple(t.shape), dtype=np.uint8)))
                else:
                    t.copy_(torch.from_numpy(rng.integers(-10**6, 10**6, tuple(t.shape), dtype=np.int32)))
            m.set_qparams_in(ltq.QParams(float(rng.uniform(0.001, 1)), int(rng.integers(0, 256))))
            m.set_qparams_out(ltq.QParams(float(rng.uniform(0.001, 1)), int(rng.integers(0, 256))))
            m.set_qparams_params([ltq.QParams(float(rng.uniform(0.001, 1)), int(rng.integers(0, 256)))], 1)
    return mods


def _same(a, b):
    for ma, mb in zip(a, b):
        for ta, tb in zip(ma.get_all_weights(), mb.get_all_weights()):
            assert ta.dtype == tb.dtype and torch.equal(ta, tb)
        for name in ("qparams_in_", "qparams_wt_", "qparams_out_"):
            qa, qb = getattr(ma, name), getattr(mb, name)
            assert (np.float32(qa.scale), qa.zero_point) == (np.float32(qb.scale), qb.zero_point), name


def test_round_trip(tmp_path):
    import ltq
    src = _modules(1)
    path = str(tmp_path / "q.ckpt")
    assert ltq.save_checkpoint(src, path) == 0
    dst = _modules(2, fill=False)
    assert ltq.load_checkpoint(dst, path) == 0
    _same(src, dst)
    # 1 byte per uint8 weight, 4 per int32 bias element, nothing else of size
    payload = sum(t.numel() * t.element_size() for m in src for t in m.get_all_weights())
    assert payload < os.path.getsize(path) < payload + 400


def test_mismatches_are_refused(tmp_path):
    import ltq
    src = _modules(3)
    path = str(tmp_path / "q.ckpt")
    ltq.save_checkpoint(src, path)
    with pytest.raises(ValueError, match="modules"):
        ltq.load_checkpoint(_modules(4, fill=False)[:2], path)
    other = _modules(5, fill=False)
    other[1] = ltq.FullyConnected_q(21, 7, True)
    other[1].init()
    with pytest.raises(ValueError, match="tensor mismatch"):
        ltq.load_checkpoint(other, path)
    with open(path, "r+b") as f:
        f.write(b"XXXX")
    with pytest.raises(ValueError, match="not a quantized checkpoint"):
        ltq.load_checkpoint(_modules(6, fill=False), path)
    with open(str(tmp_path / "short.ckpt"), "wb") as f:
        f.write(open(path, "rb").read()[:60].replace(b"XXXX", b"LTQC"))
    with pytest.raises(Exception):
        ltq.load_checkpoint(_modules(7, fill=False), str(tmp_path / "short.ckpt"))


def test_python_reads_what_the_cpp_host_writes(tmp_path):
    """The C++ program builds Conv2d_q(2 -> 5, 3 x 3, bias) + FullyConnected_q(20 -> 7, bias) + FullyConnected_q(7 -> 3)
    on the CPU, fills them from a fixed recipe (byte i of a tensor = (7 * i + tensor index) mod 251, int32 element i =
    1000 * i - 7 * tensor index), saves, reloads into fresh modules and compares; Python then reads the same file."""
    if not os.path.exists(CPP_WRITER):
        pytest.skip("C++ host side not built")
    import ltq
    path = str(tmp_path / "cpp.ckpt")
    r = subprocess.run([CPP_WRITER, path], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
    mods = _modules(8, fill=False)
    ltq.load_checkpoint(mods, path)
    ti = 0
    for mi, m in enumerate(mods):
        for t in m.get_all_weights():
            n = t.numel()
            if t.dtype == torch.uint8:
                want = ((7 * np.arange(n) + ti) % 251).astype(np.uint8)
            else:
                want = (1000 * np.arange(n) - 7 * ti).astype(np.int32)
            np.testing.assert_array_equal(t.numpy().ravel(), want)
            ti += 1
        assert (m.qparams_in_.zero_point, m.qparams_wt_.zero_point, m.qparams_out_.zero_point) == (10 + mi, 20 + mi, 30 + mi)
        assert np.float32(m.qparams_wt_.scale) == np.float32(0.5) / np.float32(mi + 1)
