"""Checkpoint I/O for quantized modules.

l-ten's ``NeuralNetwork::save_checkpoint / load_checkpoint`` (l-ten/net.h:130-265) write the raw bytes of every
parameter back to back assuming four bytes per element and nothing else, which neither fits uint8 weights nor keeps the
quantisation parameters a quantized layer cannot run without.  The format here carries both; the C++ host side
(light-tensor_b200/host) reads and writes the same bytes.

Layout (little endian)::

    "LTQCKPT1"                                   8 bytes
    uint32 modules
    per module:
        uint32 tensors                           get_all_weights() order: weights, then bias
        per tensor: uint8 dtype (0 uint8, 1 int32, 2 float32), uint8[3] zero, uint32 ndims, uint64 dims[ndims], raw data
        3 x { float32 scale, uint8 zero_point, uint8[3] zero }     input, weights, output QuantizationParams
"""
import struct

import numpy as np
import torch

from ._binding import QParams

MAGIC = b"LTQCKPT1"
_CODES = {torch.uint8: 0, torch.int32: 1, torch.float32: 2}
_NP = {0: np.uint8, 1: np.int32, 2: np.float32}


def save_checkpoint(modules, checkpoint_path):
    """modules: FullyConnected_q / Conv2d_q objects (anything with get_all_weights() and the three qparams_*_ fields),
    on any device.  Returns 0 like the reference's method."""
    with open(checkpoint_path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<I", len(modules)))
        for m in modules:
            tensors = m.get_all_weights()
            f.write(struct.pack("<I", len(tensors)))
            for t in tensors:
                f.write(struct.pack("<B3xI", _CODES[t.dtype], t.dim()))
                f.write(struct.pack(f"<{t.dim()}Q", *t.shape))
                f.write(t.detach().cpu().contiguous().numpy().tobytes())
            for q in (m.qparams_in_, m.qparams_wt_, m.qparams_out_):
                f.write(struct.pack("<fB3x", q.scale, q.zero_point))
    return 0


def load_checkpoint(modules, checkpoint_path):
    """Fills already constructed and ``init()``-ed modules (shapes and dtypes must match the file; tensors may already
    live on a GPU) and sets their quantisation parameters.  Raises ValueError on any mismatch."""
    with open(checkpoint_path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError("not a quantized checkpoint")
        (n,) = struct.unpack("<I", f.read(4))
        if n != len(modules):
            raise ValueError(f"checkpoint holds {n} modules, {len(modules)} were given")
        for mi, m in enumerate(modules):
            tensors = m.get_all_weights()
            (nt,) = struct.unpack("<I", f.read(4))
            if nt != len(tensors):
                raise ValueError(f"module {mi}: checkpoint holds {nt} tensors, the module has {len(tensors)}")
            for t in tensors:
                code, nd = struct.unpack("<B3xI", f.read(8))
                dims = struct.unpack(f"<{nd}Q", f.read(8 * nd))
                if code != _CODES[t.dtype] or tuple(dims) != tuple(t.shape):
                    raise ValueError(f"module {mi}: tensor mismatch (file dtype {code} dims {dims}, module {t.dtype} "
                                     f"{tuple(t.shape)})")
                count = int(np.prod(dims)) if nd else 1
                raw = f.read(count * np.dtype(_NP[code]).itemsize)
                if len(raw) != count * np.dtype(_NP[code]).itemsize:
                    raise ValueError("truncated checkpoint")
                t.copy_(torch.from_numpy(np.frombuffer(raw, dtype=_NP[code]).reshape(dims).copy()))
            qs = []
            for _ in range(3):
                s, z = struct.unpack("<fB3x", f.read(8))
                qs.append(QParams(s, z))
            m.set_qparams_in(qs[0])
            m.set_qparams_params([qs[1]], 1)
            m.set_qparams_out(qs[2])
            if getattr(m, "_handle", None) is not None:   # already on a GPU: the cached weight sums must follow the new bytes
                m._handle.set_weights(m.weight_ptr_, m.bias_ptr_)
    return 0
