"""Calibration and quantisation set-up, the step in front of the quantized layers.

l-ten has no helper for this: its quantized test repeats ~100 lines per network (tests/nn_tests.cpp:538-608 for the
running statistics, :786-884 for the per-layer set-up).  This module packages exactly that recipe, computing on the
device through libltq:

* ``MinMaxObserver`` -- the test's ``blob_statistics`` + ``update_statistics``: running min / max of every tensor shown
  to it, seeded with +/-FLT_MAX, turned into QuantizationParams by ``ComputeQuantizationParams``;
* ``quantize_module`` -- weights -> ``GetMinMax`` -> ``ComputeQuantizationParams`` -> ``Quantize`` (uint8) written
  through ``get_all_weights()[0]``; bias -> int32 with scale ``s_in * s_wt`` and zero point 0 written through
  ``get_all_weights()[1]``; then ``set_qparams_in / set_qparams_out / set_qparams_params``.
"""
import numpy as np
import torch

from ._binding import QParams
from .ops import ComputeQuantizationParams, GetMinMax, Quantize, QuantizeInt32

FLT_MAX = float(np.finfo(np.float32).max)


class MinMaxObserver:
    """Running minimum / maximum over the tensors passed to ``update`` (tests/nn_tests.cpp:538-587)."""

    def __init__(self):
        self.min = FLT_MAX
        self.max = -FLT_MAX

    def update(self, x):
        """x: float32 CUDA tensor of any shape.  Reads two floats back from the device (calibration is off the hot path)."""
        mn, mx = GetMinMax(x.contiguous().view(-1)).tolist()
        self.min = min(self.min, mn)
        self.max = max(self.max, mx)
        return x

    def qparams(self):
        if self.min > self.max:
            raise ValueError("the observer has not seen any data")
        return ComputeQuantizationParams(self.min, self.max)


def quantize_module(q_mod, weight, bias, qp_in, qp_out):
    """Fill a freshly ``init()``-ed quantized module (FullyConnected_q or Conv2d_q) from float parameters held on a CUDA
    device, the way tests/nn_tests.cpp:808-834 does for each layer.  Returns the weight QuantizationParams.
    The module's tensors are still on the CPU at this point (call ``to("cuda", idx)`` afterwards, as the reference's
    flow does)."""
    tensors = q_mod.get_all_weights()
    wf = weight.contiguous().view(-1).float()
    qp_wt = ComputeQuantizationParams(*GetMinMax(wf).tolist())
    wq = Quantize(wf, qp_wt)
    tensors[0].copy_(wq.view(tensors[0].shape).to(tensors[0].device))
    qps = [qp_wt]
    if len(tensors) > 1:
        if bias is None:
            raise ValueError("the module uses a bias but none was given")
        # arXiv:1712.05877: the bias shares the accumulator's scale, s_in * s_wt, with zero point 0 (nn_tests.cpp:824-826)
        qp_b = QParams(float(np.float32(qp_in.scale) * np.float32(qp_wt.scale)), 0)
        bq = QuantizeInt32(bias.contiguous().view(-1).float(), qp_b)
        tensors[1].copy_(bq.view(tensors[1].shape).to(tensors[1].device))
        qps.append(qp_b)
    q_mod.set_qparams_in(qp_in)
    q_mod.set_qparams_out(qp_out)
    q_mod.set_qparams_params(qps, len(qps))
    return qp_wt


def calibrate(forward_with_taps, batches):
    """Runs ``forward_with_taps(batch)`` -- a float32 forward pass that returns the list of tensors to observe (input
    first, then every layer output, as ``Net::forward`` does with ``layer_stats`` in tests/nn_tests.cpp:589-608) -- over
    all batches and returns one QuantizationParams per tap."""
    observers = None
    with torch.no_grad():
        for b in batches:
            taps = forward_with_taps(b)
            if observers is None:
                observers = [MinMaxObserver() for _ in taps]
            for o, t in zip(observers, taps):
                o.update(t)
    if observers is None:
        raise ValueError("no calibration batches")
    return [o.qparams() for o in observers]
