"""One host thread driving several GPUs through the C ABI's multi-device entry points (``ltq_comm_*``,
``ltq_linear_forward_rowsharded``, ``ltq_linear_forward_colsharded_allgather``): the single-process counterpart of
``ltq.sharded`` (which runs one process per GPU over ``torch.distributed``).  This is the model of l-ten itself: a
single-threaded API with a device index per tensor (l-ten/globals.h:15,89-124)."""
import ctypes as C

import torch

from ._binding import OUT_F32, OUT_I32, OUT_U8, LtqError, check, lib

_OUT_DTYPE = {OUT_U8: torch.uint8, OUT_F32: torch.float32, OUT_I32: torch.int32}


def _ptr_array(items):
    return (C.c_void_p * len(items))(*[None if i is None else (i if isinstance(i, int) else i.data_ptr()) for i in items])


class DeviceGroup:
    """``ltq_comm``: one NCCL communicator and one stream per device.  ``devices``: list of CUDA device indices."""

    def __init__(self, devices):
        self.devices = list(devices)
        self._h = C.c_void_p()
        arr = (C.c_int * len(self.devices))(*self.devices)
        check(lib().ltq_comm_init_all(C.byref(self._h), len(self.devices), arr))
        self.streams = [torch.cuda.ExternalStream(lib().ltq_comm_stream(self._h, i), device=d)
                        for i, d in enumerate(self.devices)]

    def close(self):
        if self._h:
            lib().ltq_comm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self):
        return len(self.devices)

    def wait_for_current_streams(self):
        """Orders the group's streams after whatever the caller's current streams have enqueued so far."""
        for d, s in zip(self.devices, self.streams):
            s.wait_stream(torch.cuda.current_stream(d))

    def synchronize(self, timeout_ms=0):
        check(lib().ltq_comm_synchronize(self._h, timeout_ms))

    def allreduce_minmax(self, minmax):
        """minmax: one 2-element float32 tensor per device; replaced in place by the global {min, max}."""
        check(lib().ltq_comm_allreduce_minmax(self._h, _ptr_array(minmax)))

    def forward_rowsharded(self, layers, xs, out_mode=OUT_U8, flags=0, asums=None, qp_in_devs=None, outs=None):
        """layers: one LayerHandle per device (full weights each); xs: that device's rows, uint8 [rows_d, K]."""
        n = len(self.devices)
        rows = [x.numel() // layers[0].K for x in xs]
        if outs is None:
            outs = [torch.empty((rows[i], layers[i].N), dtype=_OUT_DTYPE[out_mode], device=xs[i].device) for i in range(n)]
        check(lib().ltq_linear_forward_rowsharded(
            self._h, _ptr_array([l._h.value for l in layers]), _ptr_array(xs),
            None if asums is None else _ptr_array(asums), (C.c_uint64 * n)(*rows),
            None if qp_in_devs is None else _ptr_array(qp_in_devs), out_mode, flags, _ptr_array(outs)))
        return outs

    def forward_colsharded(self, layers, xs, out_mode=OUT_U8, flags=0, asums=None, qp_in_devs=None, outs=None,
                           locals_=None, gathered=None):
        """layers: one LayerHandle per device holding that device's slice of the weight rows (equal slices);
        xs: the full activations on every device, uint8 [M, K].  Returns the full [M, N] output on every device."""
        n = len(self.devices)
        M = xs[0].numel() // layers[0].K
        nloc = layers[0].N
        dt = _OUT_DTYPE[out_mode]
        if outs is None:
            outs = [torch.empty((M, nloc * n), dtype=dt, device=x.device) for x in xs]
        if locals_ is None:
            locals_ = [torch.empty((M, nloc), dtype=dt, device=x.device) for x in xs]
        if gathered is None:
            gathered = [torch.empty((n, M, nloc), dtype=dt, device=x.device) for x in xs]
        check(lib().ltq_linear_forward_colsharded_allgather(
            self._h, _ptr_array([l._h.value for l in layers]), _ptr_array(xs),
            None if asums is None else _ptr_array(asums), M, None if qp_in_devs is None else _ptr_array(qp_in_devs),
            out_mode, flags, _ptr_array(locals_), _ptr_array(gathered), _ptr_array(outs)))
        self._keep = (locals_, gathered)
        return outs
