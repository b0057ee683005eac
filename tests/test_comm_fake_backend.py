"""CPU: the multi-device group of the C ABI (ltq_comm_*) against a fake communication backend.

No GPU and no NCCL are involved: the library lets tests replace NCCL and the CUDA streams by a table of callbacks
(``ltq_comm_set_backend``), and a group created while a fake is installed makes no CUDA call at all.  Covered here: the
argument checks, the routing of the min/max all-reduce through one group, and the host-side watchdog of
``ltq_comm_synchronize`` -- a communicator that reports an asynchronous error, and streams that never drain within the
time limit, both end with every communicator aborted and a status code instead of a hang."""
import ctypes as C
import time

import pytest

import ltq
from ltq._binding import lib


class Backend(C.Structure):
    _fields_ = [
        ("comm_init_all", C.CFUNCTYPE(C.c_int, C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_int))),
        ("comm_destroy", C.CFUNCTYPE(C.c_int, C.c_void_p)),
        ("comm_abort", C.CFUNCTYPE(C.c_int, C.c_void_p)),
        ("comm_get_async_error", C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_int))),
        ("all_gather", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p)),
        ("all_reduce_f32", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_int, C.c_void_p, C.c_void_p)),
        ("group_start", C.CFUNCTYPE(C.c_int)),
        ("group_end", C.CFUNCTYPE(C.c_int)),
        ("stream_create", C.CFUNCTYPE(C.c_int, C.c_int, C.POINTER(C.c_void_p))),
        ("stream_destroy", C.CFUNCTYPE(C.c_int, C.c_int, C.c_void_p)),
        ("stream_query", C.CFUNCTYPE(C.c_int, C.c_int, C.c_void_p)),
        ("error_string", C.CFUNCTYPE(C.c_void_p, C.c_int)),
    ]


class Fake:
    """Records what the library asks of the backend; `busy` and `async_error` steer the watchdog."""

    def __init__(self):
        self.log, self.busy, self.async_error, self.init_rc = [], False, {}, 0
        self._msg = C.create_string_buffer(b"fake error")
        f = dict(Backend._fields_)

        def init_all(comms, ndev, devices):
            self.log.append(("init", [devices[i] for i in range(ndev)]))
            for i in range(ndev):
                comms[i] = 0x1000 + devices[i]
            return self.init_rc

        def get_async(comm, out):
            out[0] = self.async_error.get(comm, 0)
            return 0

        def stream_create(device, out):
            out[0] = 0x2000 + device
            return 0

        self.table = Backend(
            f["comm_init_all"](init_all),
            f["comm_destroy"](lambda c: self.log.append(("destroy", c)) or 0),
            f["comm_abort"](lambda c: self.log.append(("abort", c)) or 0),
            f["comm_get_async_error"](get_async),
            f["all_gather"](lambda s, r, n, c, st: self.log.append(("all_gather", n, c, st)) or 0),
            f["all_reduce_f32"](lambda s, r, n, op, c, st: self.log.append(("all_reduce", s, op, c, st)) or 0),
            f["group_start"](lambda: self.log.append(("group_start",)) or 0),
            f["group_end"](lambda: self.log.append(("group_end",)) or 0),
            f["stream_create"](stream_create),
            f["stream_destroy"](lambda d, s: self.log.append(("stream_destroy", d)) or 0),
            f["stream_query"](lambda d, s: 1 if self.busy else 0),
            f["error_string"](lambda code: C.addressof(self._msg)),
        )


@pytest.fixture
def fake():
    fk = Fake()
    assert lib().ltq_comm_set_backend(C.byref(fk.table)) == 0
    yield fk
    assert lib().ltq_comm_set_backend(None) == 0


def _group(devices):
    h = C.c_void_p()
    arr = (C.c_int * len(devices))(*devices)
    rc = lib().ltq_comm_init_all(C.byref(h), len(devices), arr)
    return rc, h


def test_group_lifecycle_and_argument_checks(fake):
    L = lib()
    rc, h = _group([0, 1, 2, 3])
    assert rc == 0 and L.ltq_comm_size(h) == 4
    assert [L.ltq_comm_device(h, i) for i in range(5)] == [0, 1, 2, 3, -1]
    assert L.ltq_comm_stream(h, 2) == 0x2002 and L.ltq_comm_stream(h, 4) is None
    assert fake.log[0] == ("init", [0, 1, 2, 3])
    assert L.ltq_comm_synchronize(h, 100) == 0                       # idle streams: returns at once
    assert L.ltq_comm_destroy(h) == 0
    assert [e for e in fake.log if e[0] == "destroy"] == [("destroy", 0x1000 + d) for d in range(4)]
    assert [e for e in fake.log if e[0] == "stream_destroy"] == [("stream_destroy", d) for d in range(4)]
    # bad arguments
    assert _group([])[0] == -1 and _group(list(range(9)))[0] == -1
    rc, _ = _group([0, 1, 1])
    assert rc == -1 and "twice" in ltq.last_error()
    fake.init_rc = 5
    rc, _ = _group([0, 1])
    assert rc == -3 and "fake error" in ltq.last_error()
    assert L.ltq_comm_synchronize(None, 0) == -1 and L.ltq_comm_destroy(None) == 0


def test_minmax_allreduce_goes_out_as_one_group(fake):
    L = lib()
    rc, h = _group([0, 1])
    bufs = (C.c_void_p * 2)(0x9000, 0xA000)
    assert L.ltq_comm_allreduce_minmax(h, bufs) == 0
    ops = [e for e in fake.log if e[0] in ("group_start", "group_end", "all_reduce")]
    assert ops[0] == ("group_start",) and ops[-1] == ("group_end",) and len(ops) == 6
    # min on element 0, max on element 1 (4 bytes further), each on its device's communicator and stream
    assert ops[1] == ("all_reduce", 0x9000, 0, 0x1000, 0x2000) and ops[2] == ("all_reduce", 0x9004, 1, 0x1000, 0x2000)
    assert ops[3] == ("all_reduce", 0xA000, 0, 0x1001, 0x2001) and ops[4] == ("all_reduce", 0xA004, 1, 0x1001, 0x2001)
    assert L.ltq_comm_allreduce_minmax(h, None) == -1
    L.ltq_comm_destroy(h)
    # a group of one has nothing to exchange
    rc, h1 = _group([3])
    n = len(fake.log)
    assert L.ltq_comm_allreduce_minmax(h1, (C.c_void_p * 1)(0x9000)) == 0 and len(fake.log) == n
    L.ltq_comm_destroy(h1)


def test_sharded_forwards_reject_missing_arguments(fake):
    L = lib()
    rc, h = _group([0, 1])
    two = (C.c_void_p * 2)(None, None)
    rows = (C.c_uint64 * 2)(4, 4)
    assert L.ltq_linear_forward_rowsharded(h, None, two, None, rows, None, 0, 0, two) == -1
    assert L.ltq_linear_forward_rowsharded(h, two, two, None, rows, None, 0, 0, two) == -1      # NULL layers
    assert L.ltq_linear_forward_colsharded_allgather(h, two, two, None, 8, None, 0, 0, two, two, two) == -1
    assert L.ltq_linear_forward_colsharded_allgather(h, two, two, None, 8, None, 7, 0, two, two, two) == -1
    L.ltq_comm_destroy(h)


def test_watchdog_aborts_on_timeout(fake):
    L = lib()
    rc, h = _group([0, 1, 2])
    fake.busy = True                                                    # streams that never drain
    t0 = time.time()
    assert L.ltq_comm_synchronize(h, 150) == -4                         # LTQ_ERR_DEVICE_TIMEOUT
    assert 0.14 < time.time() - t0 < 2.0
    assert "150 ms" in ltq.last_error()
    assert [e for e in fake.log if e[0] == "abort"] == [("abort", 0x1000 + d) for d in range(3)]
    # an aborted group refuses further work and does not destroy its communicators a second time
    assert L.ltq_comm_synchronize(h, 10) == -3 and "aborted" in ltq.last_error()
    assert L.ltq_comm_allreduce_minmax(h, (C.c_void_p * 3)(1, 2, 3)) == -3
    L.ltq_comm_destroy(h)
    assert not [e for e in fake.log if e[0] == "destroy"]


def test_watchdog_aborts_on_asynchronous_error(fake):
    L = lib()
    rc, h = _group([0, 1])
    fake.busy = True
    fake.async_error = {0x1001: 6}                                      # device 1's communicator has failed
    t0 = time.time()
    assert L.ltq_comm_synchronize(h, 0) == -3                           # no time limit needed: the error ends the wait
    assert time.time() - t0 < 1.0
    assert "device 1" in ltq.last_error() and "fake error" in ltq.last_error()
    assert [e for e in fake.log if e[0] == "abort"] == [("abort", 0x1000), ("abort", 0x1001)]
    L.ltq_comm_destroy(h)


def test_incomplete_backend_is_rejected():
    t = Backend()
    assert lib().ltq_comm_set_backend(C.byref(t)) == -1
    assert lib().ltq_comm_set_backend(None) == 0
