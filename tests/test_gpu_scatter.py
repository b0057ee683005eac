"""GPU: the multi-destination epilogue (ltq_layer_forward_scatter) and the fused column-sharded linear built on it.

* one process: several destination buffers on the same GPU, with a row pitch wider than the layer and a column offset,
  on every kernel path, against the dense result;
* two processes (gloo for the rendezvous, one or two GPUs, whatever the box has): each rank owns half of the output
  columns and stores them straight into both ranks' buffers through CUDA IPC mappings; every rank then holds the full
  unsharded result.  No kernel waits on another one, so both ranks may share one GPU."""
import os
import socket
import sys

import numpy as np
import pytest

from helpers import ltq_qp, qp_of

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("path,shape", [
    ("simt", (33, 48, 100)), ("tc", (200, 272, 256)), ("tcpair", (300, 512, 128)), ("skinny", (5, 160, 256)),
    ("auto", (64, 96, 784)),
    # pair kernel with several tile widths: with more than one destination the stores go through the row-coalescing
    # stage in shared memory (full 32-row groups) or directly (the ragged last row tile)
    ("tcpair", (2000, 2160, 64)), ("tcpair", (2048, 2016, 64)), ("tcpair", (1100, 2304, 64)),
])
@pytest.mark.parametrize("mode", ["u8", "f32"])
def test_scatter_writes_every_destination_at_the_offset(cuda, oracle, path, shape, mode):
    import ltq
    M, N, K = shape
    force = {"simt": ltq.FLAG_FORCE_SIMT, "tc": ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_SINGLE,
             "tcpair": ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR, "skinny": ltq.FLAG_FORCE_SKINNY, "auto": 0}[path]
    out_mode, dt = (ltq.OUT_U8, cuda.uint8) if mode == "u8" else (ltq.OUT_F32, cuda.float32)
    rng = np.random.default_rng(M + N + K)
    x = rng.integers(0, 256, (M, K), dtype=np.uint8)
    w = rng.integers(0, 256, (N, K), dtype=np.uint8)
    b = rng.integers(-9000, 9000, N, dtype=np.int32)
    rows = [(0.02, 128), (0.005, 127), (0.8, 9)]
    h = ltq.LayerHandle(0, K, N)
    h.set_weights(cuda.from_numpy(w).cuda(), cuda.from_numpy(b).cuda())
    h.set_qparams(*[ltq_qp(r) for r in rows])
    xd = cuda.from_numpy(x).cuda()
    dense = h.forward(xd, out_mode, force)
    for ld, off in ((N + 32, 16), (2 * N, N), (N + 7, 3)):     # aligned (vector stores) and unaligned (scalar stores)
        sentinel = 77
        bufs = [cuda.full((M, ld), sentinel, dtype=dt, device="cuda") for _ in range(3)]
        h.forward_scatter(xd, [t.data_ptr() for t in bufs], ld, off, out_mode, force)
        cuda.cuda.synchronize()
        for t in bufs:
            assert cuda.equal(t[:, off:off + N], dense), (path, ld, off)
            assert bool((t[:, :off] == sentinel).all()) and bool((t[:, off + N:] == sentinel).all()), "wrote outside its columns"
    # and the dense result itself is the reference's
    if mode == "u8":
        want, _ = oracle.port.quantized_matmul(x, w, M, N, K, [qp_of(oracle, r) for r in rows], bias=b)
        np.testing.assert_array_equal(dense.cpu().numpy(), want)
    with pytest.raises(ltq.LtqError):
        h.forward_scatter(xd, [dense.data_ptr()], N, 1, out_mode, force)   # does not fit in the row


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _fused_worker(rank, world, port, results):
    for p in (ROOT, os.path.join(ROOT, "light-tensor_b200", "python")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        import ltq
        from ltq import sharded
        dev = rank % torch.cuda.device_count()
        torch.cuda.set_device(dev)
        rng = np.random.default_rng(77)   # same stream on every rank: replicated inputs
        M, K, N = 160, 256, 512
        w = rng.integers(0, 256, (N, K), dtype=np.uint8)
        bias = rng.integers(-3000, 3000, N, dtype=np.int32)
        rows = [(0.02, 128), (0.005, 127), (0.9, 12)]
        qps = [ltq.QParams(float(np.float32(s)), z) for s, z in rows]
        oqs = [oracle.qp(np.float32(s), z) for s, z in rows]
        col = sharded.ColShardedLinear(torch.from_numpy(w).cuda(), torch.from_numpy(bias).cuda(), N, *qps, fused=True,
                                       max_rows=M, out_mode=ltq.OUT_U8)
        plain = sharded.ColShardedLinear(torch.from_numpy(w).cuda(), torch.from_numpy(bias).cuda(), N, *qps)
        for it in range(5):               # more iterations than buffers: exercises the alternation
            x = rng.integers(0, 256, (M - 16 * (it % 2), K), dtype=np.uint8)
            got = col.forward(torch.from_numpy(x).cuda(), ltq.OUT_U8, 0)
            torch.cuda.synchronize()
            want, _ = oracle.port.quantized_matmul(x, w, x.shape[0], N, K, oqs, bias=bias)
            assert np.array_equal(got.cpu().numpy(), want), f"rank {rank} iteration {it}: fused result differs"
            local = plain.layer.forward(torch.from_numpy(x).cuda(), ltq.OUT_U8, 0)
            assert np.array_equal(local.cpu().numpy(), want[:, plain.n0:plain.n1])
            dist.barrier()
        results[rank] = "ok"
    except Exception:
        import traceback
        results[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def test_fused_column_sharding_two_ranks_over_ipc(cuda):
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_fused_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for r in range(world):
        assert results.get(r) == "ok", results.get(r)


def _multicast_worker(rank, world, port, results):
    for p in (ROOT, os.path.join(ROOT, "light-tensor_b200", "python")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(rank), str(world)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import oracle
        import ltq
        from ltq import sharded
        rng = np.random.default_rng(78)   # same stream on every rank: replicated inputs
        M, K, N = 1100, 256, 1024         # more than 16 rows: tensor-core kernels; 1100 leaves a ragged last row block
        w = rng.integers(0, 256, (N, K), dtype=np.uint8)
        bias = rng.integers(-3000, 3000, N, dtype=np.int32)
        rows = [(0.02, 128), (0.005, 127), (0.9, 12)]
        qps = [ltq.QParams(float(np.float32(s)), z) for s, z in rows]
        oqs = [oracle.qp(np.float32(s), z) for s, z in rows]
        for mode, pair in ((ltq.OUT_U8, False), (ltq.OUT_F32, False), (ltq.OUT_U8, True)):
            col = sharded.ColShardedLinear(torch.from_numpy(w).cuda(), torch.from_numpy(bias).cuda(), N, *qps, fused=True,
                                           max_rows=M, out_mode=mode, multicast=True)
            used = col.multicast
            flags = (ltq.FLAG_FORCE_TC | ltq.FLAG_FORCE_TC_PAIR) if pair else 0
            for it in range(4):
                x = rng.integers(0, 256, (M - 40 * (it % 2), K), dtype=np.uint8)
                got = col.forward(torch.from_numpy(x).cuda(), mode, flags)
                torch.cuda.synchronize()
                acc = oracle.port.acc_i32(x, w, x.shape[0], N, K, 128, 127, bias=bias)
                want = (oracle.port.epilogue_u8(acc, 0.02, 0.005, 0.9, 12) if mode == ltq.OUT_U8
                        else oracle.port.epilogue_f32(acc, 0.02, 0.005))
                g = got.cpu().numpy()
                assert np.array_equal(g.view(np.uint32) if mode == ltq.OUT_F32 else g,
                                      want.view(np.uint32) if mode == ltq.OUT_F32 else want), \
                    f"rank {rank} mode {mode} pair {pair} iteration {it}: result differs (multicast={used})"
                dist.barrier()
            col.close()
        results[rank] = "ok multicast" if used else "ok peer stores"
    except Exception:
        import traceback
        results[rank] = traceback.format_exc()
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


def test_fused_column_sharding_through_an_nvlink_multicast_address(cuda):
    """Two ranks on two GPUs (skipped with fewer): the fused exchange with every rank's columns stored ONCE to a multicast
    address that NVSwitch replicates into both ranks' buffers.  Where the system offers no multicast the same code falls
    back to peer stores and the result must be the same."""
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_multicast_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for r in range(world):
        assert str(results.get(r)).startswith("ok"), results.get(r)
    print("multicast test:", dict(results))
