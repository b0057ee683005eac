"""CPU, world_size 2, gloo: the multi-rank logic of the row- and column-sharded quantized linear (partitioning, the
min/max all-reduce, the all-gather of column slices and its relayout) with the CPU oracle injected as the compute
backend.  No GPU is involved; the same module runs on GPUs with the CUDA backend and NCCL."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_covers_exactly():
    from ltq.sharded import shard_range
    for total in (1, 7, 64, 100, 4096, 11008, 65536):
        for world in (1, 2, 3, 4, 8):
            for mult in (1, 8, 16):
                blocks = [shard_range(total, r, world, mult) for r in range(world)]
                assert blocks[0][0] == 0 and blocks[-1][1] == total
                for (a, b), (c, d) in zip(blocks, blocks[1:]):
                    assert b == c and a <= b
                for (a, b) in blocks[:-1]:
                    assert (b - a) % mult == 0
                sizes = [b - a for a, b in blocks]
                assert max(sizes) - min(sizes) <= mult or total < mult * world


class OracleBackend:
    """Test stand-in for the CUDA backend: same interface, CPU oracle arithmetic."""

    def __init__(self, oracle):
        self.o = oracle

    def make_layer(self, w_q, bias_q, qp_in, qp_wt, qp_out):
        return dict(w=w_q.numpy(), b=None if bias_q is None else bias_q.numpy(), qps=(qp_in, qp_wt, qp_out))

    def forward(self, layer, x_q, out_mode, flags, out=None):
        import ltq
        qa, qw, qc = layer["qps"]
        M, K = x_q.shape
        N = layer["w"].shape[0]
        acc = self.o.port.acc_i32(x_q.numpy(), layer["w"], M, N, K, qa.zero_point, qw.zero_point, bias=layer["b"])
        relu = bool(flags & ltq.FLAG_RELU)
        if out_mode == ltq.OUT_U8:
            r = self.o.port.epilogue_u8(acc, qa.scale, qw.scale, qc.scale, qc.zero_point, relu=relu)
        elif out_mode == ltq.OUT_F32:
            r = self.o.port.epilogue_f32(acc, qa.scale, qw.scale, relu=relu)
        else:
            r = np.maximum(acc, 0) if relu else acc
        t = torch.from_numpy(np.ascontiguousarray(r))
        if out is not None:
            out.copy_(t)
            return out
        return t

    def min_max(self, x):
        mn, mx = self.o.port.get_min_max(x.numpy())
        return torch.tensor([mn, mx], dtype=torch.float32)

    def interleave(self, gathered, out):
        G, M, W = gathered.shape
        out.copy_(gathered.permute(1, 0, 2).reshape(M, G * W))
        return out


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, results):
    for p in (ROOT, os.path.join(ROOT, "light-tensor_b200", "python")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "1"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        import ltq
        from ltq import sharded
        be = OracleBackend(oracle)
        rng = np.random.default_rng(123)  # same stream on every rank: replicated inputs
        M, K, N = 48, 160, 64
        x = (rng.standard_normal((M, K)) * 2).astype(np.float32)
        w = rng.integers(0, 256, (N, K), dtype=np.uint8)
        bias = rng.integers(-3000, 3000, N, dtype=np.int32)
        qw, qo = ltq.QParams(0.01, 120), ltq.QParams(0.7, 99)

        # --- rows: dynamic activation quantisation needs the GLOBAL min/max ---
        r0, r1 = sharded.RowShardedLinear.my_rows(M)
        local_mm = be.min_max(torch.from_numpy(x[r0:r1].copy()))
        mm = sharded.global_min_max(local_mm)
        gmn, gmx = oracle.port.get_min_max(x)
        assert float(mm[0]) == float(gmn) and float(mm[1]) == float(gmx)
        oq = oracle.port.compute_qparams(mm[0].item(), mm[1].item())
        qx = ltq.QParams(oq.scale, oq.zero_point)
        xq = oracle.port.quantize_u8(x, oq)
        lin = sharded.RowShardedLinear(torch.from_numpy(w), torch.from_numpy(bias), qx, qw, qo, backend=be)
        mine = lin.forward(torch.from_numpy(xq[r0:r1].copy()), ltq.OUT_U8, ltq.FLAG_RELU)
        full, _ = oracle.port.quantized_matmul(xq, w, M, N, K, [oq, oracle.qp(qw.scale, qw.zero_point),
                                                               oracle.qp(qo.scale, qo.zero_point)], bias=bias)
        acc = oracle.port.acc_i32(xq, w, M, N, K, oq.zero_point, qw.zero_point, bias=bias)
        want = oracle.port.epilogue_u8(acc, oq.scale, qw.scale, qo.scale, qo.zero_point, relu=True)
        assert np.array_equal(mine.numpy(), want[r0:r1]), "row-sharded slice differs from the unsharded result"
        # the slices of all ranks tile the output exactly
        parts = [torch.empty((b - a, N), dtype=torch.uint8) for a, b in
                 (sharded.shard_range(M, r, world) for r in range(world))]
        dist.all_gather(parts, mine)
        assert np.array_equal(torch.cat(parts).numpy(), want)

        # --- columns: all-gather of output slices + relayout ---
        col = sharded.ColShardedLinear(torch.from_numpy(w), torch.from_numpy(bias), N, qx, qw, qo, backend=be)
        assert (col.n1 - col.n0) == N // world
        for mode, ref in ((ltq.OUT_U8, full), (ltq.OUT_I32, acc),
                          (ltq.OUT_F32, oracle.port.epilogue_f32(acc, oq.scale, qw.scale))):
            got = col.forward(torch.from_numpy(xq), mode, 0)
            assert tuple(got.shape) == (M, N)
            assert np.array_equal(got.numpy().view(np.uint8), np.ascontiguousarray(ref).view(np.uint8)), f"mode {mode}"
        # column sharding refuses slices that are not vector-aligned
        try:
            sharded.ColShardedLinear(torch.from_numpy(w[:40]), None, 40, qx, qw, qo, backend=be)
            raise AssertionError("N = 40 over 2 ranks must be rejected")
        except ValueError:
            pass
        results[rank] = "ok"
    except Exception as e:  # surface the failure in the parent
        import traceback
        results[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def test_row_and_column_sharding_world2_gloo():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for r in range(world):
        assert results.get(r) == "ok", results.get(r)


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(2, 64, 48, "u8"), (8, 33, 128, "u8"), (4, 100, 24, "f32"), (3, 7, 5, "u8"),
                                  (8, 1024, 4096, "u8")])
def test_interleave_kernel_matches_permute(cuda, case):
    import ltq
    from ltq import sharded
    G, M, W, kind = case
    if kind == "u8":
        g = cuda.randint(0, 256, (G, M, W), dtype=cuda.uint8, device="cuda")
    else:
        g = cuda.randn((G, M, W), device="cuda")
    out = cuda.empty((M, G * W), dtype=g.dtype, device="cuda")
    sharded.CudaBackend().interleave(g, out)
    assert cuda.equal(out, g.permute(1, 0, 2).reshape(M, G * W))
