"""One-process-per-GPU sharding of the quantized linear path over ``torch.distributed``.

Two partitionings, both exact (per-tensor quantisation parameters make output rows and columns independent):

* rows (M): each rank owns a contiguous block of activation rows and a full replica of the weights.  No data-path
  collective.  Only dynamic activation quantisation needs one exchange: the per-tensor min/max must be the GLOBAL one
  for the sharded result to equal the single-device result, which is two 4-byte all-reduces (MIN, MAX).
* columns (N): each rank owns a contiguous block of weight rows (output features) with their bias / row sums and sees
  the full activations.  It produces ``out[:, n0:n1]``; an all-gather (NCCL over NVLink on GPUs) collects the slices
  as ``[world][M][N/world]`` and one relayout pass restores row-major ``[M, N]``.

The compute itself is injected (``backend``): on GPUs it is the CUDA library (``CudaBackend``); the CPU tests of the
multi-rank logic inject a stand-in so that the partitioning, the collectives and the index arithmetic are exercised with
the gloo backend and no GPU.
"""
import ctypes as C

import torch
import torch.distributed as dist

from ._binding import OUT_F32, OUT_I32, OUT_U8, QParams, check, lib

_OUT_DTYPE = {OUT_U8: torch.uint8, OUT_F32: torch.float32, OUT_I32: torch.int32}


def shard_range(total, rank, world, multiple=1):
    """Contiguous block ``[lo, hi)`` of ``total`` items for ``rank``; every block but the last is a multiple of
    ``multiple`` items.  Blocks differ by at most one unit and cover ``[0, total)`` exactly."""
    units = (total + multiple - 1) // multiple
    lo = (units * rank) // world * multiple
    hi = (units * (rank + 1)) // world * multiple
    return min(lo, total), min(hi, total)


def global_min_max(local_minmax, group=None):
    """All-reduce of a 2-element {min, max} tensor: the only collective the row-sharded path ever needs (and only
    under dynamic activation quantisation)."""
    mn, mx = local_minmax[0:1].clone(), local_minmax[1:2].clone()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(mn, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
    return torch.cat([mn, mx])


class CudaBackend:
    """Compute through libltq on this rank's GPU."""

    def make_layer(self, w_q, bias_q, qp_in, qp_wt, qp_out):
        from .layer import LayerHandle
        N, K = w_q.shape
        h = LayerHandle(w_q.device.index, K, N)
        h.set_weights(w_q, bias_q)
        h.set_qparams(qp_in, qp_wt, qp_out)
        return h

    def forward(self, layer, x_q, out_mode, flags, out=None):
        return layer.forward(x_q, out_mode, flags, out=out)

    def min_max(self, x):
        from .ops import GetMinMax
        return GetMinMax(x)

    def interleave(self, gathered, out):
        G, M, W = gathered.shape
        wbytes = W * gathered.element_size()
        stream = C.c_void_p(torch.cuda.current_stream(gathered.device).cuda_stream)
        check(lib().ltq_interleave_column_blocks(gathered.data_ptr(), out.data_ptr(), G, M, wbytes,
                                                 gathered.device.index, stream))
        return out


class RowShardedLinear:
    """Weights replicated, activation rows split.  ``forward`` takes THIS rank's rows and returns this rank's rows of
    the output; nothing is exchanged."""

    def __init__(self, w_q, bias_q, qp_in, qp_wt, qp_out, backend=None, group=None):
        self.backend = backend or CudaBackend()
        self.group = group
        self.layer = self.backend.make_layer(w_q, bias_q, qp_in, qp_wt, qp_out)

    @staticmethod
    def my_rows(M, group=None):
        return shard_range(M, dist.get_rank(group), dist.get_world_size(group))

    def forward(self, x_q_local, out_mode=OUT_U8, flags=0, out=None):
        return self.backend.forward(self.layer, x_q_local, out_mode, flags, out=out)


class ColShardedLinear:
    """Weight rows (output features) split in blocks of a multiple of 16 columns, activations replicated.
    ``forward`` returns the full ``[M, N]`` output on every rank."""

    def __init__(self, w_q_full_or_local, bias_q, N_total, qp_in, qp_wt, qp_out, backend=None, group=None, is_local=False):
        self.backend = backend or CudaBackend()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.N = N_total
        if N_total % (16 * self.world) != 0:
            raise ValueError("column sharding needs N divisible by 16 * world size (equal, vector-aligned slices)")
        self.n0, self.n1 = shard_range(N_total, self.rank, self.world, 16)
        if is_local:
            w_loc, b_loc = w_q_full_or_local, bias_q
        else:
            w_loc = w_q_full_or_local[self.n0:self.n1].contiguous()
            b_loc = None if bias_q is None else bias_q[self.n0:self.n1].contiguous()
        self._keep = (w_loc, b_loc)
        self.layer = self.backend.make_layer(w_loc, b_loc, qp_in, qp_wt, qp_out)

    def forward(self, x_q, out_mode=OUT_U8, flags=0, out=None, gathered=None, local=None):
        M = x_q.shape[0]
        nloc = self.n1 - self.n0
        dt = _OUT_DTYPE[out_mode]
        if local is None:
            local = torch.empty((M, nloc), dtype=dt, device=x_q.device)
        self.backend.forward(self.layer, x_q, out_mode, flags, out=local)
        if self.world == 1:
            return local
        if gathered is None:
            gathered = torch.empty((self.world, M, nloc), dtype=dt, device=x_q.device)
        dist.all_gather_into_tensor(gathered.view(-1), local.view(-1), group=self.group)
        if out is None:
            out = torch.empty((M, self.N), dtype=dt, device=x_q.device)
        return self.backend.interleave(gathered, out)
