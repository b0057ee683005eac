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

from ._binding import FLAG_MULTICAST_DEST, OUT_F32, OUT_I32, OUT_U8, QParams, check, lib

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


class PeerBuffer:
    """One device buffer per rank, each mapped into every other rank of the group (CUDA IPC through libltq).
    ``ptrs[r]`` is the address under which THIS process reaches rank r's buffer; ``local`` is a uint8 torch view of
    this rank's own buffer.  Collective: every rank of the group must construct it at the same point."""

    def __init__(self, nbytes, device_index, group=None):
        self.device_index, self.nbytes = device_index, int(nbytes)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        own = C.c_void_p()
        handle = C.create_string_buffer(64)
        check(lib().ltq_peer_alloc(C.byref(own), self.nbytes, device_index, handle))
        self._own = own
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs, self._opened = [], []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(own.value)
                continue
            p = C.c_void_p()
            check(lib().ltq_peer_open(h, device_index, C.byref(p)))
            self._opened.append(p)
            self.ptrs.append(p.value)
        self.local = _wrap_device_memory(own.value, self.nbytes, device_index, self)

    def close(self):
        for p in self._opened:
            lib().ltq_peer_close(p, self.device_index)
        self._opened = []
        if self._own:
            lib().ltq_peer_free(self._own, self.device_index)
            self._own = None


class MulticastBuffer:
    """One device buffer per rank behind an NVLink multicast mapping: a store to ``mc_ptr`` lands in every rank's
    buffer (NVSwitch replicates it), so a rank sends its data once however many peers there are.  The buffers, the
    multicast object and their exchange between the ranks come from ``torch.distributed``'s symmetric memory (NCCL
    process groups on NVSwitch systems); ``mc_ptr`` is 0 where the system has no multicast support, and the caller
    falls back to peer stores.  Collective: every rank of the group must construct it at the same point."""

    def __init__(self, nbytes, device_index, group=None):
        import torch.distributed._symmetric_memory as symm
        self.nbytes = int(nbytes)
        grp = group if group is not None else dist.group.WORLD
        self.local = symm.empty(self.nbytes, dtype=torch.uint8, device=torch.device("cuda", device_index))
        self._hdl = symm.rendezvous(self.local, grp)
        self.mc_ptr = int(self._hdl.multicast_ptr or 0)      # 0 where the system has no multicast support
        self.ptrs = [int(p) for p in self._hdl.buffer_ptrs]

    def close(self):
        self._hdl = None
        self.local = None


def _wrap_device_memory(ptr, nbytes, device_index, owner):
    """uint8 CUDA tensor over memory this module allocated itself (no copy; `owner` is kept alive by the tensor)."""
    class _Iface:
        pass
    holder = _Iface()
    holder.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                       "strides": None}
    holder._owner = owner
    return torch.as_tensor(holder, device=torch.device("cuda", device_index))


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

    def __init__(self, w_q_full_or_local, bias_q, N_total, qp_in, qp_wt, qp_out, backend=None, group=None, is_local=False,
                 fused=False, max_rows=0, out_mode=OUT_U8, multicast=False):
        """``fused=True``: no all-gather; the GEMM epilogue stores this rank's columns straight into every rank's
        ``[max_rows, N]`` output buffer over NVLink (peer-mapped memory, two buffers used alternately), followed by one
        tiny stream-ordered collective as the barrier.  Needs the CUDA backend and ``max_rows``/``out_mode`` up front.
        ``multicast=True`` (with ``fused``): the buffers sit behind an NVLink multicast mapping and each rank issues ONE
        store per piece of output (``multimem.st``) that NVSwitch replicates to every rank, instead of one per peer;
        falls back to peer stores where multicast is not available (``self.multicast`` tells which is in use)."""
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
        self.fused = bool(fused) and self.world > 1
        if self.fused:
            if max_rows < 1:
                raise ValueError("fused column sharding needs max_rows")
            self.max_rows, self.out_mode = int(max_rows), out_mode
            self._esize = torch.empty(0, dtype=_OUT_DTYPE[out_mode]).element_size()
            dev = w_loc.device.index
            nbytes = self.max_rows * self.N * self._esize
            self.multicast = False
            if multicast:
                bufs = [MulticastBuffer(nbytes, dev, group) for _ in range(2)]
                if all(b.mc_ptr for b in bufs):
                    self._bufs, self.multicast = bufs, True
                else:
                    for b in bufs:
                        b.close()
            if not self.multicast:
                self._bufs = [PeerBuffer(nbytes, dev, group) for _ in range(2)]
            self._turn = 0
            self._flag = torch.zeros(1, dtype=torch.int32, device=w_loc.device)

    def close(self):
        """Releases the peer-mapped buffers of the fused form.  Collective: every rank calls it, after its last forward;
        nobody unmaps or frees before everyone has finished computing, and nobody frees before everyone has unmapped."""
        if not self.fused:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        if self.multicast:
            # nobody lets go of its part of the multicast mapping while another rank may still store through it
            for b in self._bufs:
                b.close()
            dist.barrier(group=self.group)
            self._bufs, self.fused = [], False
            return
        for b in self._bufs:
            for p in b._opened:
                lib().ltq_peer_close(p, b.device_index)
            b._opened = []
        dist.barrier(group=self.group)
        for b in self._bufs:
            b.close()
        self._bufs = []
        self.fused = False

    def forward(self, x_q, out_mode=OUT_U8, flags=0, out=None, gathered=None, local=None):
        M = x_q.shape[0]
        nloc = self.n1 - self.n0
        dt = _OUT_DTYPE[out_mode]
        if self.fused:
            return self._forward_fused(x_q, M, out_mode, flags)
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

    def _forward_fused(self, x_q, M, out_mode, flags):
        """Returns a view of this rank's current output buffer, valid until the forward after next."""
        if out_mode != self.out_mode or M > self.max_rows:
            raise ValueError("fused column sharding was set up for another out_mode or fewer rows")
        buf = self._bufs[self._turn]
        self._turn ^= 1
        if self.multicast:
            # one destination: the multicast address (this rank's own buffer is behind it too)
            self.layer.forward_scatter(x_q, [buf.mc_ptr], self.N, self.n0, out_mode, flags | FLAG_MULTICAST_DEST)
        else:
            # this rank's pointer first (the kernel's primary destination), then the peers' starting with the next rank:
            # at any moment the ranks then store to different peers instead of all to the same one
            world = len(buf.ptrs)
            ptrs = [buf.ptrs[self.rank]] + [buf.ptrs[(self.rank + k) % world] for k in range(1, world)]
            self.layer.forward_scatter(x_q, ptrs, self.N, self.n0, out_mode, flags)
        self._barrier(x_q.device)
        return buf.local[:M * self.N * self._esize].view(_OUT_DTYPE[out_mode]).view(M, self.N)

    def _barrier(self, device):
        """Every rank's stores have landed before anyone reads.  NCCL: a 4-byte all-reduce on the compute stream (device
        ordered, no host sync).  Other backends (tests with gloo): drain the stream, then a host barrier."""
        if dist.get_backend(self.group) == "nccl":
            dist.all_reduce(self._flag, group=self.group)
        else:
            torch.cuda.current_stream(device).synchronize()
            dist.barrier(group=self.group)
