"""Batch sharding across GPUs and the one collective of the path.

The reference is single-device (one sycl::queue per backend, include/portdnn/backend/
snn_usm_backend.h:79-80).  Here the convolution path is sharded by batch, one process per GPU:
forward and input backprop need no exchange at all (every rank holds all filters); filter
backprop reduces over the batch, so each rank's filter gradients are summed with ONE all-reduce
over a contiguous fp32 buffer.  torch.distributed (NCCL on GPUs, gloo in the CPU tests) is the
plumbing; nothing here touches peer memory directly.
"""
import numpy as np


def shard_batch(global_batch, world_size, rank):
    """Images [start, start+count) of the global batch that `rank` owns: contiguous, sizes differ
    by at most one, earlier ranks take the remainder."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("bad rank/world size")
    base, rem = divmod(global_batch, world_size)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, count


def filter_gradient_layout(filter_sizes, pad_to=None):
    """Offsets of each layer's filter gradient inside the one contiguous buffer, each rounded
    up to 64 elements (256 bytes of fp32) so that every view stays 16-byte aligned for the
    kernels; returns (offsets, total)."""
    offsets, off = [], 0
    for n in filter_sizes:
        offsets.append(off)
        off += (int(n) + 63) // 64 * 64
    total = off if pad_to is None else max(off, int(pad_to))
    return offsets, total


class FilterGradientBucket:
    """All filter gradients of a network in one fp32 tensor, reduced with a single all_reduce."""

    def __init__(self, filter_sizes, device, pad_to=None):
        import torch
        self.sizes = [int(n) for n in filter_sizes]
        self.offsets, self.total = filter_gradient_layout(self.sizes, pad_to)
        self.buffer = torch.zeros(self.total, dtype=torch.float32, device=device)

    def view(self, i):
        return self.buffer[self.offsets[i]:self.offsets[i] + self.sizes[i]]

    def span(self, first, last):
        """(start, stop) of the contiguous slice that holds the gradients of layers first..last."""
        return self.offsets[first], self.offsets[last] + (self.sizes[last] + 63) // 64 * 64

    def all_reduce(self, group=None, async_op=False, span=None, comm=None):
        """Sum over ranks of the whole buffer, or of one span of it (no-op without an initialised process
        group or with one rank).  comm: a GradientComm, to go through the library's own C-ABI collective
        instead of torch.distributed."""
        if comm is not None:
            return comm.all_reduce(self.buffer if span is None else self.buffer[span[0]:span[1]])
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
            return None
        t = self.buffer if span is None else self.buffer[span[0]:span[1]]
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


class GradientComm:
    """The library's own communicator for the filter-gradient all-reduce (pdnn_comm_* /
    pdnn_allreduce_filter_grads): NCCL reached through the C ABI rather than through torch.distributed.
    `exchange(id_bytes_or_None) -> id_bytes` hands rank 0's 128-byte id to every rank: by default it is
    a torch.distributed broadcast over the initialised process group."""

    def __init__(self, rank, world_size, exchange=None):
        import ctypes
        from . import api
        self._api, self._ct, self.world = api, ctypes, world_size
        L = api.lib()
        buf = (ctypes.c_char * 128)()
        if rank == 0:
            api._check(L.pdnn_comm_unique_id(buf))
        ident = (exchange or self._broadcast)(bytes(buf) if rank == 0 else None)
        self._comm = ctypes.c_void_p()
        api._check(L.pdnn_comm_init(ctypes.byref(self._comm), ident, world_size, rank))

    @staticmethod
    def _broadcast(ident):
        import torch
        import torch.distributed as dist
        t = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if ident is not None:
            t.copy_(torch.frombuffer(bytearray(ident), dtype=torch.uint8))
        dist.broadcast(t, src=0)
        return bytes(t.cpu().numpy().tobytes())

    def all_reduce(self, tensor):
        """Sums a contiguous fp32 CUDA tensor over the ranks in place, on the current stream."""
        import torch
        if tensor.dtype != torch.float32 or not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("the gradient buffer must be a contiguous fp32 CUDA tensor")
        self._api._check(self._api.lib().pdnn_allreduce_filter_grads(
            self._comm, self._ct.c_void_p(tensor.data_ptr()), self._ct.c_size_t(tensor.numel()),
            self._ct.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def destroy(self):
        if self._comm:
            self._api._check(self._api.lib().pdnn_comm_destroy(self._comm))
            self._comm = None


def max_over_ranks(value, device=None, group=None):
    """A timing taken on every rank -> the slowest rank's value (what a multi-GPU number must report)."""
    import torch
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class RankFailure(RuntimeError):
    """Raised on the surviving ranks when a rank reported a failure, or never reported at all, before
    a collective of the step."""


class StepGuard:
    """Host-side agreement before the filter-gradient all-reduce: every rank posts the outcome of its
    backward pass to a key-value store (torch.distributed's TCPStore or any object with set / get /
    wait) and reads the others' before it enters the collective.  A rank that raised posts "failed";
    a rank that died posts nothing and the others' wait runs out.  Either way the survivors raise
    RankFailure instead of blocking inside a collective that can never complete.  The reference is
    single-device and has no counterpart."""

    def __init__(self, store, rank, world_size, timeout_s=5.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world_size, timeout_s

    def _key(self, step, rank):
        return "pdnn/step%d/rank%d" % (step, rank)

    def report(self, step, ok=True, reason=""):
        self.store.set(self._key(step, self.rank), "ok" if ok else "failed:" + reason)

    def check(self, step):
        """Blocks until every rank has reported for `step` (at most timeout_s per rank) and raises
        RankFailure if one failed or stayed silent."""
        import datetime
        for r in range(self.world):
            key = self._key(step, r)
            try:
                self.store.wait([key], datetime.timedelta(seconds=self.timeout_s))
            except Exception as e:  # the store's wait raises on time-out
                raise RankFailure("rank %d did not report for step %d within %.1f s" % (r, step, self.timeout_s)) from e
            val = self.store.get(key)
            val = val.decode() if isinstance(val, bytes) else str(val)
            if val != "ok":
                raise RankFailure("rank %d reported %s in step %d" % (r, val, step))

    def guarded_all_reduce(self, bucket, step, compute):
        """Runs compute() (the rank's backward pass), reports its outcome, checks the others and only
        then sums the bucket.  A local exception is reported before it propagates."""
        try:
            compute()
        except Exception as e:
            self.report(step, False, type(e).__name__)
            raise
        self.report(step, True)
        self.check(step)
        return bucket.all_reduce()
