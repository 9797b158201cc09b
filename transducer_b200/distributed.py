"""Host-side helpers for batch-sharded (data-parallel) use: every rank owns a contiguous
shard of the utterances, runs the loss on it, and the only exchange is an all-reduce of the
scalar loss sum.  Works with any torch.distributed backend (NCCL on GPUs, gloo in tests);
PeerLossSum does the same exchange with the library's own kernel over peer memory."""
import ctypes

import torch
import torch.distributed as dist


def shard_range(batch, rank, world):
    """[first, first+count) of `batch` utterances owned by `rank`: contiguous, sizes differ
    by at most one, earlier ranks take the remainder."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    base, extra = divmod(batch, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def all_reduce_loss(loss_sum, group=None):
    """Sum of the per-rank loss sums (in place on the 1-element tensor the loss kernel
    wrote); returns it.  A no-op when torch.distributed is not initialised."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(loss_sum, op=dist.ReduceOp.SUM, group=group)
    return loss_sum


def mean_loss(loss_sum, global_batch, group=None):
    """Batch-mean loss over all ranks from the per-rank sums."""
    return all_reduce_loss(loss_sum.clone(), group) / float(global_batch)


class PeerLossSum(object):
    """Sum of the per-rank loss sums by plain peer stores over NVLink (tb200_loss_sum_exchange):
    one launch of one warp per rank and step instead of an all-reduce.  One process per GPU of
    ONE node; torch.distributed (any backend) is used once, to pass the CUDA IPC handles of the
    slot buffers around.  Every rank must call the object once per step, in the same order.

        reducer = PeerLossSum()                       # collective: all ranks construct it
        total = reducer(criterion.last_loss_sum)      # 1-element device tensor, same bits everywhere

    A peer that stops calling makes the next total NaN after `timeout_us` (0: the library's
    2 s limit) and shows up in check_device_status(); nothing hangs.
    """

    def __init__(self, group=None, device=None):
        from . import _lib
        self._lib = _lib
        lib = _lib.lib
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        self.seq = 0
        self.total = torch.zeros(1, device=self.device)
        with torch.cuda.device(self.device):
            mine = ctypes.c_void_p()
            _lib.check(lib.tb200_peer_alloc(ctypes.byref(mine)))
            self._mine = mine
            handle = ctypes.create_string_buffer(64)
            _lib.check(lib.tb200_peer_export(mine, handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self._imported = []
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(mine.value)
                    continue
                p = ctypes.c_void_p()
                _lib.check(lib.tb200_peer_import(ctypes.create_string_buffer(h, 64), ctypes.byref(p)))
                self._imported.append(p)
                ptrs.append(p.value)
            self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        dist.barrier(group=group)   # every buffer is open everywhere before the first store

    def __call__(self, loss_sum, timeout_us=0):
        if loss_sum.device != self.device or loss_sum.dtype is not torch.float32:
            raise ValueError("loss_sum must be a float32 tensor on %s" % self.device)
        self.seq += 1
        lib = self._lib.lib
        with torch.cuda.device(self.device):
            self._lib.check(lib.tb200_set_stream(torch.cuda.current_stream(self.device).cuda_stream))
            self._lib.check(lib.tb200_loss_sum_exchange(
                loss_sum.data_ptr(), self._ptrs, self.rank, self.world, self.seq,
                self.total.data_ptr(), int(timeout_us)))
        return self.total

    def close(self):
        """Collective: waits for all ranks, then closes the peers' buffers and frees its own."""
        if self._mine is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        lib = self._lib.lib
        with torch.cuda.device(self.device):
            for p in self._imported:
                lib.tb200_peer_close(p)
            lib.tb200_peer_free(self._mine)
        self._imported, self._mine = [], None
