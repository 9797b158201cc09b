"""Host-side helpers for batch-sharded (data-parallel) use: every rank owns a contiguous
shard of the utterances, runs the loss on it, and the only exchange is an all-reduce of the
scalar loss sum.  Works with any torch.distributed backend (NCCL on GPUs, gloo in tests)."""
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
