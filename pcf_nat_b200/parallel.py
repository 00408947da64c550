"""Batch sharding helpers. NA1D has no exchange step: every (batch, head) sequence is independent, so
ranks only agree on who owns which sequences and on the slowest rank's time (SURVEY: the reference itself
has no distributed code; the only collectives of a data-parallel run live in the model around the op)."""
import torch
import torch.distributed as dist


def shard_range(total, world, rank):
    """Contiguous [lo, hi) slice of `total` items for `rank`; sizes differ by at most one."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(tensors, heads, world, rank):
    """Slice (N=batch*heads, T, C) tensors by whole utterances (all heads of an utterance stay together)."""
    n = tensors[0].shape[0]
    if n % heads:
        raise ValueError("N=%d is not a multiple of heads=%d" % (n, heads))
    lo, hi = shard_range(n // heads, world, rank)
    return [t[lo * heads:hi * heads] for t in tensors]


def max_over_ranks(value, device=None):
    """Largest `value` among all ranks (identity without an initialised process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier():
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
