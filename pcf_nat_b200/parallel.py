"""Batch sharding helpers. NA1D has no exchange step: every (batch, head) sequence is independent, so ranks only
agree on who owns which sequences and on the slowest rank's time. The reference itself has no distributed code; the
only collectives of a data-parallel run live in the model around the operator: one all-reduce of the gradients per
training step and one all-gather of the embeddings per extraction pass."""
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


def flat_gradient_buffer(params):
    """One contiguous fp32 buffer holding every parameter's gradient: each ``p.grad`` becomes a view into it, so that a
    data-parallel step needs a single all-reduce and autograd accumulates into the views in place."""
    params = [p for p in params if p.requires_grad]
    if not params:
        raise ValueError("no trainable parameters")
    flat = torch.zeros(sum(p.numel() for p in params), dtype=torch.float32, device=params[0].device)
    off = 0
    for p in params:
        p.grad = flat[off:off + p.numel()].view_as(p)
        off += p.numel()
    return flat


def all_reduce_mean(t):
    """In-place mean of `t` over the ranks (identity without a process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return t
    if dist.get_backend() == "nccl":
        dist.all_reduce(t, op=dist.ReduceOp.AVG)
    else:   # gloo has no AVG
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        t.div_(dist.get_world_size())
    return t


def all_gather_rows(local, out=None):
    """Concatenation over the ranks, in rank order, of equally sized ``(n, d)`` blocks (the extraction path's embeddings)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        if out is None:
            return local
        out.copy_(local)
        return out
    if out is None:
        out = local.new_empty((dist.get_world_size() * local.shape[0],) + tuple(local.shape[1:]))
    dist.all_gather_into_tensor(out, local.contiguous())
    return out
