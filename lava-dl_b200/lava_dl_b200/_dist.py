"""Batch-sharded data parallelism for the hot path.

Rows (batch x neurons) are independent recurrences and neuron states are per
sample, so every rank simply runs the kernels on its own slice of the batch:
the forward pass needs no communication.  Only the gradients of the *shared*
per-layer parameters (decays, sin/cos of the rotation, axonal delays) must be
summed over ranks; all of them are flattened into one buffer and all-reduced
once per step (a few bytes to a few KB: latency bound, NVLink bandwidth is
irrelevant).  The reference has no distributed code at all; its tutorials use
single-process ``torch.nn.DataParallel``.
"""

import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """``[lo, hi)`` of rank's contiguous share of ``n`` samples (ragged tails allowed)."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(t, rank=None, world=None, dim=0):
    """This rank's slice of a batch tensor."""
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    lo, hi = shard_bounds(t.shape[dim], rank, world)
    return t.narrow(dim, lo, hi - lo)


def allreduce_param_grads(params, group=None):
    """Sum the ``.grad`` of every parameter in ``params`` over the process group
    with ONE collective.  Parameters without a gradient contribute zeros so that
    all ranks issue an identical collective.  Returns the number of elements
    reduced."""
    params = [p for p in params if p.requires_grad]
    if not params:
        return 0
    device = params[0].device
    flat = torch.cat([
        (p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).to(torch.float32) for p in params
    ])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    offset = 0
    for p in params:
        n = p.numel()
        chunk = flat[offset:offset + n].reshape(p.shape).to(device=device, dtype=p.dtype)
        if p.grad is None:
            p.grad = chunk.clone()
        else:
            p.grad.copy_(chunk)
        offset += n
    return int(flat.numel())
