"""Batch sharding of the forward across the GPUs of one node: one process per GPU, every rank
holds a full replica of the weights and runs its slice of the batch; the only collective is an
all-gather of what the caller wants back (argmax ids by default, logits on request).

The reference is single-GPU and has no counterpart of this file.  Nothing here touches CUDA
directly: the forward is whatever callable the caller passes (``FusedGPT.logits`` on a GPU, any
stand-in under the ``gloo`` backend on CPU), so the partitioning and gather logic is testable
without a GPU.
"""

import torch
import torch.distributed as dist


def shard_bounds(n_rows, rank, world_size):
    """Rows [start, end) of rank `rank`: contiguous, balanced to within one row, covering
    [0, n_rows) exactly once over all ranks; empty slices when world_size > n_rows."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(n_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(ids, rank=None, world_size=None):
    """This rank's rows of a (batch, seqlen) id tensor."""
    rank = dist.get_rank() if rank is None else rank
    world_size = dist.get_world_size() if world_size is None else world_size
    lo, hi = shard_bounds(ids.shape[0], rank, world_size)
    return ids[lo:hi]


def gather_rows(local, n_rows_total, group=None):
    """All-gather per-rank row blocks (sizes as given by shard_bounds) into the full tensor, in
    rank order, on every rank.  Uneven slices are padded to the largest one for the collective."""
    world = dist.get_world_size(group)
    sizes = [hi - lo for lo, hi in (shard_bounds(n_rows_total, r, world) for r in range(world))]
    if local.shape[0] != sizes[dist.get_rank(group)]:
        raise ValueError(f"rank holds {local.shape[0]} rows, expected {sizes[dist.get_rank(group)]}")
    widest = max(sizes)
    if local.shape[0] < widest:
        pad = torch.zeros((widest - local.shape[0], *local.shape[1:]), dtype=local.dtype, device=local.device)
        local = torch.cat([local, pad], dim=0)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)


@torch.no_grad()
def sharded_forward(logits_fn, ids, gather="argmax", group=None):
    """Run `logits_fn` (ids -> logits) on this rank's rows of the global batch `ids` and return
    the gathered result on every rank:

    gather="argmax": (batch, seqlen) int64 next-token ids (8 bytes per token cross NVLink);
    gather="logits": (batch, seqlen, vocab) logits (large: meant for checks, not for throughput);
    gather="none":   this rank's logits only, no collective.
    """
    world = dist.get_world_size(group)
    local_ids = shard_batch(ids, dist.get_rank(group), world)
    logits = logits_fn(local_ids)
    if gather == "none":
        return logits
    if gather == "argmax":
        return gather_rows(logits.argmax(dim=-1), ids.shape[0], group)
    if gather == "logits":
        return gather_rows(logits.contiguous(), ids.shape[0], group)
    raise ValueError(f"unknown gather mode {gather!r}")
