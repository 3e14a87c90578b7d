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


def gather_equal_rows(local, out=None, group=None):
    """All-gather row blocks of EQUAL size with one ``all_gather_into_tensor`` straight into `out`
    ((world * rows, ...), allocated if None): no padding, no list of parts, no concatenation.  The per-step
    collective of a batch that divides evenly over the ranks."""
    world = dist.get_world_size(group)
    local = local.contiguous()
    if out is None:
        out = torch.empty((world * local.shape[0], *local.shape[1:]), dtype=local.dtype, device=local.device)
    elif out.shape[0] != world * local.shape[0] or out.shape[1:] != local.shape[1:] or not out.is_contiguous():
        raise ValueError(f"out has shape {tuple(out.shape)}, expected ({world * local.shape[0]}, ...) contiguous")
    dist.all_gather_into_tensor(out, local, group=group)
    return out


@torch.no_grad()
def sharded_forward(fn, ids, gather="argmax", group=None, fn_returns="logits"):
    """Run `fn` on this rank's rows of the global batch `ids` and return the gathered result on every rank.

    `fn` maps ids to logits (``fn_returns="logits"``, e.g. ``FusedGPT.logits``) or straight to next-token ids
    (``fn_returns="ids"``, e.g. ``FusedGPT.next_ids``, whose argmax comes out of the lm_head's epilogue so that
    no (tokens, vocab) tensor is written or reduced a second time; or ``lambda x: model.generate(x, n)``, whose
    (rows, n) continuations are gathered the same way).

    gather="argmax": (batch, seqlen) int64 next-token ids (8 bytes per token cross NVLink);
    gather="logits": (batch, seqlen, vocab) logits (large: meant for checks, not for throughput);
    gather="none":   this rank's result only, no collective.
    """
    if fn_returns not in ("logits", "ids"):
        raise ValueError(f"unknown fn_returns {fn_returns!r}")
    if gather not in ("none", "argmax", "logits"):
        raise ValueError(f"unknown gather mode {gather!r}")
    if fn_returns == "ids" and gather == "logits":
        raise ValueError("a callable that returns ids has no logits to gather")
    world = dist.get_world_size(group)
    local_ids = shard_batch(ids, dist.get_rank(group), world)
    result = fn(local_ids)
    if gather == "none":
        return result
    if gather == "argmax":
        local = result if fn_returns == "ids" else result.argmax(dim=-1)
        if ids.shape[0] % world == 0:
            return gather_equal_rows(local, group=group)
        return gather_rows(local, ids.shape[0], group)
    return gather_rows(result.contiguous(), ids.shape[0], group)
