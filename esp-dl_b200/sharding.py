"""Batch sharding across GPUs for the forward path: one process per GPU, a replica of the weights on each,
the images split into contiguous shards, and one exchange per step - the gather of the logits.

The path has no other cross-image dependency, so there is no collective between layers.  The helpers work on any
torch.distributed backend ("nccl" on GPUs, "gloo" in the CPU tests)."""
import torch
import torch.distributed as dist


def shard_range(total, rank, world):
    """[begin, end) of the images rank `rank` owns when `total` images are split over `world` ranks.
    Shards are contiguous and differ by at most one image; the first `total % world` ranks get the extra one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_logits(local, total, group=None, out=None):
    """All ranks pass their shard's logits `local` [n_local, classes] (same dtype and device everywhere) and get the
    [total, classes] tensor of all images in image order.  Equal shards go through one all_gather_into_tensor on
    the caller's buffers; ragged shards are padded to the largest shard first."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    begin, end = shard_range(total, rank, world)
    if local.shape[0] != end - begin:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows, its shard has {end - begin}")
    classes = local.shape[1:]
    largest = shard_range(total, 0, world)[1]
    if total % world == 0:
        if out is None:
            out = torch.empty((total,) + tuple(classes), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((largest,) + tuple(classes), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    rows = [pieces[r][: shard_range(total, r, world)[1] - shard_range(total, r, world)[0]] for r in range(world)]
    return torch.cat(rows, dim=0)
