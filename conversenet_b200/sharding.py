"""Batch sharding over the GPUs of one box.

Every (sample, channel) plane of Converse2D and every image of a network is independent, so a
batch is cut into contiguous slices, one per rank, the weights are replicated, and no collective
sits on the path; a gather of the per-rank outputs is optional and off the timed path.  The
reference has no counterpart (it is single-process); this is the layer `bench.py --gpus N`, and
any data-parallel caller, uses.  Works with any `torch.distributed` backend (NCCL on the GPUs,
gloo in the CPU tests)."""
import torch
import torch.distributed as dist


def shard_batch(total, rank, world):
    """Slice [start, start + count) of a batch of `total` items for `rank` of `world`.

    Slices are contiguous, cover the batch exactly once and differ by at most one item: the
    first `total % world` ranks take one extra.  With fewer items than ranks the last ranks
    get `count == 0` and have nothing to do."""
    if total < 0 or world < 1 or not 0 <= rank < world:
        raise ValueError("shard_batch(total=%r, rank=%r, world=%r)" % (total, rank, world))
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def shard_tensor(x, rank, world):
    """This rank's slice of `x` along dimension 0 (a view)."""
    start, count = shard_batch(x.size(0), rank, world)
    return x[start:start + count]


def max_over_ranks(value, device=None, group=None):
    """Max of a per-rank float (an elapsed time) over the group; the value itself without a group."""
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def gather_batch(y_local, total, group=None):
    """All ranks' output slices concatenated in batch order (every rank gets the whole batch).

    Slices may differ by one item, so each rank pads its slice to the largest count before the
    all-gather and the padding is dropped afterwards.  Off the timed path."""
    if not (dist.is_available() and dist.is_initialized()):
        return y_local
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    counts = [shard_batch(total, r, world)[1] for r in range(world)]
    cmax = max(counts)
    tail = tuple(y_local.shape[1:])
    padded = y_local.new_zeros((cmax,) + tail)
    padded[:counts[rank]] = y_local
    parts = [y_local.new_empty((cmax,) + tail) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)
