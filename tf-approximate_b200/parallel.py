"""Batch sharding of the table convolution across the GPUs of one box.

Every output pixel depends on its own image only, so the batch is cut into contiguous slabs, each rank owns
one slab, a replica of the truth table and of the filter, and no collective sits on the compute path.  What
the ranks must agree on are the quantisation ranges (host scalars of the op): they are fixed once
(`broadcast_ranges`) instead of being reduced per batch.  `gather_outputs` is the optional all-gather of the
final layer's output."""
import torch
import torch.distributed as dist


def shard_bounds(n, world_size, rank):
    """Contiguous slab [lo, hi) of a batch of n images for `rank`; slab sizes differ by at most one."""
    base, rem = divmod(n, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(x, world_size=None, rank=None):
    """This rank's slab of an NHWC batch (a view: NHWC slabs are contiguous)."""
    world_size = dist.get_world_size() if world_size is None else world_size
    rank = dist.get_rank() if rank is None else rank
    lo, hi = shard_bounds(x.shape[0], world_size, rank)
    return x[lo:hi]


def broadcast_ranges(ranges, src=0):
    """Make the per-layer (min, max) pairs of rank `src` the ones every rank uses."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return ranges
    box = [ranges]
    dist.broadcast_object_list(box, src=src)
    return box[0]


def gather_outputs(y, total_batch=None):
    """All-gather of per-rank outputs [n_r, ...] along the batch axis (slabs may differ by one image)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return y
    world = dist.get_world_size()
    sizes = [torch.zeros(1, dtype=torch.int64, device=y.device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([y.shape[0]], dtype=torch.int64, device=y.device))
    sizes = [int(s.item()) for s in sizes]
    nmax = max(sizes)
    pad = y
    if y.shape[0] < nmax:
        pad = torch.cat([y, y.new_zeros((nmax - y.shape[0],) + tuple(y.shape[1:]))], 0)
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad.contiguous())
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], 0)
