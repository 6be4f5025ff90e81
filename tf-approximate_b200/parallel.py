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


def forward_sharded(x_slabs, filters, table, ranges, strides, padding, gather_to=None):
    """Single-process form of the batch sharding (axc_conv2d_forward_sharded): `x_slabs[i]` and `filters[i]` live on
    GPU i's device, every slab gets a stream-ordered forward call on its own device, and - if `gather_to` names a
    device - the outputs are gathered there with one peer copy per slab (axc_gather_outputs).  Returns the list of
    per-slab outputs, or the gathered tensor."""
    import ctypes as C
    from . import _lib, ops
    from .errors import raise_for_status
    L = _lib.load()
    tab = ops._table_for(table, 8)
    d = ops._desc(x_slabs[0].shape, filters[0].shape, strides, padding, "NHWC", [1, 1, 1, 1], [])
    shards = (_lib.Shard * len(x_slabs))()
    outs, keep = [], []
    for i, (x, f) in enumerate(zip(x_slabs, filters)):
        dev = x.device
        oshape = ops.conv2d_output_shape(x.shape, f.shape, strides, padding)
        y = torch.empty(oshape, dtype=torch.float32, device=dev)
        ws = torch.zeros(ops.workspace_bytes(x.shape, f.shape, strides, padding), dtype=torch.uint8, device=dev)
        xs, fs = x.contiguous(), f.contiguous()
        keep += [xs, fs, ws]
        outs.append(y)
        shards[i] = _lib.Shard(ops._device_index(dev), int(x.shape[0]), xs.data_ptr(), fs.data_ptr(), y.data_ptr(), ws.data_ptr(),
                               ws.numel(), torch.cuda.current_stream(dev).cuda_stream)
    failed = C.c_int32(-1)
    st = L.axc_conv2d_forward_sharded(tab.handle, C.byref(d), shards, len(x_slabs), *[float(v) for v in ranges], C.byref(failed))
    raise_for_status(st, "sharded ApproxConv2D", "shard %d" % failed.value)
    if gather_to is None:
        return outs
    gdev = torch.device(gather_to)
    total = sum(int(y.shape[0]) for y in outs)
    dst = torch.empty((total,) + tuple(outs[0].shape[1:]), dtype=torch.float32, device=gdev)
    image_bytes = 4 * int(outs[0][0].numel()) if total else 0
    raise_for_status(L.axc_gather_outputs(shards, len(x_slabs), image_bytes, dst.data_ptr(), ops._device_index(gdev)), "gather")
    for y in outs:      # the copies run on the slabs' streams: make the gathered tensor's device wait for them
        torch.cuda.current_stream(gdev).wait_stream(torch.cuda.current_stream(y.device))
    return dst
