"""GPU, two or more devices: the batch-sharded forward pass with the optional NCCL gather of the final output.

One process per GPU (as the benchmark launches them): the same seeded batch on every rank, frozen per-layer ranges
broadcast from rank 0, rank r convolves `parallel.shard_batch(x)`, `parallel.gather_outputs` all-gathers the final
activations.  The gathered tensor must carry the bits of the whole batch run on one GPU.  Skipped with fewer than
two GPUs."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, kind, hw, batch, out_path):
    import torch
    import torch.distributed as dist
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import parallel, workloads as W
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        net = W.Network(kind, hw)
        filters = W.make_filters(net.convs, 2300)
        tables = [ax.noisy_table(3300 + i) for i in range(len(net.convs))]
        runner = W.GpuRunner(net, tables, filters, dev)
        x = torch.from_numpy(W.make_input(batch, net.hw, net.in_channels, 1003))
        if rank == 0:
            runner.calibrate(x.to(dev))
        runner.in_ranges = parallel.broadcast_ranges(runner.in_ranges, src=0)
        y_slab = runner.forward(parallel.shard_batch(x, world, rank).to(dev))
        y_all = parallel.gather_outputs(y_slab)
        assert y_all.shape[0] == batch
        if rank == 0:
            y_one = runner.forward(x.to(dev))
            torch.cuda.synchronize()
            same = torch.equal(y_all.view(torch.int32), y_one.view(torch.int32))
            with open(out_path, "w") as fh:
                fh.write("same" if same else "different")
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [8, 7], ids=["even_slabs", "ragged_slabs"])
def test_sharded_forward_and_gather_equal_single_gpu(built, tmp_path, batch):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    out = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, _free_port(), "resnet20", 32, batch, str(out)), nprocs=2, join=True)
    assert out.read_text() == "same"


def test_sharded_entry_point_on_the_devices_present(built):
    """axc_conv2d_forward_sharded + axc_gather_outputs in one process: the batch cut into slabs over however many
    GPUs there are (on a single GPU: two slabs on the same device), gathered on device 0, against the whole batch in
    one call - bit for bit; and a shard whose workspace is missing is reported by its index, the shards before it
    having been accepted."""
    import ctypes as C
    import numpy as np
    import torch
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import _lib, ops, parallel
    ndev = max(1, min(torch.cuda.device_count(), 4))
    nshards = max(2, ndev)
    rng = np.random.Generator(np.random.PCG64(71))
    x = torch.from_numpy(rng.uniform(-1, 1, (7, 20, 20, 16)).astype(np.float32))
    f = torch.from_numpy(rng.normal(0, 0.1, (3, 3, 16, 48)).astype(np.float32))
    table = ax.Table(array=ax.noisy_table(3071))
    mm = (-1.0, 1.0, float(f.min()), float(f.max()))
    slabs, filters = [], []
    for i in range(nshards):
        lo, hi = parallel.shard_bounds(x.shape[0], nshards, i)
        dev = torch.device("cuda", i % ndev)
        slabs.append(x[lo:hi].to(dev))
        filters.append(f.to(dev))
    y = parallel.forward_sharded(slabs, filters, table, mm, [1, 1, 1, 1], "SAME", gather_to="cuda:0")
    torch.cuda.synchronize()
    want = ax.approx_conv2d_with_min_max_vars(x.cuda(0), f.cuda(0), *mm, [1, 1, 1, 1], 8, table, "SAME")
    assert torch.equal(y.view(torch.int32), want.view(torch.int32))

    # an injected host-side failure: the second shard comes without a workspace
    L = _lib.load()
    d = ops._desc(slabs[0].shape, f.shape, [1, 1, 1, 1], "SAME", "NHWC", [1, 1, 1, 1], [])
    shards = (_lib.Shard * 2)()
    outs = [torch.empty(ops.conv2d_output_shape(s.shape, f.shape, [1, 1, 1, 1], "SAME"), device=s.device) for s in slabs[:2]]
    ws0 = torch.zeros(ops.workspace_bytes(slabs[0].shape, f.shape, [1, 1, 1, 1], "SAME"), dtype=torch.uint8, device=slabs[0].device)
    shards[0] = _lib.Shard(slabs[0].device.index, int(slabs[0].shape[0]), slabs[0].data_ptr(), filters[0].data_ptr(),
                           outs[0].data_ptr(), ws0.data_ptr(), ws0.numel(), None)
    shards[1] = _lib.Shard(slabs[1].device.index, int(slabs[1].shape[0]), slabs[1].data_ptr(), filters[1].data_ptr(),
                           outs[1].data_ptr(), None, 0, None)
    failed = C.c_int32(-2)
    st = L.axc_conv2d_forward_sharded(table.handle, C.byref(d), shards, 2, *mm, C.byref(failed))
    torch.cuda.synchronize()
    assert st == 13 and failed.value == 1
    lo, hi = parallel.shard_bounds(x.shape[0], nshards, 0)
    assert torch.equal(outs[0].view(torch.int32), want[lo:hi].to(outs[0].device).view(torch.int32))
