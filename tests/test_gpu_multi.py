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
    out = tmp_path / "verdict.txt"
    mp.spawn(_worker, args=(2, _free_port(), "resnet20", 32, batch, str(out)), nprocs=2, join=True)
    assert out.read_text() == "same"
