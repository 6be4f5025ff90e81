"""CPU, two gloo ranks: the host logic of the multi-GPU path - contiguous batch slabs, one set of frozen
quantisation ranges for all ranks, optional output gather.  The convolution itself is done by the CPU checker
here; on GPUs the same host logic wraps the CUDA op (bench.py)."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from tf_approximate_b200 import parallel
    import tf_approximate_b200 as ax
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.Generator(np.random.PCG64(77))           # same data on both ranks
        x = rng.uniform(-1, 1, (5, 9, 9, 8)).astype(np.float32)   # 5 images: slabs of 3 and 2
        f = rng.normal(0, 0.1, (3, 3, 8, 12)).astype(np.float32)
        lut = ax.noisy_table(3055)
        # rank 1 starts with different (wrong) ranges; after the broadcast both use rank 0's
        ranges = [(-1.0, 1.0, float(f.min()), float(f.max()))] if rank == 0 else [(-9.0, 9.0, -9.0, 9.0)]
        ranges = parallel.broadcast_ranges(ranges, src=0)
        assert ranges == [(-1.0, 1.0, float(f.min()), float(f.max()))]
        lo, hi = parallel.shard_bounds(5, world, rank)
        assert (lo, hi) == ((0, 3) if rank == 0 else (3, 5))
        xs = parallel.shard_batch(torch.from_numpy(x)).numpy()
        assert xs.shape[0] == hi - lo
        d = O.desc(xs.shape[0], 9, 9, 8, 3, 3, 12)
        y = O.conv2d(d, lut, xs, f, *ranges[0], want=("out_exact",))["out_exact"]
        full = parallel.gather_outputs(torch.from_numpy(y)).numpy()
        want = O.conv2d(O.desc(5, 9, 9, 8, 3, 3, 12), lut, x, f, *ranges[0], want=("out_exact",))["out_exact"]
        assert full.shape == want.shape and np.array_equal(full.view(np.uint32), want.view(np.uint32))
        open(os.path.join(tmpdir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding(built, tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")


def test_shard_bounds_cover_the_batch():
    sys.path.insert(0, ROOT)
    from tf_approximate_b200.parallel import shard_bounds
    for n in (0, 1, 7, 8, 256, 1001):
        for w in (1, 2, 3, 8):
            b = [shard_bounds(n, w, r) for r in range(w)]
            assert b[0][0] == 0 and b[-1][1] == n
            assert all(b[i][1] == b[i + 1][0] for i in range(w - 1))
            assert max(hi - lo for lo, hi in b) - min(hi - lo for lo, hi in b) <= 1
