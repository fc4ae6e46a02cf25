"""The N > 1 path on CPU: two gloo ranks each run their slice of the batch (on the CPU oracle standing in for the
device) and the gathered result equals the single-process full-batch result."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from armnn_b200.sharding import gather_rows, shard_range

HERE = os.path.dirname(os.path.abspath(__file__))


def test_shard_ranges_partition_the_batch():
    for batch in (256, 7, 1, 0):
        for world in (1, 2, 3, 4, 8):
            rows = [shard_range(batch, world, r) for r in range(world)]
            assert rows[0][0] == 0 and rows[-1][1] == batch
            for (a, b), (c, d) in zip(rows, rows[1:]):
                assert b == c and a <= b
            sizes = [b - a for a, b in rows]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _worker(rank, world, port, batch, out_path):
    sys.path.insert(0, HERE)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import hostnet
    from armnn_b200 import configs, network
    a, b = shard_range(batch, world, rank)
    rng = np.random.default_rng(11)
    x_full = rng.integers(-128, 128, size=(batch, 32, 32, 3)).astype(np.int8)
    net, info = configs.resnet50(b - a, 32)
    y = hostnet.OracleNetwork(network.Optimize(net)).run({0: x_full[a:b]})[0]
    full = gather_rows(torch.from_numpy(y), batch)
    if rank == 0:
        np.save(out_path, full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_full_batch(built, tmp_path):
    import hostnet
    from armnn_b200 import configs, network
    batch, world = 3, 2
    out = str(tmp_path / "gathered.npy")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, batch, out), nprocs=world, join=True)
    rng = np.random.default_rng(11)
    x_full = rng.integers(-128, 128, size=(batch, 32, 32, 3)).astype(np.int8)
    net, info = configs.resnet50(batch, 32)
    want = hostnet.OracleNetwork(network.Optimize(net)).run({0: x_full})[0]
    assert np.array_equal(np.load(out), want)
