"""Multi-rank logic on CPU (gloo, world size 2 and 3): `conversenet_b200.sharding` cuts a batch
into per-rank slices, every rank works on its own planes with no collective on the path, and the
max-over-ranks timing reduction and the gather of uneven per-rank outputs reproduce the
single-rank result.  The per-rank operator is the numpy oracle here (no GPU in this test); what is
checked is the product's sharding code that bench.py --gpus N runs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conversenet_b200.sharding import gather_batch, max_over_ranks, shard_batch, shard_tensor
from oracle import converse2d_oracle as orc


def test_shard_batch_covers_the_batch_once():
    for total in (0, 1, 5, 8, 16, 32, 33):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                start, count = shard_batch(total, r, world)
                assert count in (total // world, total // world + 1)
                seen += list(range(start, start + count))
            assert seen == list(range(total))
    assert shard_batch(8, 7, 8) == (7, 1) and shard_batch(3, 3, 4) == (3, 0)
    with pytest.raises(ValueError):
        shard_batch(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, x, w, b, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = shard_tensor(torch.from_numpy(x), rank, world).numpy()
    if mine.shape[0]:
        y = torch.from_numpy(orc.converse2d_forward(mine, w, b, 2, 2, "circular", 1e-5, dtype=np.float64))
    else:
        y = torch.empty((0, x.shape[1], 2 * x.shape[2], 2 * x.shape[3]), dtype=torch.float64)
    t = max_over_ranks(float(rank + 1))             # stand-in for this rank's elapsed time
    full = gather_batch(y, x.shape[0])              # off the timed path: only to compare
    if rank == 0:
        np.save(out_path, full.numpy())
        assert t == float(world)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,batch", [(2, 4), (3, 5), (3, 2)])
def test_batch_sharding_over_ranks(tmp_path, world, batch):
    rng = np.random.default_rng(0)
    w, b = orc.init_weight(3, 5, rng)
    x = rng.standard_normal((batch, 3, 12, 14)).astype(np.float32)
    out_path = str(tmp_path / "gathered.npy")
    mp.spawn(_worker, args=(world, _free_port(), x, w, b, out_path), nprocs=world, join=True)
    full = orc.converse2d_forward(x, w, b, 2, 2, "circular", 1e-5, dtype=np.float64)
    assert np.array_equal(np.load(out_path), full)
