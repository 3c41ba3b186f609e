"""Multi-rank logic on CPU (gloo, world size 2): the batch is split over ranks, every rank works
on its own planes with no collective on the path, and the max-over-ranks timing reduction and the
gather of per-rank outputs reproduce the single-rank result.  The per-rank operator is the numpy
oracle here (no GPU in this test); what is checked is the sharding arithmetic bench.py relies on."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import converse2d_oracle as orc


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
    per = x.shape[0] // world
    mine = x[rank * per:(rank + 1) * per]
    y = torch.from_numpy(orc.converse2d_forward(mine, w, b, 2, 2, "circular", 1e-5, dtype=np.float64))
    t = torch.tensor([float(rank + 1)])            # stand-in for this rank's elapsed time
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    gathered = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(gathered, y)                   # off the timed path: only to compare
    if rank == 0:
        np.save(out_path, torch.cat(gathered).numpy())
        assert float(t) == float(world)
    dist.barrier()
    dist.destroy_process_group()


def test_batch_sharding_world_size_2(tmp_path):
    rng = np.random.default_rng(0)
    w, b = orc.init_weight(3, 5, rng)
    x = rng.standard_normal((4, 3, 12, 14)).astype(np.float32)
    out_path = str(tmp_path / "gathered.npy")
    mp.spawn(_worker, args=(2, _free_port(), x, w, b, out_path), nprocs=2, join=True)
    full = orc.converse2d_forward(x, w, b, 2, 2, "circular", 1e-5, dtype=np.float64)
    assert np.array_equal(np.load(out_path), full)
