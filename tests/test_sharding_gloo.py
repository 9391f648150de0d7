"""CPU, world_size 2 over gloo: the (batch, kv-head group) sharding used by bench.py at N > 1. The path has no data
collective: every rank takes a contiguous slice of the b * h_kv groups; only the timing is reduced (max over ranks)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bench import shard_groups


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = shard_groups(4 * 16, rank, world)
    t = torch.tensor([float(hi - lo), 1.0 + rank])
    dist.all_reduce(t[0:1], op=dist.ReduceOp.SUM)       # every group is owned exactly once
    dist.all_reduce(t[1:2], op=dist.ReduceOp.MAX)       # the timing reduction bench.py uses
    out[rank] = (lo, hi, t.tolist())
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_partition_the_groups():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    (lo0, hi0, t0), (lo1, hi1, t1) = out[0], out[1]
    assert (lo0, hi0, lo1, hi1) == (0, 32, 32, 64)
    assert t0 == [64.0, 2.0] and t1 == [64.0, 2.0]


def test_uneven_split_covers_everything_once():
    for n, w in ((7, 2), (64, 8), (5, 8), (16, 4)):
        seen = []
        for r in range(w):
            lo, hi = shard_groups(n, r, w)
            seen += list(range(lo, hi))
        assert seen == list(range(n))
