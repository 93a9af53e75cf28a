"""Multi-process (CPU, gloo, world_size 2) check of the N > 1 host logic: sessions are partitioned over the
ranks with no overlap and no gap, and the timing reduction the benchmark uses (max over ranks) works."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from world_engine_b200.sessions import shard_sessions


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n_sessions: int, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = shard_sessions(n_sessions, world, rank)
    owned = torch.zeros(n_sessions, dtype=torch.int64)
    owned[mine] = 1
    dist.all_reduce(owned)                                   # every session owned exactly once
    t = torch.tensor([10.0 + rank], dtype=torch.float64)     # the benchmark reports the slowest rank
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    if rank == 0:
        out.put((owned.tolist(), float(t), len(mine)))
    dist.destroy_process_group()


def test_sessions_are_partitioned_across_two_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 7, out)) for r in range(2)]
    for p in procs:
        p.start()
    owned, slowest, n0 = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert owned == [1] * 7
    assert slowest == 11.0
    assert n0 == 4


def test_shard_helper_edges():
    assert shard_sessions(0, 4, 3) == []
    assert shard_sessions(3, 8, 5) == []
    assert shard_sessions(64, 8, 7) == list(range(7, 64, 8))
    assert sorted(sum((shard_sessions(13, 4, r) for r in range(4)), [])) == list(range(13))
