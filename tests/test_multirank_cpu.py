"""The N>1 host logic on CPU: two gloo ranks partition streams and heads, then agree on the
job-wide time (max over ranks) and work (sum over ranks) exactly as the benchmark does."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from xor_net_b200 import sharding

    mine = sharding.streams_of_rank(256, world, rank)
    heads = sharding.query_heads_of_rank(32, 8, world, rank)
    gathered = [None] * world
    dist.all_gather_object(gathered, (mine, heads))
    # every rank reports its own time and work; the job-wide numbers must agree on all ranks
    times, work = sharding.aggregate([10.0 + rank, 5.0 - rank], [100.0 * (rank + 1)])
    if rank == 0:
        out.put((gathered, times, work))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_partition_and_aggregation_across_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    [p.start() for p in procs]
    gathered, times, work = out.get(timeout=120)
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    streams = sorted(s for mine, _ in gathered for s in mine)
    assert streams == list(range(256))                       # every stream on exactly one rank
    for r, (mine, heads) in enumerate(gathered):
        assert all(s % world == r for s in mine)             # round-robin rule
        assert heads == list(range(r * 32 // world, (r + 1) * 32 // world))  # contiguous head blocks
    heads = sorted(h for _, hs in gathered for h in hs)
    assert heads == list(range(32))
    assert times == [10.0 + world - 1, 5.0]                  # max over ranks
    assert work == [100.0 * world * (world + 1) / 2]         # sum over ranks


def test_sharding_helpers_single_process():
    sys.path.insert(0, ROOT)
    from xor_net_b200 import sharding

    assert sharding.streams_of_rank(10, 4, 1) == [1, 5, 9]
    assert sharding.rank_of_stream(9, 4) == 1
    assert sharding.kv_heads_of_rank(8, 8, 3) == [3]
    assert sharding.query_heads_of_rank(32, 8, 2, 1) == list(range(16, 32))
    with pytest.raises(ValueError):
        sharding.kv_heads_of_rank(5, 2, 0)
    assert sharding.aggregate([1.0], [2.0]) == ([1.0], [2.0])
    with pytest.raises(ValueError):
        sharding.streams_of_rank(4, 2, 2)
