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


def _placement_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    import xor_net_b200 as xn

    # what every rank of `bench.py --gpus N` does before it builds its streams: ONE global list of
    # N x 64 lengths (the same seed on every rank), placed by the library's own rule
    lens = bench.stream_lengths(world * 64, 128, 4096, bench.BASE_SEED + 3000)
    owners = {p: bench.place_streams(xn, lens, world, p) for p in ("least", "rr")}
    mine = [i for i, w in enumerate(owners["least"]) if w == rank]
    gathered = [None] * world
    dist.all_gather_object(gathered, (owners, mine, int(sum(int(lens[i]) for i in mine))))
    if rank == 0:
        out.put((gathered, [int(x) for x in lens]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_one_global_stream_list_is_placed_identically_on_every_rank(world):
    """The decode benchmark shards ONE list of streams over the ranks with the device group's
    placement rule.  Every rank must derive the same owners on its own (no collective on the data
    path), the ranks' shares must partition the list, and the least-loaded rule must balance the
    cached tokens better than stream-number-modulo-N does."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_placement_worker, args=(r, world, port, out)) for r in range(world)]
    [p.start() for p in procs]
    gathered, lens = out.get(timeout=180)
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    owners0 = gathered[0][0]
    assert all(g[0] == owners0 for g in gathered)                       # the same plan on every rank
    assert sorted(i for g in gathered for i in g[1]) == list(range(world * 64))
    tokens = [g[2] for g in gathered]
    assert sum(tokens) == sum(lens)
    assert max(tokens) - min(tokens) <= 4096                             # within one stream of each other
    rr = [sum(lens[i] for i in range(len(lens)) if owners0["rr"][i] == r) for r in range(world)]
    assert max(tokens) <= max(rr)
    assert owners0["rr"] == [i % world for i in range(world * 64)]
