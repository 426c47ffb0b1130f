"""Multi-GPU partitioning of the attention path: one process per GPU, no data-path collective.

Decode shards by stream: stream ``i`` lives on GPU ``i mod world`` for its whole life (its pages
are in that GPU's pool), so a decode step needs no exchange between GPUs.  A long prefill can be
split by KV-head group: GPU ``g`` owns a contiguous block of KV heads and their query heads; only the
per-head outputs are gathered at the end.  The only collectives here are the ones a benchmark
needs to agree on a result (maximum time over ranks, total work), and they run on whatever
``torch.distributed`` backend the caller initialised (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def streams_of_rank(n_streams: int, world: int, rank: int) -> List[int]:
    """Global stream ids owned by ``rank``: round-robin, ``gpu = stream_id mod n_gpus``."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("need 0 <= rank < world")
    return list(range(rank, n_streams, world))


def rank_of_stream(stream_id: int, world: int) -> int:
    return stream_id % world


def kv_heads_of_rank(num_kv_heads: int, world: int, rank: int) -> List[int]:
    """KV heads (and with them the query-head groups) a rank computes in a head-split prefill:
    contiguous blocks, so that the gathered per-rank outputs are already in head order."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("need 0 <= rank < world")
    if num_kv_heads % world != 0:
        raise ValueError("the number of KV heads must be a multiple of the number of GPUs")
    per = num_kv_heads // world
    return list(range(rank * per, (rank + 1) * per))


def query_heads_of_rank(num_heads: int, num_kv_heads: int, world: int, rank: int) -> List[int]:
    group = num_heads // num_kv_heads
    return [h * group + g for h in kv_heads_of_rank(num_kv_heads, world, rank) for g in range(group)]


def aggregate(times_ms: Sequence[float], work: Sequence[float], device=None) -> Tuple[List[float], List[float]]:
    """Job-wide figures from per-rank ones: element-wise MAX of ``times_ms`` and SUM of ``work``.

    Without an initialised process group (single process) the inputs are returned unchanged.
    """
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(times_ms), list(work)
    t = torch.tensor(list(times_ms), dtype=torch.float64, device=device)
    w = torch.tensor(list(work), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(w, op=dist.ReduceOp.SUM)
    return t.tolist(), w.tolist()
