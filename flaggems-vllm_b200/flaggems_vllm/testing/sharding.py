"""Token sharding across GPUs: one process per GPU, one K cache per GPU, no data-path collective.

The operator needs no exchange between ranks (every token is independent and each rank owns
the cache its tokens go to), so the only cross-rank step is bookkeeping: the job's time is the
slowest rank's, its work is the sum over ranks, and a failure on any rank fails the job.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def aggregate(seconds: float, tokens: int, nbytes: int, launches: int, status: int = 0, device="cpu") -> dict:
    """Combine per-rank measurements.  Works without a process group (single rank).

    Returns max-over-ranks seconds, summed tokens / bytes / launches, the largest shard's tokens and
    bytes (the kernel the step waits for), the OR of the ranks' status words, and the sum over ranks of
    tokens/seconds (what the ranks deliver when they do not wait for each other, i.e. uneven shards
    without a per-step barrier)."""
    rate = tokens / seconds if seconds > 0 else 0.0
    t = torch.tensor([seconds, float(tokens), float(nbytes), float(launches), float(status), rate], dtype=torch.float64,
                     device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        mx, sm = t.clone(), t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        world = dist.get_world_size()
    else:
        mx, sm, world = t, t, 1
    return {
        "world": world, "seconds": float(mx[0]), "tokens": int(sm[1]), "bytes": int(sm[2]), "launches": int(sm[3]),
        "largest_tokens": int(mx[1]), "largest_bytes": int(mx[2]), "failed": bool(mx[4] != 0),
        "sum_of_rank_rates": float(sm[5]),
    }
