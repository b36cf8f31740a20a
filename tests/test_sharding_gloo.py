"""The N>1 path on CPU: two gloo ranks build their own shard of the token-sharded workload, run the
CPU oracle on it (standing in for the kernel, which has no CPU path) and aggregate.  No GPU."""
from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _rank_main(rank: int, world: int, init_file: str, out_dir: str, fail_rank: int):
    sys.path[:0] = [str(ROOT / "flaggems-vllm_b200"), str(ROOT)]
    from flaggems_vllm.testing import sharding, workloads
    from oracle import c_oracle

    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    total = 4096 * world + 1500
    w = workloads.make("sharded", device="cpu", seed=0, rank=rank, world=world, total_tokens=total, num_heads=2,
                       num_blocks=256)
    sizes = workloads.shard_sizes(total, world, seed=0)
    assert w.num_tokens == sizes[rank]
    status = 0
    try:
        if rank == fail_rank:
            raise RuntimeError("injected host-side failure on this rank")
        c_oracle.prologue(*w.args(), threads=1)
    except RuntimeError:
        status = 1
    agg = sharding.aggregate(0.001 * (rank + 1), w.num_tokens, w.algorithmic_bytes(), 1, status)
    torch.save({"agg": agg, "tokens": w.num_tokens, "kv_head": w.kv[:4].clone(), "bytes": w.algorithmic_bytes()},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _run(world: int, fail_rank: int = -1):
    with tempfile.TemporaryDirectory() as tmp:
        init_file = os.path.join(tmp, "rendezvous")
        mp.spawn(_rank_main, args=(world, init_file, tmp, fail_rank), nprocs=world, join=True)
        return [torch.load(os.path.join(tmp, f"rank{r}.pt")) for r in range(world)]


def test_two_ranks_shard_tokens_and_aggregate():
    res = _run(2)
    total = 4096 * 2 + 1500
    assert sum(r["tokens"] for r in res) == total and res[0]["tokens"] != res[1]["tokens"]
    assert not torch.equal(res[0]["kv_head"], res[1]["kv_head"]), "ranks must draw different tokens"
    for r in res:
        a = r["agg"]
        assert a["world"] == 2 and a["tokens"] == total and a["launches"] == 2 and not a["failed"]
        assert abs(a["seconds"] - 0.002) < 1e-12, "job time is the slowest rank's"
        assert a["bytes"] == sum(x["bytes"] for x in res)
        assert a["largest_tokens"] == max(x["tokens"] for x in res)
        want = sum(x["tokens"] / (0.001 * (i + 1)) for i, x in enumerate(res))
        assert abs(a["sum_of_rank_rates"] - want) < 1e-6 * want


def test_failure_on_one_rank_is_seen_by_all_and_others_finish():
    res = _run(2, fail_rank=1)
    assert all(r["agg"]["failed"] for r in res)
    assert res[0]["agg"]["tokens"] == 4096 * 2 + 1500  # the healthy rank still completed and reported


def test_single_rank_needs_no_process_group():
    sys.path[:0] = [str(ROOT / "flaggems-vllm_b200")]
    from flaggems_vllm.testing import sharding

    a = sharding.aggregate(0.5, 10, 100, 3)
    assert a == {"world": 1, "seconds": 0.5, "tokens": 10, "bytes": 100, "launches": 3, "largest_tokens": 10,
                 "largest_bytes": 100, "failed": False, "sum_of_rank_rates": 20.0}
