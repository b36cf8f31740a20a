"""Seeded workload generators and the algorithmic-byte count.  No GPU."""
from __future__ import annotations

import torch

from flaggems_vllm.testing import workloads


def test_shard_sizes_are_uneven_floored_and_exact():
    for world in (1, 2, 4, 8):
        sizes = workloads.shard_sizes(32768 * world, world, seed=0)
        assert len(sizes) == world and sum(sizes) == 32768 * world and min(sizes) >= 4096
        assert sizes == workloads.shard_sizes(32768 * world, world, seed=0)
    assert len(set(workloads.shard_sizes(262144, 8, seed=0))) > 1


def test_algorithmic_bytes_formula():
    slots = torch.tensor([3, -1, 7, 9], dtype=torch.int64)
    # 5 tokens, 128 heads: 5*(2048*128+264) + 4 slot entries*8 + 3 valid*1608
    assert workloads.algorithmic_bytes(5, 128, slots) == 5 * (262144 + 264) + 32 + 3 * 1608
    full = torch.arange(8192, dtype=torch.int64)
    assert workloads.algorithmic_bytes(8192, 128, full) == 8192 * 264024


def test_small_workloads_have_the_documented_structure():
    w = workloads.make("cpu_ref")
    assert w.q.shape == (256, 8, 512) and w.k_cache.shape == (64, 64 * 584) and w.cos_sin_cache.shape == (4096, 64)
    assert w.slot_mapping.unique().numel() == 256 and int(w.position_ids.max()) < 4096
    p = workloads.make("prefill", num_tokens=4096 + 100, num_heads=2, num_blocks=128)
    assert p.meta["sequences"] == 3
    runs = p.position_ids[:2048]
    assert torch.equal(runs, runs[0] + torch.arange(2048))
    assert torch.equal(p.slot_mapping[:64], p.slot_mapping[0] + torch.arange(64)) and int(p.slot_mapping[0]) % 64 == 0
    assert p.slot_mapping.unique().numel() == p.num_tokens
    lp = workloads.make("long_prefill", num_tokens=1000, num_heads=1, num_blocks=32)
    assert int((lp.slot_mapping < 0).sum()) == 100 and lp.meta["outlier_rows"] == 10
    valid = lp.slot_mapping[lp.slot_mapping >= 0]
    assert valid.unique().numel() == valid.numel()
    assert float(lp.kv.float().abs().max()) > 50.0
    s0 = workloads.make("sharded", rank=0, world=2, num_heads=1, num_blocks=256, total_tokens=8192 + 4096)
    s1 = workloads.make("sharded", rank=1, world=2, num_heads=1, num_blocks=256, total_tokens=8192 + 4096)
    assert s0.num_tokens + s1.num_tokens == 8192 + 4096
    assert not torch.equal(s0.kv[:16], s1.kv[:16])
