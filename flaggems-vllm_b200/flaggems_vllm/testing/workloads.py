"""Seeded synthetic workloads for the DeepSeek-V4 attention prologue.

The five named workloads stand in for real serving traffic (no dataset exists for
this operator; the upstream benchmark also feeds it seeded random tensors,
benchmark/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:195-236).
Tensors follow the operator's contract
(src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:289-333):
q bf16 [N,H,512], kv bf16 [N,512], k_cache uint8 [blocks, block_size*584],
slot_mapping / position_ids int64, cos/sin fp32 [max_pos, 64] = 32 cos | 32 sin.

Random draws use a `torch.Generator` of the target device seeded with `seed`, so
a workload is reproducible per device type; tests copy the device tensors to the
host for the CPU oracle, which therefore always sees the same bits as the GPU.
The cache is pre-filled with random bytes so that untouched bytes are observable.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

HEAD_DIM, ROPE_DIM, NOPE_DIM = 512, 64, 448
TOKEN_DATA_BYTES, SCALE_BYTES, TOKEN_BYTES = 576, 8, 584

WORKLOADS = ("cpu_ref", "decode", "prefill", "long_prefill", "sharded")


@dataclass
class Workload:
    name: str
    q: torch.Tensor
    kv: torch.Tensor
    k_cache: torch.Tensor
    slot_mapping: torch.Tensor
    position_ids: torch.Tensor
    cos_sin_cache: torch.Tensor
    eps: float
    cache_block_size: int
    meta: dict = field(default_factory=dict)

    def args(self):
        """Positional arguments of the operator, in its order."""
        return (self.q, self.kv, self.k_cache, self.slot_mapping, self.position_ids,
                self.cos_sin_cache, self.eps, self.cache_block_size)

    @property
    def num_tokens(self) -> int:
        return self.q.shape[0]

    @property
    def num_heads(self) -> int:
        return self.q.shape[1]

    def algorithmic_bytes(self) -> int:
        return algorithmic_bytes(self.num_tokens, self.num_heads, self.slot_mapping)


def algorithmic_bytes(num_tokens: int, num_heads: int, slot_mapping: torch.Tensor) -> int:
    """Bytes the operator must move: per token q read+write (2048*H), position (8)
    and its cos/sin row (256); +8 for each slot_mapping entry; +1608 for each
    entry >= 0 (1024 kv read + 576 cache data + 8 scale bytes)."""
    n_ins = int(slot_mapping.shape[0])
    n_valid = int((slot_mapping >= 0).sum().item())
    return num_tokens * (2048 * num_heads + 264) + 8 * n_ins + 1608 * n_valid


def cos_sin_table(max_pos: int, theta: float = 10000.0, device="cpu") -> torch.Tensor:
    """fp32 [max_pos, 64]; row p = cos(p*f_i) for 32 frequencies f_i = theta^(-2i/64), then
    the 32 sines.  Always computed on the host so every device sees identical rows."""
    inv = 1.0 / (theta ** (torch.arange(0, ROPE_DIM, 2, dtype=torch.float32) / ROPE_DIM))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.cat((ang.cos(), ang.sin()), dim=-1).to(device)


def shard_sizes(total_tokens: int, world: int, seed: int = 0, alpha: float = 5.0, floor: int = 4096) -> list[int]:
    """Uneven token counts per GPU: Dirichlet(alpha) shares of `total_tokens`, each at
    least `floor`, summing exactly to `total_tokens`."""
    if world == 1:
        return [total_tokens]
    assert total_tokens >= floor * world
    share = np.random.default_rng(seed).dirichlet([alpha] * world)
    sizes = np.maximum(floor, np.rint(share * total_tokens).astype(np.int64))
    # hand the rounding / floor surplus back to (or take it from) the largest shards
    diff = int(total_tokens - sizes.sum())
    while diff != 0:
        i = int(np.argmax(sizes))
        if diff > 0:
            sizes[i] += diff
            diff = 0
        else:
            take = min(-diff, int(sizes[i] - floor))
            sizes[i] -= take
            diff += take
    return [int(s) for s in sizes]


def _gen(device, seed: int) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def _randn_bf16(shape, g, device, chunk_rows: int = 1 << 14) -> torch.Tensor:
    """N(0,1) bf16 filled chunk by chunk (keeps the fp32 temporary small)."""
    out = torch.empty(shape, dtype=torch.bfloat16, device=device)
    flat = out.view(shape[0], -1)
    for a in range(0, shape[0], chunk_rows):
        rows = flat[a : a + chunk_rows]
        rows.copy_(torch.randn(rows.shape, generator=g, device=device, dtype=torch.float32))
    return out


def _random_cache(num_blocks: int, block_bytes: int, g, device) -> torch.Tensor:
    out = torch.empty(num_blocks, block_bytes, dtype=torch.uint8, device=device)
    step = max(1, (1 << 28) // block_bytes)
    for a in range(0, num_blocks, step):
        rows = out[a : a + step]
        rows.copy_(torch.randint(0, 256, rows.shape, generator=g, device=device, dtype=torch.uint8))
    return out


def _sequence_runs(n: int, run: int, start_hi: int, g, device):
    """Positions as runs of `run` contiguous values from random starts in [0, start_hi)."""
    n_runs = (n + run - 1) // run
    starts = torch.randint(0, start_hi, (n_runs,), generator=g, device=device, dtype=torch.int64)
    pos = (starts[:, None] + torch.arange(run, device=device, dtype=torch.int64)[None, :]).flatten()[:n]
    return pos.contiguous(), n_runs


def make(name: str, device="cpu", seed: int = 0, *, num_tokens: int | None = None,
         num_heads: int | None = None, num_blocks: int | None = None, rank: int = 0, world: int = 1,
         total_tokens: int | None = None) -> Workload:
    """Build one of the named workloads.

    cpu_ref       N=256  H=8   max_pos 4096    64 blocks     slots = first N of a permutation
    decode        N=256  H=128 max_pos 65536   16384 blocks  distinct random slots, random positions
    prefill       N=8192 H=128 max_pos 65536   16384 blocks  4 sequences x 2048 contiguous positions,
                                                             slots contiguous inside random blocks
    long_prefill  N=32768 H=128 max_pos 131072 65536 blocks  10% slots = -1, 1% of rows x50 (q and kv)
    sharded       rank `rank` of `world`: N = its Dirichlet share of `total_tokens`
                  (default 32768 per GPU), H=128, max_pos 65536, 65536-block cache of its own
    `num_tokens` / `num_heads` / `num_blocks` override the sizes (used by reduced-size tests).
    """
    bs = 64
    dev = torch.device(device)
    if name == "sharded":
        total = total_tokens if total_tokens is not None else 32768 * world
        n_default = shard_sizes(total, world, seed=seed)[rank]
        seed = seed * 1000 + rank + 1
    g = _gen(dev, seed)
    spec = {
        "cpu_ref": (256, 8, 4096, 64),
        "decode": (256, 128, 65536, 16384),
        "prefill": (8192, 128, 65536, 16384),
        "long_prefill": (32768, 128, 131072, 65536),
        "sharded": (n_default if name == "sharded" else 0, 128, 65536, 65536),
    }[name]
    n = num_tokens if num_tokens is not None else spec[0]
    h = num_heads if num_heads is not None else spec[1]
    max_pos = spec[2]
    num_blocks = num_blocks if num_blocks is not None else spec[3]
    assert num_blocks * bs >= n, "cache too small for distinct slots"

    q = _randn_bf16((n, h, HEAD_DIM), g, dev)
    kv = _randn_bf16((n, HEAD_DIM), g, dev)
    k_cache = _random_cache(num_blocks, bs * TOKEN_BYTES, g, dev)
    cs = cos_sin_table(max_pos, device=dev)
    meta: dict = {"num_blocks": num_blocks, "max_pos": max_pos, "seed": seed}

    def distinct_slots(count):
        return torch.randperm(num_blocks * bs, generator=g, device=dev)[:count].to(torch.int64).contiguous()

    if name == "cpu_ref":
        pos = torch.randint(0, max_pos, (n,), generator=g, device=dev, dtype=torch.int64)
        slots = distinct_slots(n)
    elif name == "decode":
        pos = torch.randint(0, max_pos, (n,), generator=g, device=dev, dtype=torch.int64)
        slots = distinct_slots(n)
    elif name == "prefill":
        pos, n_runs = _sequence_runs(n, 2048, 32768, g, dev)
        blocks_needed = (n + bs - 1) // bs
        table = torch.randperm(num_blocks, generator=g, device=dev)[:blocks_needed].to(torch.int64)
        i = torch.arange(n, device=dev, dtype=torch.int64)
        slots = (table[i // bs] * bs + i % bs).contiguous()
        meta["sequences"] = n_runs
    elif name == "long_prefill":
        pos = torch.randint(0, max_pos, (n,), generator=g, device=dev, dtype=torch.int64)
        slots = distinct_slots(n)
        pad = torch.randperm(n, generator=g, device=dev)[: n // 10]
        slots[pad] = -1
        hot = torch.randperm(n, generator=g, device=dev)[: max(1, n // 100)]
        q[hot] = (q[hot].float() * 50.0).to(torch.bfloat16)
        kv[hot] = (kv[hot].float() * 50.0).to(torch.bfloat16)
        meta["outlier_rows"] = int(hot.numel())
        meta["padding_tokens"] = int(pad.numel())
    else:  # sharded
        pos, n_runs = _sequence_runs(n, 2048, 32768, g, dev)
        slots = distinct_slots(n)
        meta.update(rank=rank, world=world, sequences=n_runs)
    return Workload(name, q, kv, k_cache, slots, pos, cs, 1e-6, bs, meta)
