"""The operator stated with torch tensor ops on CPU.  TEST INFRASTRUCTURE ONLY.

A restatement, in this project's own words, of the torch reference path that the
upstream project keeps in tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py
(`ref_impl`, T:316-333, with its helpers T:93-243).  It uses the same torch
primitives in the same order (pow/mean/rsqrt; two rounded products then add or
subtract; clamp/div/log2/ceil; Tensor.to(float8_e4m3fn)), so on the same torch
build it reproduces that path bit for bit - which the golden-vector tests check.
It is the "reference's CPU torch path" that the benchmark times beside the GPU
kernel.  Unlike the upstream oracle it leaves `kv` untouched.
"""
from __future__ import annotations

import torch

HEAD_DIM, ROPE_DIM, NOPE_DIM = 512, 64, 448
GROUP, N_GROUPS = 64, 7
DATA_BYTES, SCALE_BYTES = 576, 8
Q_ROWS_PER_CHUNK = 1 << 19  # rows of q normalised at once (T:292-299 bounds temporaries the same way)


def _rotate(tail_f32: torch.Tensor, cs: torch.Tensor) -> torch.Tensor:
    """GPT-J rotation (T:93-140) of `tail_f32` [..., 64] by cs rows [tokens, 64] = cos|sin."""
    c, s = cs[:, :32], cs[:, 32:]
    while c.dim() < tail_f32.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    pairs = tail_f32.unflatten(-1, (32, 2))
    ev, od = pairs[..., 0], pairs[..., 1]
    return torch.stack((ev * c - od * s, ev * s + od * c), dim=-1).flatten(-2)


def q_inplace(q: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor, eps: float) -> None:
    """Weight-less RMSNorm (T:143-148) + tail rotation of every q row, in place."""
    n, h, _ = q.shape
    step = max(1, Q_ROWS_PER_CHUNK // max(h, 1))
    for a in range(0, n, step):
        rows = q[a : a + step]
        xf = rows.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
        cs = cos_sin_cache[positions[a : a + step]].float()
        rows[..., NOPE_DIM:] = _rotate(xf[..., NOPE_DIM:], cs).to(q.dtype)
        rows[..., :NOPE_DIM] = xf[..., :NOPE_DIM].to(q.dtype)


def kv_insert(kv, k_cache, slot_mapping, positions, cos_sin_cache, block_size: int) -> None:
    """Rotate the raw tail, quantise the raw head with UE8M0 scales, scatter (T:178-243)."""
    n_ins = slot_mapping.shape[0]
    tok = torch.nonzero(slot_mapping >= 0).flatten()
    if tok.numel() == 0:
        return
    slot = slot_mapping[tok]
    rows = kv[:n_ins][tok]
    blk, pos = slot // block_size, slot % block_size
    data_off = pos * DATA_BYTES
    scale_off = block_size * DATA_BYTES + pos * SCALE_BYTES

    cs = cos_sin_cache[positions[:n_ins][tok]].float()
    tail = _rotate(rows[:, NOPE_DIM:].float(), cs).to(torch.bfloat16).contiguous()
    span = torch.arange(2 * ROPE_DIM)
    k_cache[blk[:, None], (data_off + NOPE_DIM)[:, None] + span] = tail.view(torch.uint8)

    g = rows[:, :NOPE_DIM].float().unflatten(-1, (N_GROUPS, GROUP))
    amax = g.abs().amax(dim=-1).clamp(min=1e-4)
    exponent = torch.ceil(torch.log2(amax / 448.0))
    code = (exponent.to(torch.int32) + 127).clamp(0, 255)
    scale = (code << 23).view(torch.float32)  # exact power of two (T:154-163)
    fp8 = (g / scale[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    k_cache[blk[:, None], data_off[:, None] + torch.arange(NOPE_DIM)] = fp8.flatten(1)
    k_cache[blk[:, None], scale_off[:, None] + torch.arange(N_GROUPS)] = (exponent + 127.0).clamp(0.0, 255.0).to(torch.uint8)
    k_cache[blk, scale_off + N_GROUPS] = 0


def prologue(q, kv, k_cache, slot_mapping, position_ids, cos_sin_cache, eps, cache_block_size) -> None:
    """Operator semantics on CPU tensors: q and k_cache change in place, kv does not."""
    q_inplace(q, position_ids, cos_sin_cache, eps)
    kv_insert(kv, k_cache, slot_mapping, position_ids, cos_sin_cache, cache_block_size)


def cos_sin_table(max_pos: int, theta: float = 10000.0) -> torch.Tensor:
    """fp32 [max_pos, 64]: 32 cos then 32 sin of pos * theta^(-2i/64) (layout of T:68-90)."""
    inv = 1.0 / (theta ** (torch.arange(0, ROPE_DIM, 2, dtype=torch.float32) / ROPE_DIM))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.cat((ang.cos(), ang.sin()), dim=-1)
