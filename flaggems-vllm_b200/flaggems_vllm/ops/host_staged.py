"""The prologue for callers whose tokens live in (pinned) host memory.

`HostStagedPrologue` streams q / kv / slot_mapping / position_ids to the device in token
chunks, runs the fused kernel on each chunk and streams the rewritten q back, with the
host->device copy, the kernel and the device->host copy of neighbouring chunks overlapped
on three CUDA streams (PCIe is full duplex).  The paged K cache and the cos/sin table stay
resident on the device, as they do in serving.  Device staging buffers are allocated once,
at construction.
"""
from __future__ import annotations

import torch

from .fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert import fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert


class HostStagedPrologue:
    def __init__(self, num_heads: int, chunk_tokens: int = 1024, device="cuda", depth: int = 3):
        self.device = torch.device(device)
        self.chunk = int(chunk_tokens)
        self.heads = int(num_heads)
        self.depth = depth
        dev = self.device
        self.q = [torch.empty(self.chunk, self.heads, 512, dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self.kv = [torch.empty(self.chunk, 512, dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self.slots = [torch.empty(self.chunk, dtype=torch.int64, device=dev) for _ in range(depth)]
        self.pos = [torch.empty(self.chunk, dtype=torch.int64, device=dev) for _ in range(depth)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(depth)]
        self.ev_run = [torch.cuda.Event() for _ in range(depth)]
        self.ev_out = [torch.cuda.Event() for _ in range(depth)]
        self.launches = 0

    def __call__(self, q_host, kv_host, k_cache, slot_mapping_host, position_ids_host, cos_sin_cache, eps,
                 cache_block_size, q_out_host=None):
        """Same meaning as the operator, with q, kv, slot_mapping and position_ids on the host
        (pinned for real overlap).  q_out_host (default: q_host, i.e. in place) receives the
        rewritten q.  Returns after everything has landed in host memory."""
        n = q_host.shape[0]
        n_ins = slot_mapping_host.shape[0]
        assert q_host.shape[1] == self.heads and kv_host.shape[0] == n and n_ins <= n
        q_out_host = q_host if q_out_host is None else q_out_host
        caller = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(caller)
        self.s_run.wait_stream(caller)
        self.launches = 0
        for i, a in enumerate(range(0, n, self.chunk)):
            b = min(a + self.chunk, n)
            k, m = i % self.depth, b - a
            ins = max(0, min(b, n_ins) - a)
            with torch.cuda.stream(self.s_in):
                if i >= self.depth:
                    self.s_in.wait_event(self.ev_out[k])  # staging set k was drained
                self.q[k][:m].copy_(q_host[a:b], non_blocking=True)
                self.kv[k][:m].copy_(kv_host[a:b], non_blocking=True)
                self.pos[k][:m].copy_(position_ids_host[a:b], non_blocking=True)
                if ins:
                    self.slots[k][:ins].copy_(slot_mapping_host[a : a + ins], non_blocking=True)
                self.ev_in[k].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[k])
                fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert(
                    self.q[k][:m], self.kv[k][:m], k_cache, self.slots[k][:ins], self.pos[k][:m], cos_sin_cache, eps,
                    cache_block_size)
                self.launches += 1
                self.ev_run[k].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[k])
                q_out_host[a:b].copy_(self.q[k][:m], non_blocking=True)
                self.ev_out[k].record(self.s_out)
        caller.wait_stream(self.s_out)
        caller.wait_stream(self.s_run)
        self.s_out.synchronize()
        return q_out_host
