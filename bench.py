#!/usr/bin/env python
"""Benchmark of the fused DeepSeek-V4 attention prologue on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass of the operator over one batch of synthetic tokens.
  N = 1 : workload "long_prefill" (32768 tokens x 128 heads, 10 % slots = -1, 1 % outlier rows)
  N > 1 : workload "sharded": 32768*N tokens split unevenly (seeded Dirichlet(5), each >= 4096)
          over the ranks, one K cache per GPU, no collective on the data path (weak scaling).
Rank 0 prints ONE JSON line: tokens/s over all GPUs (`value`, inputs resident in HBM), the
roofline of the kernel (algorithmic bytes / CUDA-event time against the measured copy
bandwidth), the same metric end to end from pinned host buffers (`e2e`), a CPU baseline, the
SM clocks sampled during the timed region and the number of kernel launches timed.
`--impl reference` times the CPU torch statement of the reference path instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path[:0] = [str(ROOT / "flaggems-vllm_b200"), str(ROOT)]

import torch  # noqa: E402

METRIC = "fused qnorm/RoPE/FP8-insert tokens/s"
HBM_FALLBACK_GBS = 6650.0  # an earlier B200 copy measurement, used only if MEASURED_PEAKS.json is absent
NOMINAL_HBM_GBS = 8000.0
CPU_SAMPLE_TOKENS = 2048
# DRAM traffic per token (dram__bytes_read.sum + dram__bytes_write.sum) of one ncu capture of the kernel, scaled by
# the tokens of the reported launch: traffic grows in proportion to tokens (no byte is shared between tokens).  The
# capture is of a smaller workload than the timed one because a profiler replays each launch about 40 times.
# To refresh after a kernel change: the --set full command in TRAFFIC_SOURCE["command"], then read both counters.
NCU_DRAM_BYTES_PER_TOKEN = 257191  # (1.084411 + 1.022503) GB over 8192 tokens x 128 heads
TRAFFIC_SOURCE = {
    "kind": "one ncu capture, scaled by tokens; not measured in this run",
    "kernel": "prologue_rows_kernel<2 rows/warp, 4 warps, 10 CTAs/SM, unchecked, in place, launch mode 2, shared-memory table staging>",
    "workload": "prefill: 8192 tokens x 128 heads (1 GiB of q, 2.2 GB on the device)",
    "captured": "2026-11-25, 1 x B200, CUDA 12.9, ncu --set full --clock-control none, second of two captured launches",
    "command": "ncu --set full --clock-control none -k regex:prologue_rows_kernel -s 3 -c 2 python bench.py --workload prefill "
               "--steps 2 --warmup 3 --no-e2e --no-cpu-baseline --no-extra",
    "dram_bytes_read": 1084411000, "dram_bytes_write": 1022503000, "tokens": 8192,
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", default=None, help="override the N=1 workload (decode, prefill, long_prefill)")
    ap.add_argument("--variant", type=int, default=None, help="kernel variant id (default: library's choice)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the decode / prefill side measurements")
    ap.add_argument("--upstream-shapes", action="store_true",
                    help="time the shapes of the reference's own benchmark for this operator; prints JSON and exits")
    ap.add_argument("--siblings-only", action="store_true",
                    help="time only the sibling operators (used to profile them); prints their JSON and exits")
    ap.add_argument("--sibling", default=None,
                    help="with --siblings-only: only the operators whose name contains this string, e.g. "
                         "'fused_inv_rope_fp8_quant[fp32' (one operator and its tensors: the form to run under a profiler)")
    return ap.parse_args()


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return HBM_FALLBACK_GBS, "fallback"


class ClockSampler:
    """nvidia-smi polling of one GPU during the timed region (reads settings, changes none)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            uuid = torch.cuda.get_device_properties(index).uuid
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id=GPU-{uuid}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])), mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def bind_to_gpu_numa_node(device_index: int):
    """Pin this process to the CPU cores next to its GPU (the "CPU Affinity" column of `nvidia-smi topo -m`), so that
    the pinned host buffers of the end-to-end leg are allocated on the GPU's own NUMA node and the ranks of a
    multi-GPU run do not all stream through one socket.  Reads settings only; returns the core list or None."""
    try:
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        q = subprocess.run(["nvidia-smi", "--query-gpu=index,uuid", "--format=csv,noheader"], capture_output=True, text=True,
                           timeout=20).stdout
        smi_index = next(int(line.split(",")[0]) for line in q.splitlines() if uuid in line)
        topo = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout.splitlines()
        header = next(line for line in topo if "CPU Affinity" in line)
        col = next(i for i, c in enumerate(header.split("\t")) if "CPU Affinity" in c)
        row = next(line for line in topo if line.split("\t")[0].strip() == f"GPU{smi_index}")
        spec = [c.strip() for c in row.split("\t")][col]
        cores = set()
        for part in spec.split(","):
            lo, _, hi = part.partition("-")
            cores.update(range(int(lo), int(hi or lo) + 1))
        cores &= os.sched_getaffinity(0)
        if cores:
            os.sched_setaffinity(0, cores)
            return sorted(cores)
    except Exception:
        pass
    return None


def time_steps(fn, steps: int, warmup: int, stream, sync_all):
    """W untimed steps, then exactly K steps between two CUDA events on the launching stream,
    bracketed by a barrier + device synchronise on both sides.  Returns seconds for the K steps."""
    for _ in range(warmup):
        fn()
    sync_all()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(steps):
        fn()
    t1.record(stream)
    sync_all()
    return t0.elapsed_time(t1) * 1e-3


def best_of_runs(fn, steps: int, warmup: int, stream, sync_all, runs: int = 3):
    """The side measurements (sibling operators) are short and run once per process, right after their tensors were
    made: the fastest of `runs` timed runs of `steps` launches each (seconds for `steps` launches), so that a clock
    ramp or an allocator warm-up in the first run does not become the reported figure.  Not used for the headline."""
    best = time_steps(fn, steps, warmup, stream, sync_all)
    for _ in range(runs - 1):
        best = min(best, time_steps(fn, steps, 0, stream, sync_all))
    return best


def per_launch_times(fn, launches: int, stream, sync_all):
    """Every launch between its own pair of CUDA events (after the timed region, not part of it): median and best, the
    statistics the reference's harness reports, beside the mean over back-to-back launches that `value` uses."""
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(launches)]
    sync_all()
    for a, b in events:
        a.record(stream)
        fn()
        b.record(stream)
    sync_all()
    ms = sorted(a.elapsed_time(b) for a, b in events)
    return {"launches": launches, "median_ms": ms[len(ms) // 2], "best_ms": ms[0], "worst_ms": ms[-1]}


def reference_cpu_path():
    """The reference's CPU implementation of the operator as (function, kind, description).  kind "reference": the
    upstream project's own torch function `ref_impl`, loaded from its unmodified test file (from an upstream checkout,
    or from the digest-checked copy that oracle/make_ref.py places under oracle/_ref/).  kind "port": the restatement
    in oracle/torch_path.py, used only where neither is present.  `ref_impl` rotates the kv tensor it is given, so the
    wrapper hands it a copy (the operator leaves kv untouched)."""
    from oracle import ref_loader, torch_path

    found = ref_loader.hot_path_test_root()
    if found is not None:
        try:
            upstream = ref_loader.load_upstream_test_module()

            def ref(q, kv, cache, slots, pos, cs, eps, bs):
                upstream.ref_impl(q, kv.clone(), cache, slots, pos, cs, eps, bs)

            return ref, "reference", f"upstream ref_impl (torch CPU path of the reference's own test file, {found[1]})"
        except Exception as e:  # an unreadable copy must not silently become the reference
            print(f"# upstream ref_impl could not be loaded ({e!r}); timing the restatement instead", file=sys.stderr)
    return torch_path.prologue, "port", "restatement of the reference's torch CPU path (oracle/torch_path.py)"


def cpu_baseline(workload, budget_s: float = 12.0):
    """The reference's CPU torch path (see reference_cpu_path) on the first CPU_SAMPLE_TOKENS tokens of the workload,
    all host threads; best of >= 5 runs within a budget."""
    cpu_path, kind, what = reference_cpu_path()

    n = min(CPU_SAMPLE_TOKENS, workload.num_tokens)
    n_ins = min(n, workload.slot_mapping.shape[0])
    q = workload.q[:n].cpu()
    kv = workload.kv[:n].cpu()
    slots = workload.slot_mapping[:n_ins].cpu()
    pos = workload.position_ids[:n].cpu()
    cs = workload.cos_sin_cache.cpu()
    valid = slots >= 0
    compact = torch.full_like(slots, -1)
    compact[valid] = torch.arange(int(valid.sum()))
    cache = torch.zeros(n // 64 + 1, 64 * 584, dtype=torch.uint8)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    best, runs, t_start = float("inf"), 0, time.perf_counter()
    while runs < 5 or (time.perf_counter() - t_start < budget_s and runs < 50):
        qq = q.clone()
        t = time.perf_counter()
        cpu_path(qq, kv, cache, compact, pos, cs, workload.eps, 64)
        best = min(best, time.perf_counter() - t)
        runs += 1
    out = {"value": n / best, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
           "sample": f"first {n} tokens x {workload.num_heads} heads of the workload, {what}, best of {runs} runs",
           "ms_per_sample": best * 1e3}
    # for scale: the plain-C oracle (OpenMP over tokens) on the same sample
    from oracle import c_oracle

    c_best = float("inf")
    for _ in range(5):
        qq = q.clone()
        t = time.perf_counter()
        c_oracle.prologue(qq, kv, cache, compact, pos, cs, workload.eps, 64, threads=threads)
        c_best = min(c_best, time.perf_counter() - t)
    out["c_oracle_tokens_per_s"] = n / c_best
    return out


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU torch path (see reference_cpu_path) on a bounded sample per step."""
    if rank != 0:
        return
    from flaggems_vllm.testing import workloads

    cpu_path, kind, what = reference_cpu_path()

    name = args.workload or ("long_prefill" if world == 1 else "sharded")
    n = CPU_SAMPLE_TOKENS
    w = workloads.make("long_prefill" if name != "sharded" else "sharded", device="cpu", seed=0, num_tokens=n,
                       num_blocks=n // 64 + 8, world=world if name == "sharded" else 1,
                       total_tokens=None if name != "sharded" else 32768 * world)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    q0 = w.q.clone()

    def step():
        q = q0.clone()
        t = time.perf_counter()
        cpu_path(q, w.kv, w.k_cache, w.slot_mapping, w.position_ids, w.cos_sin_cache, w.eps, 64)
        return time.perf_counter() - t

    for _ in range(args.warmup):
        step()
    total = sum(step() for _ in range(args.steps))
    value = n * args.steps / total
    sample = f"{n} tokens x {w.num_heads} heads per step (bounded sample of the workload), {what}"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "num_heads": w.num_heads, "sample_tokens": n},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def hbm_ceiling(native, nbytes: int, stream):
    """This GPU's streaming rates for the prologue's access pattern without arithmetic
    (dsv4_hbm_probe): in place (1 read : 1 write, the operator's mix), read-only, write-only, and 2 read : 1 write
    (the mix of the narrowing sibling operators)."""
    from flaggems_vllm.testing import hbm_probe

    rows = max(1, nbytes // 1024)
    buf = torch.empty(rows * 1536, dtype=torch.uint8, device="cuda")
    out = {}
    for mode, name, traffic in ((0, "inplace_gbs", 2), (1, "read_gbs", 1), (2, "write_gbs", 1), (3, "read2_write1_gbs", 1.5)):
        def fn():
            hbm_probe.probe(mode, buf.data_ptr(), rows, stream.cuda_stream)
        secs = time_steps(fn, 10, 3, stream, torch.cuda.synchronize)
        out[name] = traffic * rows * 1024 * 10 / secs / 1e9
    out["buffer_bytes"] = rows * 1024
    return out


def sibling_ops(steps, warmup, only=None):
    """The operators either side of the prologue (the step before, the cache reader, the attention epilogue, the sparse-indexer
    prologue), 8192 tokens x 128 heads,
    device-resident inputs larger than L2, CUDA-event time (fastest of three runs of `steps` launches); GB/s = algorithmic
    bytes / time.
    `only`: time just the operators whose name contains this string, and allocate nothing for the others (the form to
    put under a profiler: one operator, at most a few GB on the device)."""
    import flaggems_vllm
    from flaggems_vllm.testing.workloads import cos_sin_table

    dev, n, h = "cuda", 8192, 128
    stream = torch.cuda.current_stream()
    g = torch.Generator(device=dev).manual_seed(0)
    out = {}
    cs = cos_sin_table(65536, device=dev)

    def want(*names):
        return only is None or any(only in name or name in only for name in names)

    if want("fused_inv_rope_fp8_quant"):
        _sibling_epilogue(flaggems_vllm, out, steps, warmup, stream, g, cs, n, h, only)
    if want("fused_q_kv_rmsnorm"):
        _sibling_rmsnorm(flaggems_vllm, out, steps, warmup, stream, g)
    if want("dequantize_and_gather_k_cache"):
        _sibling_gather(flaggems_vllm, out, steps, warmup, stream, g)
    if want("fused_indexer_q_rope_quant"):
        _sibling_indexer_q(flaggems_vllm, out, steps, warmup, stream, g, cs, only)
    if want("indexer_k_quant_and_cache", "cp_gather_indexer_k_quant_cache"):
        _sibling_indexer_k(flaggems_vllm, out, steps, warmup, stream, g, only)
    if want("compute_global_topk_indices_and_lens", "combine_topk_swa_indices"):
        _sibling_index_ops(flaggems_vllm, out, steps, warmup, stream, g, only)
    if want("per_token_group_quant_fp8"):
        _sibling_group_quant(flaggems_vllm, out, steps, warmup, stream, g, only)
    if want("top_k_per_row_decode"):
        _sibling_topk(flaggems_vllm, out, steps, warmup, stream, g, only)
    return out


def _sibling_epilogue(flaggems_vllm, out, steps, warmup, stream, g, cs, n, h, only):
    # epilogue: read 1 KiB, write 512 B + 4 fp32 scales per (token, head) row
    dev = "cuda"
    o = torch.randn(n, h, 512, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    pos = torch.randint(0, 65536, (n,), generator=g, device=dev, dtype=torch.int64)
    for packed, key, scale_bytes in ((True, "fused_inv_rope_fp8_quant[ue8m0 scales]", 4), (False, "fused_inv_rope_fp8_quant[fp32 scales]", 16)):
        if only is not None and only not in key:
            continue
        secs = best_of_runs(lambda: flaggems_vllm.fused_inv_rope_fp8_quant(o, pos, cs, 8, 16, tma_aligned_scales=packed), steps,
                          warmup, stream, torch.cuda.synchronize)
        nbytes = n * h * (1024 + 512 + scale_bytes) + n * 264
        out[key] = {"rows": n * h, "us_per_launch": secs / steps * 1e6, "hbm_gbs": nbytes * steps / secs / 1e9,
                    "note": "includes torch.empty of the two outputs per call"}


def _sibling_rmsnorm(flaggems_vllm, out, steps, warmup, stream, g):
    # step before: weighted RMSNorm of [N,1536] and [N,512]; 64 Ki tokens so the working set exceeds L2
    dev, nt = "cuda", 65536
    qr = torch.randn(nt, 1536, generator=g, device=dev).to(torch.bfloat16)
    kv = torch.randn(nt, 512, generator=g, device=dev).to(torch.bfloat16)
    qw, kw = torch.ones(1536, device=dev, dtype=torch.bfloat16), torch.ones(512, device=dev, dtype=torch.bfloat16)
    secs = best_of_runs(lambda: flaggems_vllm.fused_q_kv_rmsnorm(qr, kv, qw, kw, 1e-6), steps, warmup, stream, torch.cuda.synchronize)
    out["fused_q_kv_rmsnorm"] = {"tokens": nt, "us_per_launch": secs / steps * 1e6,
                                 "hbm_gbs": nt * 2048 * 2 * 2 * steps / secs / 1e9,
                                 "note": "includes torch.empty_like of the two outputs per call"}


def _sibling_gather(flaggems_vllm, out, steps, warmup, stream, g):
    # reader: 16 requests x 16384 tokens gathered through a block table; 584 B read, 1 KiB written per token
    dev, reqs, seq, bs = "cuda", 16, 16384, 64
    blocks = reqs * seq // bs
    cache = torch.randint(0, 256, (blocks, bs * 584), generator=g, device=dev, dtype=torch.uint8)
    table = torch.randperm(blocks, generator=g, device=dev).to(torch.int32).view(reqs, seq // bs).contiguous()
    lens = torch.full((reqs,), seq, device=dev, dtype=torch.int32)
    dst = torch.empty(reqs, seq, 512, device=dev, dtype=torch.bfloat16)
    secs = best_of_runs(lambda: flaggems_vllm.dequantize_and_gather_k_cache(dst, cache, lens, None, table, bs), steps, warmup, stream,
                      torch.cuda.synchronize)
    out["dequantize_and_gather_k_cache"] = {"tokens": reqs * seq, "us_per_launch": secs / steps * 1e6,
                                            "hbm_gbs": reqs * seq * (584 + 1024) * steps / secs / 1e9}


def _sibling_indexer_q(flaggems_vllm, out, steps, warmup, stream, g, cs, only):
    # sparse-indexer siblings: 64 Ki tokens, 64 index heads x 128 (q), one 128-wide key per token (k)
    dev, nt, ih = "cuda", 65536, 64
    iq = torch.randn(nt, ih, 128, generator=g, device=dev).to(torch.bfloat16)
    ipos = torch.randint(0, 65536, (nt,), generator=g, device=dev, dtype=torch.int64)
    iw = torch.randn(nt, ih, generator=g, device=dev).to(torch.bfloat16)
    for fp4, key, out_b in ((False, "fused_indexer_q_rope_quant[fp8]", 128), (True, "fused_indexer_q_rope_quant[mxfp4]", 68)):
        if only is not None and only not in key:
            continue
        secs = best_of_runs(lambda: flaggems_vllm.fused_indexer_q_rope_quant(ipos, iq, cs, iw, 0.088, 0.125, use_fp4=fp4), steps, warmup,
                          stream, torch.cuda.synchronize)
        out[key] = {"rows": nt * ih, "us_per_launch": secs / steps * 1e6, "hbm_gbs": nt * ih * (256 + out_b + 6) * steps / secs / 1e9,
                    "note": "includes torch.empty of the outputs per call"}


def _sibling_indexer_k(flaggems_vllm, out, steps, warmup, stream, g, only):
    dev, nk = "cuda", 1 << 20
    ik = torch.randn(nk, 128, generator=g, device=dev).to(torch.bfloat16)
    icache = torch.zeros(nk // 64, 64, 132, device=dev, dtype=torch.uint8)
    # slots as a prefill produces them (tokens fill randomly chosen blocks in order) and fully random slots
    table = torch.randperm(nk // 64, generator=g, device=dev).to(torch.int64)
    order = torch.arange(nk, device=dev, dtype=torch.int64)
    for key, islots in (("indexer_k_quant_and_cache[block-contiguous slots]", (table[order // 64] * 64 + order % 64).contiguous()),
                        ("indexer_k_quant_and_cache[random slots]", torch.randperm(nk, generator=g, device=dev).to(torch.int64))):
        if only is not None and only not in key:
            continue
        secs = best_of_runs(lambda: flaggems_vllm.indexer_k_quant_and_cache(ik, icache, islots, 128, "ue8m0"), steps, warmup, stream,
                          torch.cuda.synchronize)
        out[key] = {"tokens": nk, "us_per_launch": secs / steps * 1e6, "hbm_gbs": nk * (256 + 132 + 8) * steps / secs / 1e9}
    del ik
    if only is not None and only not in "cp_gather_indexer_k_quant_cache" and "cp_gather_indexer_k_quant_cache" not in only:
        return
    # reader of that cache: 16 requests x 64 Ki tokens gathered into token order (132 B read + 132 B written per token)
    reqs = 16
    cu = (torch.arange(reqs + 1, device=dev, dtype=torch.int32) * (nk // reqs)).contiguous()
    btable = table.to(torch.int32).view(reqs, nk // 64 // reqs).contiguous()
    gk = torch.empty(nk, 128, device=dev, dtype=torch.float8_e4m3fn)
    gs = torch.empty(nk, 4, device=dev, dtype=torch.uint8)
    secs = best_of_runs(lambda: flaggems_vllm.cp_gather_indexer_k_quant_cache(icache, gk, gs, btable, cu), steps, warmup, stream,
                      torch.cuda.synchronize)
    out["cp_gather_indexer_k_quant_cache"] = {"tokens": nk, "us_per_launch": secs / steps * 1e6, "hbm_gbs": nk * 264 * steps / secs / 1e9}


def _sibling_index_ops(flaggems_vllm, out, steps, warmup, stream, g, only):
    # index bookkeeping of the sparse attention: 32768 tokens, 16 requests
    dev, nt, reqs, tk = "cuda", 32768, 16, 2048
    if only is None or only in "compute_global_topk_indices_and_lens" or "compute_global_topk_indices_and_lens" in only:
        _sibling_global_topk(flaggems_vllm, out, steps, warmup, stream, g, dev, nt, reqs, tk)
    if only is not None and only not in "combine_topk_swa_indices" and "combine_topk_swa_indices" not in only:
        return
    tk, window = 512, 128
    tki = torch.randint(0, 8192, (nt, tk), generator=g, device=dev, dtype=torch.int32)
    qsl = (torch.arange(reqs + 1, device=dev, dtype=torch.int32) * (nt // reqs)).contiguous()
    seq = torch.full((reqs,), 8192, device=dev, dtype=torch.int32)
    gat = torch.full((reqs,), nt // reqs + window, device=dev, dtype=torch.int32)
    secs = best_of_runs(lambda: flaggems_vllm.combine_topk_swa_indices(tki, qsl, seq, gat, window, 4, tk, 8192, 2048), steps, warmup, stream,
                      torch.cuda.synchronize)
    out["combine_topk_swa_indices"] = {"tokens": nt, "topk": tk, "window": window, "us_per_launch": secs / steps * 1e6,
                                       "hbm_gbs": nt * (4 * tk + 4 * (tk + window) + 4) * steps / secs / 1e9,
                                       "note": "includes torch.empty of the outputs per call; positions 6144-8191, so every row has 512 + 128 entries"}


def _sibling_global_topk(flaggems_vllm, out, steps, warmup, stream, g, dev, nt, reqs, tk):
    local = torch.randint(0, 65536, (nt, tk), generator=g, device=dev, dtype=torch.int32)
    local[torch.rand(nt, tk, generator=g, device=dev) < 0.1] = -1
    t2r = torch.randint(0, reqs, (nt,), generator=g, device=dev, dtype=torch.int32)
    btable = torch.randperm(reqs * 1024, generator=g, device=dev).to(torch.int32).view(reqs, 1024).contiguous()
    secs = best_of_runs(lambda: flaggems_vllm.compute_global_topk_indices_and_lens(local, t2r, btable, 64), steps, warmup, stream,
                      torch.cuda.synchronize)
    out["compute_global_topk_indices_and_lens"] = {"tokens": nt, "topk": tk, "us_per_launch": secs / steps * 1e6,
                                                   "hbm_gbs": nt * (8 * tk + 8) * steps / secs / 1e9,
                                                   "note": "includes torch.empty of the outputs per call"}


def _sibling_group_quant(flaggems_vllm, out, steps, warmup, stream, g, only):
    # activation quantiser in front of the FP8 projections: 32768 tokens x 7168, groups of 128
    dev = "cuda"
    xa = torch.randn(32768, 7168, generator=g, device=dev).to(torch.bfloat16)
    for ue8m0, key in ((True, "per_token_group_quant_fp8[ue8m0 scales]"), (False, "per_token_group_quant_fp8[fp32 scales]")):
        if only is not None and only not in key:
            continue
        secs = best_of_runs(lambda: flaggems_vllm.per_token_group_quant_fp8(xa, 128, scale_ue8m0=ue8m0), steps, warmup, stream, torch.cuda.synchronize)
        out[key] = {"tokens": 32768, "columns": 7168, "us_per_launch": secs / steps * 1e6,
                    "hbm_gbs": xa.numel() * (2 + 1 + 4 / 128) * steps / secs / 1e9, "note": "includes torch.empty of the two outputs per call"}


def _sibling_topk(flaggems_vllm, out, steps, warmup, stream, g, only):
    # top-k selection over the indexer logits: one decode row, a decode batch, a prefill chunk (rotating inputs larger than L2)
    dev = "cuda"
    try:
        import vllm._custom_ops  # noqa: F401  (loads torch.ops._C)

        library = torch.ops._C.top_k_per_row_decode if hasattr(torch.ops._C, "top_k_per_row_decode") else None
    except Exception:
        library = None
    for rows, vocab, tk in ((1, 262144, 512), (496, 262144, 512), (4096, 32768, 2048)):
        key = f"top_k_per_row_decode[{rows}x{vocab}, k={tk}]"
        if only is not None and only not in key:
            continue
        sets = max(1, min(8, (1 << 30) // (rows * vocab * 4)))
        logits = [torch.randn(rows, vocab, generator=g, device=dev) for _ in range(sets)]
        seq = torch.full((rows,), vocab, device=dev, dtype=torch.int32)
        idx = torch.empty(rows, tk, device=dev, dtype=torch.int32)
        turn = [0]

        def ours():
            turn[0] += 1
            x = logits[turn[0] % sets]
            flaggems_vllm.top_k_per_row_decode(x, 1, seq, idx, rows, x.stride(0), x.stride(1), tk)

        def theirs():
            turn[0] += 1
            x = logits[turn[0] % sets]
            library(x, 1, seq, idx, rows, x.stride(0), x.stride(1), tk)

        secs = best_of_runs(ours, steps, warmup, stream, torch.cuda.synchronize)
        entry = {"rows": rows, "vocab": vocab, "top_k": tk, "us_per_launch": secs / steps * 1e6,
                 "hbm_gbs": rows * (vocab + tk) * 4 * steps / secs / 1e9}
        if library is not None and only is None:
            entry["vllm_kernel_us_per_launch"] = best_of_runs(theirs, steps, warmup, stream, torch.cuda.synchronize) / steps * 1e6
        out[key] = entry
        del logits


def measure_e2e(flaggems_vllm, w, args, dev, stream, sync_all, tokens_all_ranks):
    """The same step through the public host-buffer front end: q/kv/slots/positions start in pinned host
    memory, the rewritten q ends in pinned host memory (in place), copies inside the timed region."""
    import torch.distributed as dist

    distributed = dist.is_available() and dist.is_initialized()
    try:
        hq = torch.empty(w.q.shape, dtype=w.q.dtype, pin_memory=True)
    except RuntimeError as e:  # not enough pinnable host memory on this box
        return {"value": None, "unit": "tokens/s", "unavailable": f"pinned allocation failed: {str(e).splitlines()[0]}"}
    hq.copy_(w.q)
    hkv = w.kv.cpu().pin_memory()
    hslots = w.slot_mapping.cpu().pin_memory()
    hpos = w.position_ids.cpu().pin_memory()
    pipe = flaggems_vllm.HostStagedPrologue(w.num_heads, chunk_tokens=1024, device=dev)
    e2e_steps = max(2, min(args.steps, 5))

    def e2e_step():
        pipe(hq, hkv, w.k_cache, hslots, hpos, w.cos_sin_cache, w.eps, 64)

    for _ in range(min(args.warmup, 2) or 1):
        e2e_step()
    sync_all()
    # the staged call makes the caller's stream wait for its last copy, so two events on that stream
    # bracket the host->device copies, the kernels and the device->host copies
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    t1.record(stream)
    sync_all()
    secs = t0.elapsed_time(t1) * 1e-3 / e2e_steps
    h2d = hq.numel() * 2 + hkv.numel() * 2 + hslots.numel() * 8 + hpos.numel() * 8
    d2h = hq.numel() * 2
    my_secs, my_h2d, my_d2h = secs, h2d, d2h
    es = torch.tensor([secs, float(h2d), float(d2h)], dtype=torch.float64, device=dev)
    world = dist.get_world_size() if distributed else 1
    if world > 1:
        em, esum = es.clone(), es.clone()
        dist.all_reduce(em, op=dist.ReduceOp.MAX)
        dist.all_reduce(esum, op=dist.ReduceOp.SUM)
        secs, h2d, d2h = float(em[0]), float(esum[1]), float(esum[2])
    out = {"value": tokens_all_ranks / secs, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
           "ms_per_step": secs * 1e3, "chunk_tokens": 1024, "launches_per_step": pipe.launches,
           "note": "q/kv/slots/positions from pinned host memory, rewritten q back to the same pinned buffer; "
                   "K cache and cos/sin table device-resident"}
    # What the host side of this box can move with no kernel and no pipeline at all: every rank copies half of its
    # pinned q to the device while the other half comes back (then the halves swap), all ranks at once.  Beside
    # it, what the staged pipeline moved per rank in the timed region above.  Equal figures mean the box's host
    # memory / PCIe fabric is the limit of `e2e`, not the pipeline.
    bare = bare_copy_rates(hq, w.q, dev, sync_all)
    mine = torch.tensor([my_h2d / my_secs / 1e9, my_d2h / my_secs / 1e9, bare[0], bare[1], float(w.num_tokens)],
                        dtype=torch.float64, device=dev)
    every = [torch.zeros_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(every, mine)
    else:
        every = [mine]
    rows = [[round(float(v), 2) for v in t.tolist()] for t in every]
    out["staged_gbs_per_rank"] = [[r[0], r[1]] for r in rows]
    out["bare_copy_gbs_per_rank"] = [[r[2], r[3]] for r in rows]
    out["tokens_per_rank"] = [int(r[4]) for r in rows]
    out["bare_copy_gbs_all_ranks"] = [round(sum(r[2] for r in rows), 1), round(sum(r[3] for r in rows), 1)]
    out["staged_gbs_all_ranks"] = [round(h2d / secs / 1e9, 1), round(d2h / secs / 1e9, 1)]
    out["bare_copy_note"] = ("[host->device, device->host] GB/s; bare = plain cudaMemcpyAsync of pinned q in both directions at "
                             "once on every rank at once, no kernel, measured after the timed region")
    return out


def bare_copy_rates(hq, dq, dev, sync_all, passes: int = 2):
    """(host->device GB/s, device->host GB/s) of this rank while all ranks copy at once: one half of the pinned
    buffer goes to the device while the other half comes back, then the halves swap; each direction on its own
    stream between its own events.  `dq` is a device buffer of the same shape whose contents are no longer needed."""
    half = hq.shape[0] // 2
    if half == 0:
        return 0.0, 0.0
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(2)]
    sync_all()
    ev[0][0].record(s_in), ev[1][0].record(s_out)
    for k in range(passes):
        up, down = (slice(0, half), slice(half, 2 * half)) if k % 2 == 0 else (slice(half, 2 * half), slice(0, half))
        with torch.cuda.stream(s_in):
            dq[up].copy_(hq[up], non_blocking=True)
        with torch.cuda.stream(s_out):
            hq[down].copy_(dq[down], non_blocking=True)
        # the halves swap only when both copies of this pass are done
        s_in.wait_stream(s_out), s_out.wait_stream(s_in)
    ev[0][1].record(s_in), ev[1][1].record(s_out)
    sync_all()
    nbytes = passes * half * hq[0].numel() * hq.element_size()
    return nbytes / (ev[0][0].elapsed_time(ev[0][1]) * 1e-3) / 1e9, nbytes / (ev[1][0].elapsed_time(ev[1][1]) * 1e-3) / 1e9


def library_kernel_time(w, steps, warmup, stream):
    """vLLM's own CUDA kernel for this operator (the nine-argument torch.ops._C form of the installed wheel), timed
    on the same device-resident workload as a same-box comparison; None when the wheel does not provide it."""
    try:
        import vllm._custom_ops  # noqa: F401

        kernel = torch.ops._C.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert
        fn = lambda: kernel(w.q, w.kv, w.k_cache, w.slot_mapping, w.position_ids, w.cos_sin_cache, w.num_heads, w.eps, 64)  # noqa: E731
        fn()
        torch.cuda.synchronize()
    except Exception as e:
        return {"unavailable": str(e).splitlines()[0][:120] if str(e) else type(e).__name__}
    secs = time_steps(fn, steps, warmup, stream, torch.cuda.synchronize)
    return {"name": "vllm torch.ops._C.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert (out of place, 9 arguments)",
            "ms_per_step": secs / steps * 1e3, "note": "allocates and writes a new q tensor instead of rewriting q in place"}


def upstream_shapes(op, reps: int = 20):
    """The shapes the reference benchmarks this operator at (benchmark/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:137-163,
    195-236): N in {1..131072} x H in {64, 128}, block 64, positions = slots = arange, table of max(4096, N) rows.
    As that harness does (triton do_bench): L2 flushed by writing a 256 MB buffer before every timed call, median of
    the per-call CUDA-event times.  Its baseline, vLLM's own kernel, is timed the same way where the wheel has it."""
    from flaggems_vllm.testing.workloads import cos_sin_table

    dev = "cuda"
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    try:
        import vllm._custom_ops  # noqa: F401

        lib_kernel = torch.ops._C.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert
    except Exception:
        lib_kernel = None

    def median_us(fn):
        for _ in range(3):
            fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return statistics.median(times)

    rows = []
    # 256 tokens is not among the reference's shapes: it is the decode batch of this repository's benchmark configurations
    for n in (1, 4, 17, 64, 256, 1024, 2048, 8192, 32768, 65536, 98304, 131072):
        for h in (64, 128):
            q = torch.empty(n, h, 512, dtype=torch.bfloat16, device=dev)
            for a in range(0, n, 8192):
                q[a : a + 8192].normal_()
            kv = torch.randn(n, 512, device=dev).to(torch.bfloat16)
            pos = torch.arange(n, dtype=torch.int64, device=dev)
            cs = cos_sin_table(max(4096, n), device=dev)
            cache = torch.zeros((n + 63) // 64 + 1, 64 * 584, dtype=torch.uint8, device=dev)
            ours = median_us(lambda: op(q, kv, cache, pos, pos, cs, 1e-6, 64))
            row = {"num_tokens": n, "num_heads": h, "ours_us": ours, "ours_gbs": (n * (2048 * h + 1880)) / ours / 1e3}
            if lib_kernel is not None:
                try:
                    row["vllm_us"] = median_us(lambda: lib_kernel(q, kv, cache, pos, pos, cs, h, 1e-6, 64))
                    row["speedup_vs_vllm"] = row["vllm_us"] / ours
                except Exception as e:
                    row["vllm_us"] = None
                    row["vllm_error"] = str(e).splitlines()[0][:80]
            rows.append(row)
            del q, kv, cache
            torch.cuda.empty_cache()
    return rows


def side_measurement(name, steps, warmup, op, native):
    """decode / prefill configurations, reported beside the headline (N=1, rank 0 only).
    The 256-token decode batch fits in L2, so it rotates over enough independent q/kv sets to
    exceed L2 between reuses."""
    from flaggems_vllm.testing import workloads

    w = workloads.make(name, device="cuda", seed=0)
    sets = 1
    q_sets, kv_sets, slot_sets = [w.q], [w.kv], [w.slot_mapping]
    set_bytes = w.q.numel() * 2
    if set_bytes < 512 * 1024 * 1024:
        sets = max(2, (512 * 1024 * 1024 + set_bytes - 1) // set_bytes)
        perm = torch.randperm(w.k_cache.shape[0] * 64, device="cuda")
        for i in range(1, sets):
            q_sets.append(torch.randn_like(w.q))
            kv_sets.append(torch.randn_like(w.kv))
            slot_sets.append(perm[i * w.num_tokens : (i + 1) * w.num_tokens].to(torch.int64).contiguous())
    state = {"i": 0}

    def fn():
        i = state["i"] % sets
        state["i"] += 1
        op(q_sets[i], kv_sets[i], w.k_cache, slot_sets[i], w.position_ids, w.cos_sin_cache, w.eps, 64)

    stream = torch.cuda.current_stream()
    secs = time_steps(fn, steps, warmup, stream, torch.cuda.synchronize)
    nbytes = w.algorithmic_bytes()
    out = {"tokens": w.num_tokens, "us_per_launch": secs / steps * 1e6, "tokens_per_s": w.num_tokens * steps / secs,
           "hbm_gbs": nbytes * steps / secs / 1e9, "rotating_sets": sets}
    if sets > 1:
        # The same rotation captured once in a CUDA graph (how serving runs decode steps) and replayed gives the
        # device-side time per launch.  Both ways of calling are timed in each launch mode of the library
        # (dsv4_set_pdl): 2 = the default, dependent launch with ordinary stream semantics; 0 = plain launches;
        # 1 = dependent launch that also reads positions and table rows early (positions and table are not written
        # inside the rotation).
        side = torch.cuda.Stream()
        replays = max(2, steps // sets)

        def graph_us():
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(sets):
                        fn()
            stream.wait_stream(side)
            return time_steps(graph.replay, replays, 2, stream, torch.cuda.synchronize) / (replays * sets) * 1e6

        out["us_per_launch_cuda_graph"] = graph_us()
        out["hbm_gbs_cuda_graph"] = nbytes / out["us_per_launch_cuda_graph"] / 1e3
        default_mode = native.set_pdl(0)
        try:
            out["us_per_launch_plain_launch"] = time_steps(fn, steps, warmup, stream, torch.cuda.synchronize) / steps * 1e6
            out["us_per_launch_cuda_graph_plain_launch"] = graph_us()
            native.set_pdl(1)
            out["us_per_launch_early_reads"] = time_steps(fn, steps, warmup, stream, torch.cuda.synchronize) / steps * 1e6
            out["us_per_launch_cuda_graph_early_reads"] = graph_us()
        finally:
            native.set_pdl(default_mode)
        out["launch_mode"] = default_mode
        # The ceiling for a launch of THIS size: the arithmetic-free in-place copy with the same row access pattern
        # over the same number of q rows, rotating over as many buffers, replayed from a CUDA graph the same way.
        # A launch this short is bounded by launch, ramp-up and drain as much as by bandwidth; the probe pays the same.
        from flaggems_vllm.testing import hbm_probe

        rows = w.num_tokens * w.num_heads
        with torch.cuda.stream(side):
            side.wait_stream(stream)
            for q in q_sets[:2]:
                hbm_probe.probe(0, q.data_ptr(), rows, side.cuda_stream)
            graph_probe = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_probe, stream=side):
                for q in q_sets:
                    hbm_probe.probe(0, q.data_ptr(), rows, torch.cuda.current_stream().cuda_stream)
        stream.wait_stream(side)
        csecs = time_steps(graph_probe.replay, replays, 2, stream, torch.cuda.synchronize)
        out["copy_probe_us_per_launch_cuda_graph"] = csecs / (replays * sets) * 1e6
        out["frac_of_copy_probe_same_size"] = out["copy_probe_us_per_launch_cuda_graph"] / out["us_per_launch_cuda_graph"]
        out["frac_of_copy_probe_same_size_plain_launch"] = (out["copy_probe_us_per_launch_cuda_graph"] /
                                                            out["us_per_launch_cuda_graph_plain_launch"])
        # the library kernel of the same operator (vLLM's, out of place, nine arguments) over the same rotation
        try:
            import vllm._custom_ops  # noqa: F401

            lib_kernel = torch.ops._C.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert

            def lib_fn():
                i = state["i"] % sets
                state["i"] += 1
                lib_kernel(q_sets[i], kv_sets[i], w.k_cache, slot_sets[i], w.position_ids, w.cos_sin_cache, w.num_heads, w.eps, 64)

            out["vllm_kernel_us_per_launch"] = time_steps(lib_fn, steps, warmup, stream, torch.cuda.synchronize) / steps * 1e6
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                graph_lib = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph_lib, stream=side):
                    for _ in range(sets):
                        lib_fn()
            stream.wait_stream(side)
            out["vllm_kernel_us_per_launch_cuda_graph"] = (time_steps(graph_lib.replay, replays, 2, stream, torch.cuda.synchronize)
                                                           / (replays * sets) * 1e6)
        except Exception as e:
            out["vllm_kernel_error"] = str(e).splitlines()[0][:120]
    return out


def main():
    args = parse_args()
    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    assert args.warmup >= 0 and args.steps >= 1

    import flaggems_vllm
    from flaggems_vllm import _native
    from flaggems_vllm.testing import sharding, workloads

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    numa_cores = bind_to_gpu_numa_node(local_rank) if distributed else None
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    if args.variant is not None:
        _native.set_variant(args.variant)
    op = flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert

    if args.siblings_only:
        out = {"sibling_ops": sibling_ops(args.steps, args.warmup, args.sibling)}
        if args.sibling is None:
            out["hbm_ceiling"] = hbm_ceiling(_native, 1 << 30, torch.cuda.current_stream(dev))
        print(json.dumps(out), flush=True)
        return
    if args.upstream_shapes:
        print(json.dumps({"upstream_benchmark_shapes": upstream_shapes(op)}), flush=True)
        return
    if world == 1:
        name = args.workload or "long_prefill"
        w = workloads.make(name, device=dev, seed=0)
    else:
        name = "sharded"
        w = workloads.make("sharded", device=dev, seed=0, rank=rank, world=world, total_tokens=32768 * world)
    stream = torch.cuda.current_stream(dev)

    def sync_all():
        torch.cuda.synchronize(dev)
        if distributed:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def step():
        op(*w.args())

    # ---- device-resident throughput ("value") and the roofline of the kernel
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        time.sleep(0.3)  # let nvidia-smi start polling before the (short) timed region
    launches0 = _native.launch_count()
    secs = time_steps(step, args.steps, args.warmup, stream, sync_all)
    launches = _native.launch_count() - launches0 - args.warmup
    clocks = sampler.stop() if sampler else None
    launch_stats = per_launch_times(step, 30, stream, sync_all)
    my_bytes = w.algorithmic_bytes()
    agg = sharding.aggregate(secs, w.num_tokens, my_bytes, launches, status=_native.device_error(), device=dev)
    secs_max, tokens, nbytes, launches_total = agg["seconds"], float(agg["tokens"]), float(agg["bytes"]), agg["launches"]
    largest_tokens, largest_bytes = float(agg["largest_tokens"]), float(agg["largest_bytes"])
    if agg["failed"]:
        raise SystemExit("a kernel reported a device-side error; no number is printed")

    # ---- end to end from pinned host buffers through the public API
    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(flaggems_vllm, w, args, dev, stream, sync_all, tokens)

    # ---- the same total with EVEN shards (N > 1 only): what the uneven split of the headline costs
    even = None
    num_heads, cache_blocks = w.num_heads, int(w.k_cache.shape[0])
    if distributed and not args.no_extra:
        del w
        torch.cuda.empty_cache()
        w_even = workloads.make("long_prefill", device=dev, seed=rank)  # 32768 tokens x 128 heads on every rank
        even_steps = min(args.steps, 50)
        even_secs = time_steps(lambda: op(*w_even.args()), even_steps, max(args.warmup, 3), stream, sync_all)
        even_agg = sharding.aggregate(even_secs, w_even.num_tokens, w_even.algorithmic_bytes(), even_steps, status=_native.device_error(), device=dev)
        even = {"tokens_total": int(even_agg["tokens"]), "tokens_per_rank": w_even.num_tokens, "steps": even_steps,
                "ms_per_step": even_agg["seconds"] / even_steps * 1e3, "value": float(even_agg["tokens"]) * even_steps / even_agg["seconds"],
                "note": "same kernel and total token count, every rank 32768 tokens; the headline uses the uneven seeded Dirichlet(5) split"}
        if not args.no_e2e:
            even_e2e = measure_e2e(flaggems_vllm, w_even, args, dev, stream, sync_all, float(even_agg["tokens"]))
            even["e2e"] = {k: even_e2e.get(k) for k in ("value", "unit", "ms_per_step", "h2d_bytes_per_step", "d2h_bytes_per_step",
                                                         "staged_gbs_all_ranks", "bare_copy_gbs_all_ranks", "unavailable") if k in even_e2e}
        del w_even

    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    peak, peak_kind = hbm_peak()
    # the kernel on the rank with the most bytes is the one the step waits for
    achieved = largest_bytes / (secs_max / args.steps) / 1e9
    traffic = None
    if NCU_DRAM_BYTES_PER_TOKEN is not None and num_heads == 128:
        traffic = NCU_DRAM_BYTES_PER_TOKEN * largest_tokens
    line = {
        "metric": METRIC, "value": tokens * args.steps / secs_max, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs_max / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "num_heads": num_heads, "tokens_total": int(tokens),
                   "tokens_largest_shard": int(largest_tokens), "cache_blocks_per_gpu": cache_blocks,
                   "cache_block_size": 64, "parallelism": f"token-sharded x{world}, no collective",
                   "l2": "inputs (>= 1 GiB of q per GPU) exceed the 126 MB L2; no flush between steps",
                   "variant": _native.lib().dsv4_get_variant()},
        "hbm_gbs_aggregate": nbytes * args.steps / secs_max / 1e9,
        "tokens_per_s_sum_of_rank_rates": agg["sum_of_rank_rates"] * args.steps,
        "hbm_frac_of_nominal_8tbs": achieved / NOMINAL_HBM_GBS,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "traffic_source": TRAFFIC_SOURCE if traffic is not None else None,
                     "peak_source": f"{peak_kind} copy bandwidth",
                     "algorithmic_bytes_per_launch": int(largest_bytes),
                     "kernel_ms": secs_max / args.steps * 1e3, "kernel_ms_per_launch_rank0": launch_stats},
        "clocks": clocks, "gpu_launches": launches_total, "e2e": e2e, "even_shards": even,
        "host_numa_binding": (f"rank 0 bound to {len(numa_cores)} cores next to its GPU" if numa_cores else None),
    }
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(w)
    if not args.no_extra and world == 1:
        lib_k = library_kernel_time(w, min(args.steps, 50), 5, stream)
        if "ms_per_step" in lib_k:
            lib_k["ours_over_library_speed"] = lib_k["ms_per_step"] / (secs_max / args.steps * 1e3)
        line["same_box_library_kernel"] = lib_k
        q_bytes = w.q.numel() * 2
        del w
        torch.cuda.empty_cache()
        ceiling = hbm_ceiling(_native, q_bytes, stream)
        line["roofline"]["inplace_copy_ceiling_gbs"] = ceiling["inplace_gbs"]
        line["roofline"]["frac_of_inplace_ceiling"] = achieved / ceiling["inplace_gbs"]
        line["hbm_ceiling"] = ceiling
        line["other_configs"] = {n: side_measurement(n, max(args.steps, 50), max(args.warmup, 5), op, _native)
                                 for n in ("decode", "prefill")}
        torch.cuda.empty_cache()
        line["sibling_ops"] = sibling_ops(20, 5)
    print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
