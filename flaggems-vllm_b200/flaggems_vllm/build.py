"""Builds the CUDA libraries in place with nvcc for sm_100a: `python -m flaggems_vllm.build`.

  libdsv4_prologue.so            the operators (the product)
  testing/libdsv4_hbm_probe.so   aids: the bandwidth probe the benchmark compares the kernels with, and the on-device
                                 check of the quantisers' division shortcut that a test runs

Cross-compiles without a GPU.  The CUDA runtime is linked statically so the libraries
load (and export their symbols) on a machine that has no driver.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG.parent / "csrc"
OUT = PKG / "libdsv4_prologue.so"
PROBE_OUT = PKG / "testing" / "libdsv4_hbm_probe.so"
PROBE_SOURCES = ("hbm_probe.cu", "division_probe.cu")
SOURCES = ("abi.cu", "prologue_rows.cu", "prologue_bulk.cu", "gather_dequant.cu", "q_kv_rmsnorm.cu", "inv_rope_fp8_quant.cu", "indexer_k_quant.cu",
           "indexer_q_rope_quant.cu", "cp_gather_indexer.cu", "topk_indices.cu", "topk_per_row.cu", "topk_per_row_short.cu", "group_quant_fp8.cu")
HEADERS = ("dsv4_common.cuh", "../../include/dsv4_prologue.h", "../../include/dsv4_hbm_probe.h")


def nvcc_path() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; it is required to build libdsv4_prologue.so")
    return exe


def command(extra_flags=(), out: Path = OUT, sources=SOURCES) -> list[str]:
    return [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "-shared", "-cudart", "static", *extra_flags,
        "-o", str(out), *[str(CSRC / s) for s in sources],
    ]


def up_to_date(out: Path = OUT, sources=SOURCES) -> bool:
    if not out.exists():
        return False
    newest = max((CSRC / f).resolve().stat().st_mtime for f in tuple(sources) + HEADERS)
    return out.stat().st_mtime >= newest


def build(force: bool = False, verbose: bool = False, extra_flags=()) -> Path:
    """Build whichever of the two libraries is older than its sources; returns the operator library's path."""
    env = dict(os.environ)
    env.pop("CC", None), env.pop("CXX", None)  # let nvcc pick the system host compiler
    for out, sources in ((OUT, SOURCES), (PROBE_OUT, PROBE_SOURCES)):
        if not force and up_to_date(out, sources):
            continue
        cmd = command(extra_flags, out, sources)
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if verbose or res.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed building {out.name}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True,
                extra_flags=("-Xptxas", "-v") if "--ptxas" in sys.argv else ()))
