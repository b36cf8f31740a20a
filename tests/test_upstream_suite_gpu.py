"""The upstream project's own test files, unmodified, run against this package on the GPU.

oracle/make_ref.py copies the upstream tests byte for byte into oracle/_ref/ (digests recorded in the recipe and
checked again here).  Each case below starts a fresh pytest process on one of those files with this package first on
the import path, from a scratch working directory (the upstream conftest appends a result file to its working
directory, tests/conftest.py:220-234 upstream), without the cache plugin, and with a pytest.ini of ours in place of the
upstream one, whose `pythonpath = src` would put the upstream package in front (pytest.ini:17 upstream).  The upstream
tests compare the operator with their own torch reference on the GPU (ref_impl,
tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:316-333), so a pass here means "the reference's tests
pass on this build".
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

from oracle import make_ref

ROOT = Path(__file__).resolve().parent.parent
PKG_DIR = ROOT / "flaggems-vllm_b200"

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not make_ref.present(), reason="oracle/_ref has not been made (python oracle/make_ref.py)")]


def run_upstream(test_file: str, tmp_path: Path, select: str | None = None, deselect: tuple[str, ...] = (), timeout: int = 1500):
    assert not make_ref.verify(), "a file under oracle/_ref differs from the upstream revision"
    # the child process needs the device memory this process may still hold in torch's cache (the largest upstream case
    # keeps three 16 GiB tensors alive)
    import torch

    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    target = make_ref.OUT / "tests" / test_file
    cmd = [sys.executable, "-m", "pytest", str(target), "-q", "-p", "no:cacheprovider", "-rs", "--no-header",
           "-c", str(make_ref.OUT / "pytest.ini"), "--rootdir", str(make_ref.OUT)]
    if select:
        cmd += ["-k", select]
    if deselect:
        cmd += ["-k", " and ".join(f"not {d}" for d in deselect)]
    env = dict(os.environ)
    env["PYTHONPATH"] = str(PKG_DIR)  # this package, and nothing else of this repository
    env["PYTHONDONTWRITEBYTECODE"] = "1"
    res = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=timeout)
    tail = res.stdout[-4000:] + res.stderr[-2000:]
    counts = {k: int(v) for v, k in re.findall(r"(\d+) (passed|failed|skipped|error|errors|deselected)", res.stdout.splitlines()[-1] if res.stdout.strip() else "")}
    return res.returncode, counts, tail


def test_package_under_test_is_this_one(tmp_path):
    """The process the upstream tests run in imports flaggems_vllm from this repository and loads its CUDA library."""
    env = dict(os.environ, PYTHONPATH=str(PKG_DIR))
    out = subprocess.run([sys.executable, "-c", "import flaggems_vllm, flaggems_vllm._native as n; print(flaggems_vllm.__file__); print(n.version())"],
                         cwd=tmp_path, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert str(PKG_DIR) in out.stdout.splitlines()[0]


def test_hot_path_upstream_tests_all_sizes(tmp_path):
    """tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py upstream, every test and every size
    (test_combined_q_and_kv reaches 131072 tokens x 128 heads = 16 GiB of q): q path :358-402, kv path :419-462,
    DP padding :468-515 (whole cache bit-exact), combined :521-573.  test_backend_override_matches_reference is
    skipped by upstream itself on NVIDIA (no override bound), test_matches_vllm_reference skips itself where the
    installed vLLM's operator has another signature (:661-676)."""
    rc, counts, tail = run_upstream(f"test_{make_ref.OP}.py", tmp_path)
    print(f"upstream test_{make_ref.OP}.py: {counts}")
    assert rc == 0, tail
    assert counts.get("failed", 0) == 0 and counts.get("error", 0) == 0 and counts.get("errors", 0) == 0, tail
    # 8 q-path + 8 kv-path + 8 DP-padding + 36 combined cases
    assert counts.get("passed", 0) >= 60, tail


SIBLINGS = [
    ("test_deepseek_v4_attention_dequantize_and_gather_k_cache.py", ()),
    ("test_deepseek_v4_attention_fused_q_kv_rmsnorm.py", ()),
    ("test_fused_indexer_q_rope_quant.py", ()),
    ("test_indexer_k_quant_and_cache.py", ()),
    ("test_cp_gather_indexer_k_quant_cache.py", ()),
    # test_unfused_path (:563 upstream) builds its expectation from flaggems_vllm.apply_rotary_pos_emb, a generic
    # rotary operator that is not on this path and that this package does not provide
    ("test_fused_inv_rope_fp8_quant.py", ("test_unfused_path",)),
]


@pytest.mark.parametrize("test_file,deselect", SIBLINGS, ids=[s[0][5:-3] for s in SIBLINGS])
def test_sibling_upstream_tests(tmp_path, test_file, deselect):
    """The upstream test files of the neighbouring operators (reader of the cache, the weighted norms before the
    path, the sparse-indexer prologue), unmodified, against this package."""
    rc, counts, tail = run_upstream(test_file, tmp_path, deselect=deselect)
    print(f"upstream {test_file}: {counts}")
    assert rc == 0, tail
    assert counts.get("failed", 0) == 0 and counts.get("passed", 0) > 0, tail
