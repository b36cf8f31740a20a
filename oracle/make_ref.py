"""Recipe: place the upstream project's own test files, byte for byte, under oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  The upstream project is Python; its CPU implementation of the attention
prologue is the torch function `ref_impl` inside its test file
(tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:316-333, helpers :68-243).  This script
copies that file, the conftest and package marker it needs (tests/conftest.py, tests/__init__.py) and the
test files of the neighbouring operators out of an upstream checkout into the git-ignored folder oracle/_ref/,
so that

* the upstream tests can be run, unmodified, against this package on a machine that has a GPU but no
  upstream checkout (tests/test_upstream_suite_gpu.py), and
* the CPU baseline and the `--impl reference` arm of bench.py time the upstream code itself instead of a
  restatement of it.

Nothing is edited on the way: every copied file is checked against the SHA-256 recorded below, and the same
digests are checked again where the files are used.  The only file written here that does not come from upstream is
oracle/_ref/pytest.ini, which keeps pytest from adopting the upstream `pythonpath = src` setting
(pytest.ini:17 upstream) - the package under test must be this one.

    python oracle/make_ref.py [UPSTREAM_ROOT]

UPSTREAM_ROOT defaults to $DSV4_UPSTREAM_ROOT, then to a checkout named `reference` beside this repository.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
UPSTREAM_ENV = "DSV4_UPSTREAM_ROOT"
OP = "fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert"
HOT_PATH_TEST = f"tests/test_{OP}.py"

# upstream path -> SHA-256 of the revision the golden vectors of this repository were made from
FILES = {
    "tests/__init__.py": "722438002fad4d34dd245e2e2345c4dcba542295822fdb7e2e8c90ab658a9cfa",
    "tests/conftest.py": "358217de80629d13ec28fed8b01f8dbdb9175fa0d5658071f5bbdbdcc4979b18",
    "tests/accuracy_utils.py": "957f6897a53d6b0a039cbc76aa3fb609a49480d9ce7cfc3223531cbea174c195",
    "tests/test_fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py": "7065ef5bdb256877ee777b1b3ba40eeadc907ecc494d868d13b9b9f6f8225667",
    "tests/test_deepseek_v4_attention_dequantize_and_gather_k_cache.py": "8234ae3940a60aab54228a6b49dd7ec9371f56505b89fd07ca80272fe00a0489",
    "tests/test_deepseek_v4_attention_fused_q_kv_rmsnorm.py": "99370670e579f4446d4ca32fdda599e45e404283914de174202ba2816c50c688",
    "tests/test_fused_inv_rope_fp8_quant.py": "a2a2416278993ad6190d5d5a1ea35fb01ea1fc5238bfd5563ae428333f03cfcf",
    "tests/test_fused_indexer_q_rope_quant.py": "d2834b4d239e1b1be215385c0e596a690e6cab478a01662e7822451c8c9f4732",
    "tests/test_indexer_k_quant_and_cache.py": "083ac398c24ad4953ceeeaa8abb36b03ee6115ffd128dd8ad417dd678eff56c9",
    "tests/test_cp_gather_indexer_k_quant_cache.py": "831057f1e2389d60637e85a60a85753df096b9c99f8c5fefcdd070d663c7713c",
}

PYTEST_INI = "[pytest]\nfilterwarnings = ignore::pytest.PytestUnknownMarkWarning\n"


def sha256(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


def find_upstream(arg: str | None = None) -> Path | None:
    candidates = [arg, os.environ.get(UPSTREAM_ENV), HERE.parent.parent / "reference"]
    for c in candidates:
        if c and (Path(c) / HOT_PATH_TEST).exists():
            return Path(c)
    return None


def verify(out: Path = OUT) -> list[str]:
    """Names of expected files that are missing from `out` or whose bytes differ from the recorded digest."""
    bad = []
    for rel, digest in FILES.items():
        p = out / rel
        if not p.exists() or (digest is not None and sha256(p) != digest):
            bad.append(rel)
    return bad


def present(out: Path = OUT) -> bool:
    return (out / HOT_PATH_TEST).exists() and not verify(out)


def make(upstream: Path | None = None, out: Path = OUT) -> Path:
    upstream = upstream or find_upstream()
    if upstream is None:
        raise FileNotFoundError("no upstream checkout found (set DSV4_UPSTREAM_ROOT)")
    for rel, digest in FILES.items():
        src = upstream / rel
        got = sha256(src)
        if digest is not None and got != digest:
            raise RuntimeError(f"{rel}: upstream file differs from the recorded revision ({got})")
        dst = out / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
    (out / "pytest.ini").write_text(PYTEST_INI)
    (out / "MANIFEST.json").write_text(json.dumps({rel: sha256(out / rel) for rel in FILES}, indent=1) + "\n")
    return out


if __name__ == "__main__":
    root = find_upstream(sys.argv[1] if len(sys.argv) > 1 else None)
    if "--print-digests" in sys.argv:
        for rel in FILES:
            print(f'    "{rel}": "{sha256(root / rel)}",')
    else:
        print(make(root))
