"""Loads the upstream test file and hands out its own torch reference functions.

TEST INFRASTRUCTURE ONLY, and usable only where the upstream source tree, or the
verified copy of its test files that oracle/make_ref.py places under oracle/_ref/,
is present: it is how the golden vectors under tests/golden/ were produced, how
the restatements in this folder are checked against the real thing, and how the
CPU baseline of bench.py reaches the upstream `ref_impl`.  The upstream
package itself cannot be imported without a GPU and its SQL dependency, so the
test module is executed with small stand-in modules for the names it imports;
its pure-torch reference functions (`ref_impl` and helpers) need nothing else.
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

from . import make_ref

UPSTREAM_ENV = make_ref.UPSTREAM_ENV  # names the directory of an upstream checkout
OP = make_ref.OP


def upstream_root() -> Path | None:
    """An upstream checkout ($DSV4_UPSTREAM_ROOT, else a folder `reference` beside this repository), or None."""
    return make_ref.find_upstream()


def hot_path_test_root() -> tuple[Path, str] | None:
    """Where the upstream test file of the hot path can be read: (root, kind).  kind "checkout" = an upstream
    checkout; "copy" = the verified byte-for-byte copy oracle/make_ref.py placed under oracle/_ref/."""
    root = upstream_root()
    if root is not None:
        return root, "checkout"
    if make_ref.present():
        return make_ref.OUT, "copy"
    return None


def load_upstream_test_module():
    """The upstream test module object (has ref_impl, make_cos_sin_cache, k_cache_compare...)."""
    found = hot_path_test_root()
    if found is None:
        raise FileNotFoundError("neither an upstream checkout nor oracle/_ref is present")
    root = found[0]
    saved = {k: sys.modules.get(k) for k in list(sys.modules) if k == "flaggems_vllm" or k.startswith("flaggems_vllm.")}
    for k in saved:
        del sys.modules[k]

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    def _unbound(*_a, **_k):
        raise RuntimeError("stand-in: the operator is not bound in the reference loader")

    dev_fn = types.SimpleNamespace(empty_cache=lambda: None, synchronize=lambda: None)
    runtime = mod("flaggems_vllm.runtime", torch_device_fn=dev_fn)
    pkg = mod("flaggems_vllm", device="cpu", vendor_name="nvidia", runtime=runtime, __path__=[])
    setattr(pkg, OP, _unbound)
    mod("flaggems_vllm.ops", __path__=[])
    mod(f"flaggems_vllm.ops.{OP}", **{OP: _unbound})
    mod("flaggems_vllm.utils", __path__=[])
    mod("flaggems_vllm.utils.device_info", get_device_capability=lambda: (10, 0))
    mod("_dsv4_upstream_tests", __path__=[])
    mod("_dsv4_upstream_tests.conftest", QUICK_MODE=True)
    try:
        spec = importlib.util.spec_from_file_location(
            "_dsv4_upstream_tests.t", root / "tests" / f"test_{OP}.py"
        )
        module = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = module
        spec.loader.exec_module(module)
    finally:
        for k in [k for k in sys.modules if k == "flaggems_vllm" or k.startswith("flaggems_vllm.")]:
            del sys.modules[k]
        sys.modules.update({k: v for k, v in saved.items() if v is not None})
    return module


def load_upstream_helper_test(test_file: str, op_module: str, op_names: tuple[str, ...], package_attrs: dict | None = None,
                               sibling_modules: dict | None = None, op_bindings: dict | None = None):
    """Execute another upstream test file (e.g. tests/test_deepseek_v4_attention_*.py) with stand-ins for
    the package names it imports, to reach the pure-torch helpers it defines (expected-value builders,
    reference functions).  `op_module` is the dotted module the test imports its operator from;
    `package_attrs` are extra attributes of the stand-in `flaggems_vllm`; `sibling_modules` maps names of
    modules the test imports relatively (e.g. "accuracy_utils") to attribute dicts; `op_bindings` maps operator
    names to CPU callables that take the operator's place (the way a restatement is run through the upstream
    test's own expected-value code), the others raise when called."""
    root = upstream_root()
    if root is None or not (root / "tests" / test_file).exists():
        raise FileNotFoundError("upstream tree not present")
    saved = {k: sys.modules.get(k) for k in list(sys.modules) if k == "flaggems_vllm" or k.startswith("flaggems_vllm.")}
    for k in saved:
        del sys.modules[k]

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    def _unbound(*_a, **_k):
        raise RuntimeError("stand-in: the operator is not bound in the reference loader")

    import torch

    def assert_equal(a, b, **_k):
        assert torch.equal(a, b), "tensors differ"

    testing = mod("flaggems_vllm.testing", assert_equal=assert_equal,
                  assert_close=lambda a, b, dtype=None, equal_nan=False, **k: torch.testing.assert_close(a, b, equal_nan=equal_nan))
    pkg = mod("flaggems_vllm", device="cpu", vendor_name="nvidia", testing=testing, __path__=[])
    mod("flaggems_vllm.ops", __path__=[])
    ops_pkg = sys.modules["flaggems_vllm.ops"]
    bound = {n: (op_bindings or {}).get(n, _unbound) for n in op_names}
    for n in op_names:
        setattr(ops_pkg, n, bound[n])
        setattr(pkg, n, bound[n])
    for k, v in (package_attrs or {}).items():
        setattr(pkg, k, v)
    if op_module != "flaggems_vllm.ops":
        mod(op_module, **bound)
    mod("flaggems_vllm.utils", __path__=[])
    mod("flaggems_vllm.utils.device_info", get_device_capability=lambda: (10, 0))
    mod("_dsv4_upstream_tests", __path__=[])
    mod("_dsv4_upstream_tests.conftest", QUICK_MODE=True)
    for name, attrs in (sibling_modules or {}).items():
        setattr(sys.modules["_dsv4_upstream_tests"], name, mod(f"_dsv4_upstream_tests.{name}", **attrs))
    try:
        spec = importlib.util.spec_from_file_location(f"_dsv4_upstream_tests.{Path(test_file).stem}", root / "tests" / test_file)
        module = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = module
        spec.loader.exec_module(module)
    finally:
        for k in [k for k in sys.modules if k == "flaggems_vllm" or k.startswith("flaggems_vllm.")]:
            del sys.modules[k]
        sys.modules.update({k: v for k, v in saved.items() if v is not None})
    return module
