"""Host side of the drop-in: import surface and argument checks of the Python entry point
(reference: src/flaggems_vllm/ops/fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert.py:320-333,
src/flaggems_vllm/__init__.py:25-46).  No GPU: every call must fail before reaching the device."""
from __future__ import annotations

import inspect

import pytest
import torch

import flaggems_vllm
from flaggems_vllm.ops.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert import (
    fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert as op,
)


def test_import_surface():
    assert flaggems_vllm.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert is op
    assert flaggems_vllm.ops_deepseek_v4_qnorm_rope_kv_rope_quant_insert is op
    assert flaggems_vllm.ops.fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert is op
    assert flaggems_vllm.device == "cuda" and flaggems_vllm.vendor_name == "nvidia"
    assert flaggems_vllm.runtime.device.vendor_name == "nvidia"
    assert hasattr(flaggems_vllm.runtime.torch_device_fn, "synchronize")
    assert hasattr(flaggems_vllm.runtime.torch_device_fn, "empty_cache")
    from flaggems_vllm.utils.device_info import get_device_capability  # noqa: F401


def test_compat_helpers():
    import flaggems_vllm.testing as fg_testing

    a = torch.tensor([1.0, 2.0], dtype=torch.bfloat16)
    fg_testing.assert_close(a, a.float() * 1.005, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        fg_testing.assert_close(a, a.float() * 1.1, dtype=torch.bfloat16)
    fg_testing.assert_equal(a, a.clone())
    with flaggems_vllm.use_gems():
        assert flaggems_vllm.SUPPORTED_FP8_DTYPE == torch.float8_e4m3fn


def test_signature_is_the_reference_one():
    names = list(inspect.signature(op).parameters)
    assert names == ["q", "kv", "k_cache", "slot_mapping", "position_ids", "cos_sin_cache", "eps", "cache_block_size"]


def _args(n=4, h=2, bs=16, nb=2):
    return dict(
        q=torch.zeros(n, h, 512, dtype=torch.bfloat16), kv=torch.zeros(n, 512, dtype=torch.bfloat16),
        k_cache=torch.zeros(nb, bs * 584, dtype=torch.uint8), slot_mapping=torch.arange(n),
        position_ids=torch.arange(n), cos_sin_cache=torch.zeros(64, 64), eps=1e-6, cache_block_size=bs,
    )


BAD = {
    "q_not_contiguous": lambda a: a.update(q=torch.zeros(4, 512, 2, dtype=torch.bfloat16).transpose(1, 2)),
    "head_dim": lambda a: a.update(q=torch.zeros(4, 2, 256, dtype=torch.bfloat16)),
    "kv_shape": lambda a: a.update(kv=torch.zeros(3, 512, dtype=torch.bfloat16)),
    "q_dtype": lambda a: a.update(q=torch.zeros(4, 2, 512, dtype=torch.float16)),
    "kv_dtype": lambda a: a.update(kv=torch.zeros(4, 512, dtype=torch.float32)),
    "cache_dtype": lambda a: a.update(k_cache=torch.zeros(2, 16 * 584, dtype=torch.int8)),
    "slot_dim": lambda a: a.update(slot_mapping=torch.zeros(4, 1, dtype=torch.int64)),
    "slot_longer_than_tokens": lambda a: a.update(slot_mapping=torch.arange(5)),
    "slot_dtype": lambda a: a.update(slot_mapping=torch.arange(4, dtype=torch.int32)),
    "position_shape": lambda a: a.update(position_ids=torch.arange(5)),
    "position_dtype": lambda a: a.update(position_ids=torch.arange(4, dtype=torch.int32)),
    "cos_sin_cols": lambda a: a.update(cos_sin_cache=torch.zeros(64, 32)),
    "cos_sin_dtype": lambda a: a.update(cos_sin_cache=torch.zeros(64, 64, dtype=torch.float64)),
    "cache_block_too_small": lambda a: a.update(k_cache=torch.zeros(2, 16 * 576, dtype=torch.uint8)),
    "cache_not_2d": lambda a: a.update(k_cache=torch.zeros(2, 16, 584, dtype=torch.uint8)),
}


@pytest.mark.parametrize("case", sorted(BAD))
def test_bad_arguments_raise_assertion_error(case):
    a = _args()
    BAD[case](a)
    with pytest.raises(AssertionError):
        op(*a.values())


def test_cpu_tensors_are_refused_not_silently_computed():
    """No CPU fallback: valid shapes on the host still raise."""
    a = _args()
    before = a["q"].clone()
    with pytest.raises(AssertionError, match="no CPU path"):
        op(*a.values())
    assert torch.equal(a["q"], before)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from flaggems_vllm import _native

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", tmp_path / "libdsv4_prologue.so")
    with pytest.raises(_native.NativeLibraryMissing):
        _native.lib()
