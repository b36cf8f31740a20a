"""Test helpers shipped with the package: seeded workloads, the parity comparators, and the two assertion
helpers the reference's operator tests import from here (src/flaggems_vllm/testing/__init__.py:79-92)."""
import torch

from . import compare, sharding, workloads  # noqa: F401

# relative tolerance per dtype used by assert_close (absolute tolerance: atol * reduce_dim)
RESOLUTION = {
    torch.bool: 0, torch.uint8: 0, torch.int8: 0, torch.int16: 0, torch.int32: 0, torch.int64: 0,
    torch.float8_e4m3fn: 1e-3, torch.float8_e5m2: 1e-3, torch.float16: 1e-3, torch.bfloat16: 0.016,
    torch.float32: 1.3e-6, torch.float64: 1e-7,
}


def assert_close(res, ref, dtype, equal_nan=False, reduce_dim=1, atol=1e-4):
    """`res` has dtype `dtype` and equals `ref` (cast to it) within the dtype's resolution."""
    dtype = torch.float32 if dtype is None else dtype
    assert res.dtype == dtype
    torch.testing.assert_close(res, ref.to(dtype), atol=atol * reduce_dim, rtol=RESOLUTION[dtype], equal_nan=equal_nan)


def assert_equal(res, ref, equal_nan=False):
    torch.testing.assert_close(res, ref, atol=0, rtol=0, equal_nan=equal_nan)
