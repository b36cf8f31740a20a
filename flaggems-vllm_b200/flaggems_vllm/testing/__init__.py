"""Test helpers shipped with the package: seeded workloads and the parity comparators."""
from . import compare, sharding, workloads  # noqa: F401
