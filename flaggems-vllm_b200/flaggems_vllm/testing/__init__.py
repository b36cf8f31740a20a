"""Test helpers shipped with the package: seeded workloads and the parity comparators."""
from . import compare, workloads  # noqa: F401
