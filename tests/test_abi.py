"""The C-ABI library: loads without a GPU, exports every symbol the header declares, and
rejects bad arguments before launching anything.  No GPU, no compute calls."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from flaggems_vllm import _native
from flaggems_vllm.testing import hbm_probe

ROOT = Path(__file__).resolve().parent.parent
HEADERS = sorted((ROOT / "include").glob("*.h"))


# which library implements which header
LIBRARY_OF = {"dsv4_prologue.h": _native.LIB_PATH, "dsv4_hbm_probe.h": hbm_probe.LIB_PATH}


def declared_functions() -> list[tuple[str, str]]:
    """(header name, function) for every function a header under include/ declares."""
    names = []
    for h in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names += [(h.name, f) for f in sorted(set(re.findall(r"\b(dsv4_[a-z0-9_]+)\s*\(", text)))]
    return names


def test_header_declares_the_expected_entry_points():
    assert HEADERS, "include/*.h missing"
    assert {h.name for h in HEADERS} == set(LIBRARY_OF)
    assert set(_native.EXPORTS) == {f for h, f in declared_functions() if h == "dsv4_prologue.h"}


@pytest.mark.parametrize("header,symbol", declared_functions())
def test_library_exports_every_declared_symbol(header, symbol):
    lib = ctypes.CDLL(str(LIBRARY_OF[header]))
    assert getattr(lib, symbol) is not None


def test_operator_library_exports_no_measurement_aid():
    lib = ctypes.CDLL(str(_native.LIB_PATH))
    assert not hasattr(lib, "dsv4_hbm_probe")


def test_version_and_error_strings():
    assert "sm_100a" in _native.version()
    lib = _native.lib()
    for code in (0, -1, -2, -3, -4, -5):
        assert lib.dsv4_error_string(code)


def test_rejections_happen_before_any_launch():
    lib = _native.lib()
    before = _native.launch_count()
    bad_size = lib.dsv4_qnorm_rope_kv_insert(None, None, None, None, None, None, 1e-6, -1, 8, 0, 64, 64 * 584, None)
    assert bad_size == -2
    more_slots_than_tokens = lib.dsv4_qnorm_rope_kv_insert(None, None, None, None, None, None, 1e-6, 4, 8, 5, 64, 64 * 584, None)
    assert more_slots_than_tokens == -2
    null_ptr = lib.dsv4_qnorm_rope_kv_insert(None, None, None, None, None, None, 1e-6, 4, 8, 4, 64, 64 * 584, None)
    assert null_ptr == -1
    empty = lib.dsv4_qnorm_rope_kv_insert(None, None, None, None, None, None, 1e-6, 0, 8, 0, 64, 64 * 584, None)
    assert empty == 0
    assert lib.dsv4_gather_dequant_k_cache(None, None, -1, None, 512, 64, 64 * 584, None) == -2
    assert lib.dsv4_gather_dequant_k_cache(None, None, 3, None, 512, 64, 64 * 584, None) == -1
    assert lib.dsv4_gather_dequant_k_cache(None, None, 0, None, 512, 64, 64 * 584, None) == 0
    # q on an odd address, or a table off its 4-byte grid (fake non-null addresses are never dereferenced: validation
    # fails first); q and kv may start on any even address, which takes the any-alignment kernel
    assert lib.dsv4_qnorm_rope_kv_insert(0x1001, 0x2000, 0x3000, 0x4000, 0x5000, 0x6000, 1e-6, 4, 8, 4, 64, 64 * 584, None) == -3
    assert lib.dsv4_qnorm_rope_kv_insert(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 0x6002, 1e-6, 4, 8, 4, 64, 64 * 584, None) == -3
    # the range-checked and the out-of-place forms keep the 16-byte requirement
    assert lib.dsv4_qnorm_rope_kv_insert_checked(0x1008, 0x2000, 0x3000, 0x4000, 0x5000, 0x6000, 1e-6, 4, 8, 4, 64, 64 * 584,
                                                 100, 4096, 0x7000, None) == -3
    # cache block smaller than block_size * 584 bytes
    assert lib.dsv4_qnorm_rope_kv_insert(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 0x6000, 1e-6, 4, 8, 4, 64, 64 * 576, None) == -2
    assert _native.launch_count() == before


def test_variant_selection_round_trip():
    prev = _native.set_variant(_native.VARIANT_ROWS)
    assert _native.lib().dsv4_get_variant() == _native.VARIANT_ROWS
    with pytest.raises(_native.Dsv4Error):
        _native.set_variant(99)
    _native.set_variant(prev)
