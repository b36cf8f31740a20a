"""ctypes binding of libdsv4_hbm_probe.so (include/dsv4_hbm_probe.h): the bandwidth probe with the prologue's access
pattern and no arithmetic.  A measurement aid for the benchmark and its test; the operators do not use it."""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libdsv4_hbm_probe.so"
_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m flaggems_vllm.build`")
        L = ctypes.CDLL(str(LIB_PATH))
        L.dsv4_hbm_probe.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        L.dsv4_hbm_probe.restype = ctypes.c_int
        L.dsv4_division_probe.argtypes = [ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L.dsv4_division_probe.restype = ctypes.c_int
        _lib = L
    return _lib


def division_probe(eps: float, form: int, counts_ptr: int, stream: int) -> None:
    """Launch the on-device check of the division shortcut (see dsv4_division_probe); `counts_ptr` -> three zeroed
    64-bit words on the device: pairs examined, differing e4m3 bytes, reciprocals more than one ulp off."""
    code = lib().dsv4_division_probe(float(eps), int(form), counts_ptr, stream)
    if code != 0:
        raise RuntimeError(f"dsv4_division_probe failed with code {code}")


def probe(mode: int, buffer_ptr: int, rows: int, stream: int) -> None:
    """Launch the probe (mode 0 in place, 1 read, 2 write, 3 two reads : one write) over `rows` rows of 1 KiB."""
    code = lib().dsv4_hbm_probe(int(mode), buffer_ptr, int(rows), stream)
    if code != 0:
        raise RuntimeError(f"dsv4_hbm_probe failed with code {code}")
