"""CPU checks of the C ABI: the library builds for sm_100a, loads, exports every symbol
the header declares, and validates arguments before touching the device."""
import ctypes as C
import re
from pathlib import Path

from pratchya_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def test_exports_every_declared_symbol(built_lib):
    header = (ROOT / "include" / "pratchya_b200.h").read_text()
    declared = set(re.findall(r"PB_API\s+[\w\s\*]+?\b(pb_\w+)\s*\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.DECLARED_SYMBOLS), declared ^ set(_lib.DECLARED_SYMBOLS)
    for name in declared:
        assert hasattr(built_lib, name), f"{name} is declared but not exported"


def test_version_and_status_strings(built_lib):
    assert built_lib.pb_version() >= 100
    assert built_lib.pb_status_string(0) == b"ok"
    assert b"timed out" in built_lib.pb_status_string(7)


def test_group_geometry_matches_reference_rule(built_lib):
    m, k = C.c_int64(), C.c_int64()
    for (r, c, a, b), want in {
        (2048, 2048, 1, 128): (4096, 8), (2048, 8192, 128, 128): (1, 1024), (4096, 16384, 128, 128): (4, 1024),
        (2048, 2048, 128, 1): (4096, 8), (4, 4, 4, 4): (1, 1), (3, 48, 1, 16): (9, 1), (1, 512, 1, 128): (1, 4),
    }.items():
        assert built_lib.pb_group_geometry(r, c, a, b, C.byref(m), C.byref(k)) == 0
        assert (m.value, k.value) == want
    assert built_lib.pb_group_geometry(10, 10, 4, 4, C.byref(m), C.byref(k)) == 2      # PB_ERR_BAD_SHAPE
    assert b"not divisible" in built_lib.pb_last_error()


def test_argument_errors_are_reported_without_a_device(built_lib):
    assert built_lib.pb_quantize(None, 0, 1, 8, 8, 1, 8, 0, None, None, None, None, 0, None) == 1
    one = C.c_void_p(16)
    assert built_lib.pb_quantize(one, 7, 1, 8, 8, 1, 8, 0, one, one, one, None, 0, None) == 4
    assert built_lib.pb_quantize(one, 0, 1, 8, 9, 1, 8, 0, one, one, one, None, 0, None) == 2
    assert built_lib.pb_quantize(one, 0, 1, 8, 8, 0, 8, 0, one, one, one, None, 0, None) == 3
    assert built_lib.pb_quantize(one, 0, 1, 8, 8, 1, 8, 0, one, one, one, None, 0, None) == 5      # workspace needed
    assert built_lib.pb_dequantize(None, 0, None, None, 1, 8, 8, 1, 8, 0, None, None) == 1
    assert built_lib.pb_quantize_workspace_size(1, 2048, 2048, 1, 128) == 0
    assert built_lib.pb_quantize_workspace_size(1, 2048, 2048, 128, 128) == 256 * 8
