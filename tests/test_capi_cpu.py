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


def test_argument_errors_of_the_fused_entry_points(built_lib):
    """The fused calls validate before launching: the status codes say why a caller must take the plain calls."""
    one = C.c_void_p(4096)
    op = _lib.Operand(4096, 4096, 4096, 1024, 1024, 128, 128, 0, 1)
    # pb_quantize_for_gemm / pb_relu2_requantize: whole super-groups per row only
    assert built_lib.pb_quantize_for_gemm(one, 1, 128, 512, 0, one, one, one, op, one, 1 << 20, None) == 2
    assert built_lib.pb_quantize_for_gemm(None, 1, 128, 1024, 0, one, one, one, op, one, 1 << 20, None) == 1
    assert built_lib.pb_quantize_for_gemm(one, 1, 128, 1024, 0, one, one, one, op, one, 16, None) == 5          # workspace too small
    assert built_lib.pb_relu2_requantize(one, 128, 512, 0, one, one, one, None, None, 0, None) == _lib.PB_ERR_UNSUPPORTED
    assert built_lib.pb_relu2_requantize(one, 128, 1024, 3, one, one, one, None, None, 0, None) == 4
    # pb_fake_quantize: f32 on (1,128) with 8-block super-groups, nothing else
    assert built_lib.pb_fake_quantize(one, 1, 1, 128, 1024, 1, 128, 0, one, 0, None) == _lib.PB_ERR_UNSUPPORTED   # bf16 input
    assert built_lib.pb_fake_quantize(one, 0, 1, 128, 1024, 128, 128, 0, one, 0, None) == _lib.PB_ERR_UNSUPPORTED
    assert built_lib.pb_fake_quantize(one, 0, 1, 128, 1000, 1, 128, 0, one, 0, None) == 2
    # pb_quantize_dual: bf16, rows % 128 == 0, cols % 1024 == 0
    assert built_lib.pb_quantize_dual(one, 0, 1, 128, 1024, 0, one, one, one, one, one, one, one, 1 << 20, None) == _lib.PB_ERR_UNSUPPORTED
    assert built_lib.pb_quantize_dual(one, 1, 1, 128, 512, 0, one, one, one, one, one, one, one, 1 << 20, None) == _lib.PB_ERR_UNSUPPORTED
    assert built_lib.pb_quantize_dual(one, 1, 1, 128, 1024, 0, one, one, one, one, one, one, None, 0, None) == 5
    # pb_elementwise: four ops
    assert built_lib.pb_elementwise(7, one, 0, one, one, one, 0, one, one, 1, 16, 16, 16, 16, one, None) == _lib.PB_ERR_UNSUPPORTED
    assert built_lib.pb_elementwise(0, one, 0, one, one, one, 0, one, one, 1, 16, 17, 16, 16, one, None) == 2
    assert built_lib.pb_elementwise(0, None, 0, one, one, one, 0, one, one, 1, 16, 16, 16, 16, one, None) == 1
    # pb_gemm_tn_ex: unknown flag bits
    a = _lib.Operand(4096, 4096, 4096, 256, 1024, 1, 128, 0, 0)
    assert built_lib.pb_gemm_tn_ex(a, op, one, 0, 1024, one, 1 << 20, 8, None) == _lib.PB_ERR_UNSUPPORTED
    assert b"flag" in built_lib.pb_last_error()
