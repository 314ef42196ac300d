"""ctypes binding of libpratchya_b200.so (the C ABI declared in include/pratchya_b200.h).

There is no CPU fallback: if the library has not been built, or CUDA is not
usable, the ops raise.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libpratchya_b200.so"
_DIAG_LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libpratchya_b200_diag.so"
_lib = None
_diag_lib = None

PB_F32, PB_BF16 = 0, 1
PB_E4M3, PB_E5M2 = 0, 1


PB_ERR_UNSUPPORTED = 8


class PbError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"pratchya_b200 status {status}: {text}")
        self.status = status


class Operand(C.Structure):
    """Mirror of `pb_operand`."""
    _fields_ = [
        ("q", C.c_void_p), ("sc8", C.c_void_p), ("sc32", C.c_void_p),
        ("rows", C.c_int64), ("depth", C.c_int64),
        ("grid_a", C.c_int), ("grid_b", C.c_int), ("format", C.c_int), ("transposed_blocks", C.c_int),
    ]


_i64, _int, _ptr, _sz = C.c_int64, C.c_int, C.c_void_p, C.c_size_t
_SIGNATURES = {
    "pb_version": (C.c_int, []),
    "pb_last_error": (C.c_char_p, []),
    "pb_status_string": (C.c_char_p, [_int]),
    "pb_group_geometry": (_int, [_i64, _i64, _int, _int, C.POINTER(_i64), C.POINTER(_i64)]),
    "pb_quantize_workspace_size": (_sz, [_i64, _i64, _i64, _int, _int]),
    "pb_quantize": (_int, [_ptr, _int, _i64, _i64, _i64, _int, _int, _int, _ptr, _ptr, _ptr, _ptr, _sz, _ptr]),
    "pb_quantize_static": (_int, [_ptr, _int, _i64, _i64, _i64, _int, _int, _int, _ptr, _ptr, _ptr, _ptr]),
    "pb_quantize_transposed_workspace_size": (_sz, [_i64, _i64, _i64, _int]),
    "pb_quantize_transposed": (_int, [_ptr, _int, _i64, _i64, _i64, _int, _int, _ptr, _ptr, _ptr, _ptr, _sz, _ptr]),
    "pb_quantize_dual": (_int, [_ptr, _int, _i64, _i64, _i64, _int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _sz, _ptr]),
    "pb_dequantize": (_int, [_ptr, _int, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _int, _ptr, _ptr]),
    "pb_dequantize_bwd": (_int, [_ptr, _int, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr]),
    "pb_gemm_workspace_size": (_sz, [C.POINTER(Operand), C.POINTER(Operand)]),
    "pb_gemm_tn": (_int, [C.POINTER(Operand), C.POINTER(Operand), _ptr, _int, _i64, _ptr, _sz, _ptr]),
    "pb_gemm_tn_ex": (_int, [C.POINTER(Operand), C.POINTER(Operand), _ptr, _int, _i64, _ptr, _sz, C.c_uint, _ptr]),
    "pb_quantize_for_gemm": (_int, [_ptr, _int, _i64, _i64, _int, _ptr, _ptr, _ptr, C.POINTER(Operand), _ptr, _sz, _ptr]),
    "pb_relu2_requantize": (_int, [_ptr, _i64, _i64, _int, _ptr, _ptr, _ptr, C.POINTER(Operand), _ptr, _sz, _ptr]),
    "pb_elementwise": (_int, [_int, _ptr, _int, _ptr, _ptr, _ptr, _int, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr]),
    "pb_momentum_workspace_size": (_sz, [_i64, _i64, _i64, _int, _int]),
    "pb_momentum_update": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _int,
                                  C.c_float, C.c_float, C.c_float, C.c_float, _ptr, _ptr, _ptr, _ptr, _ptr, _sz, _ptr]),
    "pb_momentum_update_stacked": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _int,
                                          C.c_float, C.c_float, C.c_float, C.c_float, _ptr, _ptr, _ptr, _ptr, _ptr, _sz, _ptr]),
    "pb_fake_quantize": (_int, [_ptr, _int, _i64, _i64, _i64, _int, _int, _int, _ptr, _int, _ptr]),
    "pb_gemm_check": (_int, [_ptr]),
    "pb_transpose_bytes": (_int, [_ptr, _i64, _i64, _ptr, _ptr]),
    "pb_token_shift_lerp": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _ptr, _ptr]),
    "pb_token_shift_lerp_bwd_workspace_size": (_sz, [_i64, _i64, _i64, _int]),
    "pb_token_shift_lerp_bwd": (_int, [_ptr] * 4 + [_i64, _i64, _i64, _int] + [_ptr] * 4 + [_sz, _ptr]),
    "pb_relu2_quantize_dual": (_int, [_ptr, _i64, _i64] + [_ptr] * 7),
    "pb_dequantize_bwd_quantize_dual": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _int] + [_ptr] * 7),
    "pb_shift_lerp_quantize": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _ptr, _ptr, _ptr, C.c_uint, _ptr, _ptr, _ptr, _ptr]),
    "pb_wkv_prepare": (_int, [_ptr] * 11 + [_i64, _i64, _i64, _int] + [_ptr] * 8),
    "pb_wkv_prepare_bwd_workspace_size": (_sz, [_i64, _i64, _i64, _int]),
    "pb_wkv_prepare_bwd": (_int, [_ptr] * 11 + [_i64, _i64, _i64, _int] + [_ptr] * 17 + [_sz, _ptr]),
    "pb_rms_norm": (_int, [_ptr, _ptr, _i64, _i64, C.c_float, _ptr, _ptr, _ptr]),
    "pb_rms_norm_bwd_workspace_size": (_sz, [_i64, _i64]),
    "pb_rms_norm_bwd": (_int, [_ptr] * 4 + [_i64, _i64] + [_ptr] * 3 + [_sz, _ptr]),
    "pb_relu2": (_int, [_ptr, _i64, _ptr, _ptr]),
    "pb_relu2_bwd": (_int, [_ptr, _ptr, _i64, _ptr, _ptr]),
    "pb_wkv_finish_workspace_size": (_sz, [_i64, _i64, _i64, _int]),
    "pb_wkv_finish": (_int, [_ptr] * 8 + [C.c_float, _i64, _i64, _i64, _int] + [_ptr] * 3 + [_sz, _ptr]),
    "pb_wkv_finish_bwd_workspace_size": (_sz, [_i64, _i64, _i64, _int]),
    "pb_wkv_finish_bwd": (_int, [_ptr] * 10 + [_i64, _i64, _i64, _int] + [_ptr] * 9 + [_sz, _ptr]),
    "pb_smoothed_xent": (_int, [_ptr, _ptr, _ptr, _i64, _i64, C.c_float, _ptr, _ptr, _ptr]),
    "pb_smoothed_xent_bwd": (_int, [_ptr] * 5 + [C.c_float, _i64, _i64, C.c_float, _ptr, _ptr]),
    "pb_wkv7_forward": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "pb_wkv7_checkpoint_floats": (_sz, [_i64, _i64, _i64, _int]),
    "pb_wkv7_backward": (_int, [_ptr] * 10 + [_i64, _i64, _i64, _int] + [_ptr] * 8),
}
# extra exports of the diagnostics build (libpratchya_b200_diag.so): test hooks, not part of the C ABI
_DIAG_SIGNATURES = {
    "pb_debug_division_check": (_int, [C.c_uint64, C.c_uint64, _ptr, _ptr]),
    "pb_debug_gemm_profile": (_int, [C.POINTER(C.c_uint64), _ptr]),
    "pb_debug_gemm_control": (_int, [C.c_uint, _int]),
}

# every symbol include/pratchya_b200.h declares (checked by the CPU test-suite)
DECLARED_SYMBOLS = tuple(_SIGNATURES)


def lib_path() -> Path:
    return _LIB_PATH


def _open(path: Path, signatures):
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m pratchya_b200.csrc.build` "
            "(there is no CPU fallback for the pratchya_b200 ops)")
    lib = C.CDLL(str(path))
    for name, (res, args) in signatures.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue          # reported by the symbol test; calling it raises AttributeError
        fn.restype, fn.argtypes = res, args
    return lib


def load():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        _lib = _open(_LIB_PATH, _SIGNATURES)
    return _lib


def load_diagnostics():
    """The diagnostics build of the same sources (cycle counters, fault injection, device self-checks).
    A separate library with its own device state; the ops of this package never use it."""
    global _diag_lib
    if _diag_lib is None:
        _diag_lib = _open(_DIAG_LIB_PATH, {**_SIGNATURES, **_DIAG_SIGNATURES})
    return _diag_lib


def check(status: int):
    if status != 0:
        raise PbError(status, load().pb_last_error().decode(errors="replace"))
