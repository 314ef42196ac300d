"""pb_quantize_static: the quantizer for hosts that cannot hand over or allocate scratch
memory around the call (an FFI custom call registered without a scratch buffer, a fixed-buffer
replay loop, an allocator that must not be re-entered from inside an op).  Its scratch is a
device array compiled into the library, so the test drives it through the C ABI with nothing but
input and output pointers and checks it against pb_quantize, which uses a caller workspace.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test."""
import numpy as np
import pytest
import torch

from pratchya_b200 import _lib

pytestmark = pytest.mark.gpu


def _run_both(lib, x, grid):
    a, b = grid
    rows, cols = x.shape[-2:]
    batch = x.numel() // (rows * cols)
    nb = rows * cols // (a * b) * batch
    stream = torch.cuda.current_stream().cuda_stream
    code = _lib.PB_BF16 if x.dtype == torch.bfloat16 else _lib.PB_F32

    def outputs():
        return (torch.full(x.shape, 0xAB, dtype=torch.uint8, device="cuda"),
                torch.full((nb,), 0xCD, dtype=torch.uint8, device="cuda"),
                torch.full((nb,), -1.0, dtype=torch.float32, device="cuda"))

    q0, s0, f0 = outputs()
    ws_bytes = lib.pb_quantize_workspace_size(batch, rows, cols, a, b)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    _lib.check(lib.pb_quantize(x.data_ptr(), code, batch, rows, cols, a, b, _lib.PB_E4M3,
                               q0.data_ptr(), s0.data_ptr(), f0.data_ptr(), ws.data_ptr(), ws_bytes, stream))
    q1, s1, f1 = outputs()
    _lib.check(lib.pb_quantize_static(x.data_ptr(), code, batch, rows, cols, a, b, _lib.PB_E4M3,
                                      q1.data_ptr(), s1.data_ptr(), f1.data_ptr(), stream))
    torch.cuda.synchronize()
    return (q0, s0, f0), (q1, s1, f1)


def test_static_scratch_quantize_matches_workspace_quantize_twice_in_a_row(built_lib):
    torch.manual_seed(0)
    # first call: a (128,128) weight with 256 blocks; second call: fewer, differently scaled blocks
    # on another grid, so stale amax bits or divisors from the first call would show up
    cases = [(torch.randn(2048, 2048, device="cuda") * 0.02, (128, 128)),
             (torch.randn(3, 64, 96, device="cuda").to(torch.bfloat16) * 5.0, (16, 16)),
             (torch.randn(512, 1024, device="cuda"), (1, 128))]          # scratch-free grid goes through as well
    for x, grid in cases:
        (q0, s0, f0), (q1, s1, f1) = _run_both(built_lib, x.contiguous(), grid)
        m, k = _lib_geometry(built_lib, x.shape[-2], x.shape[-1], grid)
        groups = x.numel() // (x.shape[-2] * x.shape[-1]) * m
        assert torch.equal(q0, q1), f"fp8 bytes differ on grid {grid}"
        assert torch.equal(s0, s1), f"e8m0 bytes differ on grid {grid}"
        assert torch.equal(f0[:groups], f1[:groups]), f"fp32 scales differ on grid {grid}"


def _lib_geometry(lib, rows, cols, grid):
    import ctypes as C
    m, k = C.c_int64(), C.c_int64()
    _lib.check(lib.pb_group_geometry(rows, cols, grid[0], grid[1], C.byref(m), C.byref(k)))
    return m.value, k.value


def test_static_scratch_rejects_oversized_inputs(built_lib):
    x = torch.zeros(4096, 4096, device="cuda")          # (4,4) blocks: 1,048,576 > 65,536
    q = torch.empty(4096, 4096, dtype=torch.uint8, device="cuda")
    s = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    f = torch.empty(1 << 20, dtype=torch.float32, device="cuda")
    st = built_lib.pb_quantize_static(x.data_ptr(), _lib.PB_F32, 1, 4096, 4096, 4, 4, _lib.PB_E4M3,
                                      q.data_ptr(), s.data_ptr(), f.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 8 and b"exceed the built-in scratch" in built_lib.pb_last_error()
