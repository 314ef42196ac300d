"""The abort path of the CTA-pair GEMM kernel: a bounded wait that runs out.

The diagnostics build of the library (same sources, -DPB_DIAGNOSTICS) can leave the first pipeline
slot of a launch unarmed and unfilled -- no copy is in flight for it, its barrier simply never
completes -- and can shrink the poll budget of the waits to about two milliseconds.  Every role of
both CTAs then runs out of patience, raises the abort flag, leaves its loop, the pair meets at the
cluster barrier, tensor memory is released and the kernel returns: nothing traps, faults or spins
without a limit, and the context stays usable.  The test checks the status word and that the next
launch is bit-identical to the one before."""
import pytest
import torch

from helpers import synth, to_torch
from pratchya_b200 import _lib
from pratchya_b200._qualia import quantize_impl
from pratchya_b200._qualia._ops import transpose_bytes

pytestmark = pytest.mark.gpu

PB_ERR_DEVICE_TIMEOUT = 7


def test_a_bounded_wait_that_runs_out_is_reported_and_the_next_launch_is_clean(built_lib, diag_lib):
    m, k, n = 512, 1024, 512
    x = to_torch(synth((m, k), seed=1)).to(torch.bfloat16)
    w = to_torch(synth((k, n), seed=2, scale=0.02, outliers=0)).to(torch.bfloat16)
    xq, wq = quantize_impl(x, (1, 128)), quantize_impl(w, (128, 128))
    w_t = transpose_bytes(wq[0])
    a = _lib.Operand(xq[0].data_ptr(), xq[1].data_ptr(), xq[2].data_ptr(), m, k, 1, 128, _lib.PB_E4M3, 0)
    b = _lib.Operand(w_t.data_ptr(), wq[1].data_ptr(), wq[2].data_ptr(), n, k, 128, 128, _lib.PB_E4M3, 1)
    ws_bytes = diag_lib.pb_gemm_workspace_size(a, b)
    assert ws_bytes > 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def run():
        d = torch.zeros(m, n, dtype=torch.float32, device="cuda")
        assert diag_lib.pb_gemm_tn(a, b, d.data_ptr(), _lib.PB_F32, n, ws.data_ptr(), ws_bytes, st) == 0
        return d

    before = run()
    assert diag_lib.pb_gemm_check(st) == 0
    assert before.abs().max().item() > 0
    try:
        assert diag_lib.pb_debug_gemm_control(1 << 10, 8) == 0      # ~2 ms budget; first slot never arrives
        run()
        assert diag_lib.pb_gemm_check(st) == PB_ERR_DEVICE_TIMEOUT
        assert b"ran out" in diag_lib.pb_last_error()
        assert diag_lib.pb_gemm_check(st) == 0                        # reading the status clears it
    finally:
        diag_lib.pb_debug_gemm_control(0, 0)
    after = run()
    assert diag_lib.pb_gemm_check(st) == 0
    assert torch.equal(before, after)
    # the product library's own status word was never touched
    assert built_lib.pb_gemm_check(st) == 0
