"""Host-side rules that need no GPU: grid adaptation, scale geometry, tensor-core eligibility,
the qx name lookup, and the refusal to run on CPU tensors."""
import pytest
import torch

from oracle import qarr_oracle as o
from pratchya_b200 import QArrayImpl, qx
from pratchya_b200._qualia import _ops
from pratchya_b200._qualia._qarr import _adapt_grid


@pytest.mark.parametrize("grid,shape", [((128, 128), (2048, 96)), ((1, 128), (7,)), ((16, 16), ()), ((4, 4), (3, 6, 10)), ((128, 1), (256, 32))])
def test_adapt_grid_matches_oracle(grid, shape):
    assert _adapt_grid(grid, shape) == o.adapt_grid(grid, shape)


@pytest.mark.parametrize("rows,cols,grid", [(2048, 2048, (1, 128)), (2048, 8192, (128, 128)), (4096, 16384, (128, 128)), (3, 48, (1, 16)), (8, 8, (1, 1))])
def test_group_geometry_matches_oracle(rows, cols, grid):
    assert _ops.group_geometry(rows, cols, grid) == o.group_geometry(rows, cols, grid)


def test_group_geometry_rejects_indivisible_shapes():
    with pytest.raises(ValueError):
        _ops.group_geometry(10, 10, (4, 4))


def test_tensor_core_eligibility():
    e4 = torch.float8_e4m3fn
    x = torch.empty(256, 1024, dtype=e4)
    w = torch.empty(1024, 512, dtype=e4)
    assert _ops._tensor_core_eligible(x, w, (1, 128), (128, 128))
    assert _ops._tensor_core_eligible(torch.empty(4, 64, 1024, dtype=e4), w, (1, 128), (128, 128))     # batched activations
    assert not _ops._tensor_core_eligible(x, w, (1, 16), (16, 16))
    assert not _ops._tensor_core_eligible(torch.empty(3, 384, dtype=e4), torch.empty(384, 128, dtype=e4), (1, 128), (128, 128))  # 9 blocks: K = 1
    assert not _ops._tensor_core_eligible(x, torch.empty(1024, 100, dtype=e4), (1, 128), (128, 128))


def test_cpu_tensors_are_refused():
    with pytest.raises(RuntimeError):
        QArrayImpl(torch.zeros(8, 128), (1, 128))
    with pytest.raises(RuntimeError):
        _ops.dequantize_impl(torch.zeros(8, 128).to(torch.float8_e4m3fn), torch.zeros(1, 8, dtype=torch.uint8), torch.zeros(1, 1, 1), torch.float32, (1, 128))


def test_unquantized_box_and_qx_lookup():
    box = QArrayImpl(torch.arange(6.0).reshape(2, 3), quant=False)
    assert box.shape == (2, 3) and not box._is_quantized() and box[1].get_value().tolist() == [3.0, 4.0, 5.0]
    assert box.astype(torch.float64).dtype == torch.float64
    out = qx.relu(torch.tensor([-1.0, 2.0]))
    assert isinstance(out, QArrayImpl) and out.get_value().tolist() == [0.0, 2.0]
    with pytest.raises(AttributeError):
        qx.definitely_not_a_function
