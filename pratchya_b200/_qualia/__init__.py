from ._qarr import QArrayImpl, fp8_matmul
from ._ops import (quantize_impl, dequantize_impl, dequantize_impl_bwd, quantize_transposed_impl, matmul_impl,
                   matmul_mixed_impl, rmatmul_mixed_impl, add_impl, mul_impl, sub_impl, truediv_impl,
                   floordiv_impl, mod_impl, pow_impl, group_geometry, LinearStep, fake_quantize_impl, quantize_dual_impl)
from . import _qual as qx
