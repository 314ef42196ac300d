from ._qarr import QArrayImpl, fp8_matmul, fp8_matmul_bwd
from ._ops import (quantize_impl, dequantize_impl, dequantize_impl_bwd, quantize_transposed_impl, matmul_impl,
                   matmul_mixed_impl, rmatmul_mixed_impl, add_impl, mul_impl, sub_impl, truediv_impl,
                   floordiv_impl, mod_impl, pow_impl, group_geometry, LinearStep, fake_quantize_impl, quantize_dual_impl,
                   quantize_impl_bwd, matmul_impl_bwd, matmul_mixed_impl_bwd, rmatmul_mixed_impl_bwd, make_elementwise_impl_bwd,
                   add_impl_bwd, mul_impl_bwd, sub_impl_bwd, truediv_impl_bwd, floordiv_impl_bwd, mod_impl_bwd, pow_impl_bwd,
                   reduce_broadcast, set_literal_dot_precision)
from . import _qual as qx
