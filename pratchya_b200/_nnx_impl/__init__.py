from ._module import Linear, LowRankFFN, lecun_normal, linear_fp8
