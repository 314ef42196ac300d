from ._module import Linear, LowRankFFN, lecun_normal
