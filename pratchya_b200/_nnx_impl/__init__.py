from ._module import ChannelMixFFN, Linear, LowRankFFN, lecun_normal, linear_fp8
