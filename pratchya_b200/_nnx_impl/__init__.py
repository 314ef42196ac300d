from ._module import ChannelMixFFN, Linear, LowRankFFN, lecun_normal, linear_fp8
from ._optimizer import lion_update, momentum_update, momentum_update_stacked
from ._wkv7 import wkv_state_scan
