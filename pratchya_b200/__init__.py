"""B200-native (sm_100a) implementation of pratchya's FP8 block-quantization path.

Public surface mirrors pratchya/__init__.py: `QArrayImpl` and `qx`.
"""
from ._qualia import QArrayImpl, qx

__all__ = ["QArrayImpl", "qx"]
