"""B200-native WTConv wavelet-convolution layers.

``WTConv2d`` / ``WTConv1d`` keep the reference constructor and ``state_dict``
(wtconv/wtconv2d.py:8-36, wtconv/wtconv1d.py:8-36) and run their forward (and the
backward of ``WTConv2d``) in hand-written sm_100a kernels behind the C ABI of
``include/wtconv_b200.h``.
"""
from .modules import WTConv1d, WTConv2d  # noqa: F401

__all__ = ["WTConv2d", "WTConv1d"]
