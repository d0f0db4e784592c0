"""d2conv3d_b200 -- B200 (sm_100a) kernels for the D2Conv3D hot path behind the
reference's Python API.

    from d2conv3d_b200 import dconv_native, fast_depthwise_conv3d
    d2conv3d_b200.install_as_dropin()   # then `import dconv_native` resolves here

All compute is done by libd2conv3d.so (C ABI in include/d2conv3d.h); there is no
CPU or PyTorch fallback.
"""
import sys

from . import _lib
from ._lib import get_keep_samples, get_math_mode, set_keep_samples, set_math_mode
from . import dconv_native, fast_depthwise_conv3d
from .dconv_native import (DConv3d, DeformConv3d, MDConv3d, deform_conv3d, dyn_dilated_conv3d)
from .fast_depthwise_conv3d import DepthwiseConv3d

__all__ = ["dconv_native", "fast_depthwise_conv3d", "deform_conv3d", "dyn_dilated_conv3d", "DeformConv3d",
           "DConv3d", "MDConv3d", "DepthwiseConv3d", "set_math_mode", "get_math_mode", "set_keep_samples", "get_keep_samples",
           "install_as_dropin"]


def install_as_dropin():
    """Registers this package's mirrors under the reference's top-level module names, so
    that unmodified caller code (`import dconv_native`, `from fast_depthwise_conv3d import
    DepthwiseConv3d`) picks them up."""
    for name, mod in (("dconv_native", dconv_native), ("fast_depthwise_conv3d", fast_depthwise_conv3d)):
        sys.modules[name] = mod
        for sub in ("_ops", "deform_conv", "modules", "grid", "util", "conv"):
            full = f"{mod.__name__}.{sub}"
            if full in sys.modules:
                sys.modules[f"{name}.{sub}"] = sys.modules[full]
