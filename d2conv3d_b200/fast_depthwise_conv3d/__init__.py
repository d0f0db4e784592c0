"""Drop-in for the reference's `fast_depthwise_conv3d` package."""
from . import _ops  # noqa: F401
from .conv import DepthwiseConv3d

__all__ = ["DepthwiseConv3d"]
