"""Drop-in for the reference's `dconv_native` package (same public names)."""
from . import _ops  # noqa: F401
from .deform_conv import (DeformConv1d, DeformConv3d, DeformConvNd, deform_conv1d, deform_conv3d,
                          dyn_dilated_conv3d)
from .modules import (DConv3d, MDConv3d, SizeConditionedDConv3d, SizeConditionedMDConv3d,
                      XYSizeConditionedDConv3d, XYSizeConditionedMDConv3d, XXZSizeConditionedDConv3d,
                      XXZSizeConditionedMDConv3d, XYZSizeConditionedDConv3d, XYZSizeConditionedMDConv3d)

__all__ = [
    "deform_conv1d", "deform_conv3d",
    "DeformConv1d", "DeformConv3d",
    "DConv3d", "MDConv3d",
    "SizeConditionedDConv3d", "SizeConditionedMDConv3d",
]
