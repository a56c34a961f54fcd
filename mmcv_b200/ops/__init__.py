"""The deformable-convolution names of ``mmcv.ops`` and their sibling sampler (reference:
mmcv/ops/__init__.py)."""
from .deform_conv import DeformConv2d, DeformConv2dFunction, DeformConv2dPack, deform_conv2d
from .modulated_deform_conv import (ModulatedDeformConv2d, ModulatedDeformConv2dFunction,
                                    ModulatedDeformConv2dPack, modulated_deform_conv2d)
from .multi_scale_deform_attn import (MultiScaleDeformableAttention,
                                      MultiScaleDeformableAttnFunction)
from .saconv import SAConv2d

__all__ = ['DeformConv2d', 'DeformConv2dFunction', 'DeformConv2dPack', 'deform_conv2d',
           'ModulatedDeformConv2d', 'ModulatedDeformConv2dFunction',
           'ModulatedDeformConv2dPack', 'modulated_deform_conv2d', 'SAConv2d',
           'MultiScaleDeformableAttention', 'MultiScaleDeformableAttnFunction']
