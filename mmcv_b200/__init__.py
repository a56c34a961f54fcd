"""B200-native forward of deformable convolution v1/v2 behind the ``mmcv.ops`` interface.

``mmcv_b200.ops`` carries the layer classes and functions under the reference's names;
``mmcv_b200._ext`` is the stand-in for the reference's compiled extension;
``install()`` points an installed ``mmcv`` at it.
"""
from . import _lib

__version__ = '0.1.0'


def frozen_weights():
    """Context manager for serving and evaluation: while it is active, each layer's weights
    are cast and re-laid-out for the tensor-core kernel once instead of on every call
    (see ``mmcv_b200._ext.frozen_weights``)."""
    from . import _ext
    return _ext.frozen_weights()


def install():
    """Make an installed ``mmcv`` use this library for the deformable-conv forward.

    Replaces the module-global ``ext_module`` that ``mmcv.ops.modulated_deform_conv``,
    ``mmcv.ops.deform_conv`` and ``mmcv.ops.multi_scale_deform_attn`` look their compiled entry
    points up on (mmcv/ops/modulated_deform_conv.py:17-19, mmcv/ops/deform_conv.py:19-22,
    mmcv/ops/multi_scale_deform_attn.py:19-20).  Returns
    the list of patched modules; raises ImportError if ``mmcv`` is not importable.
    """
    import importlib
    from . import _ext
    patched = []
    for name in ('mmcv.ops.modulated_deform_conv', 'mmcv.ops.deform_conv',
                 'mmcv.ops.multi_scale_deform_attn'):
        mod = importlib.import_module(name)
        mod.ext_module = _ext
        patched.append(name)
    return patched
