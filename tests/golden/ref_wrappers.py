"""Load the reference's UNCHANGED Python wrappers for the deformable-conv path
on top of an arbitrary extension module (test infrastructure).

The reference package cannot be imported as a whole here (its registry/logging
dependency ``mmengine`` is not installed), but the two wrapper files
``mmcv/ops/modulated_deform_conv.py`` and ``mmcv/ops/deform_conv.py`` only need
a handful of names from it, none of which does arithmetic.  ``load`` puts small
stand-ins for those names into ``sys.modules``, registers ``ext`` as
``mmcv._ext`` (the name ``mmcv/utils/ext_loader.py:12-16`` imports) and executes
the two wrapper files from the reference checkout, unmodified.
"""
import functools
import importlib.util
import os
import sys
import types

import torch

_NAMES = ['mmengine', 'mmengine.logging', 'mmengine.registry', 'mmengine.utils',
          'mmengine.utils.dl_utils', 'mmengine.model', 'mmcv', 'mmcv.utils', 'mmcv.utils.ext_loader',
          'mmcv._ext', 'mmcv.ops', 'mmcv.ops.modulated_deform_conv',
          'mmcv.ops.deform_conv', 'mmcv.ops.multi_scale_deform_attn']


class _Registry:
    def __init__(self):
        self.modules = {}

    def register_module(self, name=None, **_):
        def deco(cls):
            self.modules[name or cls.__name__] = cls
            return cls
        return deco

    def get(self, name):
        return self.modules[name]


def _digit_version(v):
    out = []
    for part in str(v).split('+')[0].split('.'):
        digits = ''.join(ch for ch in part if ch.isdigit())
        out.append(int(digits) if digits else 0)
    return tuple(out)


def _deprecated_api_warning(name_dict, cls_name=None):
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            for old, new in name_dict.items():
                if old in k:
                    k[new] = k.pop(old)
            return fn(*a, **k)
        return wrapped
    return deco


def _module(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    return m


def _exec(name, path, package):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    mod.__package__ = package
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


class _BaseModule(torch.nn.Module):
    def __init__(self, init_cfg=None):
        super().__init__()
        self.init_cfg = init_cfg
        self._is_init = False


def _constant_init(module, val, bias=0):
    if getattr(module, 'weight', None) is not None:
        torch.nn.init.constant_(module.weight, val)
    if getattr(module, 'bias', None) is not None:
        torch.nn.init.constant_(module.bias, bias)


def _xavier_init(module, gain=1, bias=0, distribution='normal'):
    if getattr(module, 'weight', None) is not None:
        if distribution == 'uniform':
            torch.nn.init.xavier_uniform_(module.weight, gain=gain)
        else:
            torch.nn.init.xavier_normal_(module.weight, gain=gain)
    if getattr(module, 'bias', None) is not None:
        torch.nn.init.constant_(module.bias, bias)


def default_root():
    """Where the reference's wrapper files are: the checkout named by DCN_REFERENCE_ROOT, else
    the copies the checker's build recipe left under oracle/_ref/pywrap; None if neither exists."""
    root = os.environ.get('DCN_REFERENCE_ROOT', '')
    if root and os.path.isfile(os.path.join(root, 'mmcv/ops/deform_conv.py')):
        return root
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    wrap = os.path.join(here, 'oracle', '_ref', 'pywrap')
    return wrap if os.path.isfile(os.path.join(wrap, 'mmcv/ops/deform_conv.py')) else None


def load(ext, ref_root=None):
    """Returns (modulated_deform_conv module, deform_conv module, registry)."""
    ref_root = ref_root or default_root()
    if ref_root is None:
        raise FileNotFoundError('the reference wrapper files are not available')
    for n in _NAMES:
        sys.modules.pop(n, None)
    reg = _Registry()
    sys.modules['mmengine'] = _module('mmengine', __path__=[], ConfigDict=dict)
    sys.modules['mmengine.model'] = _module(
        'mmengine.model', BaseModule=_BaseModule, constant_init=_constant_init,
        xavier_init=_xavier_init)
    sys.modules['mmengine.logging'] = _module(
        'mmengine.logging', print_log=lambda *a, **k: None)
    sys.modules['mmengine.registry'] = _module('mmengine.registry', MODELS=reg)
    sys.modules['mmengine.utils'] = _module(
        'mmengine.utils', __path__=[], digit_version=_digit_version,
        deprecated_api_warning=_deprecated_api_warning)
    sys.modules['mmengine.utils.dl_utils'] = _module(
        'mmengine.utils.dl_utils', TORCH_VERSION=torch.__version__)
    sys.modules['mmcv'] = _module('mmcv', __path__=[])
    sys.modules['mmcv._ext'] = ext
    utils = _module('mmcv.utils', __path__=[], IS_MLU_AVAILABLE=False,
                    IS_MUSA_AVAILABLE=False, IS_NPU_AVAILABLE=False,
                    IS_MPS_AVAILABLE=False,
                    IS_CUDA_AVAILABLE=torch.cuda.is_available())
    sys.modules['mmcv.utils'] = utils
    utils.ext_loader = _exec('mmcv.utils.ext_loader',
                             os.path.join(ref_root, 'mmcv/utils/ext_loader.py'),
                             'mmcv.utils')
    sys.modules['mmcv.ops'] = _module('mmcv.ops', __path__=[])
    v2 = _exec('mmcv.ops.modulated_deform_conv',
               os.path.join(ref_root, 'mmcv/ops/modulated_deform_conv.py'),
               'mmcv.ops')
    v1 = _exec('mmcv.ops.deform_conv',
               os.path.join(ref_root, 'mmcv/ops/deform_conv.py'), 'mmcv.ops')
    return v2, v1, reg


def load_msda(ext, ref_root=None):
    """The reference's unchanged mmcv/ops/multi_scale_deform_attn.py on top of `ext` (which must
    have ms_deform_attn_forward / ms_deform_attn_backward); call after load()."""
    ref_root = ref_root or default_root()
    path = os.path.join(ref_root, 'mmcv/ops/multi_scale_deform_attn.py')
    if not os.path.isfile(path):
        raise FileNotFoundError('the reference wrapper file of multi-scale deformable attention is not available')
    sys.modules['mmcv._ext'] = ext
    return _exec('mmcv.ops.multi_scale_deform_attn', path, 'mmcv.ops')


def unload():
    for n in _NAMES:
        sys.modules.pop(n, None)
