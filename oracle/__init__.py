"""CPU checkers for the deformable-convolution forward (test infrastructure).

``port_forward``  -- the plain-C restatement (``dcn_oracle.c``) through ctypes.
``ref_forward``   -- the unmodified reference CPU extension built into
                     ``oracle/_ref`` (present only where it was compiled).

Nothing in the shipped package imports this module; tests, the smoke check
and the benchmark's CPU-baseline leg do.
"""
import ctypes
import importlib.util
import os

import torch

from .build_oracle import PORT_SO, REF_NAME, REF_SO, build_port

_port = None
_ref = None


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def out_size(in_size, pad, dil, k, stride):
    return (in_size + 2 * pad - (dil * (k - 1) + 1)) // stride + 1


def load_port():
    global _port
    if _port is None:
        if not os.path.exists(PORT_SO):
            build_port()
        lib = ctypes.CDLL(PORT_SO)
        f = ctypes.c_void_p
        lib.dcn_oracle_forward_f32.argtypes = [f] * 6 + [ctypes.c_int] * 15
        lib.dcn_oracle_forward_f32.restype = ctypes.c_int
        lib.dcn_oracle_bilinear.argtypes = [f, ctypes.c_int, ctypes.c_int,
                                            ctypes.c_float, ctypes.c_float]
        lib.dcn_oracle_bilinear.restype = ctypes.c_float
        lib.dcn_oracle_num_threads.restype = ctypes.c_int
        _port = lib
    return _port


def have_ref():
    return os.path.exists(REF_SO)


def load_ref():
    """The reference CPU extension as a Python module (five reference names)."""
    global _ref
    if _ref is None:
        if not have_ref():
            raise RuntimeError('reference CPU extension not built: run '
                               'python oracle/build_oracle.py where the '
                               'reference checkout is present')
        spec = importlib.util.spec_from_file_location(REF_NAME, REF_SO)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ref = mod
    return _ref


def _prep(x, offset, mask, weight, bias):
    f = lambda t: None if t is None else t.detach().to('cpu', torch.float32).contiguous()
    return f(x), f(offset), f(mask), f(weight), f(bias)


def port_forward(x, offset, mask, weight, bias=None, stride=1, padding=0,
                 dilation=1, groups=1, deform_groups=1):
    """fp32 forward through the C restatement; mask=None is the v1 operator."""
    lib = load_port()
    x, offset, mask, weight, bias = _prep(x, offset, mask, weight, bias)
    sh, sw = _pair(stride); ph, pw = _pair(padding); dh, dw = _pair(dilation)
    N, C, H, W = x.shape
    Co, _, kh, kw = weight.shape
    Ho, Wo = out_size(H, ph, dh, kh, sh), out_size(W, pw, dw, kw, sw)
    out = torch.empty(N, Co, Ho, Wo, dtype=torch.float32)
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    rc = lib.dcn_oracle_forward_f32(p(x), p(offset), p(mask), p(weight), p(bias),
                                    p(out), N, C, H, W, Co, kh, kw, sh, sw, ph,
                                    pw, dh, dw, groups, deform_groups)
    if rc != 0:
        raise RuntimeError(f'dcn_oracle_forward_f32 rejected the arguments ({rc})')
    return out


def ref_forward(x, offset, mask, weight, bias=None, stride=1, padding=0,
                dilation=1, groups=1, deform_groups=1, im2col_step=None):
    """fp32 forward through the unmodified reference CPU extension."""
    ext = load_ref()
    x, offset, mask, weight, bias = _prep(x, offset, mask, weight, bias)
    sh, sw = _pair(stride); ph, pw = _pair(padding); dh, dw = _pair(dilation)
    N, C, H, W = x.shape
    Co, _, kh, kw = weight.shape
    Ho, Wo = out_size(H, ph, dh, kh, sh), out_size(W, pw, dw, kw, sw)
    out = x.new_empty(N, Co, Ho, Wo)
    e = x.new_empty(0)
    if mask is None:
        assert bias is None, 'the v1 operator has no bias'
        step = min(im2col_step or 32, N)
        while N % step:
            step -= 1
        ext.deform_conv_forward(x, weight, offset, out, e, e.clone(), kW=kw, kH=kh,
                                dW=sw, dH=sh, padW=pw, padH=ph, dilationW=dw,
                                dilationH=dh, group=groups,
                                deformable_group=deform_groups, im2col_step=step)
    else:
        ext.modulated_deform_conv_forward(
            x, weight, bias if bias is not None else e, e.clone(), offset, mask,
            out, e.clone(), kernel_h=kh, kernel_w=kw, stride_h=sh, stride_w=sw,
            pad_h=ph, pad_w=pw, dilation_h=dh, dilation_w=dw, group=groups,
            deformable_group=deform_groups, with_bias=bias is not None)
    return out


def best_forward(*a, **k):
    """Reference extension when it was built, the C restatement otherwise."""
    return (ref_forward if have_ref() else port_forward)(*a, **k)
