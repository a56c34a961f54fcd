"""Stand-in for the reference's compiled extension module, for this path only.

Exposes the five functions that the reference's Python wrappers look up on
``mmcv._ext`` (``mmcv/ops/modulated_deform_conv.py:17-19``,
``mmcv/ops/deform_conv.py:19-22``) with the positional order and keyword names
of the reference's module definition (``mmcv/ops/csrc/pytorch/pybind.cpp:525-545,
641-656``).  All five call the CUDA library through its C ABI; the backward entries
additionally use torch.matmul for the two matrix products the reference gives to addmm_.
"""
import contextlib
import ctypes
import os

import torch

from . import _lib

_FP32_MATH = {'ffma': _lib.MATH_FFMA, 'tf32x3': _lib.MATH_TF32X3}
_fp32_math = os.environ.get('DCN_B200_FP32_MATH', 'tf32x3').lower()
_check_status = os.environ.get('DCN_B200_CHECK_STATUS', '0') == '1'


def set_fp32_math(mode: str) -> None:
    """Contraction arithmetic for fp32 tensors: 'tf32x3' (tensor cores, three TF32 products
    per step; the default) or 'ffma' (SIMT cores).  Both meet the fp32 error bound."""
    global _fp32_math
    if mode not in _FP32_MATH:
        raise ValueError(f'unknown fp32 math mode {mode!r}')
    _fp32_math = mode


def set_check_status(flag: bool) -> None:
    """Read the device status word after every call (synchronises)."""
    global _check_status
    _check_status = bool(flag)


def _dtype_code(t):
    if t.dtype == torch.float32:
        return _lib.DTYPE_F32
    if t.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    if t.dtype == torch.float16:
        return _lib.DTYPE_F16
    raise RuntimeError(f'dcn_b200: unsupported dtype {t.dtype} (float32, bfloat16 and float16 '
                       'only)')


def _require_cuda(**tensors):
    dev = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f'dcn_b200: {name} must be a CUDA tensor (this build has no '
                               'CPU implementation)')
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f'dcn_b200: {name} is on {t.device}, expected {dev}')
    return dev


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class _FrozenWeights:
    """What frozen_weights() keeps: dtype casts of parameters and their weight images, each
    keyed by the source's device address and held together with the source tensor, so that
    the address cannot be handed to another tensor while the entry lives."""

    def __init__(self):
        self.casts = {}
        self.images = {}


_frozen = None


@contextlib.contextmanager
def frozen_weights():
    """Inside this block the caller promises that no weight changes (serving, evaluation).
    Each layer's weights are then cast and re-laid-out for the tensor-core kernel once, on
    first use, instead of on every call; everything cached is dropped at exit.  Writing to a
    weight inside the block leaves the cached copy stale: leave the block first."""
    global _frozen
    outer, _frozen = _frozen, (_frozen or _FrozenWeights())
    try:
        yield
    finally:
        _frozen = outer


def cast_weight(t, dtype):
    """t in `dtype`; cached while frozen_weights() is active."""
    if t is None or t.dtype == dtype:
        return t
    if _frozen is None or torch.is_grad_enabled() and t.requires_grad:
        return t.to(dtype)
    key = (t.data_ptr(), t.dtype, dtype, tuple(t.shape))
    hit = _frozen.casts.get(key)
    if hit is None:
        hit = _frozen.casts[key] = (t, t.detach().to(dtype))
    return hit[1]


def _weight_image(lib, p, weight, dev, stream):
    """Attach the cached weight image for this problem to p (making it on first use)."""
    key = (weight.data_ptr(), p.dtype, p.math_mode, p.N, p.C, p.H, p.W, p.Co, p.kh, p.kw,
           p.stride_h, p.stride_w, p.pad_h, p.pad_w, p.dil_h, p.dil_w, p.groups,
           p.deform_groups, tuple(p.in_stride), bool(p.offset), bool(p.mask))
    hit = _frozen.images.get(key)
    if hit is None:
        nbytes = ctypes.c_size_t(0)
        _lib.check(lib.dcn_weight_image_bytes(ctypes.byref(p), ctypes.byref(nbytes)))
        image = None
        if nbytes.value:
            image = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
            _lib.check(lib.dcn_prepare_weights(ctypes.byref(p), _ptr(image), nbytes.value,
                                               stream))
        hit = _frozen.images[key] = (weight, image)
    if hit[1] is not None:
        p.weight_image = _ptr(hit[1])
        p.weight_image_bytes = hit[1].numel()


def forward(input, offset, mask, weight, bias, output, stride, padding, dilation,
            groups, deform_groups, math_mode=None, act=_lib.ACT_NONE, act_range=(0, 0),
            offset_batch_stride=0, mask_batch_stride=0, out_batch_stride=0,
            offset_strides=(0, 0), mask_strides=(0, 0), mask_act=_lib.ACT_NONE, padded=None):
    """Launch one forward on the current stream.  offset=None means an ordinary
    convolution, mask=None the unmodulated (v1) operator.  offset_strides / mask_strides are
    (channel, pixel) element strides inside a sample, (0, 0) = dense planes; mask_act =
    ACT_SIGMOID says the mask tensor holds logits; padded = the zero-bordered channels-last copy
    of `input` from pad_channels_last(), when the caller has one.  Returns the workspace tensor."""
    lib = _lib.load()
    dev = _require_cuda(input=input, offset=offset, mask=mask, weight=weight, bias=bias,
                        output=output)
    code = _dtype_code(input)
    for name, t in (('offset', offset), ('mask', mask), ('weight', weight), ('bias', bias),
                    ('output', output)):
        if t is not None and t.dtype != input.dtype:
            raise RuntimeError(f'dcn_b200: {name} has dtype {t.dtype}, input has {input.dtype}')
    if math_mode is None:
        math_mode = _FP32_MATH[_fp32_math] if code == _lib.DTYPE_F32 else _lib.MATH_AUTO
    p = _lib.DcnFwdParams()
    p.input, p.offset, p.mask = _ptr(input), _ptr(offset), _ptr(mask)
    p.weight, p.bias, p.output = _ptr(weight), _ptr(bias), _ptr(output)
    p.dtype, p.math_mode = code, math_mode
    p.N, p.C, p.H, p.W = input.shape
    p.Co = weight.shape[0]
    p.kh, p.kw = weight.shape[2], weight.shape[3]
    p.stride_h, p.stride_w = stride
    p.pad_h, p.pad_w = padding
    p.dil_h, p.dil_w = dilation
    p.groups, p.deform_groups = groups, deform_groups
    for i, s in enumerate(input.stride()):
        p.in_stride[i] = s
    p.offset_batch_stride = offset_batch_stride
    p.mask_batch_stride = mask_batch_stride
    p.out_batch_stride = out_batch_stride
    p.offset_channel_stride, p.offset_pixel_stride = offset_strides
    p.mask_channel_stride, p.mask_pixel_stride = mask_strides
    p.mask_act = mask_act
    if padded is not None:
        p.padded_input, p.padded_input_bytes = _ptr(padded), padded.numel()
    p.act, p.act_lo, p.act_hi = act, act_range[0], act_range[1]
    p.device = dev.index if dev.index is not None else torch.cuda.current_device()
    nbytes = ctypes.c_size_t(0)
    _lib.check(lib.dcn_fwd_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)))
    with torch.cuda.device(dev):
        ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        if _frozen is not None and input.numel():
            _weight_image(lib, p, weight, dev, stream)
        _lib.check(lib.dcn_fwd(ctypes.byref(p), _ptr(ws), nbytes.value, stream))
        if _check_status:
            st = ctypes.c_int32(0)
            _lib.check(lib.dcn_read_status(_ptr(ws), stream, ctypes.byref(st)))
            if st.value != 0:
                raise RuntimeError(f'dcn_b200: device-side wait {st.value} timed out; the '
                                   'output is not valid')
    return ws


def _out_hw(input, weight, stride, padding, dilation):
    """Output height and width, as the reference computes them
    (mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:87-90)."""
    kh, kw = weight.shape[2], weight.shape[3]
    ho = (input.size(2) + 2 * padding[0] - (dilation[0] * (kh - 1) + 1)) // stride[0] + 1
    wo = (input.size(3) + 2 * padding[1] - (dilation[1] * (kw - 1) + 1)) // stride[1] + 1
    return ho, wo


def _check_shapes(input, weight, offset, mask, output, stride, padding, dilation, deform_groups):
    """The kernels index offset, mask and output from the problem geometry alone, so a tensor
    of another shape (an offset made for another stride, a smaller batch, the wrong number of
    deform groups) would be read or written out of bounds: reject it here."""
    if min(stride) <= 0 or min(dilation) <= 0:
        return   # the library reports these with the reference's messages
    N = input.size(0)
    T = weight.size(2) * weight.size(3)
    ho, wo = _out_hw(input, weight, stride, padding, dilation)
    if ho < 1 or wo < 1:
        return   # "output size is too small": reported by the library
    want = {'offset': (N, deform_groups * 2 * T, ho, wo), 'mask': (N, deform_groups * T, ho, wo),
            'output': (N, weight.size(0), ho, wo)}
    for name, t in (('offset', offset), ('mask', mask), ('output', output)):
        if t is not None and tuple(t.shape) != want[name]:
            raise RuntimeError(f'dcn_b200: {name} has shape {tuple(t.shape)}, expected '
                               f'{want[name]} for this input, kernel, stride, padding, dilation '
                               'and deformable_group')


def forward_from_branch(input, branch, n_offset, weight, bias, output, stride, padding, dilation,
                        groups, deform_groups, padded=None):
    """Deformable convolution whose offsets are the first n_offset channels of `branch` (the
    raw output of a Pack layer's offset convolution, NCHW-contiguous or channels-last) and
    whose mask logits are the remaining channels (none: the v1 operator).  The kernel reads
    both where they lie and applies the sigmoid itself.  Returns False, having done nothing,
    when this problem does not run on the tensor-core kernel."""
    if branch.dim() != 4 or branch.dtype != input.dtype:
        return False
    N, Ct, Ho, Wo = branch.shape
    T = weight.size(2) * weight.size(3)
    if n_offset != deform_groups * 2 * T or Ct not in (n_offset, n_offset + deform_groups * T):
        raise RuntimeError(f'dcn_b200: the branch has {Ct} channels with {n_offset} offset '
                           f'channels; expected {deform_groups * 2 * T} offset channels and none '
                           f'or {deform_groups * T} mask channels')
    if (N, Ho, Wo) != (input.size(0),) + _out_hw(input, weight, stride, padding, dilation):
        raise RuntimeError(f'dcn_b200: the branch is {N} x {Ho} x {Wo} (batch, height, width), '
                           'which is not the output size of this problem')
    _check_shapes(input, weight, None, None, output, stride, padding, dilation, deform_groups)
    input = _input_layout(input)
    if N == 0 or (N > 1 and branch.stride(0) != Ct * Ho * Wo):
        return False   # (an empty batch takes the ordinary route)
    if branch.is_contiguous():
        strides = (Ho * Wo, 1)
    elif branch.is_contiguous(memory_format=torch.channels_last):
        strides = (1, Ct)
    else:
        return False
    modulated = n_offset < Ct
    offset = branch
    # a one-element view that starts at the first mask channel (same storage, no copy)
    mask = (branch.as_strided((1,), (1,), branch.storage_offset() + n_offset * strides[0])
            if modulated else None)
    try:
        forward(input, offset, mask, weight, bias, output, stride, padding, dilation, groups,
                deform_groups, offset_batch_stride=Ct * Ho * Wo,
                mask_batch_stride=Ct * Ho * Wo if modulated else 0, offset_strides=strides,
                mask_strides=strides if modulated else (0, 0),
                mask_act=_lib.ACT_SIGMOID if modulated else _lib.ACT_NONE, padded=padded)
    except _lib.Unsupported:
        return False
    return True


def to_channels_last(x):
    """x [N, C, H, W] as a dense channels-last tensor (same shape, NHWC memory), made by this
    library's layout kernel; x itself when it already is one."""
    if x.dim() != 4:
        raise RuntimeError(f'dcn_b200: expected a 4-D tensor, got {x.dim()}-D')
    if x.is_contiguous(memory_format=torch.channels_last) or x.numel() == 0:
        return x
    lib = _lib.load()
    dev = _require_cuda(input=x)
    out = torch.empty_like(x, memory_format=torch.channels_last)
    strides = (ctypes.c_int64 * 4)(*x.stride())
    with torch.cuda.device(dev):
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(lib.dcn_to_channels_last(
            _ptr(x), _ptr(out), _dtype_code(x), x.size(0), x.size(1), x.size(2), x.size(3),
            strides, dev.index if dev.index is not None else torch.cuda.current_device(), stream))
    return out


def pad_channels_last(x):
    """The zero-bordered channels-last copy of x [N, C, H, W] that the 16-bit tensor-core kernels
    sample (a flat uint8 tensor), made once for all operators that read the same activations;
    None when x is not a 16-bit CUDA tensor with a multiple of 8 channels."""
    if x.dim() != 4 or not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16):
        return None
    if x.size(1) % 8 != 0 or x.numel() == 0:
        return None
    lib = _lib.load()
    nbytes = ctypes.c_size_t(0)
    _lib.check(lib.dcn_padded_bytes(_dtype_code(x), x.size(0), x.size(1), x.size(2), x.size(3),
                                    ctypes.byref(nbytes)))
    dev = x.device
    with torch.cuda.device(dev):
        out = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
        strides = (ctypes.c_int64 * 4)(*x.stride())
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(lib.dcn_pad_channels_last(
            _ptr(x), _ptr(out), _dtype_code(x), x.size(0), x.size(1), x.size(2), x.size(3), strides,
            dev.index if dev.index is not None else torch.cuda.current_device(), stream))
    return out


def conv_forward(x, weight, bias, stride, padding, dilation, padded=None, act=_lib.ACT_NONE,
                 act_range=(0, 0)):
    """Ordinary convolution of x with `weight` (+ bias) on this library's kernels: the
    tensor-map convolution when the problem fits it (16-bit, channels a multiple of 64 or one
    group), else the general kernel with zero offsets.  Returns [N, Cout, Ho, Wo]."""
    lib = _lib.load()
    ho, wo = _out_hw(x, weight, stride, padding, dilation)
    out = x.new_empty((x.size(0), weight.size(0), ho, wo))
    if x.numel() == 0 or out.numel() == 0:
        return out
    dev = _require_cuda(input=x, weight=weight, bias=bias)
    x = _input_layout(x)
    weight = weight.contiguous()
    bias = None if bias is None else bias.contiguous()
    if x.dtype in (torch.bfloat16, torch.float16):
        p = _lib.DcnFwdParams()
        p.input, p.weight, p.bias, p.output = _ptr(x), _ptr(weight), _ptr(bias), _ptr(out)
        p.dtype, p.math_mode = _dtype_code(x), _lib.MATH_AUTO
        p.N, p.C, p.H, p.W = x.shape
        p.Co, p.kh, p.kw = weight.shape[0], weight.shape[2], weight.shape[3]
        p.stride_h, p.stride_w = stride
        p.pad_h, p.pad_w = padding
        p.dil_h, p.dil_w = dilation
        p.groups, p.deform_groups = 1, 1
        for i, s in enumerate(x.stride()):
            p.in_stride[i] = s
        p.act, p.act_lo, p.act_hi = act, act_range[0], act_range[1]
        p.device = dev.index if dev.index is not None else torch.cuda.current_device()
        if padded is not None:
            p.padded_input, p.padded_input_bytes = _ptr(padded), padded.numel()
        nbytes = ctypes.c_size_t(0)
        rc = lib.dcn_conv_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes))
        if rc == 0:
            with torch.cuda.device(dev):
                ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
                stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
                _lib.check(lib.dcn_conv_fwd(ctypes.byref(p), _ptr(ws), nbytes.value, stream))
                if _check_status:
                    st = ctypes.c_int32(0)
                    _lib.check(lib.dcn_read_status(_ptr(ws), stream, ctypes.byref(st)))
                    if st.value != 0:
                        raise RuntimeError(f'dcn_b200: device-side wait {st.value} timed out; the '
                                           'output is not valid')
            return out
        if rc != -2:
            _lib.check(rc)
    forward(x, None, None, weight, bias, out, stride, padding, dilation, 1, 1, act=act,
            act_range=act_range, padded=padded)
    return out


def _per_sample(t):
    """(tensor, batch stride in elements) for a tensor whose samples are each contiguous;
    a channel slice of a larger NCHW tensor qualifies and is passed without a copy."""
    if t.dim() == 4 and t.size(0) > 0:
        st, sh = t.stride(), t.shape
        if st[3] == 1 and st[2] == sh[3] and st[1] == sh[2] * sh[3] and st[0] >= sh[1] * st[1]:
            return t, st[0]
    t = t.contiguous()
    return t, 0


def _input_layout(x):
    if x.is_contiguous() or x.is_contiguous(memory_format=torch.channels_last):
        return x
    return x.contiguous()


def modulated_deform_conv_forward(input, weight, bias, ones, offset, mask, output, columns,
                                  kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w,
                                  dilation_h, dilation_w, group, deformable_group, with_bias):
    """Same contract as the reference entry of this name
    (mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:395-412): writes the result into
    ``output`` in place; ``ones`` and ``columns`` are accepted and left untouched."""
    if weight.size(2) != kernel_h or weight.size(3) != kernel_w:
        raise RuntimeError(f"Input shape and kernel shape won't match: ({kernel_h} x {kernel_w} "
                           f'vs {weight.size(2)} x {weight.size(3)}).')
    if input.size(1) != weight.size(1) * group:
        raise RuntimeError(f"Input shape and kernel channels won't match: ({input.size(1)} vs "
                           f'{weight.size(1) * group}).')
    if not output.is_contiguous():
        raise RuntimeError('dcn_b200: output must be contiguous')
    b = bias.contiguous() if (with_bias and bias is not None and bias.numel() > 0) else None
    if with_bias and b is None:
        raise RuntimeError('dcn_b200: with_bias is set but bias is empty')
    _check_shapes(input, weight, offset, mask, output, (stride_h, stride_w), (pad_h, pad_w),
                  (dilation_h, dilation_w), deformable_group)
    offset, off_bs = _per_sample(offset)
    mask, msk_bs = _per_sample(mask)
    forward(_input_layout(input), offset, mask, weight.contiguous(), b, output,
            (stride_h, stride_w), (pad_h, pad_w), (dilation_h, dilation_w), group,
            deformable_group, offset_batch_stride=off_bs, mask_batch_stride=msk_bs)


def deform_conv_forward(input, weight, offset, output, columns, ones, kW, kH, dW, dH, padW,
                        padH, dilationW, dilationH, group, deformable_group, im2col_step):
    """Same contract as the reference entry of this name
    (mmcv/ops/csrc/pytorch/deform_conv.cpp:140-260), including its contiguity and shape
    checks (:45-138, :145-166); ``im2col_step`` is validated and otherwise unused."""
    for name, t in (('input', input), ('offset', offset), ('weight', weight),
                    ('output', output)):
        if not t.is_cuda:
            raise RuntimeError(f'{name} must be a CUDA tensor (this build has no CPU '
                               'implementation)')
        if not t.is_contiguous() and not (
                name == 'input' and t.is_contiguous(memory_format=torch.channels_last)):
            raise RuntimeError(f'{name} must be contiguous')
    if weight.dim() != 4:
        raise RuntimeError('4D weight tensor (nOutputPlane,nInputPlane,kH,kW) expected, but got: '
                           f'{weight.dim()}')
    if weight.size(2) != kH or weight.size(3) != kW:
        raise RuntimeError('kernel size should be consistent with weight, but got '
                           f'kH: {kH} kW: {kW} weight.size(2): {weight.size(2)}, '
                           f'weight.size(3): {weight.size(3)}')
    if input.dim() != 4:
        raise RuntimeError(f'4D input tensor expected but got: {input.dim()}')
    n_in = weight.size(1) * group
    if input.size(1) != n_in:
        raise RuntimeError(f'invalid number of input planes, expected: {n_in}, but got: '
                           f'{input.size(1)}')
    if input.size(2) < kH or input.size(3) < kW:
        raise RuntimeError('input image is smaller than kernel')
    ho = (input.size(2) + 2 * padH - (dilationH * (kH - 1) + 1)) // dH + 1 if dH > 0 else 0
    wo = (input.size(3) + 2 * padW - (dilationW * (kW - 1) + 1)) // dW + 1 if dW > 0 else 0
    if dH > 0 and dW > 0 and ho >= 1 and wo >= 1:
        if offset.size(2) != ho or offset.size(3) != wo:
            raise RuntimeError(f'invalid spatial size of offset, expected height: {ho} width: '
                               f'{wo}, but got height: {offset.size(2)} width: {offset.size(3)}')
        if offset.size(1) != deformable_group * 2 * kH * kW:
            raise RuntimeError('invalid number of channels of offset')
    if offset.size(0) != input.size(0):
        raise RuntimeError('invalid batch size of offset')
    if im2col_step <= 0 or input.size(0) % im2col_step != 0:
        raise RuntimeError('batch size must be divisible by im2col_step')
    _check_shapes(input, weight, offset, None, output, (dH, dW), (padH, padW),
                  (dilationH, dilationW), deformable_group)
    forward(input, offset, None, weight, None, output, (dH, dW), (padH, padW),
            (dilationH, dilationW), group, deformable_group)


def conv_offset_forward(x, weight, bias, stride, padding, dilation, sigmoid_from=None, padded=None):
    """The offset(/mask) branch of the Pack layers as an ordinary convolution on this library's
    kernels, optionally with the sigmoid of the mask channels [sigmoid_from, Cout) fused into
    the epilogue.  Returns [N, Cout, Ho, Wo]."""
    act = _lib.ACT_SIGMOID if sigmoid_from is not None else _lib.ACT_NONE
    rng = (sigmoid_from, weight.size(0)) if sigmoid_from is not None else (0, 0)
    return conv_forward(x, weight, bias, stride, padding, dilation, padded=padded, act=act, act_range=rng)


# ---------------------------------------------------------------------------------------
# Backward.  Three sampling kernels of the library (columns, input scatter, coordinate
# gradients) around two plain matrix products, which go to torch.matmul (cuBLAS) exactly
# where the reference calls addmm_.  Everything is computed in fp32 and cast at the end.
# ---------------------------------------------------------------------------------------
_BWD_CHUNK_BYTES = 1 << 29   # column workspace per chunk of samples


def _params(input, offset, mask, weight, stride, padding, dilation, groups, deform_groups):
    p = _lib.DcnFwdParams()
    p.input, p.offset, p.mask = _ptr(input), _ptr(offset), _ptr(mask)
    p.weight = _ptr(weight)
    p.dtype, p.math_mode = _dtype_code(input), _lib.MATH_FFMA
    p.N, p.C, p.H, p.W = input.shape
    p.Co, p.kh, p.kw = weight.shape[0], weight.shape[2], weight.shape[3]
    p.stride_h, p.stride_w = stride
    p.pad_h, p.pad_w = padding
    p.dil_h, p.dil_w = dilation
    p.groups, p.deform_groups = groups, deform_groups
    for i, st in enumerate(input.stride()):
        p.in_stride[i] = st
    dev = input.device
    p.device = dev.index if dev.index is not None else torch.cuda.current_device()
    return p


def _backward(input, offset, mask, weight, grad_output, stride, padding, dilation, groups,
              deform_groups, want_input=True, want_weight=True):
    """Returns fp32 (grad_input, grad_offset, grad_mask, grad_weight); entries not wanted are
    None.  mask=None is the unmodulated operator."""
    lib = _lib.load()
    dev = _require_cuda(input=input, offset=offset, mask=mask, weight=weight,
                        grad_output=grad_output)
    input = _input_layout(input)
    offset = offset.contiguous()
    mask = None if mask is None else mask.contiguous()
    N, C, H, W = input.shape
    Co, Cg, kh, kw = weight.shape
    T, K = kh * kw, Cg * kh * kw
    Ho, Wo = grad_output.shape[2], grad_output.shape[3]
    P = Ho * Wo
    p = _params(input, offset, mask, weight, stride, padding, dilation, groups, deform_groups)
    w2 = weight.detach().float().reshape(groups, Co // groups, K) if want_input else None
    go_all = grad_output.detach().float().contiguous()
    g_in = torch.zeros(N, C, H, W, device=dev, dtype=torch.float32) if want_input else None
    g_off = torch.empty(offset.shape, device=dev, dtype=torch.float32) if want_input else None
    g_msk = (torch.empty(mask.shape, device=dev, dtype=torch.float32)
             if (want_input and mask is not None) else None)
    g_w = torch.zeros(groups, Co // groups, K, device=dev, dtype=torch.float32) if want_weight else None
    per_sample = C * T * P * 4
    step = max(1, min(N, _BWD_CHUNK_BYTES // max(per_sample, 1)))
    # autocast stays off in here: a backward called inside an autocast block would otherwise
    # turn the fp32 matrix products below into half tensors
    with torch.cuda.device(dev), torch.autocast('cuda', enabled=False):
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        for n0 in range(0, N, step):
            n1 = min(N, n0 + step)
            go = go_all[n0:n1].reshape(n1 - n0, groups, Co // groups, P)
            if want_input:
                # grad_columns[s, g] = W[g]^T @ grad_out[s, g]      (K x Cog) @ (Cog x P)
                gcol = torch.matmul(w2.transpose(1, 2).unsqueeze(0), go).contiguous()
                _lib.check(lib.dcn_bwd_coord(ctypes.byref(p), n0, n1, _ptr(gcol), _ptr(g_off),
                                             _ptr(g_msk), stream))
                _lib.check(lib.dcn_bwd_input(ctypes.byref(p), n0, n1, _ptr(gcol), _ptr(g_in),
                                             stream))
                del gcol
            if want_weight:
                col = torch.empty(n1 - n0, groups, K, P, device=dev, dtype=torch.float32)
                _lib.check(lib.dcn_bwd_columns(ctypes.byref(p), n0, n1, _ptr(col), stream))
                # grad_weight[g] += sum_s grad_out[s, g] @ columns[s, g]^T
                g_w += torch.matmul(go, col.transpose(2, 3)).sum(0)
                del col
    if g_w is not None:
        g_w = g_w.reshape(weight.shape)
    return g_in, g_off, g_msk, g_w


def modulated_deform_conv_backward(input, weight, bias, ones, offset, mask, columns, grad_input,
                                   grad_weight, grad_bias, grad_offset, grad_mask, grad_output,
                                   kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w,
                                   dilation_h, dilation_w, group, deformable_group, with_bias):
    """Same contract as the reference entry of this name
    (mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp:140-251): fills the five gradient
    tensors in place (weight and bias gradients are accumulated, as in the reference)."""
    if weight.size(2) != kernel_h or weight.size(3) != kernel_w:
        raise RuntimeError(f"Input shape and kernel shape won't match: ({kernel_h} x {kernel_w} "
                           f'vs {weight.size(2)} x {weight.size(3)}).')
    if input.size(1) != weight.size(1) * group:
        raise RuntimeError(f"Input shape and kernel channels won't match: ({input.size(1)} vs "
                           f'{weight.size(1) * group}).')
    gi, go_, gm, gw = _backward(input, offset, mask, weight, grad_output, (stride_h, stride_w),
                                (pad_h, pad_w), (dilation_h, dilation_w), group, deformable_group)
    grad_input.copy_(gi)
    grad_offset.copy_(go_)
    grad_mask.copy_(gm)
    grad_weight.add_(gw.to(grad_weight.dtype))
    if with_bias:
        grad_bias.add_(grad_output.detach().float().sum((0, 2, 3)).to(grad_bias.dtype))


def deform_conv_backward_input(input, offset, gradOutput, gradInput, gradOffset, weight, columns,
                               kW, kH, dW, dH, padW, padH, dilationW, dilationH, group,
                               deformable_group, im2col_step):
    """Same contract as the reference entry of this name
    (mmcv/ops/csrc/pytorch/deform_conv.cpp:262-393)."""
    for name, t in (('input', input), ('offset', offset), ('gradOutput', gradOutput),
                    ('gradInput', gradInput), ('gradOffset', gradOffset), ('weight', weight)):
        if not t.is_contiguous():
            raise RuntimeError(f'{name} must be contiguous')
    if im2col_step <= 0 or input.size(0) % im2col_step != 0:
        raise RuntimeError('batch size must be divisible by im2col_step')
    gi, go_, _, _ = _backward(input, offset, None, weight, gradOutput, (dH, dW), (padH, padW),
                              (dilationH, dilationW), group, deformable_group, want_weight=False)
    gradInput.copy_(gi)
    gradOffset.copy_(go_)


def deform_conv_backward_parameters(input, offset, gradOutput, gradWeight, columns, ones, kW, kH,
                                    dW, dH, padW, padH, dilationW, dilationH, group,
                                    deformable_group, scale, im2col_step):
    """Same contract as the reference entry of this name
    (mmcv/ops/csrc/pytorch/deform_conv.cpp:395-525): gradWeight += scale * gradient."""
    for name, t in (('input', input), ('offset', offset), ('gradOutput', gradOutput),
                    ('gradWeight', gradWeight)):
        if not t.is_contiguous():
            raise RuntimeError(f'{name} must be contiguous')
    if im2col_step <= 0 or input.size(0) % im2col_step != 0:
        raise RuntimeError('batch size must be divisible by im2col_step')
    # (this entry receives no weight tensor; only its shape is needed, and gradWeight has it)
    _, _, _, gw = _backward(input, offset, None, gradWeight, gradOutput, (dH, dW),
                            (padH, padW), (dilationH, dilationW), group, deformable_group,
                            want_input=False)
    gradWeight.add_((gw * scale).to(gradWeight.dtype))



# ---------------------------------------------------------------------------------------------
# Multi-scale deformable attention (the sibling sampler; reference entry points
# mmcv/ops/csrc/pytorch/ms_deform_attn.cpp:38-60, CUDA bodies
# mmcv/ops/csrc/pytorch/cuda/ms_deform_attn_cuda.cu:203-351)

def _msda_check(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                attention_weights, im2col_step, extra=()):
    names = ['value', 'spatial_shapes', 'level_start_index', 'sampling_loc', 'attn_weight']
    tensors = [value, value_spatial_shapes, value_level_start_index, sampling_locations,
               attention_weights]
    for name, t in list(zip(names, tensors)) + list(extra):
        if not t.is_contiguous():
            raise RuntimeError(f'{name} tensor has to be contiguous')
        if not t.is_cuda:
            raise RuntimeError(f'{name} must be a CUDA tensor')
    if value.dim() != 4 or sampling_locations.dim() != 6 or attention_weights.dim() != 5:
        raise RuntimeError('ms_deform_attn: value must be 4-D, sampling_loc 6-D, attn_weight 5-D')
    if value_spatial_shapes.dtype != torch.int64 or value_level_start_index.dtype != torch.int64:
        raise RuntimeError('ms_deform_attn: spatial_shapes and level_start_index must be int64')
    for name, t in (('sampling_loc', sampling_locations), ('attn_weight', attention_weights)):
        if t.dtype != value.dtype:
            raise RuntimeError(f'ms_deform_attn: {name} has dtype {t.dtype}, value has {value.dtype}')
    batch = value.size(0)
    step = min(batch, int(im2col_step))
    if batch > 0 and (step <= 0 or batch % step != 0):
        raise RuntimeError(f'batch({batch}) must divide im2col_step({step})')
    B, S, M, D = value.shape
    L = value_spatial_shapes.size(0)
    Q, P = sampling_locations.size(1), sampling_locations.size(4)
    if tuple(sampling_locations.shape) != (B, Q, M, L, P, 2) or \
            tuple(attention_weights.shape) != (B, Q, M, L, P) or \
            tuple(value_spatial_shapes.shape) != (L, 2) or value_level_start_index.numel() != L:
        raise RuntimeError('ms_deform_attn: argument shapes do not match each other')
    return B, S, M, D, L, Q, P


def ms_deform_attn_forward(value, value_spatial_shapes, value_level_start_index,
                           sampling_locations, attention_weights, im2col_step):
    """Same contract as the reference entry of this name: returns the attention output
    [batch, num_query, num_heads * channels] in value's dtype; ``im2col_step`` is validated
    (the batch must be a multiple of min(batch, im2col_step)) and otherwise unused."""
    lib = _lib.load()
    B, S, M, D, L, Q, P = _msda_check(value, value_spatial_shapes, value_level_start_index,
                                      sampling_locations, attention_weights, im2col_step)
    code = _dtype_code(value)
    dev = value.device
    with torch.cuda.device(dev):
        out = value.new_empty((B, Q, M * D))
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(lib.dcn_msda_forward(_ptr(value), _ptr(value_spatial_shapes),
                                        _ptr(value_level_start_index), _ptr(sampling_locations),
                                        _ptr(attention_weights), _ptr(out), code, B, S, M, D, L, Q, P,
                                        dev.index if dev.index is not None else torch.cuda.current_device(),
                                        stream))
    return out


def ms_deform_attn_backward(value, value_spatial_shapes, value_level_start_index,
                            sampling_locations, attention_weights, grad_output, grad_value,
                            grad_sampling_loc, grad_attn_weight, im2col_step):
    """Same contract as the reference entry of this name: adds to ``grad_value`` and writes
    ``grad_sampling_loc`` / ``grad_attn_weight`` in place (the caller passes them zeroed)."""
    lib = _lib.load()
    B, S, M, D, L, Q, P = _msda_check(value, value_spatial_shapes, value_level_start_index,
                                      sampling_locations, attention_weights, im2col_step,
                                      extra=[('grad_output', grad_output)])
    code = _dtype_code(value)
    dev = value.device
    if grad_output.dtype != value.dtype:
        raise RuntimeError('ms_deform_attn: grad_output must have value\'s dtype')
    with torch.cuda.device(dev):
        f32 = value.dtype == torch.float32
        direct = f32 and all(t.is_contiguous() and t.dtype == torch.float32
                             for t in (grad_value, grad_sampling_loc, grad_attn_weight))
        if direct:
            gv, gl, ga = grad_value, grad_sampling_loc, grad_attn_weight
            gl.zero_()
            ga.zero_()
        else:
            # the kernels produce fp32 gradients; 16-bit tensors get them rounded once
            gv = torch.zeros(value.shape, dtype=torch.float32, device=dev)
            gl = torch.zeros(sampling_locations.shape, dtype=torch.float32, device=dev)
            ga = torch.zeros(attention_weights.shape, dtype=torch.float32, device=dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(lib.dcn_msda_backward(_ptr(value), _ptr(value_spatial_shapes),
                                         _ptr(value_level_start_index), _ptr(sampling_locations),
                                         _ptr(attention_weights), _ptr(grad_output), _ptr(gv), _ptr(gl),
                                         _ptr(ga), code, B, S, M, D, L, Q, P,
                                         dev.index if dev.index is not None else torch.cuda.current_device(),
                                         stream))
        if not direct:
            grad_value.add_(gv.to(grad_value.dtype))
            grad_sampling_loc.copy_(gl)
            grad_attn_weight.copy_(ga)
