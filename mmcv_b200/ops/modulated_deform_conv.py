"""Modulated deformable convolution (DCNv2) with the interface of
``mmcv.ops.modulated_deform_conv`` (reference: mmcv/ops/modulated_deform_conv.py).

Names, argument order, defaults, dtype rule (everything follows ``offset``'s
dtype, reference lines 136-139), error types and state-dict layout are the
reference's; the computation goes to the sm_100a library through ``_ext``.
"""
import math
import os
from typing import Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.autograd import Function
from torch.autograd.function import once_differentiable
from torch.nn.modules.utils import _pair, _single

from .. import _ext as ext_module


def conv_output_size(input, weight, stride, padding, dilation):
    """[N, Co, Ho, Wo]; ValueError when a spatial size is not positive
    (reference: modulated_deform_conv.py:216-230)."""
    size = [input.size(0), weight.size(0)]
    for d in range(input.dim() - 2):
        span = dilation[d] * (weight.size(d + 2) - 1) + 1
        size.append((input.size(d + 2) + 2 * padding[d] - span) // stride[d] + 1)
    if any(s <= 0 for s in size):
        raise ValueError('convolution input is too small (output would be ' +
                         'x'.join(str(s) for s in size) + ')')
    return size


class ModulatedDeformConv2dFunction(Function):

    @staticmethod
    def symbolic(g, input, offset, mask, weight, bias, stride, padding, dilation, groups,
                 deform_groups):
        """ONNX export node, same name and attributes as the reference emits
        (mmcv/ops/modulated_deform_conv.py:25-37)."""
        tensors = [input, offset, mask, weight] + ([bias] if bias is not None else [])
        return g.op('mmcv::MMCVModulatedDeformConv2d', *tensors, stride_i=stride,
                    padding_i=padding, dilation_i=dilation, groups_i=groups,
                    deform_groups_i=deform_groups)

    @staticmethod
    def forward(ctx, input, offset, mask, weight, bias=None, stride=1, padding=0,
                dilation=1, groups=1, deform_groups=1):
        if input is not None and input.dim() != 4:
            raise ValueError(f'Expected 4D tensor as input, got {input.dim()}D tensor instead.')
        ctx.stride, ctx.padding, ctx.dilation = _pair(stride), _pair(padding), _pair(dilation)
        ctx.groups, ctx.deform_groups = groups, deform_groups
        ctx.with_bias = bias is not None
        if bias is None:
            bias = input.new_empty(0)
        # offset's dtype decides (this is how autocast reaches the op)
        input = input.type_as(offset)
        weight = ext_module.cast_weight(weight, input.dtype)
        bias, mask = ext_module.cast_weight(bias, input.dtype), mask.type_as(input)
        ctx.save_for_backward(input, offset, mask, weight, bias)
        output = input.new_empty(conv_output_size(input, weight, ctx.stride, ctx.padding,
                                                  ctx.dilation))
        ctx._bufs = [input.new_empty(0), input.new_empty(0)]
        ext_module.modulated_deform_conv_forward(
            input, weight, bias, ctx._bufs[0], offset, mask, output, ctx._bufs[1],
            kernel_h=weight.size(2), kernel_w=weight.size(3),
            stride_h=ctx.stride[0], stride_w=ctx.stride[1],
            pad_h=ctx.padding[0], pad_w=ctx.padding[1],
            dilation_h=ctx.dilation[0], dilation_w=ctx.dilation[1],
            group=groups, deformable_group=deform_groups, with_bias=ctx.with_bias)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        input, offset, mask, weight, bias = ctx.saved_tensors
        grads = [torch.zeros_like(t) for t in (input, offset, mask, weight, bias)]
        ext_module.modulated_deform_conv_backward(
            input, weight, bias, ctx._bufs[0], offset, mask, ctx._bufs[1], grads[0], grads[3],
            grads[4], grads[1], grads[2], grad_output.contiguous(),
            kernel_h=weight.size(2), kernel_w=weight.size(3),
            stride_h=ctx.stride[0], stride_w=ctx.stride[1],
            pad_h=ctx.padding[0], pad_w=ctx.padding[1],
            dilation_h=ctx.dilation[0], dilation_w=ctx.dilation[1],
            group=ctx.groups, deformable_group=ctx.deform_groups, with_bias=ctx.with_bias)
        return (grads[0], grads[1], grads[2], grads[3], grads[4] if ctx.with_bias else None,
                None, None, None, None, None)


modulated_deform_conv2d = ModulatedDeformConv2dFunction.apply


# How an inference-time Pack layer computes its offset branch: 'kernel' (default) = this
# library's tensor-map convolution, reading the same zero-bordered channels-last copy of the
# input as the deformable kernel (the copy is made once per layer); 'library' = the branch's own
# nn.Conv2d arithmetic (cuDNN) on a channels-last copy of the input.
OFFSET_BRANCH = os.environ.get('DCN_B200_OFFSET_BRANCH', 'kernel')


def branch_conv(x, conv, dtype):
    """conv(x) for an inference-time offset branch (library convolution, no autograd graph);
    x is already in the layout shared with the deformable kernel."""
    return F.conv2d(x, ext_module.cast_weight(conv.weight, dtype),
                    ext_module.cast_weight(conv.bias, dtype), conv.stride, conv.padding,
                    conv.dilation, conv.groups)


def split_branch(out, sigmoid_from=None):
    """NCHW-contiguous (offset, mask) tensors from a branch output; mask is None when
    sigmoid_from is None (the v1 layer)."""
    if sigmoid_from is None:
        return out.contiguous(), None
    offset = out[:, :sigmoid_from].contiguous()
    mask = torch.empty((out.size(0), out.size(1) - sigmoid_from) + tuple(out.shape[2:]),
                       dtype=out.dtype, device=out.device)
    torch.sigmoid(out[:, sigmoid_from:], out=mask)
    return offset, mask


def library_offset_branch(x, conv, dtype, sigmoid_from=None):
    """branch_conv + split_branch."""
    return split_branch(branch_conv(x, conv, dtype), sigmoid_from)


def deform_from_branch(x, out, n_offset, weight, bias, stride, padding, dilation, groups,
                       deform_groups, padded=None):
    """The deformable convolution fed by the raw branch output `out` (offsets, then mask
    logits), which the tensor-core kernel reads where it lies, sigmoid included: no split,
    copy or sigmoid pass.  Returns None when the problem runs on another kernel."""
    weight = ext_module.cast_weight(weight, x.dtype)
    bias = ext_module.cast_weight(bias, x.dtype)
    y = x.new_empty(conv_output_size(x, weight, _pair(stride), _pair(padding), _pair(dilation)))
    done = ext_module.forward_from_branch(x, out, n_offset, weight, bias, y, _pair(stride),
                                          _pair(padding), _pair(dilation), groups, deform_groups,
                                          padded=padded)
    return y if done else None


def fused_branch_applies(x, conv):
    """The inference path of a Pack layer (shared channels-last input, no autograd graph)
    applies when nothing needs the branch's gradient; otherwise the branch stays a plain
    nn.Conv2d call so that autograd sees it."""
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        return False
    if torch.is_autocast_enabled('cuda') and torch.get_autocast_dtype('cuda') not in (
            torch.bfloat16, torch.float16):
        return False
    needs_grad = torch.is_grad_enabled() and (
        x.requires_grad or any(p.requires_grad for p in conv.parameters()))
    return not needs_grad


def shared_layout(x):
    """bf16 inputs are put in channels-last order once, so that the offset branch and the
    deformable convolution both read them without a restaging pass of their own."""
    if x.dtype in (torch.bfloat16, torch.float16) and x.size(1) % 8 == 0:
        return ext_module.to_channels_last(x)
    return x


def branch_dtype(x):
    return torch.get_autocast_dtype('cuda') if torch.is_autocast_enabled('cuda') else x.dtype


def _rename_kw(kwargs, old, new):
    if old in kwargs:
        kwargs[new] = kwargs.pop(old)


class ModulatedDeformConv2d(nn.Module):
    """DCNv2 layer taking (x, offset, mask); reference lines 236-286."""

    def __init__(self, in_channels: int, out_channels: int,
                 kernel_size: Union[int, Tuple[int]], stride: int = 1, padding: int = 0,
                 dilation: int = 1, groups: int = 1, deform_groups: int = 1,
                 bias: Union[bool, str] = True, **kwargs):
        _rename_kw(kwargs, 'deformable_groups', 'deform_groups')  # deprecated spelling
        deform_groups = kwargs.pop('deform_groups', deform_groups)
        if kwargs:
            raise TypeError(f'unexpected arguments {sorted(kwargs)}')
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size = _pair(kernel_size)
        self.stride, self.padding, self.dilation = _pair(stride), _pair(padding), _pair(dilation)
        self.groups, self.deform_groups = groups, deform_groups
        self.transposed = False            # nn.Conv2d compatibility
        self.output_padding = _single(0)
        self.weight = nn.Parameter(torch.Tensor(out_channels, in_channels // groups,
                                                *self.kernel_size))
        if bias:
            self.bias = nn.Parameter(torch.Tensor(out_channels))
        else:
            self.register_parameter('bias', None)
        self.init_weights()

    def init_weights(self):
        fan = self.in_channels * self.kernel_size[0] * self.kernel_size[1]
        bound = 1.0 / math.sqrt(fan)
        self.weight.data.uniform_(-bound, bound)
        if self.bias is not None:
            self.bias.data.zero_()

    def forward(self, x: torch.Tensor, offset: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        return modulated_deform_conv2d(x, offset, mask, self.weight, self.bias, self.stride,
                                       self.padding, self.dilation, self.groups,
                                       self.deform_groups)


def _upgrade_offset_keys(state_dict, prefix, local_metadata):
    """Checkpoints older than version 2 stored the offset branch as ``<name>_offset``."""
    version = local_metadata.get('version', None)
    if version is None or version < 2:
        for leaf in ('weight', 'bias'):
            new, old = f'{prefix}conv_offset.{leaf}', f'{prefix[:-1]}_offset.{leaf}'
            if new not in state_dict and old in state_dict:
                state_dict[new] = state_dict.pop(old)


def register_layer(name, cls):
    """Registers the layer under the reference's registry name ('DCN', 'DCNv2') when the
    registry package (mmengine) is installed, so that config-driven construction
    (mmcv/cnn/bricks/conv.py:14-51) finds it; a no-op otherwise."""
    try:
        from mmengine.registry import MODELS
    except Exception:   # mmengine is optional here
        return cls
    MODELS.register_module(name, force=True, module=cls)
    return cls


class ModulatedDeformConv2dPack(ModulatedDeformConv2d):
    """DCNv2 layer that predicts its own offsets and mask with a plain convolution
    (registry name 'DCNv2'; reference lines 289-363)."""

    _version = 2

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        taps = self.kernel_size[0] * self.kernel_size[1]
        self.conv_offset = nn.Conv2d(self.in_channels, self.deform_groups * 3 * taps,
                                     kernel_size=self.kernel_size, stride=self.stride,
                                     padding=self.padding, dilation=self.dilation, bias=True)
        self.init_weights()

    def init_weights(self) -> None:
        super().init_weights()
        if hasattr(self, 'conv_offset'):
            self.conv_offset.weight.data.zero_()
            self.conv_offset.bias.data.zero_()

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        two_thirds = self.conv_offset.out_channels // 3 * 2
        # chunk(3) + cat of the first two chunks == the first two thirds of the channels
        if fused_branch_applies(x, self.conv_offset):
            # the branch and the deformable kernel read one channels-last copy of the input
            dtype = branch_dtype(x)
            x = x.to(dtype)
            padded = None
            if OFFSET_BRANCH == 'kernel':
                # one zero-bordered channels-last copy feeds the branch and the deformable kernel
                padded = ext_module.pad_channels_last(x)
                out = ext_module.conv_offset_forward(
                    x, ext_module.cast_weight(self.conv_offset.weight, dtype),
                    ext_module.cast_weight(self.conv_offset.bias, dtype),
                    self.stride, self.padding, self.dilation, padded=padded)
            else:
                x = shared_layout(x)
                out = branch_conv(x, self.conv_offset, dtype)
            # the deformable kernel reads offsets and mask logits where the branch left them
            y = deform_from_branch(x, out, two_thirds, self.weight, self.bias, self.stride,
                                   self.padding, self.dilation, self.groups,
                                   self.deform_groups, padded=padded)
            if y is not None:
                return y
            offset, mask = split_branch(out, two_thirds)
        else:
            out = self.conv_offset(x)
            offset = out[:, :two_thirds].contiguous()
            mask = torch.sigmoid(out[:, two_thirds:])
        return modulated_deform_conv2d(x, offset, mask, self.weight, self.bias, self.stride,
                                       self.padding, self.dilation, self.groups,
                                       self.deform_groups)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        _upgrade_offset_keys(state_dict, prefix, local_metadata)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)


register_layer('DCNv2', ModulatedDeformConv2dPack)
