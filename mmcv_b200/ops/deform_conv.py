"""Deformable convolution v1 with the interface of ``mmcv.ops.deform_conv``
(reference: mmcv/ops/deform_conv.py).  Same names, argument order, defaults and
error types; the computation is the mask-free case of the sm_100a kernel."""
from typing import Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor
from torch.autograd import Function
from torch.autograd.function import once_differentiable
from torch.nn.modules.utils import _pair, _single

from .. import _ext as ext_module
from . import modulated_deform_conv as mdc
from .modulated_deform_conv import (_rename_kw, _upgrade_offset_keys, branch_dtype,
                                    conv_output_size, fused_branch_applies, register_layer,
                                    shared_layout)


class DeformConv2dFunction(Function):

    @staticmethod
    def symbolic(g, input, offset, weight, stride, padding, dilation, groups, deform_groups,
                 bias=False, im2col_step=32):
        """ONNX export node, same name and attributes as the reference emits
        (mmcv/ops/deform_conv.py:28-50)."""
        return g.op('mmcv::MMCVDeformConv2d', input, offset, weight, stride_i=stride,
                    padding_i=padding, dilation_i=dilation, groups_i=groups,
                    deform_groups_i=deform_groups, bias_i=bias, im2col_step_i=im2col_step)

    @staticmethod
    def forward(ctx, input, offset, weight, stride=1, padding=0, dilation=1, groups=1,
                deform_groups=1, bias=False, im2col_step=32):
        if input is not None and input.dim() != 4:
            raise ValueError(f'Expected 4D tensor as input, got {input.dim()}D tensor instead.')
        assert bias is False, 'Only support bias is False.'
        ctx.stride, ctx.padding, ctx.dilation = _pair(stride), _pair(padding), _pair(dilation)
        ctx.groups, ctx.deform_groups, ctx.im2col_step = groups, deform_groups, im2col_step
        input = input.type_as(offset)   # offset's dtype decides (autocast)
        weight = ext_module.cast_weight(weight, input.dtype)
        ctx.save_for_backward(input, offset, weight)
        output = input.new_empty(conv_output_size(input, weight, ctx.stride, ctx.padding,
                                                  ctx.dilation))
        ctx.bufs_ = [input.new_empty(0), input.new_empty(0)]
        cur_im2col_step = min(ctx.im2col_step, input.size(0))
        assert (input.size(0) % cur_im2col_step) == 0, \
            'batch size must be divisible by im2col_step'
        ext_module.deform_conv_forward(
            input, weight, offset, output, ctx.bufs_[0], ctx.bufs_[1],
            kW=weight.size(3), kH=weight.size(2), dW=ctx.stride[1], dH=ctx.stride[0],
            padW=ctx.padding[1], padH=ctx.padding[0], dilationW=ctx.dilation[1],
            dilationH=ctx.dilation[0], group=ctx.groups, deformable_group=ctx.deform_groups,
            im2col_step=cur_im2col_step)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        input, offset, weight = ctx.saved_tensors
        grad_input = grad_offset = grad_weight = None
        step = min(ctx.im2col_step, input.size(0))
        assert (input.size(0) % step) == 0, 'batch size must be divisible by im2col_step'
        common = dict(kW=weight.size(3), kH=weight.size(2), dW=ctx.stride[1], dH=ctx.stride[0],
                      padW=ctx.padding[1], padH=ctx.padding[0], dilationW=ctx.dilation[1],
                      dilationH=ctx.dilation[0], group=ctx.groups,
                      deformable_group=ctx.deform_groups)
        grad_output = grad_output.contiguous()
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            grad_input = torch.zeros_like(input)
            grad_offset = torch.zeros_like(offset)
            ext_module.deform_conv_backward_input(input, offset, grad_output, grad_input,
                                                  grad_offset, weight, ctx.bufs_[0],
                                                  im2col_step=step, **common)
        if ctx.needs_input_grad[2]:
            grad_weight = torch.zeros_like(weight)
            ext_module.deform_conv_backward_parameters(input, offset, grad_output, grad_weight,
                                                       ctx.bufs_[0], ctx.bufs_[1], scale=1,
                                                       im2col_step=step, **common)
        return grad_input, grad_offset, grad_weight, None, None, None, None, None, None, None


deform_conv2d = DeformConv2dFunction.apply


class DeformConv2d(nn.Module):
    """DCNv1 layer taking (x, offset); offsets are (y, x) pairs per tap in row-major tap
    order, shape (B, deform_groups*kh*kw*2, Ho, Wo).  Reference lines 229-364."""

    def __init__(self, in_channels: int, out_channels: int,
                 kernel_size: Union[int, Tuple[int, ...]],
                 stride: Union[int, Tuple[int, ...]] = 1,
                 padding: Union[int, Tuple[int, ...]] = 0,
                 dilation: Union[int, Tuple[int, ...]] = 1, groups: int = 1,
                 deform_groups: int = 1, bias: bool = False, im2col_step: int = 32,
                 **kwargs) -> None:
        _rename_kw(kwargs, 'deformable_groups', 'deform_groups')  # deprecated spelling
        deform_groups = kwargs.pop('deform_groups', deform_groups)
        if kwargs:
            raise TypeError(f'unexpected arguments {sorted(kwargs)}')
        super().__init__()
        assert not bias, f'bias={bias} is not supported in DeformConv2d.'
        assert in_channels % groups == 0, \
            f'in_channels {in_channels} cannot be divisible by groups {groups}'
        assert out_channels % groups == 0, \
            f'out_channels {out_channels} cannot be divisible by groups {groups}'
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size = _pair(kernel_size)
        self.stride, self.padding, self.dilation = _pair(stride), _pair(padding), _pair(dilation)
        self.groups, self.deform_groups, self.im2col_step = groups, deform_groups, im2col_step
        self.transposed = False            # nn.Conv2d compatibility
        self.output_padding = _single(0)
        self.weight = nn.Parameter(torch.Tensor(out_channels, in_channels // groups,
                                                *self.kernel_size))
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, nonlinearity='relu')

    def forward(self, x: Tensor, offset: Tensor) -> Tensor:
        # An input smaller than the kernel is zero-padded up to the kernel size and the
        # extra output rows/columns are cut off again (reference lines 336-349).
        grow_h = max(self.kernel_size[0] - x.size(2), 0)
        grow_w = max(self.kernel_size[1] - x.size(3), 0)
        if grow_h or grow_w:
            x = F.pad(x, (0, grow_w, 0, grow_h), 'constant', 0).contiguous()
            offset = F.pad(offset, (0, grow_w, 0, grow_h), 'constant', 0).contiguous()
        out = deform_conv2d(x, offset, self.weight, self.stride, self.padding, self.dilation,
                            self.groups, self.deform_groups, False, self.im2col_step)
        if grow_h or grow_w:
            out = out[:, :, :out.size(2) - grow_h, :out.size(3) - grow_w].contiguous()
        return out

    def __repr__(self):
        fields = [f'in_channels={self.in_channels}', f'out_channels={self.out_channels}',
                  f'kernel_size={self.kernel_size}', f'stride={self.stride}',
                  f'padding={self.padding}', f'dilation={self.dilation}',
                  f'groups={self.groups}', f'deform_groups={self.deform_groups}',
                  'bias=False)']
        return self.__class__.__name__ + '(' + ',\n'.join(fields)


class DeformConv2dPack(DeformConv2d):
    """DCNv1 layer that predicts its own offsets (registry name 'DCN'; reference
    lines 367-442)."""

    _version = 2

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        taps = self.kernel_size[0] * self.kernel_size[1]
        self.conv_offset = nn.Conv2d(self.in_channels, self.deform_groups * 2 * taps,
                                     kernel_size=self.kernel_size, stride=_pair(self.stride),
                                     padding=_pair(self.padding), dilation=_pair(self.dilation),
                                     bias=True)
        self.init_offset()

    def init_offset(self):
        self.conv_offset.weight.data.zero_()
        self.conv_offset.bias.data.zero_()

    def forward(self, x: Tensor) -> Tensor:  # type: ignore[override]
        if fused_branch_applies(x, self.conv_offset):
            dtype = branch_dtype(x)
            x = x.to(dtype)
            padded = None
            if mdc.OFFSET_BRANCH == 'kernel':
                # one zero-bordered channels-last copy feeds the branch and the deformable kernel
                padded = ext_module.pad_channels_last(x)
                offset = ext_module.conv_offset_forward(
                    x, ext_module.cast_weight(self.conv_offset.weight, dtype),
                    ext_module.cast_weight(self.conv_offset.bias, dtype),
                    _pair(self.stride), _pair(self.padding), _pair(self.dilation), padded=padded)
            else:
                x = shared_layout(x)
                offset = mdc.branch_conv(x, self.conv_offset, dtype)
            if x.size(0) > 0 and x.size(0) % min(self.im2col_step, x.size(0)) == 0:
                y = mdc.deform_from_branch(x, offset, offset.size(1), self.weight, None,
                                           self.stride, self.padding, self.dilation,
                                           self.groups, self.deform_groups, padded=padded)
                if y is not None:
                    return y
            offset = offset.contiguous()
        else:
            offset = self.conv_offset(x)
        return deform_conv2d(x, offset, self.weight, self.stride, self.padding, self.dilation,
                             self.groups, self.deform_groups, False, self.im2col_step)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        _upgrade_offset_keys(state_dict, prefix, local_metadata)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)


register_layer('DCN', DeformConv2dPack)
