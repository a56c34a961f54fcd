"""Switchable atrous convolution with the interface of ``mmcv.ops.saconv.SAConv2d``: the one
other in-tree caller of ``deform_conv2d`` (reference: mmcv/ops/saconv.py:14-148).

The layer is a weight-standardised convolution (reference base class:
mmcv/cnn/bricks/conv_ws.py:57-150) evaluated twice, with the given dilation and with three
times the dilation and padding, and blended by a learned per-pixel switch; with
``use_deform=True`` both evaluations are deformable convolutions whose offsets come from two
small 3x3 branches.  Parameter and buffer names are the reference's, so its checkpoints load.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .deform_conv import deform_conv2d
from .modulated_deform_conv import register_layer


def _fill(conv, weight, bias=0.0):
    nn.init.constant_(conv.weight, weight)
    if conv.bias is not None:
        nn.init.constant_(conv.bias, bias)


def _row_stats(weight):
    """Per-output-channel mean and sqrt(var + 1e-5) of a weight, shaped for broadcasting."""
    flat = weight.reshape(weight.size(0), -1)
    mean = flat.mean(dim=1).view(-1, 1, 1, 1)
    std = torch.sqrt(flat.var(dim=1) + 1e-5).view(-1, 1, 1, 1)
    return mean, std


class SAConv2d(nn.Conv2d):
    """SAC layer (registry name 'SAC').  Arguments as nn.Conv2d (zero padding only), plus
    ``use_deform``: evaluate both branches as deformable convolutions."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1,
                 groups=1, bias=True, use_deform=False):
        super().__init__(in_channels, out_channels, kernel_size, stride=stride, padding=padding,
                         dilation=dilation, groups=groups, bias=bias)
        # adaptive weight standardisation: w -> gamma * (w - mean) / std + beta
        self.register_buffer('weight_gamma', torch.ones(self.out_channels, 1, 1, 1))
        self.register_buffer('weight_beta', torch.zeros(self.out_channels, 1, 1, 1))
        self.use_deform = use_deform
        self.switch = nn.Conv2d(self.in_channels, 1, kernel_size=1, stride=stride, bias=True)
        self.weight_diff = nn.Parameter(torch.Tensor(self.weight.size()))
        self.pre_context = nn.Conv2d(self.in_channels, self.in_channels, kernel_size=1, bias=True)
        self.post_context = nn.Conv2d(self.out_channels, self.out_channels, kernel_size=1, bias=True)
        if self.use_deform:
            self.offset_s = nn.Conv2d(self.in_channels, 18, kernel_size=3, padding=1, stride=stride,
                                      bias=True)
            self.offset_l = nn.Conv2d(self.in_channels, 18, kernel_size=3, padding=1, stride=stride,
                                      bias=True)
        self.init_weights()

    def init_weights(self):
        _fill(self.switch, 0, bias=1)
        self.weight_diff.data.zero_()
        _fill(self.pre_context, 0)
        _fill(self.post_context, 0)
        if self.use_deform:
            _fill(self.offset_s, 0)
            _fill(self.offset_l, 0)

    def _get_weight(self, weight):
        mean, std = _row_stats(weight)
        return self.weight_gamma * ((weight - mean) / std) + self.weight_beta

    def _branch(self, x, avg_x, weight, offset_conv, padding, dilation):
        if self.use_deform:
            return deform_conv2d(x, offset_conv(avg_x), weight, self.stride, padding, dilation,
                                 self.groups, 1)
        return F.conv2d(x, weight, None, self.stride, padding, dilation, self.groups)

    def forward(self, x):
        # pre-context: global average -> 1x1 conv -> added everywhere
        x = x + self.pre_context(F.adaptive_avg_pool2d(x, output_size=1)).expand_as(x)
        # switch: 5x5 average over a reflect-padded copy, then a 1x1 conv
        avg_x = F.avg_pool2d(F.pad(x, pad=(2, 2, 2, 2), mode='reflect'), kernel_size=5, stride=1,
                             padding=0)
        switch = self.switch(avg_x)
        weight = self._get_weight(self.weight)
        out_s = self._branch(x, avg_x, weight, getattr(self, 'offset_s', None), self.padding,
                             self.dilation)
        out_l = self._branch(x, avg_x, weight + self.weight_diff, getattr(self, 'offset_l', None),
                             tuple(3 * p for p in self.padding),
                             tuple(3 * d for d in self.dilation))
        out = switch * out_s + (1 - switch) * out_l
        # post-context
        return out + self.post_context(F.adaptive_avg_pool2d(out, output_size=1)).expand_as(out)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        """A checkpoint without weight_gamma / weight_beta (plain pretrained weights) gets them
        from the statistics of the loaded weight, so that the standardised weight equals the
        pretrained one (reference: conv_ws.py:116-150)."""
        self.weight_gamma.data.fill_(-1)
        local_missing = []
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, local_missing,
                                      unexpected_keys, error_msgs)
        if self.weight_gamma.data.mean() > 0:
            missing_keys.extend(local_missing)
            return
        mean, std = _row_stats(self.weight.data)
        self.weight_beta.data.copy_(mean)
        self.weight_gamma.data.copy_(std)
        missing_keys.extend(k for k in local_missing
                            if not k.endswith(('weight_gamma', 'weight_beta')))


register_layer('SAC', SAConv2d)
