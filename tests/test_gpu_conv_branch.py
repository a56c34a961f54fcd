"""The offset / mask branch of the Pack layers on this library's tensor-map convolution, and the
Pack layers at the shapes of the ResNet-50-DCNv2 stack (stages 3-5).

The branch is checked against a plain fp32 convolution on the same (16-bit rounded) inputs and
weights; the layer is checked against the CPU checker fed the branch's own offsets and mask
(rounded to the tensors' 16-bit type, as the deformable kernel reads them), which isolates the
deformable kernel from the branch's rounding.  Bound for 16-bit tensors: relative L2 <= 2e-2.
"""
import pytest
import torch
import torch.nn.functional as F

import oracle
from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _rand(shape, gen, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(shape, generator=gen) * scale).to(dtype)


@pytest.mark.parametrize('C,Co,H,W,k,s,p,d', [
    (128, 27, 40, 36, 3, 1, 1, 1),     # the modulated Pack branch
    (64, 18, 33, 21, 3, 1, 1, 1),      # the v1 Pack branch, odd sizes (tiles overhang the image)
    (256, 27, 20, 28, 3, 2, 1, 1),     # strided
    (64, 27, 24, 24, 3, 1, 2, 2),      # dilated
    (64, 64, 17, 19, 1, 1, 0, 1),      # 1x1, no padding
    (192, 32, 16, 16, 5, 1, 2, 1),     # 5x5
    (40, 27, 12, 12, 3, 1, 1, 1),      # channels not a multiple of 64: last chunk zero-filled
    (64, 300, 9, 11, 3, 1, 1, 1),      # more output channels than one tile holds
    (64, 1, 8, 8, 3, 1, 1, 1),         # a single output channel
    (128, 27, 3, 3, 3, 1, 1, 1),       # an image smaller than a tile
    (64, 27, 31, 5, 3, 3, 1, 1),       # stride 3, narrow image
    (64, 54, 16, 16, 3, 1, 0, 1),      # no padding
    (64, 27, 10, 10, 3, 1, 3, 1),      # padding beyond the copy's one-pixel border
    (64, 27, 10, 10, 3, 2, 4, 3),      # stride, dilation and wide padding together
])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_tensor_map_convolution_matches_fp32_convolution(C, Co, H, W, k, s, p, d, dtype):
    from mmcv_b200 import _ext
    gen = torch.Generator().manual_seed(C * 1000 + Co)
    x = _rand((3, C, H, W), gen, dtype=dtype)
    w = _rand((Co, C, k, k), gen, 0.05, dtype=dtype)
    b = _rand((Co,), gen, 0.1, dtype=dtype)
    ref = F.conv2d(x.float(), w.float(), b.float(), stride=s, padding=p, dilation=d)
    xd = x.cuda()
    for padded in (None, _ext.pad_channels_last(xd)):
        y = _ext.conv_forward(xd, w.cuda(), b.cuda(), (s, s), (p, p), (d, d), padded=padded)
        assert y.shape == ref.shape and y.dtype == dtype
        assert rel_l2(y, ref) <= 5e-3, (padded is not None, rel_l2(y, ref))
    # channels-last input gives the same bits
    y2 = _ext.conv_forward(xd.contiguous(memory_format=torch.channels_last), w.cuda(), b.cuda(),
                           (s, s), (p, p), (d, d))
    assert torch.equal(y2, y)


def test_fused_sigmoid_on_a_channel_range():
    from mmcv_b200 import _ext
    gen = torch.Generator().manual_seed(5)
    x = _rand((2, 64, 20, 20), gen)
    w = _rand((27, 64, 3, 3), gen, 0.05)
    b = _rand((27,), gen, 0.1)
    ref = F.conv2d(x.float(), w.float(), b.float(), padding=1)
    ref[:, 18:] = torch.sigmoid(ref[:, 18:])
    y = _ext.conv_offset_forward(x.cuda(), w.cuda(), b.cuda(), (1, 1), (1, 1), (1, 1), sigmoid_from=18)
    assert rel_l2(y, ref) <= 5e-3


@pytest.mark.parametrize('C,H,W', [(128, 168, 100), (256, 84, 50), (512, 42, 25)])
def test_pack_layer_at_the_stack_shapes(C, H, W):
    """ModulatedDeformConv2dPack, bf16, at the three layer shapes of the 13-layer stack (two
    samples instead of sixteen: the CPU checker is the slow part)."""
    from mmcv_b200 import _ext
    from mmcv_b200.ops import ModulatedDeformConv2dPack
    from mmcv_b200.ops import modulated_deform_conv as mdc
    assert mdc.OFFSET_BRANCH == 'kernel'
    torch.manual_seed(C)
    m = ModulatedDeformConv2dPack(C, C, 3, padding=1, deform_groups=1, bias=True)
    m.conv_offset.weight.data.normal_(0, 0.01)
    m.conv_offset.bias.data.normal_(0, 0.5)
    m = m.cuda().to(torch.bfloat16).eval()
    x = torch.relu(torch.randn(2, C, H, W)).to(torch.bfloat16).cuda()
    with torch.no_grad():
        y = m(x)
        # (i) the branch, as the layer computes it
        br = _ext.conv_offset_forward(x, m.conv_offset.weight, m.conv_offset.bias, (1, 1), (1, 1),
                                      (1, 1), padded=_ext.pad_channels_last(x))
    br_ref = F.conv2d(x.float().cpu(), m.conv_offset.weight.float().cpu(),
                      m.conv_offset.bias.float().cpu(), padding=1)
    assert rel_l2(br, br_ref) <= 5e-3
    # (ii) the layer against the checker fed the branch's own offsets and mask
    off = br[:, :18].float().cpu()
    msk = torch.sigmoid(br[:, 18:].float()).cpu()
    ref = oracle.best_forward(x.float().cpu(), off, msk, m.weight.float().cpu(), m.bias.float().cpu(),
                              1, 1, 1, 1, 1)
    assert y.shape == ref.shape
    assert rel_l2(y, ref) <= 2e-2, rel_l2(y, ref)
    # the library branch gives the same layer output up to the branch's rounding
    mdc.OFFSET_BRANCH = 'library'
    try:
        with torch.no_grad():
            y_lib = m(x)
    finally:
        mdc.OFFSET_BRANCH = 'kernel'
    assert rel_l2(y_lib, y) <= 2e-2


def test_v1_pack_layer_with_own_branch():
    from mmcv_b200.ops import DeformConv2dPack
    torch.manual_seed(3)
    m = DeformConv2dPack(64, 96, 3, padding=1, deform_groups=2)
    m.conv_offset.weight.data.normal_(0, 0.02)
    m.conv_offset.bias.data.normal_(0, 0.5)
    m = m.cuda().to(torch.bfloat16).eval()
    x = torch.randn(2, 64, 30, 26).to(torch.bfloat16).cuda()
    with torch.no_grad():
        y = m(x)
        off = F.conv2d(x, m.conv_offset.weight, m.conv_offset.bias, padding=1)
    ref = oracle.best_forward(x.float().cpu(), off.float().cpu(), None, m.weight.float().cpu(), None,
                              1, 1, 1, 1, 2)
    # (the offsets of the checker come from the library convolution: its bf16 rounding differs
    # from the kernel's by at most one unit in the last place, which moves a sampling position
    # by up to 0.03 pixel)
    assert rel_l2(y, ref) <= 2e-2
