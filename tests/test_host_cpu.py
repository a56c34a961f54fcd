"""Host-side logic that needs no GPU: the library loads and exports every declared
symbol, planning, argument errors, interface parity with the reference wrappers."""
import ctypes
import os
import re

import pytest
import torch

from mmcv_b200 import _ext, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, 'include', 'dcn_b200.h')).read()
    declared = set(re.findall(r'\b(dcn_[a-z0-9_]+)\s*\(', header))
    assert declared == set(_lib.EXPORTS)
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name)
    assert lib.dcn_abi_version() == int(re.search(r'#define DCN_ABI_VERSION (\d+)', header).group(1))


def params(dtype=_lib.DTYPE_BF16, N=2, C=64, H=16, W=16, Co=64, k=3, s=1, p=1, d=1, g=1, dg=1,
           math=_lib.MATH_AUTO):
    q = _lib.DcnFwdParams()
    q.dtype, q.math_mode = dtype, math
    q.N, q.C, q.H, q.W, q.Co = N, C, H, W, Co
    q.kh = q.kw = k
    q.stride_h = q.stride_w = s
    q.pad_h = q.pad_w = p
    q.dil_h = q.dil_w = d
    q.groups, q.deform_groups = g, dg
    q.in_stride[0], q.in_stride[1], q.in_stride[2], q.in_stride[3] = C * H * W, H * W, W, 1
    return q


def plan(q):
    info = _lib.DcnPlanInfo()
    rc = _lib.load().dcn_fwd_plan(ctypes.byref(q), ctypes.byref(info))
    return rc, info


def test_plan_routes_and_sizes():
    rc, info = plan(params())
    assert rc == 0 and info.path == _lib.PATH_TCGEN05
    assert (info.tile_m, info.tile_n, info.tile_k) == (128, 64, 64)
    assert info.smem_bytes <= 232448 and info.stages_input == 1
    assert info.workspace_bytes >= 2 * 64 * 16 * 16 * 2 + 64 * 64 * 9 * 2
    rc, info = plan(params(dtype=_lib.DTYPE_F32))
    assert rc == 0 and info.path == _lib.PATH_TCGEN05 and info.tile_k == 32   # 3xTF32
    assert info.kernel_version == 1
    rc, info = plan(params(dtype=_lib.DTYPE_F32, math=_lib.MATH_FFMA))
    assert rc == 0 and info.path == _lib.PATH_SIMT_TILED
    rc, info = plan(params(dtype=_lib.DTYPE_F32, math=_lib.MATH_FFMA, N=1, C=4, Co=4, H=5, W=5))
    assert rc == 0 and info.path == _lib.PATH_SIMT_DIRECT      # too small for 64x64 tiles
    rc, info = plan(params(C=48, Co=48))                 # a partly filled last 64-channel chunk
    assert rc == 0 and info.path == _lib.PATH_TCGEN05
    rc, info = plan(params(C=20, Co=20))                 # channels not a multiple of 8
    assert rc == 0 and info.path == _lib.PATH_SIMT_TILED
    rc, info = plan(params(N=256, C=256, H=128, W=128, Co=256, dg=8))
    assert rc == 0 and info.path == _lib.PATH_TCGEN05 and info.tile_n == 256
    assert info.grid == 148 and info.smem_bytes <= 232448
    # 16-bit tensors run on the second-generation kernel: 4 epilogue + MMA + 2 loader + 1 idle
    # + 16 gather warps that build their own tap entries
    assert info.kernel_version == 2 and info.producer_layout == 16 and info.block == 24 * 32
    assert info.operand_stages >= 2 and info.weight_stages == 2
    rc, info = plan(params(N=8, C=256, H=100, W=168, Co=256, dg=4))
    assert rc == 0 and info.kernel_version == 2
    assert info.window_h >= 10 + 6 and info.window_w >= 18 + 6 and info.window_w % 2 == 0
    # more than 64 channels per deform group: the first-generation kernel's shared tap table wins
    rc, info = plan(params(N=8, C=256, H=100, W=168, Co=256, dg=1))
    assert rc == 0 and info.path == _lib.PATH_TCGEN05 and info.kernel_version == 1
    # a strided layer samples too widely for the shared-memory window: first-generation kernel
    rc, info = plan(params(C=512, Co=512, H=64, W=64, s=2, p=2, d=2, dg=4))
    assert rc == 0 and info.kernel_version == 1 and (info.Ho, info.Wo) == (32, 32)
    # a deform group of 16 channels starts inside a 32-channel unit: first-generation kernel
    rc, info = plan(params(C=64, Co=64, dg=4))
    assert rc == 0 and info.path == _lib.PATH_TCGEN05 and info.kernel_version == 1
    rc, info = plan(params(dtype=_lib.DTYPE_F32, math=_lib.MATH_TF32X3, C=256, Co=256, H=100, W=168))
    assert rc == 0 and info.path == _lib.PATH_TCGEN05 and info.tile_k == 32
    assert info.smem_bytes <= 232448
    rc, info = plan(params(dtype=_lib.DTYPE_F32, math=_lib.MATH_TF32X3, C=6, Co=12))
    assert rc == 0 and info.path == _lib.PATH_SIMT_TILED       # degrades to FFMA
    rc, info = plan(params(C=512, Co=512, H=64, W=64, s=2, p=2, d=2, dg=4))
    assert rc == 0 and (info.Ho, info.Wo) == (32, 32) and info.tile_n == 256


def test_plan_rejects_what_the_reference_rejects():
    lib = _lib.load()
    for kw, text in [(dict(k=0), 'kernel size'), (dict(s=0), 'stride'), (dict(d=0), 'dilation'),
                     (dict(C=6, dg=4), 'deformable group'), (dict(H=1, W=1, p=0), 'too small'),
                     (dict(C=6, g=4), "won't match")]:
        rc, _ = plan(params(**kw))
        assert rc == -1, kw
        assert text in lib.dcn_last_error().decode()
    rc, _ = plan(params(dtype=7))
    assert rc == -2
    rc, info = plan(params(dtype=_lib.DTYPE_F16))
    assert rc == 0 and info.path == _lib.PATH_TCGEN05
    rc, _ = plan(params(C=20, Co=20, math=_lib.MATH_BF16))
    assert rc == -2
    rc, _ = plan(params(math=_lib.MATH_TF32X3))          # bf16 tensors with the fp32-only mode
    assert rc == -1


def test_forward_on_cpu_tensors_fails_loudly():
    x = torch.randn(1, 4, 5, 5)
    w = torch.randn(4, 4, 3, 3)
    out = torch.empty(1, 4, 5, 5)
    e = x.new_empty(0)
    with pytest.raises(RuntimeError, match='CUDA tensor'):
        _ext.modulated_deform_conv_forward(
            x, w, e, e, torch.zeros(1, 18, 5, 5), torch.ones(1, 9, 5, 5), out, e, kernel_h=3,
            kernel_w=3, stride_h=1, stride_w=1, pad_h=1, pad_w=1, dilation_h=1, dilation_w=1,
            group=1, deformable_group=1, with_bias=False)
    with pytest.raises(RuntimeError, match='CUDA tensor'):
        _ext.deform_conv_forward(x, w, torch.zeros(1, 18, 5, 5), out, e, e, kW=3, kH=3, dW=1,
                                 dH=1, padW=1, padH=1, dilationW=1, dilationH=1, group=1,
                                 deformable_group=1, im2col_step=1)


def test_offset_mask_output_shapes_are_checked_before_any_launch():
    """The kernels take every size from the problem geometry, so a tensor of another shape must
    be rejected on the host (no launch happens here: the tensors are CPU tensors and the shape
    error comes first)."""
    x = torch.randn(2, 4, 6, 6)
    w = torch.randn(4, 4, 3, 3)
    e = x.new_empty(0)

    def call(offset, mask, out, dg=1, stride=1):
        _ext.modulated_deform_conv_forward(
            x, w, e, e, offset, mask, out, e, kernel_h=3, kernel_w=3, stride_h=stride,
            stride_w=stride, pad_h=1, pad_w=1, dilation_h=1, dilation_w=1, group=1,
            deformable_group=dg, with_bias=False)

    good_off, good_msk, good_out = torch.zeros(2, 18, 6, 6), torch.ones(2, 9, 6, 6), torch.empty(2, 4, 6, 6)
    for off, msk, out, kw, what in [
            (torch.zeros(2, 18, 3, 3), good_msk, good_out, {}, 'offset'),       # made for stride 2
            (torch.zeros(1, 18, 6, 6), good_msk, good_out, {}, 'offset'),       # smaller batch
            (good_off, torch.ones(2, 18, 6, 6), good_out, {}, 'mask'),          # two deform groups' worth
            (good_off, good_msk, torch.empty(2, 4, 5, 6), {}, 'output'),
            (good_off, good_msk, good_out, dict(dg=2), 'offset'),               # wrong deformable_group
            (good_off, good_msk, good_out, dict(stride=2), 'offset')]:
        with pytest.raises(RuntimeError, match=f'{what} has shape'):
            call(off, msk, out, **kw)
    with pytest.raises(RuntimeError, match='CUDA tensor'):     # all shapes right: next check
        call(good_off, good_msk, good_out)
    # the branch form: channel count and spatial size of the branch output
    with pytest.raises(RuntimeError, match='offset channels'):
        _ext.forward_from_branch(x, torch.zeros(2, 20, 6, 6), 18, w, None, good_out, (1, 1), (1, 1),
                                 (1, 1), 1, 1)
    with pytest.raises(RuntimeError, match='not the output size'):
        _ext.forward_from_branch(x, torch.zeros(2, 27, 3, 3), 18, w, None, good_out, (1, 1), (1, 1),
                                 (1, 1), 1, 1)
    with pytest.raises(RuntimeError, match='output has shape'):
        _ext.forward_from_branch(x, torch.zeros(2, 27, 6, 6), 18, w, None, torch.empty(2, 4, 3, 3),
                                 (1, 1), (1, 1), (1, 1), 1, 1)


def test_kernel_shape_mismatch_is_runtime_error():
    x = torch.randn(1, 4, 5, 5)
    w = torch.randn(4, 4, 3, 3)
    e = x.new_empty(0)
    with pytest.raises(RuntimeError, match="kernel shape won't match"):
        _ext.modulated_deform_conv_forward(
            x, w, e, e, x, x, x, e, kernel_h=2, kernel_w=3, stride_h=1, stride_w=1, pad_h=1,
            pad_w=1, dilation_h=1, dilation_w=1, group=1, deformable_group=1, with_bias=False)
    with pytest.raises(RuntimeError, match="kernel channels won't match"):
        _ext.modulated_deform_conv_forward(
            x, w, e, e, x, x, x, e, kernel_h=3, kernel_w=3, stride_h=1, stride_w=1, pad_h=1,
            pad_w=1, dilation_h=1, dilation_w=1, group=2, deformable_group=1, with_bias=False)


def test_backward_entries_fail_loudly_on_cpu_tensors():
    x = torch.randn(1, 4, 5, 5)
    w = torch.randn(4, 4, 3, 3)
    e = x.new_empty(0)
    off, msk = torch.zeros(1, 18, 5, 5), torch.ones(1, 9, 5, 5)
    with pytest.raises(RuntimeError, match='CUDA tensor'):
        _ext.modulated_deform_conv_backward(
            x, w, e, e, off, msk, e, torch.zeros_like(x), torch.zeros_like(w), e,
            torch.zeros_like(off), torch.zeros_like(msk), torch.zeros(1, 4, 5, 5), kernel_h=3,
            kernel_w=3, stride_h=1, stride_w=1, pad_h=1, pad_w=1, dilation_h=1, dilation_w=1,
            group=1, deformable_group=1, with_bias=False)
    with pytest.raises(RuntimeError, match='CUDA tensor'):
        _ext.deform_conv_backward_input(x, off, torch.zeros(1, 4, 5, 5), torch.zeros_like(x),
                                        torch.zeros_like(off), w, e, kW=3, kH=3, dW=1, dH=1,
                                        padW=1, padH=1, dilationW=1, dilationH=1, group=1,
                                        deformable_group=1, im2col_step=1)
    with pytest.raises(RuntimeError, match='CUDA tensor'):
        _ext.deform_conv_backward_parameters(x, off, torch.zeros(1, 4, 5, 5), torch.zeros_like(w),
                                             e, e, kW=3, kH=3, dW=1, dH=1, padW=1, padH=1,
                                             dilationW=1, dilationH=1, group=1,
                                             deformable_group=1, scale=1, im2col_step=1)


def test_module_interface_matches_reference_contract():
    from mmcv_b200.ops import (DeformConv2d, DeformConv2dPack, ModulatedDeformConv2d,
                               ModulatedDeformConv2dPack)
    m = ModulatedDeformConv2dPack(8, 6, 3, stride=2, padding=1, dilation=1, groups=2,
                                  deformable_groups=2, bias=True)
    assert m.deform_groups == 2 and m.conv_offset.out_channels == 2 * 3 * 9
    assert m.weight.shape == (6, 4, 3, 3) and m.bias.shape == (6,)
    assert float(m.conv_offset.weight.detach().abs().sum()) == 0 and float(m.bias.detach().abs().sum()) == 0
    assert set(m.state_dict()) == {'weight', 'bias', 'conv_offset.weight', 'conv_offset.bias'}
    v1 = DeformConv2dPack(4, 4, 3, padding=1, deform_groups=2)
    assert v1.conv_offset.out_channels == 2 * 2 * 9 and not hasattr(v1, 'bias')
    with pytest.raises(AssertionError):
        DeformConv2d(1, 1, 2, bias=True)
    with pytest.raises(AssertionError):
        DeformConv2d(3, 2, 3, groups=2)
    with pytest.raises(AssertionError):
        DeformConv2d(3, 4, 3, groups=3)
    with pytest.raises(ValueError, match='Expected 4D tensor'):
        ModulatedDeformConv2d(1, 1, 1)(torch.zeros(1, 3, 3), torch.zeros(1), torch.zeros(1))
    with pytest.raises(ValueError, match='too small'):
        ModulatedDeformConv2d(1, 1, 5)(torch.zeros(1, 1, 3, 3), torch.zeros(1, 50, 1, 1),
                                       torch.zeros(1, 25, 1, 1))


def test_state_dict_key_upgrade():
    # checkpoints older than version 2 name the offset branch "<layer>_offset"; the layer
    # renames those keys when it is handed the dict (same rule as the reference layer)
    from mmcv_b200.ops import DeformConv2dPack, ModulatedDeformConv2dPack
    for cls in (ModulatedDeformConv2dPack, DeformConv2dPack):
        layer = cls(4, 4, 3, padding=1)
        sd = {k: v.clone() for k, v in layer.state_dict().items()}
        legacy = {}
        for k, v in sd.items():
            if k.startswith('conv_offset.'):
                legacy['conv2_offset.' + k.split('.', 1)[1]] = v + 1
            else:
                legacy['conv2.' + k] = v
        missing, unexpected, errors = [], [], []
        layer._load_from_state_dict(legacy, 'conv2.', {}, True, missing, unexpected, errors)
        assert 'conv2.conv_offset.weight' in legacy and 'conv2_offset.weight' not in legacy
        layer.conv_offset._load_from_state_dict(legacy, 'conv2.conv_offset.', {}, True, missing,
                                                unexpected, errors)
        assert not missing and not errors
        assert torch.equal(layer.conv_offset.weight, sd['conv_offset.weight'] + 1)
        # a version-2 dict is left alone
        legacy2 = {'conv2_offset.weight': sd['conv_offset.weight']}
        layer._load_from_state_dict(legacy2, 'conv2.', {'version': 2}, False, [], [], [])
        assert 'conv2_offset.weight' in legacy2


def test_reference_wrappers_accept_this_extension():
    # The reference's unchanged Python wrappers load on top of this _ext (all five names are
    # found) and reach it; on CPU tensors the call must fail loudly instead of falling back.
    import sys
    sys.path.insert(0, os.path.join(ROOT, 'tests', 'golden'))
    import ref_wrappers
    if ref_wrappers.default_root() is None:
        pytest.skip('the reference wrapper files are not available (oracle/build_oracle.py copies them)')
    v2, v1, reg = ref_wrappers.load(_ext)
    try:
        assert set(reg.modules) == {'DCN', 'DCNv2'}
        layer = v2.ModulatedDeformConv2dPack(4, 4, 3, padding=1)
        with pytest.raises(RuntimeError, match='CUDA tensor'):
            layer(torch.randn(1, 4, 6, 6))
        with pytest.raises(RuntimeError, match='CUDA tensor'):
            v1.DeformConv2dPack(4, 4, 3, padding=1)(torch.randn(1, 4, 6, 6))
    finally:
        ref_wrappers.unload()


def test_onnx_symbolic_names_match_the_reference():
    from mmcv_b200.ops import DeformConv2dFunction, ModulatedDeformConv2dFunction

    class G:
        def op(self, name, *tensors, **attrs):
            return name, len(tensors), attrs

    name, n, attrs = ModulatedDeformConv2dFunction.symbolic(G(), 1, 2, 3, 4, 5, (1, 1), (1, 1),
                                                            (1, 1), 1, 2)
    assert name == 'mmcv::MMCVModulatedDeformConv2d' and n == 5
    assert set(attrs) == {'stride_i', 'padding_i', 'dilation_i', 'groups_i', 'deform_groups_i'}
    name, n, attrs = ModulatedDeformConv2dFunction.symbolic(G(), 1, 2, 3, 4, None, 1, 1, 1, 1, 1)
    assert n == 4
    name, n, attrs = DeformConv2dFunction.symbolic(G(), 1, 2, 3, 1, 0, 1, 1, 1)
    assert name == 'mmcv::MMCVDeformConv2d' and n == 3
    assert attrs['bias_i'] is False and attrs['im2col_step_i'] == 32
