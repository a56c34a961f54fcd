"""Backward of the deformable convolutions on the GPU against the reference's gradients:
the reference tests' own vectors (forward + backward through the Pack layers, as those tests
do) and the seeded fixtures generated from the unmodified reference."""
import numpy as np
import pytest
import torch

from conftest import golden_case_names, golden_cases

pytestmark = pytest.mark.gpu


def grad_close(got, ref, what):
    got, ref = got.detach().float().cpu(), ref.float()
    bound = 2e-4 * ref.abs().max().item() + 2e-5
    err = (got - ref).abs().max().item()
    assert err <= bound, f'{what}: max error {err:.3e} exceeds {bound:.3e}'


@pytest.mark.parametrize('name', [n for n in golden_case_names() if 'nonfinite' not in n])
def test_gradients_match_reference_fixtures(name):
    from mmcv_b200.ops import deform_conv2d, modulated_deform_conv2d
    m, t = golden_cases().get(name)
    leaf = {k: (None if t[k] is None else t[k].cuda().requires_grad_(True))
            for k in ('x', 'offset', 'mask', 'weight', 'bias')}
    if t['mask'] is not None:
        y = modulated_deform_conv2d(leaf['x'], leaf['offset'], leaf['mask'], leaf['weight'],
                                    leaf['bias'], m['stride'], m['padding'], m['dilation'],
                                    m['groups'], m['deform_groups'])
    else:
        y = deform_conv2d(leaf['x'], leaf['offset'], leaf['weight'], m['stride'], m['padding'],
                          m['dilation'], m['groups'], m['deform_groups'], False, 32)
    y.backward(t['grad_out'].cuda())
    for k in ('x', 'offset', 'mask', 'weight', 'bias'):
        if leaf[k] is not None:
            grad_close(leaf[k].grad, t['grad_' + k], f'{name} grad_{k}')


def test_reference_known_answer_v2_forward_and_backward(kat):
    # the reference's DCNv2 test flow (its test file, lines 51-85), backward included
    from mmcv_b200.ops import ModulatedDeformConv2dPack
    x = torch.tensor(kat['v2_input'], device='cuda', requires_grad=True)
    dcn = ModulatedDeformConv2dPack(1, 1, kernel_size=(2, 2), stride=1, padding=1,
                                    deform_groups=1, bias=False).cuda()
    dcn.weight.data.fill_(1.)
    out = dcn(x)
    out.sum().backward()
    c = lambda v: v.detach().cpu().numpy()
    assert np.allclose(c(out), kat['v2_expected'], 1e-2)
    assert np.allclose(c(x.grad), kat['v2_input_grad'], 1e-2)
    assert np.allclose(c(dcn.weight.grad), kat['v2_dcn_w_grad'], 1e-2)
    assert np.allclose(c(dcn.conv_offset.weight.grad), kat['v2_dcn_offset_w_grad'], 1e-2)
    assert np.allclose(c(dcn.conv_offset.bias.grad), kat['v2_dcn_offset_b_grad'], 1e-2)


def test_reference_known_answer_v1_forward_and_backward(kat):
    # the reference's DCNv1 test flow (its test file, lines 52-110) at its CUDA threshold 1e-3
    from mmcv_b200.ops import DeformConv2dPack
    batch = 10
    x = torch.tensor(np.repeat(kat['v1_input'], batch, axis=0), device='cuda', requires_grad=True)
    model = DeformConv2dPack(in_channels=1, out_channels=1, kernel_size=2, stride=1, padding=0,
                             im2col_step=2)
    model.conv_offset.weight.data = torch.tensor(kat['v1_offset_weight'])
    model.conv_offset.bias.data = torch.tensor(kat['v1_offset_bias'])
    model.weight.data = torch.tensor(kat['v1_deform_weight'])
    model.cuda()
    out = model(x)
    out.backward(torch.ones_like(out))
    c = lambda v: v.detach().cpu().numpy()
    thr = 1e-3
    assert np.allclose(c(out), np.repeat(kat['v1_expected'], batch, axis=0), thr)
    assert np.allclose(c(x.grad), np.repeat(kat['v1_x_grad'], batch, axis=0), thr)
    assert np.allclose(c(model.conv_offset.weight.grad) / batch, kat['v1_offset_weight_grad'], thr)
    assert np.allclose(c(model.conv_offset.bias.grad) / batch, kat['v1_offset_bias_grad'], thr)
    assert np.allclose(c(model.weight.grad) / batch, kat['v1_deform_weight_grad'], thr)
    # and against the reference's unrounded gradients on the same case
    assert np.allclose(c(x.grad), kat['v1_ref_x_grad'], rtol=1e-4, atol=1e-5)
    assert np.allclose(c(model.weight.grad), kat['v1_ref_deform_weight_grad'], rtol=1e-4, atol=1e-5)


def test_bf16_backward_runs_and_is_close():
    from mmcv_b200.ops import modulated_deform_conv2d
    m, t = golden_cases().get('v2_c64')
    leaf = {k: (None if t[k] is None else t[k].cuda().to(torch.bfloat16).requires_grad_(True))
            for k in ('x', 'offset', 'mask', 'weight', 'bias')}
    y = modulated_deform_conv2d(leaf['x'], leaf['offset'], leaf['mask'], leaf['weight'],
                                leaf['bias'], m['stride'], m['padding'], m['dilation'],
                                m['groups'], m['deform_groups'])
    y.backward(t['grad_out'].cuda().to(torch.bfloat16))
    for k in ('x', 'weight', 'mask'):
        g, r = leaf[k].grad.float().cpu(), t['grad_' + k]
        assert leaf[k].grad.dtype == torch.bfloat16
        assert ((g - r).norm() / r.norm()).item() < 5e-2, k
