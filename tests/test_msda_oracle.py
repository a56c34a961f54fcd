"""The CPU checker of multi-scale deformable attention against the fixtures generated from the
reference's own pure-PyTorch implementation (outputs and gradients), and the host-side checks of
the extension entry points."""
import os

import numpy as np
import pytest
import torch

from oracle.msda import msda_forward

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'msda_cases.npz')


def msda_case_names():
    return sorted({k.split('/')[0] for k in np.load(GOLDEN).files})


def msda_case(name):
    z = np.load(GOLDEN)
    return {k.split('/')[1]: torch.from_numpy(z[k]) for k in z.files if k.startswith(name + '/')}


@pytest.mark.parametrize('name', msda_case_names())
def test_checker_reproduces_the_reference_outputs_and_gradients(name):
    t = msda_case(name)
    v = t['value'].double().requires_grad_(True)
    loc = t['loc'].double().requires_grad_(True)
    a = t['attn'].double().requires_grad_(True)
    out = msda_forward(v, t['shapes'], loc, a)
    assert torch.allclose(out.float(), t['out'], rtol=1e-5, atol=1e-7)
    out.backward(t['grad_out'].double())
    assert torch.allclose(v.grad.float(), t['grad_value'], rtol=1e-4, atol=1e-6)
    assert torch.allclose(a.grad.float(), t['grad_attn'], rtol=1e-4, atol=1e-6)
    # gradients of the locations: grid_sample and the kernel's formula agree except exactly on
    # cell borders, where the bilinear surface has a kink (either one-sided derivative is valid)
    lw = loc.detach()[..., 0] * t['shapes'][:, 1].view(1, 1, 1, -1, 1) - 0.5
    lh = loc.detach()[..., 1] * t['shapes'][:, 0].view(1, 1, 1, -1, 1) - 0.5
    smooth = ((lw - lw.round()).abs() > 1e-6) & ((lh - lh.round()).abs() > 1e-6)
    d = (loc.grad.float() - t['grad_loc']).abs()
    assert (d[smooth] <= 1e-4 * t['grad_loc'].abs().max() + 1e-6).all()


def test_extension_entries_reject_cpu_tensors_and_bad_arguments():
    from mmcv_b200 import _ext
    from mmcv_b200.ops import MultiScaleDeformableAttention, MultiScaleDeformableAttnFunction
    t = msda_case('ref_test')
    starts = torch.tensor([0, 24])
    with pytest.raises(RuntimeError, match='CUDA tensor'):
        _ext.ms_deform_attn_forward(t['value'], t['shapes'], starts, t['loc'], t['attn'], 2)
    with pytest.raises(RuntimeError, match='CUDA tensor'):
        MultiScaleDeformableAttnFunction.apply(t['value'], t['shapes'], starts, t['loc'], t['attn'], 2)
    with pytest.raises(ValueError):
        MultiScaleDeformableAttention(embed_dims=256, num_heads=7)
    m = MultiScaleDeformableAttention(embed_dims=6, num_levels=2, num_heads=3, value_proj_ratio=0.5)
    assert m.value_proj.out_features == 3 and m.output_proj.in_features == 3
    assert m.sampling_offsets.out_features == 3 * 2 * 4 * 2
    assert torch.count_nonzero(m.sampling_offsets.weight) == 0
    assert torch.count_nonzero(m.attention_weights.weight) == 0
    # the bias of the offsets points each head in its own direction, growing with the point index
    g = m.sampling_offsets.bias.view(3, 2, 4, 2)
    assert torch.allclose(g[:, :, 1], 2 * g[:, :, 0]) and torch.allclose(g[0, 0, 0], torch.tensor([1., 0.]))
    q = torch.rand(5, 1, 6)
    with pytest.raises(RuntimeError, match='no CPU path'):
        m(q, q, q, reference_points=torch.rand(1, 5, 2, 2),
          spatial_shapes=torch.tensor([[2, 2], [1, 1]]), level_start_index=torch.tensor([0, 4]))
