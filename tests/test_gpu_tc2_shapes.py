"""Shapes that exercise the corners of the table-free 16-bit kernel (dcn_fwd_tc2): a conv group
whose last 32-channel half-chunk is partly empty, several conv groups in the unit table, an odd
number of K units (the last k-stage has one unit only), a 5x5 kernel (a wide window), two- and
four-tap kernels (a gather group then passes input windows it never reads),
deform groups of 8 / 16 / 24 channels next to the 32-channel units they must fit in, images that
tiles overhang, far and non-finite offsets, and non-finite input samples.  Each case asserts that
the plan routes it to that kernel, and compares with the CPU checker on the rounded inputs
(relative L2 <= 2e-2; finiteness patterns equal).
"""
import ctypes

import pytest
import torch

import oracle
from conftest import rel_l2
from mmcv_b200 import _lib
from test_gpu_parity import plan_path, rounded, run_cuda

pytestmark = pytest.mark.gpu

# name: N, C, H, W, Co, k, pad, groups, dg, offset sigma, special
CASES = {
    'ragged_group_48': (2, 96, 20, 22, 64, 3, 1, 2, 2, 2.0, ''),
    'three_groups': (1, 96, 17, 19, 48, 3, 1, 3, 3, 1.5, ''),
    'odd_units': (2, 96, 12, 14, 40, 3, 1, 1, 3, 1.0, ''),
    'kernel_1x2': (1, 96, 11, 13, 16, (1, 2), (0, 1), 1, 3, 1.0, ''),
    'kernel_2x2': (1, 64, 11, 13, 16, 2, 1, 1, 2, 1.0, ''),
    'kernel_3x1': (2, 128, 21, 17, 32, (3, 1), (1, 0), 1, 4, 1.5, ''),
    'kernel_1x3_two_images': (3, 160, 10, 40, 16, (1, 3), (0, 1), 1, 5, 1.5, ''),
    'kernel_5x5': (1, 64, 18, 20, 32, 5, 2, 1, 2, 2.0, ''),
    'dg_of_8_channels': (1, 64, 14, 14, 64, 3, 1, 1, 2, 1.0, 'int'),
    'far_and_nonfinite_offsets': (2, 64, 16, 16, 64, 3, 1, 1, 2, 6.0, 'far nonfinite'),
    'nonfinite_input': (1, 128, 13, 15, 32, 3, 1, 1, 4, 2.0, 'input_nonfinite int'),
    'wide_image_overhang': (1, 64, 9, 37, 24, 3, 1, 1, 1, 3.0, ''),
    'dilation_2': (2, 64, 19, 23, 32, 3, 2, 1, 2, 2.0, 'dil2'),
    'dilation_3_small_image': (1, 64, 7, 9, 16, 3, 3, 1, 2, 1.0, 'dil3'),
    'tiny_image_many_samples': (37, 32, 3, 5, 8, 3, 1, 1, 1, 1.0, ''),
    'tall_narrow': (2, 64, 70, 3, 16, 3, 1, 1, 2, 2.0, 'far'),
    'no_padding_shrinks': (1, 64, 16, 18, 16, 3, 0, 1, 2, 1.5, ''),
    'big_padding_grows': (1, 32, 8, 8, 16, 3, 3, 1, 1, 1.5, ''),
}


def make(name):
    N, C, H, W, Co, k, p, g, dg, sigma, special = CASES[name]
    kh, kw = (k, k) if isinstance(k, int) else k
    ph, pw = (p, p) if isinstance(p, int) else p
    gen = torch.Generator().manual_seed(sum(map(ord, name)))
    dil = 2 if 'dil2' in special else (3 if 'dil3' in special else 1)
    Ho, Wo = oracle.out_size(H, ph, dil, kh, 1), oracle.out_size(W, pw, dil, kw, 1)
    x = torch.randn(N, C, H, W, generator=gen)
    off = torch.randn(N, dg * 2 * kh * kw, Ho, Wo, generator=gen) * sigma
    if 'int' in special:
        off = torch.where(torch.rand(off.shape, generator=gen) < 0.2, off.round(), off)
    if 'far' in special:
        off = off + (torch.rand(off.shape, generator=gen) < 0.2) * (H + W + 5.0)
    if 'nonfinite' in special.split():
        flat = off.view(-1)
        idx = torch.randperm(flat.numel(), generator=gen)[:flat.numel() // 25]
        flat[idx] = torch.tensor([float('nan'), float('inf'), float('-inf')])[idx % 3]
    msk = torch.sigmoid(torch.randn(N, dg * kh * kw, Ho, Wo, generator=gen))
    if 'input_nonfinite' in special:
        flat = x.view(-1)
        idx = torch.randperm(flat.numel(), generator=gen)[:6]
        flat[idx] = torch.tensor([float('nan'), float('inf'), float('-inf')])[idx % 3]
        msk = torch.where(torch.rand(msk.shape, generator=gen) < 0.1, torch.zeros_like(msk), msk)
    w = torch.randn(Co, C // g, kh, kw, generator=gen) * (1.0 / (C // g * kh * kw)) ** 0.5
    b = torch.randn(Co, generator=gen) * 0.1
    t = dict(x=x, offset=off, mask=msk, weight=w, bias=b)
    m = dict(stride=(1, 1), padding=(ph, pw), dilation=(dil, dil), groups=g, deform_groups=dg)
    return m, t


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('name', sorted(CASES))
def test_table_free_kernel_corner_shapes(name, dtype):
    m, t = make(name)
    info = plan_path(t['x'], t['weight'], m, dtype)
    assert info.path == _lib.PATH_TCGEN05, info.path
    if 'dil3' not in CASES[name][10]:   # (a window around a 3-dilated footprint does not fit: either kernel may take it)
        assert info.kernel_version == 2, info.kernel_version
    r = rounded(t, dtype)
    ref = oracle.best_forward(r['x'], r['offset'], r['mask'], r['weight'], r['bias'], m['stride'],
                              m['padding'], m['dilation'], m['groups'], m['deform_groups'])
    out = run_cuda(t, m, dtype).float().cpu()
    finite = torch.isfinite(ref)
    assert torch.equal(torch.isfinite(out), finite)
    if 'nonfinite_input' in name:
        # NaN where the reference has NaN (an in-image corner under a non-finite sample, whatever its weight)
        assert torch.equal(torch.isnan(out), torch.isnan(ref))
    assert rel_l2(out[finite], ref[finite]) <= 2e-2


def test_one_tap_kernels_stay_on_the_first_generation_kernel():
    # every K unit of a 1x1 kernel is a half-chunk of its own; the window ring does not take that
    t = dict(x=torch.zeros(2, 96, 12, 14), weight=torch.zeros(40, 96, 1, 1))
    m = dict(stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, deform_groups=3)
    info = plan_path(t['x'], t['weight'], m, torch.bfloat16)
    assert info.path == _lib.PATH_TCGEN05 and info.kernel_version == 1
