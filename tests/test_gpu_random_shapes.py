"""Seeded sweep over small random problems: kernel size, stride, padding, dilation, groups,
deform groups, odd spatial sizes, inputs smaller than the (dilated) kernel, offsets that are
grid-aligned, far out of range, NaN or Inf.  Every case runs in fp32 (default 3xTF32 / FFMA
routing and forced FFMA) and bf16 and is compared with the CPU checker."""
import random

import pytest
import torch

import oracle
from conftest import fp32_close, rel_l2
from mmcv_b200 import _lib
from test_gpu_parity import rounded, run_cuda

pytestmark = pytest.mark.gpu


def random_case(rng):
    while True:
        kh, kw = rng.randint(1, 4), rng.randint(1, 4)
        s, p, d = rng.randint(1, 3), rng.randint(0, 3), rng.randint(1, 3)
        g, dg = rng.choice([1, 1, 2, 4]), rng.choice([1, 1, 2, 4])
        unit = g * dg // __import__('math').gcd(g, dg)
        mult = rng.choice([1, 2, 4, 8, 16])
        C = unit * mult
        Co = g * rng.randint(1, 5)
        H, W = rng.randint(2, 18), rng.randint(2, 18)
        Ho, Wo = oracle.out_size(H, p, d, kh, s), oracle.out_size(W, p, d, kw, s)
        if Ho >= 1 and Wo >= 1 and C <= 128:
            break
    N = rng.randint(1, 3)
    seed = rng.randint(0, 10 ** 6)
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(N, C, H, W, generator=gen)
    off = torch.randn(N, dg * 2 * kh * kw, Ho, Wo, generator=gen) * rng.choice([0.5, 2.0, 8.0])
    kind = rng.choice(['plain', 'int', 'far', 'nonfinite'])
    if kind == 'int':
        off = torch.where(torch.rand(off.shape, generator=gen) < 0.3, off.round(), off)
    elif kind == 'far':
        off = off + (torch.rand(off.shape, generator=gen) < 0.2) * (H + W + 5.0)
    elif kind == 'nonfinite':
        flat = off.view(-1)
        idx = torch.randperm(flat.numel(), generator=gen)[:max(1, flat.numel() // 20)]
        flat[idx] = torch.tensor([float('nan'), float('inf'), float('-inf')])[idx % 3]
    with_mask = rng.random() < 0.7
    msk = torch.sigmoid(torch.randn(N, dg * kh * kw, Ho, Wo, generator=gen)) if with_mask else None
    w = torch.randn(Co, C // g, kh, kw, generator=gen) * (1.0 / (C // g * kh * kw)) ** 0.5
    b = torch.randn(Co, generator=gen) * 0.1 if (with_mask and rng.random() < 0.7) else None
    t = dict(x=x, offset=off, mask=msk, weight=w, bias=b)
    m = dict(stride=(s, s), padding=(p, p), dilation=(d, d), groups=g, deform_groups=dg)
    return m, t


@pytest.mark.parametrize('index', range(48))
def test_random_problem(index):
    rng = random.Random(4242 + index)
    m, t = random_case(rng)
    args = (m['stride'], m['padding'], m['dilation'], m['groups'], m['deform_groups'])
    ref = oracle.port_forward(t['x'], t['offset'], t['mask'], t['weight'], t['bias'], *args)
    for math in (_lib.MATH_AUTO, _lib.MATH_FFMA):
        out = run_cuda(t, m, torch.float32, math=math)
        ok, frac = fp32_close(out, ref)
        assert ok, f'fp32 math {math}: error is {frac:.3f}x the bound'
    r = rounded(t, torch.bfloat16)
    refb = oracle.port_forward(r['x'], r['offset'], r['mask'], r['weight'], r['bias'], *args)
    outb = run_cuda(t, m, torch.bfloat16).float().cpu()
    assert torch.equal(torch.isfinite(outb), torch.isfinite(refb))
    # small outputs can be dominated by a few bf16 roundings: add an absolute floor
    err = (outb - refb).norm().item()
    assert err <= 2e-2 * refb.norm().item() + 2e-3 * refb.numel() ** 0.5
