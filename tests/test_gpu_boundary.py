"""The drop-in boundary on a GPU.

(a) The reference's UNCHANGED Python wrappers (mmcv/ops/modulated_deform_conv.py,
    mmcv/ops/deform_conv.py), loaded on top of ``mmcv_b200._ext`` in place of ``mmcv._ext``, run the
    reference tests' own flows (tests/test_ops/test_modulated_deform_conv.py:51-85, :87-127 and
    tests/test_ops/test_deform_conv.py:52-110) and the seeded fixtures.
(b) The flat C entry points a binding of the reference's C++ functions would call
    (``dcn_modulated_deform_conv_forward``, ``dcn_deform_conv_forward``,
    ``dcn_forward_workspace_bytes``), through ctypes with raw device pointers, in fp32, bf16, fp16.
"""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from conftest import fp32_close, golden_cases, rel_l2
from mmcv_b200 import _ext, _lib

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
import ref_wrappers  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture
def ref_ops():
    if ref_wrappers.default_root() is None:
        pytest.skip('the reference wrapper files are not available (oracle/build_oracle.py copies them)')
    v2, v1, _ = ref_wrappers.load(_ext)
    assert v2.ext_module is _ext and v1.ext_module is _ext
    yield v2, v1
    ref_wrappers.unload()


def _assert_v2_vectors(out, x, dcn, kat):
    c = lambda v: v.detach().float().cpu().numpy()
    assert np.allclose(c(out), kat['v2_expected'], 1e-2)
    assert np.allclose(c(x.grad), kat['v2_input_grad'], 1e-2)
    assert np.allclose(c(dcn.weight.grad), kat['v2_dcn_w_grad'], 1e-2)
    assert np.allclose(c(dcn.conv_offset.weight.grad), kat['v2_dcn_offset_w_grad'], 1e-2)
    assert np.allclose(c(dcn.conv_offset.bias.grad), kat['v2_dcn_offset_b_grad'], 1e-2)


@pytest.mark.parametrize('dtype', [torch.float, torch.half])
def test_reference_v2_flow_over_this_extension(ref_ops, kat, dtype):
    # tests/test_ops/test_modulated_deform_conv.py:51-85 (its float and half runs)
    v2, _ = ref_ops
    x = torch.tensor(kat['v2_input'], dtype=dtype, device='cuda')
    x.requires_grad = True
    dcn = v2.ModulatedDeformConv2dPack(1, 1, kernel_size=(2, 2), stride=1, padding=1,
                                       deform_groups=1, bias=False).to('cuda')
    dcn.weight.data.fill_(1.)
    dcn.type(dtype)
    out = dcn(x)
    out.sum().backward()
    _assert_v2_vectors(out, x, dcn, kat)


@pytest.mark.parametrize('dtype', [torch.float, torch.half])
def test_reference_v2_mixed_precision_flow(ref_ops, kat, dtype):
    # tests/test_ops/test_modulated_deform_conv.py:87-127, :182-184: the input in `dtype`, the
    # layer left in fp32, everything under autocast
    v2, _ = ref_ops
    with torch.autocast('cuda', enabled=True):
        x = torch.tensor(kat['v2_input']).to('cuda').type(dtype)
        x.requires_grad = True
        dcn = v2.ModulatedDeformConv2dPack(1, 1, kernel_size=(2, 2), stride=1, padding=1,
                                           deform_groups=1, bias=False).to('cuda')
        dcn.weight.data.fill_(1.)
        out = dcn(x)
        out.sum().backward()
    _assert_v2_vectors(out, x, dcn, kat)


@pytest.mark.parametrize('batch,im2col_step', [(10, 2), (10, 10), (1, 1)])
def test_reference_v1_flow_over_this_extension(ref_ops, kat, batch, im2col_step):
    _, v1 = ref_ops
    x = torch.tensor(np.repeat(kat['v1_input'], batch, axis=0), device='cuda', requires_grad=True)
    model = v1.DeformConv2dPack(in_channels=1, out_channels=1, kernel_size=2, stride=1, padding=0,
                                im2col_step=im2col_step)
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


def test_reference_v1_rejects_a_batch_the_step_does_not_divide(ref_ops, kat):
    # the reference pads the batch up to a multiple of im2col_step itself (deform_conv.py:88-96 is
    # the functional's assertion; the layer pads in forward) -- the functional must still assert
    _, v1 = ref_ops
    x = torch.randn(3, 4, 6, 6, device='cuda')
    w = torch.randn(4, 4, 3, 3, device='cuda')
    off = torch.zeros(3, 18, 6, 6, device='cuda')
    with pytest.raises(AssertionError):
        v1.deform_conv2d(x, off, w, 1, 1, 1, 1, 1, False, 2)


@pytest.mark.parametrize('name', ['v2_basic', 'v2_s2_d2_dg4_int', 'v2_g2_dg2', 'v2_c128_co40_dg4',
                                  'v1_basic', 'v1_g2_dg2_d2', 'v1_c64'])
def test_reference_functionals_on_the_fixtures(ref_ops, name):
    v2, v1 = ref_ops
    m, t = golden_cases().get(name)
    leaf = {k: (None if t[k] is None else t[k].cuda().requires_grad_(True))
            for k in ('x', 'offset', 'mask', 'weight', 'bias')}
    if t['mask'] is not None:
        y = v2.modulated_deform_conv2d(leaf['x'], leaf['offset'], leaf['mask'], leaf['weight'],
                                       leaf['bias'], m['stride'], m['padding'], m['dilation'],
                                       m['groups'], m['deform_groups'])
    else:
        y = v1.deform_conv2d(leaf['x'], leaf['offset'], leaf['weight'], m['stride'], m['padding'],
                             m['dilation'], m['groups'], m['deform_groups'], False, 32)
    ok, frac = fp32_close(y, t['out'])
    assert ok, f'{name}: forward error is {frac:.2f}x the bound'
    y.backward(t['grad_out'].cuda())
    for k in ('x', 'offset', 'mask', 'weight', 'bias'):
        if leaf[k] is not None:
            ref = t['grad_' + k]
            err = (leaf[k].grad.cpu() - ref).abs().max().item()
            assert err <= 2e-4 * ref.abs().max().item() + 2e-5, (name, k, err)


# ---------------------------------------------------------------------------------------------
# (b) the flat C entry points, raw pointers

_ELEM = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16}


def _vp(t):
    return ctypes.c_void_p(None if t is None else t.data_ptr())


def _flat_workspace(lib, elem, modulated, x, Co, kh, kw, m):
    n = ctypes.c_size_t(0)
    rc = lib.dcn_forward_workspace_bytes(elem, modulated, x.shape[0], x.shape[1], x.shape[2], x.shape[3],
                                         Co, kh, kw, m['stride'][0], m['stride'][1], m['padding'][0],
                                         m['padding'][1], m['dilation'][0], m['dilation'][1],
                                         m['groups'], m['deform_groups'], ctypes.byref(n))
    _lib.check(rc)
    assert n.value >= 4
    return torch.empty(n.value + 256, dtype=torch.uint8, device=x.device)


def _aligned(ws):
    return (ws.data_ptr() + 255) & ~255


def _check_against_fixture(out, t, m, dtype, name):
    if dtype == torch.float32:
        ok, frac = fp32_close(out, t['out'])
        assert ok, f'{name}: error is {frac:.2f}x the bound'
        return
    r = {k: (None if v is None else v.to(dtype).float()) for k, v in t.items()}
    ref = oracle.best_forward(r['x'], r['offset'], r['mask'], r['weight'], r['bias'], m['stride'],
                              m['padding'], m['dilation'], m['groups'], m['deform_groups'])
    assert rel_l2(out, ref) <= 2e-2, (name, rel_l2(out, ref))


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('name', ['v2_basic', 'v2_s2_d2_dg4_int', 'v2_k5x3_rect', 'v2_c64',
                                  'v2_c128_g2_dg2_s2'])
def test_flat_modulated_entry(name, dtype):
    lib = _lib.load()
    m, t = golden_cases().get(name)
    dev = torch.device('cuda:0')
    cv = lambda v: None if v is None else v.to(dev, dtype).contiguous()
    x, off, msk, w, b = (cv(t[k]) for k in ('x', 'offset', 'mask', 'weight', 'bias'))
    Co, kh, kw = w.shape[0], w.shape[2], w.shape[3]
    out = torch.full(t['out'].shape, float('nan'), device=dev, dtype=dtype)
    elem = _ELEM[dtype]
    ws = _flat_workspace(lib, elem, 1, x, Co, kh, kw, m)
    stream = torch.cuda.current_stream()
    rc = lib.dcn_modulated_deform_conv_forward(
        _vp(x), _vp(w), _vp(b), _vp(off), _vp(msk), _vp(out), elem, x.shape[0], x.shape[1],
        x.shape[2], x.shape[3], Co, kh, kw, m['stride'][0], m['stride'][1], m['padding'][0],
        m['padding'][1], m['dilation'][0], m['dilation'][1], m['groups'], m['deform_groups'],
        int(b is not None), 0, ctypes.c_void_p(_aligned(ws)), ws.numel() - 256,
        ctypes.c_void_p(stream.cuda_stream))
    _lib.check(rc)
    st = ctypes.c_int32(-1)
    _lib.check(lib.dcn_read_status(ctypes.c_void_p(_aligned(ws)), ctypes.c_void_p(stream.cuda_stream),
                                   ctypes.byref(st)))
    assert st.value == 0
    _check_against_fixture(out, t, m, dtype, name)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('name', ['v1_basic', 'v1_g2_dg2_d2', 'v1_k2_nopad', 'v1_c64'])
def test_flat_v1_entry(name, dtype):
    lib = _lib.load()
    m, t = golden_cases().get(name)
    dev = torch.device('cuda:0')
    cv = lambda v: None if v is None else v.to(dev, dtype).contiguous()
    x, off, w = (cv(t[k]) for k in ('x', 'offset', 'weight'))
    Co, kh, kw = w.shape[0], w.shape[2], w.shape[3]
    out = torch.full(t['out'].shape, float('nan'), device=dev, dtype=dtype)
    elem = _ELEM[dtype]
    ws = _flat_workspace(lib, elem, 0, x, Co, kh, kw, m)
    stream = torch.cuda.current_stream()
    # width before height in the scalar arguments, as in the reference's binding
    rc = lib.dcn_deform_conv_forward(
        _vp(x), _vp(w), _vp(off), _vp(out), elem, x.shape[0], x.shape[1], x.shape[2], x.shape[3],
        Co, kw, kh, m['stride'][1], m['stride'][0], m['padding'][1], m['padding'][0],
        m['dilation'][1], m['dilation'][0], m['groups'], m['deform_groups'], x.shape[0], 0,
        ctypes.c_void_p(_aligned(ws)), ws.numel() - 256, ctypes.c_void_p(stream.cuda_stream))
    _lib.check(rc)
    torch.cuda.synchronize()
    _check_against_fixture(out, t, m, dtype, name)


def test_flat_entries_report_errors():
    lib = _lib.load()
    x = torch.zeros(3, 4, 6, 6, device='cuda')
    w = torch.zeros(4, 4, 3, 3, device='cuda')
    off = torch.zeros(3, 18, 6, 6, device='cuda')
    out = torch.zeros(3, 4, 6, 6, device='cuda')
    ws = torch.empty(1 << 20, dtype=torch.uint8, device='cuda')
    null = ctypes.c_void_p(None)
    # im2col_step that does not divide the batch
    rc = lib.dcn_deform_conv_forward(_vp(x), _vp(w), _vp(off), _vp(out), 0, 3, 4, 6, 6, 4, 3, 3, 1, 1,
                                     1, 1, 1, 1, 1, 1, 2, 0, _vp(ws), ws.numel(), null)
    assert rc != 0 and 'im2col_step' in _lib.last_error()
    # with_bias without a bias pointer
    rc = lib.dcn_modulated_deform_conv_forward(_vp(x), _vp(w), null, _vp(off), _vp(off), _vp(out), 0, 3,
                                               4, 6, 6, 4, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, _vp(ws),
                                               ws.numel(), null)
    assert rc != 0 and 'bias' in _lib.last_error()
    # a workspace that is too small
    rc = lib.dcn_modulated_deform_conv_forward(_vp(x), _vp(w), null, _vp(off), _vp(off), _vp(out), 0, 3,
                                               4, 6, 6, 4, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, _vp(ws),
                                               16, null)
    assert rc != 0
    # fp64 is not taken
    n = ctypes.c_size_t(0)
    rc = lib.dcn_forward_workspace_bytes(7, 1, 1, 4, 6, 6, 4, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, ctypes.byref(n))
    assert rc != 0


# ---------------------------------------------------------------------------------------------
# (c) a bounded wait that runs out

def plan_kernel_version(x, w, m):
    p = _lib.DcnFwdParams()
    p.dtype = _ELEM[x.dtype]
    p.N, p.C, p.H, p.W = x.shape
    p.Co, p.kh, p.kw = w.shape[0], w.shape[2], w.shape[3]
    p.stride_h, p.stride_w = m['stride']
    p.pad_h, p.pad_w = m['padding']
    p.dil_h, p.dil_w = m['dilation']
    p.groups, p.deform_groups = m['groups'], m['deform_groups']
    for i, st in enumerate(x.stride()):
        p.in_stride[i] = st
    info = _lib.DcnPlanInfo()
    _lib.check(_lib.load().dcn_fwd_plan(ctypes.byref(p), ctypes.byref(info)))
    return info.kernel_version


def test_a_wait_that_runs_out_reports_its_code_and_leaves_the_gpu_usable():
    """The weight-tile loader is told (debug flag 1) to withhold the last copy of the first tile:
    the tensor-core issuer's wait for that weight stage can never be satisfied.  With the wait limit
    lowered to 5 ms the kernel must give up, record the code of that wait (5: tensor-core issuer
    waiting for a weight stage), release its tensor memory and return; the next forward, with the
    flag cleared, must be correct -- which it could not be if tensor memory had stayed allocated
    (the allocation of the next launch on that SM would spin until its own limit)."""
    lib = _lib.load()
    m, t = golden_cases().get('v2_c64')
    dev = torch.device('cuda:0')
    cv = lambda v: v.to(dev, torch.bfloat16).contiguous()
    x, off, msk, w, b = (cv(t[k]) for k in ('x', 'offset', 'mask', 'weight', 'bias'))
    out = torch.zeros(t['out'].shape, device=dev, dtype=torch.bfloat16)
    assert plan_kernel_version(x, w, m) == 2   # the flag lives in the 16-bit kernel without a tap table
    _ext.set_check_status(False)
    try:
        _lib.check(lib.dcn_debug_configure(5_000_000, 1))
        ws = _ext.forward(x, off, msk, w, b, out, m['stride'], m['padding'], m['dilation'],
                          m['groups'], m['deform_groups'])
        st = ctypes.c_int32(-1)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(lib.dcn_read_status(ctypes.c_void_p(ws.data_ptr()), stream, ctypes.byref(st)))
    finally:
        _lib.check(lib.dcn_debug_configure(0, 0))
        _ext.set_check_status(True)
    assert st.value == 5, f'expected the code of the weight-stage wait (5), got {st.value}'
    torch.cuda.synchronize()          # the context is still usable
    # the same problem again, flag cleared
    out2 = torch.zeros_like(out)
    ws = _ext.forward(x, off, msk, w, b, out2, m['stride'], m['padding'], m['dilation'],
                      m['groups'], m['deform_groups'])
    st = ctypes.c_int32(-1)
    _lib.check(lib.dcn_read_status(ctypes.c_void_p(ws.data_ptr()), stream, ctypes.byref(st)))
    assert st.value == 0
    r = {k: (None if v is None else v.to(torch.bfloat16).float()) for k, v in t.items()}
    ref = oracle.best_forward(r['x'], r['offset'], r['mask'], r['weight'], r['bias'], m['stride'],
                              m['padding'], m['dilation'], m['groups'], m['deform_groups'])
    assert rel_l2(out2, ref) <= 2e-2
    # and a problem whose grid covers every SM (each CTA allocates tensor memory on its SM)
    gen = torch.Generator().manual_seed(11)
    xb = torch.randn(2, 64, 96, 96, generator=gen).to(torch.bfloat16)
    ob = (torch.randn(2, 18, 96, 96, generator=gen) * 2).to(torch.bfloat16)
    mb = torch.sigmoid(torch.randn(2, 9, 96, 96, generator=gen)).to(torch.bfloat16)
    outb = torch.zeros(2, 64, 96, 96, device=dev, dtype=torch.bfloat16)
    ws = _ext.forward(xb.to(dev), ob.to(dev), mb.to(dev), w, b, outb, (1, 1), (1, 1), (1, 1), 1, 1)
    _lib.check(lib.dcn_read_status(ctypes.c_void_p(ws.data_ptr()), stream, ctypes.byref(st)))
    assert st.value == 0
    refb = oracle.best_forward(xb.float(), ob.float(), mb.float(), r['weight'], r['bias'],
                               (1, 1), (1, 1), (1, 1), 1, 1)
    assert rel_l2(outb, refb) <= 2e-2
