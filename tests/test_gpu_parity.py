"""Parity of the CUDA path with the CPU checkers, through the C ABI (needs a B200).

fp32: max|out-ref| <= 1e-4*max|ref| + 1e-5.  bf16: ||out-ref||2/||ref||2 <= 2e-2 with the
checker run in fp32 on the bf16-rounded inputs (the reference has no bf16 kernel).
"""
import ctypes

import pytest
import torch

import oracle
from conftest import fp32_close, golden_case_names, golden_cases, rel_l2
from mmcv_b200 import _ext, _lib

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2


def plan_path(x, w, m, dtype, math=_lib.MATH_AUTO):
    lib = _lib.load()
    p = _lib.DcnFwdParams()
    p.dtype = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16,
               torch.float16: _lib.DTYPE_F16}[dtype]
    p.math_mode = math
    p.N, p.C, p.H, p.W = x.shape
    p.Co, p.kh, p.kw = w.shape[0], w.shape[2], w.shape[3]
    p.stride_h, p.stride_w = m['stride']
    p.pad_h, p.pad_w = m['padding']
    p.dil_h, p.dil_w = m['dilation']
    p.groups, p.deform_groups = m['groups'], m['deform_groups']
    for i, s in enumerate(x.contiguous().stride()):
        p.in_stride[i] = s
    info = _lib.DcnPlanInfo()
    _lib.check(lib.dcn_fwd_plan(ctypes.byref(p), ctypes.byref(info)))
    return info


def run_cuda(t, m, dtype, math=None, channels_last=False):
    dev = torch.device('cuda:0')
    cv = lambda v: None if v is None else v.to(dev, dtype).contiguous()
    x, off, msk, w, b = (cv(t[k]) for k in ('x', 'offset', 'mask', 'weight', 'bias'))
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    N, Co = x.shape[0], w.shape[0]
    Ho = oracle.out_size(x.shape[2], m['padding'][0], m['dilation'][0], w.shape[2], m['stride'][0])
    Wo = oracle.out_size(x.shape[3], m['padding'][1], m['dilation'][1], w.shape[3], m['stride'][1])
    out = torch.full((N, Co, Ho, Wo), float('nan'), device=dev, dtype=dtype)
    ws = _ext.forward(x, off, msk, w, b, out, m['stride'], m['padding'], m['dilation'],
                      m['groups'], m['deform_groups'], math_mode=math)
    st = ctypes.c_int32(-1)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(_lib.load().dcn_read_status(ctypes.c_void_p(ws.data_ptr()), stream,
                                           ctypes.byref(st)))
    assert st.value == 0, f'device status {st.value}'
    return out


def rounded(t, dtype):
    return {k: (None if v is None else v.to(dtype).float()) for k, v in t.items()}


@pytest.mark.parametrize('math', [_lib.MATH_FFMA, _lib.MATH_AUTO])
@pytest.mark.parametrize('name', golden_case_names())
def test_golden_fp32(name, math):
    m, t = golden_cases().get(name)
    out = run_cuda(t, m, torch.float32, math=math)
    ok, frac = fp32_close(out, t['out'])
    assert ok, f'{name}: error is {frac:.2f}x the bound'


@pytest.mark.parametrize('name', golden_case_names())
def test_golden_bf16(name):
    m, t = golden_cases().get(name)
    r = rounded(t, torch.bfloat16)
    ref = oracle.best_forward(r['x'], r['offset'], r['mask'], r['weight'], r['bias'],
                              m['stride'], m['padding'], m['dilation'], m['groups'],
                              m['deform_groups'])
    out = run_cuda(t, m, torch.bfloat16)
    finite = torch.isfinite(ref)
    assert torch.equal(torch.isfinite(out.float().cpu()), finite)
    assert rel_l2(out.float().cpu()[finite], ref[finite]) <= BF16_TOL


@pytest.mark.parametrize('name', golden_case_names())
def test_golden_fp16(name):
    # fp16 tensors (the reference's half coverage): checker in fp32 on the fp16-rounded inputs;
    # fp16 keeps 3 more mantissa bits than bf16, so the bound is tighter
    m, t = golden_cases().get(name)
    r = rounded(t, torch.float16)
    ref = oracle.best_forward(r['x'], r['offset'], r['mask'], r['weight'], r['bias'],
                              m['stride'], m['padding'], m['dilation'], m['groups'],
                              m['deform_groups'])
    out = run_cuda(t, m, torch.float16)
    finite = torch.isfinite(ref)
    assert torch.equal(torch.isfinite(out.float().cpu()), finite)
    assert rel_l2(out.float().cpu()[finite], ref[finite]) <= 4e-3


def test_config3_fp16_on_tensor_cores():
    m, t = synth(4, 512, 64, 64, 512, 3, 2, 2, 2, 1, 4, 8.0, True, True, int_frac=0.05,
                 mask_sigma=2.0)
    assert plan_path(t['x'], t['weight'], m, torch.float16).path == _lib.PATH_TCGEN05
    out = run_cuda(t, m, torch.float16).float().cpu()
    r = rounded(t, torch.float16)
    ref = oracle.best_forward(r['x'], r['offset'], r['mask'], r['weight'], r['bias'],
                              m['stride'], m['padding'], m['dilation'], m['groups'],
                              m['deform_groups'])
    assert rel_l2(out, ref) <= 4e-3


@pytest.mark.parametrize('name', ['v2_c64', 'v2_c128_co40_dg4', 'v2_c128_g2_dg2_s2', 'v1_c64'])
@pytest.mark.parametrize('channels_last', [False, True])
def test_tensor_core_path_is_taken_and_matches(name, channels_last):
    m, t = golden_cases().get(name)
    info = plan_path(t['x'], t['weight'], m, torch.bfloat16)
    assert info.path == _lib.PATH_TCGEN05
    r = rounded(t, torch.bfloat16)
    ref = oracle.best_forward(r['x'], r['offset'], r['mask'], r['weight'], r['bias'],
                              m['stride'], m['padding'], m['dilation'], m['groups'],
                              m['deform_groups'])
    out = run_cuda(t, m, torch.bfloat16, channels_last=channels_last)
    assert rel_l2(out.float().cpu(), ref) <= BF16_TOL
    # the SIMT kernel on the same bf16 tensors is the on-device cross-check
    simt = run_cuda(t, m, torch.bfloat16, math=_lib.MATH_FFMA)
    assert rel_l2(out.float().cpu(), simt.float().cpu()) <= BF16_TOL


def test_partly_filled_channel_chunk():
    # 96 channels in two conv groups of 48: the 64-channel chunk of each group is 3/4 full
    m, t = synth(2, 96, 17, 19, 80, 3, 1, 1, 1, 2, 4, 2.0, True, True, seed=5)
    assert plan_path(t['x'], t['weight'], m, torch.bfloat16).path == _lib.PATH_TCGEN05
    check_against_oracle(m, t, torch.bfloat16)
    assert plan_path(t['x'], t['weight'], m, torch.float32).path == _lib.PATH_TCGEN05
    check_against_oracle(m, t, torch.float32)


@pytest.mark.parametrize('name', ['v2_c64', 'v2_c128_co40_dg4'])
def test_fp32_tensors_with_bf16_contraction(name):
    m, t = golden_cases().get(name)
    out = run_cuda(t, m, torch.float32, math=_lib.MATH_BF16)
    assert rel_l2(out.cpu(), t['out']) <= BF16_TOL


@pytest.mark.parametrize('name', ['v2_c64', 'v2_c128_co40_dg4', 'v2_c128_g2_dg2_s2', 'v1_c64'])
def test_fp32_tf32x3_contraction_meets_fp32_bound(name):
    # fp32 tensors, contraction on the tensor cores as three TF32 products (hi*hi + lo*hi +
    # hi*lo): must meet the same fp32 bound as the FFMA kernel
    m, t = golden_cases().get(name)
    info = plan_path(t['x'], t['weight'], m, torch.float32, math=_lib.MATH_TF32X3)
    assert info.path == _lib.PATH_TCGEN05 and info.tile_k == 32
    out = run_cuda(t, m, torch.float32, math=_lib.MATH_TF32X3)
    ok, frac = fp32_close(out, t['out'])
    assert ok, f'{name}: error is {frac:.3f}x the bound'
    cl = run_cuda(t, m, torch.float32, math=_lib.MATH_TF32X3, channels_last=True)
    assert torch.equal(cl, out)


def test_tf32x3_falls_back_to_ffma_on_odd_shapes():
    m, t = golden_cases().get('v2_k1')             # 6 channels: not a tensor-core shape
    info = plan_path(t['x'], t['weight'], m, torch.float32, math=_lib.MATH_TF32X3)
    assert info.path == _lib.PATH_SIMT_DIRECT
    out = run_cuda(t, m, torch.float32, math=_lib.MATH_TF32X3)
    ok, frac = fp32_close(out, t['out'])
    assert ok, frac


def synth(N, C, H, W, Co, k, s, p, d, g, dg, sigma, mask, bias, seed=0, int_frac=0.0,
          mask_sigma=1.0):
    gen = torch.Generator().manual_seed(seed)
    Ho, Wo = oracle.out_size(H, p, d, k, s), oracle.out_size(W, p, d, k, s)
    x = torch.randn(N, C, H, W, generator=gen)
    off = torch.randn(N, dg * 2 * k * k, Ho, Wo, generator=gen) * sigma
    if int_frac:
        sel = torch.rand(off.shape, generator=gen) < int_frac
        off = torch.where(sel, off.round(), off)
    msk = torch.sigmoid(torch.randn(N, dg * k * k, Ho, Wo, generator=gen) * mask_sigma) if mask else None
    w = torch.empty(Co, C // g, k, k)
    bound = (6.0 / (C // g * k * k)) ** 0.5
    w.copy_((torch.rand(w.shape, generator=gen) * 2 - 1) * bound)
    b = (torch.rand(Co, generator=gen) * 0.2 - 0.1) if bias else None
    t = dict(x=x, offset=off, mask=msk, weight=w, bias=b)
    m = dict(stride=(s, s), padding=(p, p), dilation=(d, d), groups=g, deform_groups=dg)
    return m, t


def check_against_oracle(m, t, dtype, samples=None, math=None):
    out = run_cuda(t, m, dtype, math=math).float().cpu()
    idx = list(range(t['x'].shape[0])) if samples is None else samples
    sub = {k: (v if (v is None or k in ('weight', 'bias')) else v[idx]) for k, v in t.items()}
    if dtype == torch.bfloat16:
        sub = rounded(sub, torch.bfloat16)
    ref = oracle.best_forward(sub['x'], sub['offset'], sub['mask'], sub['weight'], sub['bias'],
                              m['stride'], m['padding'], m['dilation'], m['groups'],
                              m['deform_groups'])
    if dtype == torch.float32:
        ok, frac = fp32_close(out[idx], ref)
        assert ok, f'error is {frac:.2f}x the bound'
    else:
        assert rel_l2(out[idx], ref) <= BF16_TOL
    return out


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_config1_full(dtype):
    m, t = synth(2, 64, 56, 56, 64, 3, 1, 1, 1, 1, 1, 2.0, True, True)
    check_against_oracle(m, t, dtype)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_config3_full_edge_offsets(dtype):
    m, t = synth(4, 512, 64, 64, 512, 3, 2, 2, 2, 1, 4, 8.0, True, True, int_frac=0.05,
                 mask_sigma=2.0)
    check_against_oracle(m, t, dtype)


def test_config1_and_config3_fp32_tf32x3():
    m, t = synth(2, 64, 56, 56, 64, 3, 1, 1, 1, 1, 1, 2.0, True, True)
    check_against_oracle(m, t, torch.float32, math=_lib.MATH_TF32X3)
    m, t = synth(4, 512, 64, 64, 512, 3, 2, 2, 2, 1, 4, 8.0, True, True, int_frac=0.05,
                 mask_sigma=2.0)
    check_against_oracle(m, t, torch.float32, math=_lib.MATH_TF32X3)


def test_config2_v1_fp32_tf32x3_two_samples():
    m, t = synth(8, 256, 100, 168, 256, 3, 1, 1, 1, 1, 1, 1.5, False, False)
    check_against_oracle(m, t, torch.float32, samples=[0, 7], math=_lib.MATH_TF32X3)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_tiled_ffma_kernel_config1_and_odd_channels(dtype):
    # the FFMA mode on a tensor-core shape, and a channel count only the SIMT kernels take
    m, t = synth(2, 64, 56, 56, 64, 3, 1, 1, 1, 1, 1, 2.0, True, True)
    assert plan_path(t['x'], t['weight'], m, dtype, math=_lib.MATH_FFMA).path == _lib.PATH_SIMT_TILED
    check_against_oracle(m, t, dtype, math=_lib.MATH_FFMA)
    m, t = synth(2, 36, 23, 31, 70, 3, 2, 1, 1, 2, 3, 3.0, True, True, seed=9)
    assert plan_path(t['x'], t['weight'], m, dtype).path == _lib.PATH_SIMT_TILED
    check_against_oracle(m, t, dtype)
    m, t = synth(1, 12, 30, 29, 10, 5, 1, 2, 1, 1, 1, 2.0, False, False, seed=10)   # 5x5, v1
    check_against_oracle(m, t, dtype)


def test_config2_v1_bf16_two_samples():
    m, t = synth(8, 256, 100, 168, 256, 3, 1, 1, 1, 1, 1, 1.5, False, False)
    check_against_oracle(m, t, torch.bfloat16, samples=[0, 7])


def test_config5_slice_and_batch_independence():
    # A slice of the large-batch workload: 6 samples; first/last checked against the
    # checker, and every sample must equal what the same sample gives when run alone.
    m, t = synth(6, 256, 128, 128, 256, 3, 1, 1, 1, 1, 8, 2.0, True, True)
    full = check_against_oracle(m, t, torch.bfloat16, samples=[0, 5])
    for n in (0, 3, 5):
        one = {k: (v if (v is None or k in ('weight', 'bias')) else v[n:n + 1]) for k, v in t.items()}
        alone = run_cuda(one, m, torch.bfloat16).float().cpu()
        assert torch.equal(alone[0], full[n])


def test_linearity_in_input_and_weight():
    m, t = synth(2, 128, 40, 36, 96, 3, 1, 1, 1, 1, 2, 2.0, True, False, seed=3)
    a = run_cuda(t, m, torch.bfloat16).float()
    t2 = dict(t, x=t['x'] * 2)            # exact in bf16
    b = run_cuda(t2, m, torch.bfloat16).float()
    assert rel_l2(b.cpu(), (2 * a).cpu()) <= 1e-2
    t3 = dict(t, mask=torch.zeros_like(t['mask']))
    z = run_cuda(t3, m, torch.bfloat16).float()
    assert torch.count_nonzero(z) == 0    # zero modulation => exactly zero without bias


def test_empty_batch():
    m, t = synth(1, 64, 8, 8, 64, 3, 1, 1, 1, 1, 1, 1.0, True, True)
    t = {k: (v if (v is None or k in ('weight', 'bias')) else v[:0]) for k, v in t.items()}
    out = run_cuda(t, m, torch.bfloat16)
    assert out.shape == (0, 64, 8, 8)
