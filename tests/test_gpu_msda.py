"""Multi-scale deformable attention on the GPU: the fixtures generated from the reference's own
pure-PyTorch implementation (fp32 outputs and gradients), 16-bit tensors against the CPU checker
on the rounded inputs, the reference tests' flows through the reference's UNCHANGED wrapper file
over this extension, and the layer.

fp32: |out - ref| <= 1e-5 |ref| + 1e-7 (outputs), gradients within 1e-4 of the largest reference
gradient (the atomic adds of grad_value are unordered).  16-bit: relative L2 <= 1e-2.
"""
import os
import sys

import pytest
import torch

from conftest import rel_l2
from mmcv_b200 import _ext
from oracle.msda import msda_forward
from test_msda_oracle import msda_case, msda_case_names

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
import ref_wrappers  # noqa: E402

pytestmark = pytest.mark.gpu


def starts_of(shapes):
    return torch.cat((shapes.new_zeros((1,)), shapes.prod(1).cumsum(0)[:-1]))


@pytest.mark.parametrize('name', msda_case_names())
def test_fp32_fixtures_forward_and_backward(name):
    from mmcv_b200.ops import MultiScaleDeformableAttnFunction
    t = msda_case(name)
    shapes = t['shapes'].cuda()
    v = t['value'].cuda().requires_grad_(True)
    loc = t['loc'].cuda().requires_grad_(True)
    a = t['attn'].cuda().requires_grad_(True)
    out = MultiScaleDeformableAttnFunction.apply(v, shapes, starts_of(shapes), loc, a, 64)
    assert out.shape == t['out'].shape and out.dtype == torch.float32
    assert torch.allclose(out.cpu(), t['out'], rtol=1e-5, atol=1e-7)
    out.backward(t['grad_out'].cuda())
    for got, key in ((v.grad, 'grad_value'), (a.grad, 'grad_attn')):
        ref = t[key]
        assert (got.cpu() - ref).abs().max() <= 1e-4 * ref.abs().max() + 1e-6, key
    # location gradients away from the cell borders (the bilinear surface has a kink there)
    lw = t['loc'][..., 0] * t['shapes'][:, 1].view(1, 1, 1, -1, 1) - 0.5
    lh = t['loc'][..., 1] * t['shapes'][:, 0].view(1, 1, 1, -1, 1) - 0.5
    smooth = ((lw - lw.round()).abs() > 1e-4) & ((lh - lh.round()).abs() > 1e-4)
    d = (loc.grad.cpu() - t['grad_loc']).abs()
    assert (d[smooth] <= 1e-4 * t['grad_loc'].abs().max() + 1e-6).all()


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('name', ['detr_like', 'odd_channels', 'wide_head', 'edges'])
def test_16bit_against_the_checker_on_rounded_inputs(name, dtype):
    t = msda_case(name)
    shapes = t['shapes']
    r = {k: t[k].to(dtype) for k in ('value', 'loc', 'attn', 'grad_out')}
    v = r['value'].cuda().requires_grad_(True)
    loc = r['loc'].cuda().requires_grad_(True)
    a = r['attn'].cuda().requires_grad_(True)
    from mmcv_b200.ops import MultiScaleDeformableAttnFunction
    out = MultiScaleDeformableAttnFunction.apply(v, shapes.cuda(), starts_of(shapes).cuda(), loc, a, 64)
    assert out.dtype == dtype
    v64 = r['value'].double().requires_grad_(True)
    l64 = r['loc'].double().requires_grad_(True)
    a64 = r['attn'].double().requires_grad_(True)
    ref = msda_forward(v64, shapes, l64, a64)
    assert rel_l2(out, ref.detach().float()) <= 1e-2
    out.backward(r['grad_out'].cuda())
    ref.backward(r['grad_out'].double())
    assert v.grad.dtype == dtype and loc.grad.dtype == dtype
    assert rel_l2(v.grad, v64.grad.float()) <= 1e-2
    assert rel_l2(a.grad, a64.grad.float()) <= 1e-2
    assert rel_l2(loc.grad, l64.grad.float()) <= 2e-2


def test_batch_chunks_and_empty_inputs():
    t = msda_case('odd_channels')
    shapes = t['shapes'].cuda()
    args = (t['value'].cuda(), shapes, starts_of(shapes), t['loc'].cuda(), t['attn'].cuda())
    full = _ext.ms_deform_attn_forward(*args, im2col_step=64)
    assert torch.equal(full, _ext.ms_deform_attn_forward(*args, im2col_step=1))
    with pytest.raises(RuntimeError, match='im2col_step'):
        _ext.ms_deform_attn_forward(t['value'].cuda().repeat(3, 1, 1, 1)[:3], shapes, starts_of(shapes),
                                    t['loc'].cuda().repeat(3, 1, 1, 1, 1, 1)[:3],
                                    t['attn'].cuda().repeat(3, 1, 1, 1, 1)[:3], im2col_step=2)
    empty = _ext.ms_deform_attn_forward(args[0], shapes, args[2], args[3][:, :0].contiguous(),
                                        args[4][:, :0].contiguous(), im2col_step=64)
    assert empty.shape == (2, 0, 15)
    # every location outside every map: exact zeros
    far = torch.full_like(args[3], 3.0)
    assert torch.count_nonzero(_ext.ms_deform_attn_forward(args[0], shapes, args[2], far, args[4], 64)) == 0


@pytest.fixture
def ref_msda():
    if ref_wrappers.default_root() is None or not os.path.isfile(
            os.path.join(ref_wrappers.default_root(), 'mmcv/ops/multi_scale_deform_attn.py')):
        pytest.skip('the reference wrapper files are not available (oracle/build_oracle.py copies them)')
    ref_wrappers.load(_ext)
    mod = ref_wrappers.load_msda(_ext)
    assert mod.ext_module is _ext
    yield mod
    ref_wrappers.unload()


def _ref_test_inputs():
    # tests/test_ops/test_ms_deformable_attn.py:199-214
    N, M, D = 1, 2, 2
    Lq, L, P = 2, 2, 2
    shapes = torch.as_tensor([(6, 4), (3, 2)], dtype=torch.long)
    level_start_index = torch.cat((shapes.new_zeros((1,)), shapes.prod(1).cumsum(0)[:-1]))
    S = sum((H * W).item() for H, W in shapes)
    torch.manual_seed(3)
    value = torch.rand(N, S, M, D) * 0.01
    sampling_locations = torch.rand(N, Lq, M, L, P, 2)
    attention_weights = torch.rand(N, Lq, M, L, P) + 1e-5
    attention_weights /= attention_weights.sum(-1, keepdim=True).sum(-2, keepdim=True)
    return value, shapes, level_start_index, sampling_locations, attention_weights


def test_reference_float_flow_over_this_extension(ref_msda):
    # tests/test_ops/test_ms_deformable_attn.py:187-227
    value, shapes, starts, loc, attn = _ref_test_inputs()
    ref = ref_msda.multi_scale_deformable_attn_pytorch(value, shapes, loc, attn).detach().cpu()
    out = ref_msda.MultiScaleDeformableAttnFunction.apply(
        value.cuda(), shapes.cuda(), starts.cuda(), loc.cuda(), attn.cuda(), 2).detach().cpu()
    assert torch.allclose(out, ref, rtol=1e-2, atol=1e-3)
    assert (out - ref).abs().max() < 1e-9
    assert ((out - ref).abs() / ref.abs()).max() < 1e-6


def test_reference_autocast_flow_over_this_extension(ref_msda):
    # tests/test_ops/test_ms_deformable_attn.py:240-288
    value, shapes, starts, loc, attn = _ref_test_inputs()
    ref = ref_msda.multi_scale_deformable_attn_pytorch(value, shapes, loc, attn).detach().cpu()
    with torch.autocast('cuda', enabled=True):
        out = ref_msda.MultiScaleDeformableAttnFunction.apply(
            value.cuda().type(torch.float), shapes.cuda(), starts.cuda(), loc.cuda(), attn.cuda(),
            2).detach().cpu()
    assert (out - ref).abs().max() < 1e-9 and ((out - ref).abs() / ref.abs()).max() < 1e-6
    with torch.autocast('cuda', enabled=True):
        out = ref_msda.MultiScaleDeformableAttnFunction.apply(
            value.cuda().type(torch.half), shapes.cuda(), starts.cuda(), loc.cuda(), attn.cuda(),
            2).detach().cpu()
    assert torch.allclose(out, ref.half(), rtol=1e-2, atol=1e-3)
    assert (out - ref).abs().max() < 1e-5 and ((out - ref).abs() / ref.abs()).max() < 1e-2


def test_reference_layer_over_this_extension_matches_its_cpu_path(ref_msda):
    # the reference's layer: its CUDA branch (this extension) against its own CPU branch
    # (tests/test_ops/test_ms_deformable_attn.py:51-99 builds the same layers)
    torch.manual_seed(0)
    layer = ref_msda.MultiScaleDeformableAttention(embed_dims=64, num_levels=2, num_heads=4,
                                                   num_points=3, dropout=0.0)
    layer.init_weights()
    for p in (layer.sampling_offsets.weight, layer.attention_weights.weight):
        p.data.normal_(0, 0.3)
    shapes = torch.tensor([[6, 5], [3, 2]])
    starts = torch.tensor([0, 30])
    q = torch.rand(7, 2, 64)
    kv = torch.rand(36, 2, 64)
    refp = torch.rand(2, 7, 2, 2)
    cpu = layer(q, kv, kv, reference_points=refp, spatial_shapes=shapes, level_start_index=starts)
    layer.cuda()
    gpu = layer(q.cuda(), kv.cuda(), kv.cuda(), reference_points=refp.cuda(),
                spatial_shapes=shapes.cuda(), level_start_index=starts.cuda())
    assert torch.allclose(gpu.cpu(), cpu, rtol=1e-4, atol=1e-5)


def test_layer_of_this_package_matches_the_checker():
    from mmcv_b200.ops import MultiScaleDeformableAttention
    torch.manual_seed(1)
    layer = MultiScaleDeformableAttention(embed_dims=64, num_levels=2, num_heads=4, num_points=3,
                                          dropout=0.0, batch_first=True)
    for p in (layer.sampling_offsets.weight, layer.attention_weights.weight):
        p.data.normal_(0, 0.3)
    shapes = torch.tensor([[6, 5], [3, 2]])
    starts = torch.tensor([0, 30])
    q = torch.rand(2, 7, 64)
    kv = torch.rand(2, 36, 64)
    refp = torch.rand(2, 7, 2, 4)
    layer.cuda()
    q_d = q.cuda().requires_grad_(True)
    gpu = layer(q_d, value=kv.cuda(), reference_points=refp.cuda(), spatial_shapes=shapes.cuda(),
                level_start_index=starts.cuda())
    gpu.sum().backward()
    assert q_d.grad is not None and torch.isfinite(q_d.grad).all()
    # the same arithmetic on the CPU with the checker in place of the kernel
    layer.cpu()
    with torch.no_grad():
        value = layer.value_proj(kv).view(2, 36, 4, -1)
        off = layer.sampling_offsets(q).view(2, 7, 4, 2, 3, 2)
        aw = layer.attention_weights(q).view(2, 7, 4, 6).softmax(-1).view(2, 7, 4, 2, 3)
        loc = refp[:, :, None, :, None, :2] + off / 3 * refp[:, :, None, :, None, 2:] * 0.5
        ref = layer.output_proj(msda_forward(value, shapes, loc, aw)) + q
    assert torch.allclose(gpu.detach().cpu(), ref, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('D', [48, 24, 16])
def test_head_widths_that_take_the_other_reduction_paths(D, dtype):
    """16-byte vectors with a number of lanes per head that is not a power of two (D = 48: 12 fp32
    or 6 bf16 lanes, atomic adds for the location / weight gradients), and small heads."""
    from mmcv_b200.ops import MultiScaleDeformableAttnFunction
    gen = torch.Generator().manual_seed(D)
    B, M, Q, P = 2, 3, 41, 2
    shapes = torch.tensor([[9, 7], [4, 5], [2, 2]])
    S = int(shapes.prod(1).sum())
    value = torch.rand(B, S, M, D, generator=gen).to(dtype)
    loc = (torch.rand(B, Q, M, 3, P, 2, generator=gen) * 1.3 - 0.15).to(dtype)
    attn = torch.rand(B, Q, M, 3 * P, generator=gen).softmax(-1).view(B, Q, M, 3, P).to(dtype)
    gout = torch.randn(B, Q, M * D, generator=gen).to(dtype)
    v = value.cuda().requires_grad_(True)
    l = loc.cuda().requires_grad_(True)
    a = attn.cuda().requires_grad_(True)
    out = MultiScaleDeformableAttnFunction.apply(v, shapes.cuda(), starts_of(shapes).cuda(), l, a, 64)
    out.backward(gout.cuda())
    v64 = value.double().requires_grad_(True)
    l64 = loc.double().requires_grad_(True)
    a64 = attn.double().requires_grad_(True)
    ref = msda_forward(v64, shapes, l64, a64)
    ref.backward(gout.double())
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_l2(out, ref.detach().float()) <= tol
    assert rel_l2(v.grad, v64.grad.float()) <= tol
    assert rel_l2(a.grad, a64.grad.float()) <= tol
    assert rel_l2(l.grad, l64.grad.float()) <= 2 * tol
