"""The layer classes and functions under the reference's names, on the GPU."""
import numpy as np
import pytest
import torch

import oracle
from conftest import fp32_close, golden_cases, rel_l2

pytestmark = pytest.mark.gpu


def test_reference_known_answer_v2_pack(kat):
    # the reference's own DCNv2 test construction (its test file, lines 51-85), forward part
    from mmcv_b200.ops import ModulatedDeformConv2dPack
    x = torch.tensor(kat['v2_input'], device='cuda')
    dcn = ModulatedDeformConv2dPack(1, 1, kernel_size=(2, 2), stride=1, padding=1,
                                    deform_groups=1, bias=False).cuda()
    dcn.weight.data.fill_(1.)
    y = dcn(x)
    assert np.allclose(y.detach().cpu().numpy(), kat['v2_expected'], 1e-2)
    assert np.allclose(y.detach().cpu().numpy(), kat['v2_ref_out'], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize('batch,step', [(10, 2), (1, 2)])
def test_reference_known_answer_v1_pack(kat, batch, step):
    from mmcv_b200.ops import DeformConv2dPack
    x = torch.tensor(np.repeat(kat['v1_input'], batch, axis=0), device='cuda')
    m = DeformConv2dPack(in_channels=1, out_channels=1, kernel_size=2, stride=1, padding=0,
                         im2col_step=step)
    m.conv_offset.weight.data = torch.tensor(kat['v1_offset_weight'])
    m.conv_offset.bias.data = torch.tensor(kat['v1_offset_bias'])
    m.weight.data = torch.tensor(kat['v1_deform_weight'])
    m.cuda()
    y = m(x).detach().cpu().numpy()
    assert np.allclose(y, np.repeat(kat['v1_expected'], batch, axis=0), 1e-3)


def test_v1_batch_not_divisible_by_step():
    from mmcv_b200.ops import DeformConv2dPack
    m = DeformConv2dPack(1, 1, 2, im2col_step=3).cuda()
    with pytest.raises(AssertionError, match='batch size must be divisible by im2col_step'):
        m(torch.zeros(10, 1, 3, 3, device='cuda'))


def test_functional_v2_matches_fixture():
    from mmcv_b200.ops import modulated_deform_conv2d
    m, t = golden_cases().get('v2_s2_d2_dg4_int')
    c = lambda v: None if v is None else v.cuda()
    y = modulated_deform_conv2d(c(t['x']), c(t['offset']), c(t['mask']), c(t['weight']),
                                c(t['bias']), m['stride'], m['padding'], m['dilation'],
                                m['groups'], m['deform_groups'])
    ok, frac = fp32_close(y, t['out'])
    assert ok, frac


def test_functional_v1_small_input_is_padded():
    from mmcv_b200.ops import DeformConv2d
    torch.manual_seed(0)
    layer = DeformConv2d(2, 3, 3, padding=1).cuda()
    x = torch.randn(1, 2, 2, 2, device='cuda')        # smaller than the 3x3 kernel
    off = torch.randn(1, 18, 2, 2, device='cuda') * 0.5
    y = layer(x, off)
    assert y.shape == (1, 3, 2, 2)
    import torch.nn.functional as F
    xp, op = F.pad(x, (0, 1, 0, 1)).cpu(), F.pad(off, (0, 1, 0, 1)).cpu()
    ref = oracle.best_forward(xp, op, None, layer.weight.detach().cpu(), None, 1, 1, 1, 1, 1)
    ok, frac = fp32_close(y, ref[:, :, :2, :2])
    assert ok, frac


def test_reference_half_test_flow_under_autocast(kat):
    # the reference's AMP test (its test file, lines 87-128): fp32 module, autocast to half,
    # forward and backward against the same vectors at its 1e-2 tolerance
    from mmcv_b200.ops import ModulatedDeformConv2dPack
    for in_dtype in (torch.float, torch.half):
        x = torch.tensor(kat['v2_input'], device='cuda').type(in_dtype)
        x.requires_grad = True
        dcn = ModulatedDeformConv2dPack(1, 1, kernel_size=(2, 2), stride=1, padding=1,
                                        deform_groups=1, bias=False).cuda()
        dcn.weight.data.fill_(1.)
        with torch.autocast('cuda', dtype=torch.half):
            out = dcn(x)
            out.sum().backward()
        assert out.dtype == torch.half
        c = lambda v: v.detach().float().cpu().numpy()
        assert np.allclose(c(out), kat['v2_expected'], 1e-2)
        assert np.allclose(c(x.grad), kat['v2_input_grad'], 1e-2)
        assert np.allclose(c(dcn.weight.grad), kat['v2_dcn_w_grad'], 1e-2)
        assert np.allclose(c(dcn.conv_offset.weight.grad), kat['v2_dcn_offset_w_grad'], 1e-2)
        assert np.allclose(c(dcn.conv_offset.bias.grad), kat['v2_dcn_offset_b_grad'], 1e-2)


def test_autocast_dtype_follows_offset():
    from mmcv_b200.ops import ModulatedDeformConv2dPack
    torch.manual_seed(1)
    dcn = ModulatedDeformConv2dPack(64, 64, 3, padding=1).cuda()
    dcn.conv_offset.weight.data.normal_(0, 0.01)
    x = torch.randn(2, 64, 20, 20, device='cuda')
    with torch.autocast('cuda', dtype=torch.bfloat16):
        y = dcn(x)
    assert y.dtype == torch.bfloat16
    y32 = dcn(x)
    assert y32.dtype == torch.float32
    assert rel_l2(y.float().cpu(), y32.detach().cpu()) < 5e-2


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_offset_branch_on_the_same_kernel(dtype):
    # ordinary convolution through the implicit-GEMM kernel (zero offsets, unit mask),
    # sigmoid fused on the mask third; checked against F.conv2d in fp32 on the same inputs
    import torch.nn.functional as F
    from mmcv_b200 import _ext
    torch.manual_seed(0)
    x = torch.relu(torch.randn(2, 128, 21, 19)).to(dtype)
    w = (torch.randn(27, 128, 3, 3) * 0.01).to(dtype)
    b = (torch.randn(27) * 0.1).to(dtype)
    out = _ext.conv_offset_forward(x.cuda(), w.cuda(), b.cuda(), (1, 1), (1, 1), (1, 1),
                                   sigmoid_from=18).float().cpu()
    ref = F.conv2d(x.float(), w.float(), b.float(), 1, 1)
    ref = torch.cat([ref[:, :18], torch.sigmoid(ref[:, 18:])], 1)
    if dtype == torch.float32:
        ok, frac = fp32_close(out, ref)
        assert ok, frac
    else:
        assert rel_l2(out, ref) <= 2e-2


@pytest.mark.parametrize('branch_mode', ['library', 'kernel'])
def test_pack_layers_inference_path(branch_mode, monkeypatch):
    # inference path of the Pack layers: the offset branch (library convolution by default, or
    # this library's kernel with zero offsets and a fused sigmoid) and the deformable kernel
    # read one channels-last copy of the input.  The branch is checked against F.conv2d; the
    # layer output against the CPU checker fed the branch's own (bf16) offsets and mask, which
    # isolates the sampling kernel from branch rounding.
    import torch.nn.functional as F
    from mmcv_b200 import _ext
    from mmcv_b200.ops import DeformConv2dPack, ModulatedDeformConv2dPack
    from mmcv_b200.ops import modulated_deform_conv as mdc
    monkeypatch.setattr(mdc, 'OFFSET_BRANCH', branch_mode)
    torch.manual_seed(0)
    for cls, dg in ((ModulatedDeformConv2dPack, 2), (DeformConv2dPack, 1)):
        layer = cls(64, 96, 3, padding=1, deform_groups=dg).cuda().to(torch.bfloat16)
        layer.conv_offset.weight.data.normal_(0, 0.02)
        layer.conv_offset.bias.data.normal_(0, 0.1)
        x = torch.relu(torch.randn(2, 64, 30, 26, device='cuda')).to(torch.bfloat16)
        modulated = cls is ModulatedDeformConv2dPack
        k = layer.conv_offset.out_channels // 3 * 2 if modulated else None
        with torch.no_grad():
            got = layer(x).float().cpu()
            if branch_mode == 'kernel':
                branch = _ext.conv_offset_forward(x, layer.conv_offset.weight,
                                                  layer.conv_offset.bias, (1, 1), (1, 1), (1, 1),
                                                  sigmoid_from=k).float().cpu()
            else:
                off_, msk_ = mdc.library_offset_branch(mdc.shared_layout(x), layer.conv_offset,
                                                       torch.bfloat16, k)
                assert off_.is_contiguous() and (msk_ is None or msk_.is_contiguous())
                branch = (torch.cat([off_, msk_], 1) if modulated else off_).float().cpu()
        o = F.conv2d(x.float().cpu(), layer.conv_offset.weight.float().cpu(),
                     layer.conv_offset.bias.float().cpu(), 1, 1)
        if modulated:
            o = torch.cat([o[:, :k], torch.sigmoid(o[:, k:])], 1)
        assert rel_l2(branch, o) <= 2e-2
        off = branch[:, :k] if modulated else branch
        msk = branch[:, k:] if modulated else None
        bias = layer.bias.float().cpu() if modulated else None
        ref = oracle.best_forward(x.float().cpu(), off.contiguous(),
                                  None if msk is None else msk.contiguous(),
                                  layer.weight.float().cpu(), bias, 1, 1, 1, 1, dg)
        assert rel_l2(got, ref) <= 2e-2


def test_forward_is_capturable_in_a_cuda_graph():
    # the C ABI neither allocates nor synchronises: a forward with a caller-held workspace can
    # be captured once and replayed on new input contents
    import ctypes
    from mmcv_b200 import _lib
    from test_zz_no_alloc import _params
    lib = _lib.load()
    dev = torch.device('cuda:0')
    m, t = golden_cases().get('v2_c64')
    t = {k: (None if v is None else v.to(dev, torch.bfloat16).contiguous())
         for k, v in t.items() if k in ('x', 'offset', 'mask', 'weight', 'bias')}
    out = torch.zeros(1, 64, 12, 12, device=dev, dtype=torch.bfloat16)
    p = _params(t, m, out, 0)
    n = ctypes.c_size_t(0)
    _lib.check(lib.dcn_fwd_workspace_bytes(ctypes.byref(p), ctypes.byref(n)))
    ws = torch.empty(n.value, dtype=torch.uint8, device=dev)
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        sptr = ctypes.c_void_p(side.cuda_stream)
        _lib.check(lib.dcn_fwd(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), n.value, sptr))
        side.synchronize()
        eager = out.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            _lib.check(lib.dcn_fwd(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), n.value,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        out.zero_()
        graph.replay()
        side.synchronize()
        assert torch.equal(out, eager)
        t['x'].mul_(2)                  # new input contents, same buffers
        graph.replay()
        side.synchronize()
        replayed = out.clone()
        _lib.check(lib.dcn_fwd(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), n.value, sptr))
        side.synchronize()
    assert not torch.equal(replayed, eager)
    assert torch.equal(replayed, out)   # replay on new contents == eager run on them


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_frozen_weights_reuse_the_weight_image(dtype):
    # inside frozen_weights() the weight re-layout runs once per layer; results are the same
    # bits as without it, and leaving the block drops the cached copies
    import mmcv_b200
    from mmcv_b200 import _ext
    from mmcv_b200.ops import ModulatedDeformConv2dPack
    torch.manual_seed(5)
    layer = ModulatedDeformConv2dPack(64, 64, 3, padding=1, deform_groups=2).cuda()
    layer.conv_offset.weight.data.normal_(0, 0.05)
    x = torch.randn(2, 64, 24, 40, device='cuda', dtype=dtype)
    with torch.no_grad(), torch.autocast('cuda', dtype=dtype, enabled=dtype != torch.float32):
        want = layer(x)
        with mmcv_b200.frozen_weights():
            first = layer(x)
            cached = len(_ext._frozen.images)
            second = layer(x)
            # the layer's own weights; for fp32 tensors also those of the offset branch, which then
            # runs on the same kernel (for 16-bit tensors the branch is the tensor-map convolution,
            # whose small weight image is rebuilt per call)
            expect = 1 if dtype == torch.bfloat16 else 2
            assert cached == expect and len(_ext._frozen.images) == expect
        assert _ext._frozen is None
        assert torch.equal(first, want) and torch.equal(second, want)
        layer.weight.data.mul_(2)
        assert not torch.equal(layer(x), want)


def test_weight_image_through_the_c_abi():
    import ctypes
    from mmcv_b200 import _lib
    lib = _lib.load()
    torch.manual_seed(6)
    N, C, H, W, Co = 2, 32, 20, 20, 48
    x = torch.randn(N, C, H, W, device='cuda', dtype=torch.bfloat16)
    w = torch.randn(Co, C, 3, 3, device='cuda', dtype=torch.bfloat16) * 0.1
    off = torch.randn(N, 18, H, W, device='cuda', dtype=torch.bfloat16)
    msk = torch.rand(N, 9, H, W, device='cuda', dtype=torch.bfloat16)
    outs = [torch.empty(N, Co, H, W, device='cuda', dtype=torch.bfloat16) for _ in range(2)]
    p = _lib.DcnFwdParams()
    p.input, p.offset, p.mask, p.weight = x.data_ptr(), off.data_ptr(), msk.data_ptr(), w.data_ptr()
    p.dtype, p.math_mode = _lib.DTYPE_BF16, _lib.MATH_AUTO
    p.N, p.C, p.H, p.W, p.Co, p.kh, p.kw = N, C, H, W, Co, 3, 3
    p.stride_h = p.stride_w = p.pad_h = p.pad_w = p.dil_h = p.dil_w = 1
    p.groups = p.deform_groups = 1
    for i, s in enumerate(x.stride()):
        p.in_stride[i] = s
    nws, nimg = ctypes.c_size_t(0), ctypes.c_size_t(0)
    _lib.check(lib.dcn_fwd_workspace_bytes(ctypes.byref(p), ctypes.byref(nws)))
    _lib.check(lib.dcn_weight_image_bytes(ctypes.byref(p), ctypes.byref(nimg)))
    assert nimg.value > 0
    ws = torch.empty(nws.value, dtype=torch.uint8, device='cuda')
    image = torch.empty(nimg.value, dtype=torch.uint8, device='cuda')
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p.output = outs[0].data_ptr()
    _lib.check(lib.dcn_fwd(ctypes.byref(p), ws.data_ptr(), nws.value, stream))
    _lib.check(lib.dcn_prepare_weights(ctypes.byref(p), image.data_ptr(), nimg.value, stream))
    info = _lib.DcnPlanInfo()
    _lib.check(lib.dcn_fwd_plan(ctypes.byref(p), ctypes.byref(info)))
    p.output, p.weight_image, p.weight_image_bytes = outs[1].data_ptr(), image.data_ptr(), nimg.value
    info2 = _lib.DcnPlanInfo()
    _lib.check(lib.dcn_fwd_plan(ctypes.byref(p), ctypes.byref(info2)))
    assert info2.launches == info.launches - 1
    _lib.check(lib.dcn_fwd(ctypes.byref(p), ws.data_ptr(), nws.value, stream))
    assert torch.equal(outs[0], outs[1])
    p.weight_image_bytes = nimg.value - 16
    assert lib.dcn_fwd(ctypes.byref(p), ws.data_ptr(), nws.value, stream) == -1   # DCN_ERR_ARG


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('shape', [(2, 64, 16, 24), (3, 72, 9, 8), (1, 20, 7, 5), (2, 130, 6, 6),
                                   (2, 8, 4, 2)])
def test_channels_last_copy_is_exact(dtype, shape):
    # the layout kernel (tiled for contiguous planes, element-wise otherwise) moves bits only
    from mmcv_b200 import _ext
    torch.manual_seed(3)
    x = torch.randn(*shape, device='cuda').to(dtype)
    got = _ext.to_channels_last(x)
    assert got.is_contiguous(memory_format=torch.channels_last)
    assert torch.equal(got, x)
    # a strided view (channel slice of a wider tensor) and a channels-last input
    wide = torch.randn(shape[0], shape[1] + 8, shape[2], shape[3], device='cuda').to(dtype)
    view = wide[:, 8:]
    assert torch.equal(_ext.to_channels_last(view), view)
    assert _ext.to_channels_last(got) is got


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('channels_last', [True, False])
def test_offsets_and_mask_logits_read_from_the_branch_output(dtype, channels_last):
    # the kernel reads offsets and mask logits where the branch convolution left them
    # (channels-last or NCHW, one tensor) and applies the sigmoid itself; compared with the
    # ordinary route fed the split, sigmoided copies
    from mmcv_b200 import _ext
    from mmcv_b200.ops import modulated_deform_conv2d, deform_conv2d
    torch.manual_seed(9)
    N, C, H, W, Co, dg = 2, 64, 18, 14, 72, 2
    x = torch.randn(N, C, H, W, device='cuda').to(dtype)
    w = (torch.randn(Co, C, 3, 3, device='cuda') * 0.05).to(dtype)
    b = torch.randn(Co, device='cuda').to(dtype)
    branch = (torch.randn(N, dg * 27, H, W, device='cuda') * 1.5).to(dtype)
    if channels_last:
        branch = branch.contiguous(memory_format=torch.channels_last)
    k = dg * 18
    want = modulated_deform_conv2d(x, branch[:, :k].contiguous(),
                                   torch.sigmoid(branch[:, k:].float()).to(dtype).contiguous(),
                                   w, b, 1, 1, 1, 1, dg)
    got = torch.empty_like(want)
    assert _ext.forward_from_branch(x, branch, k, w, b, got, (1, 1), (1, 1), (1, 1), 1, dg)
    if dtype == torch.float32:
        ok, frac = fp32_close(got, want.cpu())
        assert ok, frac
    else:
        assert rel_l2(got.float().cpu(), want.float().cpu()) <= 5e-3   # mask not rounded to bf16
    # v1: the whole tensor is offsets
    off = branch[:, :k]
    off = off.contiguous(memory_format=torch.channels_last) if channels_last else off.contiguous()
    want1 = deform_conv2d(x, off.contiguous(), w, 1, 1, 1, 1, dg)
    got1 = torch.empty_like(want1)
    assert _ext.forward_from_branch(x, off, k, w, None, got1, (1, 1), (1, 1), (1, 1), 1, dg)
    assert torch.equal(got1, want1)
    # a problem that runs on the SIMT kernels is declined, nothing is written
    x3 = torch.randn(1, 3, 8, 8, device='cuda').to(dtype)
    w3 = torch.randn(4, 3, 3, 3, device='cuda').to(dtype)
    br3 = torch.randn(1, 27, 8, 8, device='cuda').to(dtype)
    assert not _ext.forward_from_branch(x3, br3, 18, w3, None, torch.empty(1, 4, 8, 8, device='cuda',
                                                                       dtype=dtype),
                                        (1, 1), (1, 1), (1, 1), 1, 1)
