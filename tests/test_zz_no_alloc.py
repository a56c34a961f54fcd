"""The entry point that brings its own scratch memory (dcn_fwd_static_scratch).

Collected last on purpose.  It serves hosts that pass a plugin only inputs, outputs and a
stream, or that have reserved all device memory already, so the library may not allocate:
the scratch is a fixed 32 MiB array inside the library.  Here it is called through the C ABI
twice in a row on different problems (the array keeps the first call's bytes when the second
starts) and each result is compared with what dcn_fwd gives with a caller-provided
workspace.
"""
import ctypes

import pytest
import torch

from conftest import golden_cases, rel_l2
from mmcv_b200 import _lib


def _params(t, m, out, dev_index):
    p = _lib.DcnFwdParams()
    x = t['x']
    p.input, p.offset = x.data_ptr(), t['offset'].data_ptr()
    p.mask = t['mask'].data_ptr() if t['mask'] is not None else None
    p.weight = t['weight'].data_ptr()
    p.bias = t['bias'].data_ptr() if t['bias'] is not None else None
    p.output = out.data_ptr()
    p.dtype, p.math_mode = _lib.DTYPE_BF16, _lib.MATH_AUTO
    p.N, p.C, p.H, p.W = x.shape
    p.Co, p.kh, p.kw = t['weight'].shape[0], t['weight'].shape[2], t['weight'].shape[3]
    p.stride_h, p.stride_w = m['stride']
    p.pad_h, p.pad_w = m['padding']
    p.dil_h, p.dil_w = m['dilation']
    p.groups, p.deform_groups = m['groups'], m['deform_groups']
    for i, s in enumerate(x.stride()):
        p.in_stride[i] = s
    p.device = dev_index
    return p


@pytest.mark.gpu
def test_static_scratch_matches_workspace_entry_twice_in_a_row():
    lib = _lib.load()
    dev = torch.device('cuda:0')
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for name in ('v2_c128_co40_dg4', 'v2_c64'):          # two calls in a row
        m, t = golden_cases().get(name)
        t = {k: (None if v is None else v.to(dev, torch.bfloat16).contiguous())
             for k, v in t.items() if k in ('x', 'offset', 'mask', 'weight', 'bias')}
        shape = tuple(golden_cases().get(name)[1]['out'].shape)
        want = torch.full(shape, float('nan'), device=dev, dtype=torch.bfloat16)
        got = torch.full(shape, float('nan'), device=dev, dtype=torch.bfloat16)
        # existing entry point, workspace from the caller
        p = _params(t, m, want, 0)
        n = ctypes.c_size_t(0)
        _lib.check(lib.dcn_fwd_workspace_bytes(ctypes.byref(p), ctypes.byref(n)))
        assert n.value <= _lib.STATIC_SCRATCH_BYTES
        ws = torch.empty(n.value, dtype=torch.uint8, device=dev)
        _lib.check(lib.dcn_fwd(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), n.value, stream))
        # new entry point, no workspace argument at all
        q = _params(t, m, got, 0)
        scratch = ctypes.c_void_p(0)
        _lib.check(lib.dcn_fwd_static_scratch(ctypes.byref(q), stream, ctypes.byref(scratch)))
        status = ctypes.c_int32(-1)
        _lib.check(lib.dcn_read_status(scratch, stream, ctypes.byref(status)))
        assert status.value == 0
        torch.cuda.synchronize(dev)
        assert torch.isfinite(got.float()).all()
        assert rel_l2(got.float(), want.float()) <= 2e-2
        assert torch.equal(got, want)      # same kernels on the same data


def test_static_scratch_rejects_problems_beyond_its_size():
    lib = _lib.load()
    p = _lib.DcnFwdParams()
    p.dtype, p.math_mode = _lib.DTYPE_BF16, _lib.MATH_AUTO
    p.N, p.C, p.H, p.W, p.Co = 64, 256, 128, 128, 256     # 0.5 GiB channels-last copy
    p.kh = p.kw = 3
    p.stride_h = p.stride_w = p.pad_h = p.pad_w = p.dil_h = p.dil_w = 1
    p.groups, p.deform_groups = 1, 8
    p.in_stride[0], p.in_stride[1], p.in_stride[2], p.in_stride[3] = 256 * 128 * 128, 128 * 128, 128, 1
    rc = lib.dcn_fwd_static_scratch(ctypes.byref(p), None, None)
    assert rc == -3
    msg = lib.dcn_last_error().decode()
    assert 'built-in scratch array holds 33554432' in msg
