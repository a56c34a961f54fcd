"""The CPU checkers against the reference's vectors (no GPU needed)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import fp32_close, golden_case_names, golden_cases


def test_port_library_builds_and_loads():
    lib = oracle.load_port()
    assert lib.dcn_oracle_num_threads() >= 1


def test_port_reference_known_answer_v2(kat):
    # Reference test construction: zero offsets, mask 0.5, 2x2 ones kernel, pad 1.
    x = torch.from_numpy(kat['v2_input'])
    off = torch.zeros(1, 8, 4, 4)
    mask = torch.full((1, 4, 4, 4), 0.5)
    w = torch.ones(1, 1, 2, 2)
    y = oracle.port_forward(x, off, mask, w, None, 1, 1, 1, 1, 1)
    assert np.allclose(y.numpy(), kat['v2_expected'], 1e-2)
    assert np.allclose(y.numpy(), kat['v2_ref_out'], 1e-6)


def test_port_reference_known_answer_v1(kat):
    x = torch.from_numpy(np.repeat(kat['v1_input'], 10, axis=0))
    off = torch.from_numpy(kat['v1_offset'])
    w = torch.from_numpy(kat['v1_deform_weight'])
    y = oracle.port_forward(x, off, None, w, None, 1, 0, 1, 1, 1)
    want = np.repeat(kat['v1_expected'], 10, axis=0)
    # the reference holds this vector to a relative 1e-1 on CPU
    assert np.allclose(y.numpy(), want, 1e-1)
    assert np.allclose(y.numpy(), kat['v1_ref_out'], rtol=1e-5, atol=1e-6)
    assert (y.numpy()[:, 0, 0, 1] == 0).all() and (y.numpy()[:, 0, 1, :] == 0).all()


@pytest.mark.parametrize('name', golden_case_names())
def test_port_matches_reference_outputs(name):
    m, t = golden_cases().get(name)
    y = oracle.port_forward(t['x'], t['offset'], t['mask'], t['weight'], t['bias'],
                            m['stride'], m['padding'], m['dilation'], m['groups'],
                            m['deform_groups'])
    ok, frac = fp32_close(y, t['out'])
    assert ok, frac


@pytest.mark.skipif(not oracle.have_ref(), reason='reference extension not built')
@pytest.mark.parametrize('name', ['v2_basic', 'v2_s2_d2_dg4_int', 'v1_g2_dg2_d2'])
def test_reference_extension_reproduces_fixtures(name):
    m, t = golden_cases().get(name)
    y = oracle.ref_forward(t['x'], t['offset'], t['mask'], t['weight'], t['bias'],
                           m['stride'], m['padding'], m['dilation'], m['groups'],
                           m['deform_groups'])
    assert torch.equal(torch.isfinite(y), torch.isfinite(t['out']))
    assert torch.allclose(y, t['out'], rtol=0, atol=0, equal_nan=True)


def test_bilinear_corner_rules():
    lib = oracle.load_port()
    import ctypes
    plane = torch.arange(12, dtype=torch.float32).reshape(3, 4).contiguous()
    p = ctypes.c_void_p(plane.data_ptr())
    f = lambda h, w: lib.dcn_oracle_bilinear(p, 3, 4, h, w)
    assert f(1.0, 2.0) == 6.0                      # grid aligned
    assert f(0.5, 0.5) == pytest.approx(2.5)       # mean of 0,1,4,5
    assert f(-0.5, 0.0) == pytest.approx(0.0)      # top corners outside: 0.5*plane[0,0]
    assert f(2.5, 3.0) == pytest.approx(5.5)       # bottom row outside: 0.5*11
    assert f(-0.25, -0.25) == pytest.approx(0.0)
    assert f(2.0, 3.5) == pytest.approx(5.5)
