"""Generate the committed golden fixtures from the UNMODIFIED reference.

Needs a reference checkout (its root in $DCN_REFERENCE_ROOT) and the reference CPU
extension built by ``python oracle/build_oracle.py``.  Writes

* ``reference_kat.npz`` -- the known-answer vectors that the reference's own
  unit tests hold for this path, read from the test files as data
  (tests/test_ops/test_modulated_deform_conv.py:28-30 and
  tests/test_ops/test_deform_conv.py:27-35), together with what the reference
  wrappers + CPU extension produce on them (forward output, the offset/mask the
  offset branch produced, and the gradients of the reference test).
* ``msda_cases.npz`` -- seeded cases of multi-scale deformable attention: inputs, outputs and
  gradients from the reference's own pure-PyTorch implementation
  (mmcv/ops/multi_scale_deform_attn.py:113-170), among them the case of the reference's tests
  (tests/test_ops/test_ms_deformable_attn.py:101-118).
* ``dcn_cases.npz`` -- seeded small cases (inputs, parameters, forward output and
  gradients) covering kernel/stride/padding/dilation/group/deform-group
  variety, out-of-range, grid-aligned and non-finite offsets, non-finite input samples.

Run: ``python tests/golden/make_golden.py``
"""
import ast
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import oracle  # noqa: E402
import ref_wrappers  # noqa: E402

REF_ROOT = os.environ.get('DCN_REFERENCE_ROOT', '')   # the reference checkout (required)


def module_literals(path, names):
    """Module-level list literals of a reference test file, read as data."""
    tree = ast.parse(open(path).read())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.Assign) and len(node.targets) == 1:
            t = node.targets[0]
            if isinstance(t, ast.Name) and t.id in names:
                out[t.id] = ast.literal_eval(node.value)
    missing = set(names) - set(out)
    assert not missing, missing
    return out


# name, N, C, H, W, Co, (kh,kw), stride, pad, dil, groups, dg, mask, bias, sigma, special
CASES = [
    ('v2_basic', 2, 8, 9, 11, 8, (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, True, True, 1.5, ''),
    ('v2_s2_d2_dg4_int', 2, 16, 13, 12, 8, (3, 3), (2, 2), (2, 2), (2, 2), 1, 4, True, True, 4.0, 'int'),
    ('v2_g2_dg2', 1, 8, 7, 7, 12, (3, 3), (1, 1), (1, 1), (1, 1), 2, 2, True, True, 1.0, ''),
    ('v2_k1', 2, 6, 5, 6, 4, (1, 1), (1, 1), (0, 0), (1, 1), 1, 3, True, True, 1.0, ''),
    ('v2_k5x3_rect', 1, 4, 10, 9, 6, (5, 3), (1, 2), (2, 1), (1, 1), 1, 1, True, False, 2.0, ''),
    ('v2_far', 1, 4, 8, 8, 4, (3, 3), (1, 1), (1, 1), (1, 1), 1, 2, True, True, 20.0, ''),
    ('v2_nonfinite', 1, 4, 6, 6, 4, (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, True, True, 1.0, 'nonfinite'),
    ('v2_zero_offset', 1, 4, 6, 7, 4, (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, True, True, 0.0, ''),
    ('v2_c64', 1, 64, 12, 12, 64, (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, True, True, 2.0, ''),
    ('v2_c128_co40_dg4', 2, 128, 6, 7, 40, (3, 3), (1, 1), (1, 1), (1, 1), 1, 4, True, True, 2.0, 'int'),
    ('v2_c128_g2_dg2_s2', 1, 128, 9, 9, 64, (3, 3), (2, 2), (1, 1), (1, 1), 2, 2, True, False, 3.0, ''),
    ('v1_basic', 2, 8, 9, 11, 8, (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, False, False, 1.5, ''),
    ('v1_g2_dg2_d2', 2, 8, 10, 8, 4, (3, 3), (1, 1), (2, 2), (2, 2), 2, 2, False, False, 2.0, 'int'),
    ('v1_k2_nopad', 3, 3, 5, 5, 2, (2, 2), (1, 1), (0, 0), (1, 1), 1, 1, False, False, 0.7, ''),
    ('v1_c64', 1, 64, 10, 14, 32, (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, False, False, 1.5, ''),
    # Inf / NaN among the input samples, with some grid-aligned offsets (a corner of weight zero
    # over a non-finite sample gives NaN in the reference: 0 * Inf) and some zero mask values
    ('v2_input_nonfinite', 1, 8, 9, 9, 8, (3, 3), (1, 1), (1, 1), (1, 1), 1, 2, True, True, 1.5, 'input_nonfinite int'),
    ('v2_c64_input_nonfinite', 1, 64, 12, 12, 64, (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, True, True, 1.5, 'input_nonfinite int'),
    ('v1_input_nonfinite', 1, 8, 9, 9, 8, (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, False, False, 1.5, 'input_nonfinite int'),
]


def make_case(spec, seed):
    (name, N, C, H, W, Co, k, s, p, d, g, dg, with_mask, with_bias, sigma,
     special) = spec
    gen = torch.Generator().manual_seed(seed)
    kh, kw = k
    Ho = oracle.out_size(H, p[0], d[0], kh, s[0])
    Wo = oracle.out_size(W, p[1], d[1], kw, s[1])
    x = torch.randn(N, C, H, W, generator=gen)
    off = torch.randn(N, dg * 2 * kh * kw, Ho, Wo, generator=gen) * sigma
    if 'int' in special:
        sel = torch.rand(off.shape, generator=gen) < 0.05
        off = torch.where(sel, off.round(), off)
    if 'nonfinite' in special:
        flat = off.view(-1)
        idx = torch.randperm(flat.numel(), generator=gen)[:9]
        flat[idx[:3]] = float('nan')
        flat[idx[3:6]] = float('inf')
        flat[idx[6:]] = float('-inf')
    mask = (torch.sigmoid(torch.randn(N, dg * kh * kw, Ho, Wo, generator=gen))
            if with_mask else None)
    if 'input_nonfinite' in special:
        flat = x.view(-1)
        idx = torch.randperm(flat.numel(), generator=gen)[:6]
        flat[idx[:2]] = float('nan')
        flat[idx[2:4]] = float('inf')
        flat[idx[4:]] = float('-inf')
        if mask is not None:
            mask = torch.where(torch.rand(mask.shape, generator=gen) < 0.1,
                               torch.zeros_like(mask), mask)
    bound = 1.0 / (C // g * kh * kw) ** 0.5
    w = (torch.rand(Co, C // g, kh, kw, generator=gen) * 2 - 1) * bound * 3 ** 0.5
    b = (torch.rand(Co, generator=gen) * 0.2 - 0.1) if with_bias else None
    gy = torch.randn(N, Co, Ho, Wo, generator=gen)
    return dict(x=x, offset=off, mask=mask, weight=w, bias=b, grad_out=gy)


def run_case(v2, v1, spec, t):
    (name, N, C, H, W, Co, k, s, p, d, g, dg, with_mask, with_bias, sigma,
     special) = spec
    leaf = {n: (None if v is None else v.clone().requires_grad_(n != 'grad_out'))
            for n, v in t.items()}
    if with_mask:
        y = v2.modulated_deform_conv2d(leaf['x'], leaf['offset'], leaf['mask'],
                                       leaf['weight'], leaf['bias'], s, p, d, g, dg)
    else:
        y = v1.deform_conv2d(leaf['x'], leaf['offset'], leaf['weight'], s, p, d,
                             g, dg, False, 32)
    out = {'out': y.detach()}
    if 'nonfinite' not in special:   # (either kind: no gradients for non-finite cases)
        y.backward(t['grad_out'])
        for n in ('x', 'offset', 'mask', 'weight', 'bias'):
            if leaf[n] is not None:
                out['grad_' + n] = leaf[n].grad
    return out


def reference_kat(v2, v1):
    kat = {}
    a = module_literals(
        os.path.join(REF_ROOT, 'tests/test_ops/test_modulated_deform_conv.py'),
        ['input_t', 'output_t', 'input_grad', 'dcn_w_grad', 'dcn_offset_w_grad',
         'dcn_offset_b_grad'])
    # Same construction as the reference test (its lines 51-85), forward part.
    x = torch.tensor(a['input_t'], dtype=torch.float)
    dcn = v2.ModulatedDeformConv2dPack(1, 1, kernel_size=(2, 2), stride=1,
                                       padding=1, deform_groups=1, bias=False)
    dcn.weight.data.fill_(1.)
    x.requires_grad = True
    y = dcn(x)
    y.sum().backward()
    assert np.allclose(y.detach().numpy(), a['output_t'], 1e-2)
    # the reference test's gradient vectors, confirmed against the reference itself
    assert np.allclose(x.grad.numpy(), a['input_grad'], 1e-2)
    assert np.allclose(dcn.weight.grad.numpy(), a['dcn_w_grad'], 1e-2)
    assert np.allclose(dcn.conv_offset.weight.grad.numpy(), a['dcn_offset_w_grad'], 1e-2)
    assert np.allclose(dcn.conv_offset.bias.grad.numpy(), a['dcn_offset_b_grad'], 1e-2)
    for k in ('input_grad', 'dcn_w_grad', 'dcn_offset_w_grad', 'dcn_offset_b_grad'):
        kat['v2_' + k] = np.array(a[k], dtype=np.float32)
    x = x.detach()
    kat['v2_input'] = x.numpy()
    kat['v2_expected'] = np.array(a['output_t'], dtype=np.float32)
    kat['v2_ref_out'] = y.detach().numpy()

    b = module_literals(
        os.path.join(REF_ROOT, 'tests/test_ops/test_deform_conv.py'),
        ['input', 'offset_weight', 'offset_bias', 'deform_weight', 'gt_out', 'gt_x_grad',
         'gt_offset_weight_grad', 'gt_offset_bias_grad', 'gt_deform_weight_grad'])
    batch = 10
    x = torch.tensor(np.repeat(b['input'], batch, axis=0), dtype=torch.float)
    m = v1.DeformConv2dPack(in_channels=1, out_channels=1, kernel_size=2,
                            stride=1, padding=0, im2col_step=2)
    m.conv_offset.weight.data = torch.Tensor(b['offset_weight']).reshape(8, 1, 2, 2)
    m.conv_offset.bias.data = torch.Tensor(b['offset_bias']).reshape(8)
    m.weight.data = torch.Tensor(b['deform_weight']).reshape(1, 1, 2, 2)
    x.requires_grad = True
    y = m(x)
    y.backward(torch.ones_like(y))
    # The reference runs this case on CPU with a relative tolerance of 1e-1.
    assert np.allclose(y.detach().numpy(), np.repeat(b['gt_out'], batch, axis=0), 1e-1)
    assert np.allclose(x.grad.numpy(), np.repeat(b['gt_x_grad'], batch, axis=0), 1e-1)
    assert np.allclose(m.conv_offset.weight.grad.numpy() / batch, b['gt_offset_weight_grad'], 1e-1)
    assert np.allclose(m.weight.grad.numpy() / batch, b['gt_deform_weight_grad'], 1e-1)
    kat['v1_x_grad'] = np.array(b['gt_x_grad'], dtype=np.float32)
    kat['v1_offset_weight_grad'] = np.array(b['gt_offset_weight_grad'], dtype=np.float32)
    kat['v1_offset_bias_grad'] = np.array(b['gt_offset_bias_grad'], dtype=np.float32).reshape(-1)
    kat['v1_deform_weight_grad'] = np.array(b['gt_deform_weight_grad'], dtype=np.float32)
    # full-precision gradients of the reference on this case (the vectors above are rounded)
    kat['v1_ref_x_grad'] = x.grad.numpy().copy()
    kat['v1_ref_offset_weight_grad'] = m.conv_offset.weight.grad.numpy().copy()
    kat['v1_ref_offset_bias_grad'] = m.conv_offset.bias.grad.numpy().copy()
    kat['v1_ref_deform_weight_grad'] = m.weight.grad.numpy().copy()
    x = x.detach()
    kat['v1_input'] = np.array(b['input'], dtype=np.float32)
    kat['v1_offset_weight'] = np.array(b['offset_weight'], dtype=np.float32).reshape(8, 1, 2, 2)
    kat['v1_offset_bias'] = np.array(b['offset_bias'], dtype=np.float32)
    kat['v1_deform_weight'] = np.array(b['deform_weight'], dtype=np.float32).reshape(1, 1, 2, 2)
    kat['v1_expected'] = np.array(b['gt_out'], dtype=np.float32)
    kat['v1_offset'] = m.conv_offset(x).detach().numpy()
    kat['v1_ref_out'] = y.detach().numpy()
    return kat


MSDA_CASES = [
    # name, B, M, D, Q, shapes, P, location range, seed
    ('ref_test', 1, 2, 2, 2, [(6, 4), (3, 2)], 2, (0.0, 1.0), 3),      # the reference tests' own case
    ('detr_like', 1, 8, 32, 64, [(12, 16), (6, 8), (3, 4), (2, 2)], 4, (-0.15, 1.15), 11),
    ('odd_channels', 2, 3, 5, 17, [(7, 5), (4, 3), (1, 1)], 3, (-0.3, 1.3), 12),
    ('wide_head', 1, 2, 64, 33, [(9, 11), (5, 6)], 2, (-0.1, 1.1), 13),
    ('edges', 1, 4, 8, 64, [(4, 4), (2, 2)], 4, (-0.5, 1.5), 14),
]


def msda_cases(msda):
    """Inputs, outputs and gradients of multi-scale deformable attention from the reference's
    own pure-PyTorch implementation (multi_scale_deformable_attn_pytorch), computed in double
    and stored as fp32 (inputs are fp32 values, so the double result is the exact target)."""
    blob = {}
    for name, B, M, D, Q, shapes, P, (lo, hi), seed in MSDA_CASES:
        torch.manual_seed(seed)
        shp = torch.as_tensor(shapes, dtype=torch.long)
        S = int(shp.prod(1).sum())
        L = len(shapes)
        value = torch.rand(B, S, M, D) * (0.01 if name == 'ref_test' else 1.0)
        loc = torch.rand(B, Q, M, L, P, 2) * (hi - lo) + lo
        if name == 'edges':   # exact cell centres and borders among the locations
            sel = torch.rand(loc.shape) < 0.3
            loc = torch.where(sel, (loc * 8).round() / 8, loc)
        attn = torch.rand(B, Q, M, L, P) + 1e-5
        attn /= attn.sum(-1, keepdim=True).sum(-2, keepdim=True)
        gout = torch.randn(B, Q, M * D)
        v64 = value.double().requires_grad_(True)
        l64 = loc.double().requires_grad_(True)
        a64 = attn.double().requires_grad_(True)
        out = msda.multi_scale_deformable_attn_pytorch(v64, shp, l64, a64)
        out.backward(gout.double())
        for k, t in dict(value=value, shapes=shp, loc=loc, attn=attn, grad_out=gout, out=out.detach().float(),
                         grad_value=v64.grad.float(), grad_loc=l64.grad.float(),
                         grad_attn=a64.grad.float()).items():
            blob[f'{name}/{k}'] = t.numpy()
    return blob


def main():
    ext = oracle.load_ref()
    v2, v1, _ = ref_wrappers.load(ext, REF_ROOT)
    import types
    msda = ref_wrappers.load_msda(types.SimpleNamespace(ms_deform_attn_forward=None,
                                                        ms_deform_attn_backward=None), REF_ROOT)
    np.savez_compressed(os.path.join(HERE, 'msda_cases.npz'), **msda_cases(msda))
    np.savez_compressed(os.path.join(HERE, 'reference_kat.npz'), **reference_kat(v2, v1))
    blob, meta = {}, {}
    for i, spec in enumerate(CASES):
        t = make_case(spec, 1000 + i)
        r = run_case(v2, v1, spec, t)
        name = spec[0]
        meta[name] = dict(N=spec[1], C=spec[2], H=spec[3], W=spec[4], Co=spec[5],
                          kernel=spec[6], stride=spec[7], padding=spec[8],
                          dilation=spec[9], groups=spec[10], deform_groups=spec[11],
                          with_mask=spec[12], with_bias=spec[13])
        for n, v in {**t, **r}.items():
            if v is not None:
                blob[f'{name}/{n}'] = v.detach().numpy()
    blob['__meta__'] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, 'dcn_cases.npz'), **blob)
    ref_wrappers.unload()
    print('wrote', len(CASES), 'cases;',
          {f: os.path.getsize(os.path.join(HERE, f)) for f in
           ('reference_kat.npz', 'dcn_cases.npz')})


if __name__ == '__main__':
    main()
