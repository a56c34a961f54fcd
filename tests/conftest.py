import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, 'tests', 'golden')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (B200)')


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


class GoldenCases:
    """Seeded cases whose outputs came from the unmodified reference."""

    def __init__(self):
        z = np.load(os.path.join(GOLDEN, 'dcn_cases.npz'))
        self.meta = json.loads(bytes(z['__meta__']).decode())
        self.z = z

    def names(self):
        return list(self.meta)

    def get(self, name):
        m = dict(self.meta[name])
        t = {}
        for key in ('x', 'offset', 'mask', 'weight', 'bias', 'out', 'grad_out',
                    'grad_x', 'grad_offset', 'grad_mask', 'grad_weight', 'grad_bias'):
            full = f'{name}/{key}'
            t[key] = torch.from_numpy(self.z[full]) if full in self.z.files else None
        for key in ('kernel', 'stride', 'padding', 'dilation'):
            m[key] = tuple(m[key])
        return m, t


_cases = None


def golden_cases():
    global _cases
    if _cases is None:
        _cases = GoldenCases()
    return _cases


def golden_case_names():
    return golden_cases().names()


@pytest.fixture(scope='session')
def kat():
    return dict(np.load(os.path.join(GOLDEN, 'reference_kat.npz')))


def fp32_close(out, ref):
    """max|out-ref| <= 1e-4*max|ref| + 1e-5 (the fp32 acceptance bound)."""
    out = out.detach().float().cpu()
    ref = ref.detach().float().cpu()
    finite = torch.isfinite(ref)
    if not torch.equal(torch.isfinite(out), finite):
        return False, float('inf')
    if finite.sum() == 0:
        return True, 0.0
    err = (out[finite] - ref[finite]).abs().max().item()
    bound = 1e-4 * ref[finite].abs().max().item() + 1e-5
    return err <= bound, err / bound


def rel_l2(out, ref):
    out = out.detach().double().cpu()
    ref = ref.detach().double().cpu()
    return ((out - ref).norm() / ref.norm().clamp_min(1e-30)).item()
