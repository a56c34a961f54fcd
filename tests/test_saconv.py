"""SAConv2d, the other in-tree caller of deform_conv2d (reference: mmcv/ops/saconv.py; its own
test, tests/test_ops/test_saconv.py:25-39, checks output shapes only)."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import oracle
from conftest import fp32_close


def _compose(layer, x, branch):
    """The layer's formula (reference lines 97-148) written out with `branch` standing for the
    (deformable or plain) convolution of the two evaluations."""
    x = x + layer.pre_context(F.adaptive_avg_pool2d(x, 1)).expand_as(x)
    avg = F.avg_pool2d(F.pad(x, (2, 2, 2, 2), mode='reflect'), 5, 1, 0)
    sw = layer.switch(avg)
    w = layer.weight
    flat = w.reshape(w.size(0), -1)
    ws = (w - flat.mean(1).view(-1, 1, 1, 1)) / torch.sqrt(flat.var(1) + 1e-5).view(-1, 1, 1, 1)
    ws = layer.weight_gamma * ws + layer.weight_beta
    out_s = branch(x, avg, ws, 's', layer.padding, layer.dilation)
    out_l = branch(x, avg, ws + layer.weight_diff, 'l', tuple(3 * p for p in layer.padding),
                   tuple(3 * d for d in layer.dilation))
    out = sw * out_s + (1 - sw) * out_l
    return out + layer.post_context(F.adaptive_avg_pool2d(out, 1)).expand_as(out)


def _randomise(layer):
    torch.manual_seed(11)
    for p in layer.parameters():
        p.data.normal_(0, 0.2)
    layer.weight_gamma.normal_(1, 0.1)
    layer.weight_beta.normal_(0, 0.1)


def test_shapes_as_in_the_reference_test():
    from mmcv_b200.ops import SAConv2d
    x = torch.rand(1, 3, 64, 64)
    assert SAConv2d(3, 5, kernel_size=3, padding=1)(x).shape == nn.Conv2d(3, 5, 3, padding=1)(x).shape
    assert SAConv2d(3, 5, kernel_size=3, padding=2, dilation=2)(x).shape == (1, 5, 64, 64)
    x = torch.rand(1, 4, 64, 64)
    assert SAConv2d(4, 4, kernel_size=3, padding=1, groups=2)(x).shape == (1, 4, 64, 64)


def test_plain_branches_follow_the_formula():
    from mmcv_b200.ops import SAConv2d
    layer = SAConv2d(4, 6, 3, padding=1, groups=2)
    _randomise(layer)
    x = torch.randn(2, 4, 12, 10)
    with torch.no_grad():
        want = _compose(layer, x, lambda x, a, w, which, p, d: F.conv2d(x, w, None, 1, p, d, 2))
        assert torch.allclose(layer(x), want, rtol=1e-5, atol=1e-5)
    # padding and dilation are not left changed by a forward
    assert layer.padding == (1, 1) and layer.dilation == (1, 1)


def test_checkpoint_without_standardisation_buffers():
    # plain pretrained weights: gamma/beta are recovered from them and the standardised weight
    # equals the loaded one (reference: mmcv/cnn/bricks/conv_ws.py:116-150)
    from mmcv_b200.ops import SAConv2d
    layer = SAConv2d(3, 5, 3, padding=1)
    sd = {k: v.clone() for k, v in layer.state_dict().items()
          if not k.endswith(('weight_gamma', 'weight_beta'))}
    sd['weight'] = torch.randn_like(sd['weight'])
    missing, unexpected = layer.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    assert torch.allclose(layer._get_weight(layer.weight), sd['weight'], atol=1e-5)
    # a checkpoint that has them keeps them
    sd2 = layer.state_dict()
    sd2['weight_gamma'] = torch.full_like(sd2['weight_gamma'], 2.0)
    layer.load_state_dict(sd2)
    assert torch.equal(layer.weight_gamma, sd2['weight_gamma'])


def test_deform_branches_need_the_gpu():
    from mmcv_b200.ops import SAConv2d
    layer = SAConv2d(3, 5, 3, padding=1, use_deform=True)
    with pytest.raises(RuntimeError):
        layer(torch.rand(1, 3, 16, 16))


@pytest.mark.gpu
def test_deform_branches_on_the_gpu():
    from mmcv_b200.ops import SAConv2d
    # the reference's check: same shape as the plain convolution
    x = torch.rand(1, 3, 64, 64).cuda()
    layer = SAConv2d(3, 5, kernel_size=3, padding=1, use_deform=True).cuda()
    assert layer(x).shape == (1, 5, 64, 64)
    # freshly initialised offset branches give zero offsets: the layer equals its plain twin
    plain = SAConv2d(3, 5, kernel_size=3, padding=1).cuda()
    plain.load_state_dict({k: v for k, v in layer.state_dict().items() if 'offset_' not in k})
    with torch.no_grad():
        ok, frac = fp32_close(layer(x), plain(x).cpu())
        assert ok, frac
    # random weights everywhere: both evaluations against the CPU checker
    layer = SAConv2d(8, 12, 3, padding=1, use_deform=True)
    _randomise(layer)
    layer.offset_s.weight.data.mul_(0.3)
    layer.offset_l.weight.data.mul_(0.3)
    x = torch.randn(2, 8, 14, 12)

    def branch(x, avg, w, which, p, d):
        off = (layer.offset_s if which == 's' else layer.offset_l)(avg)
        return oracle.best_forward(x, off.contiguous(), None, w.contiguous(), None, 1, p, d, 1, 1)

    with torch.no_grad():
        want = _compose(layer, x, branch)
        got = layer.cuda()(x.cuda())
    ok, frac = fp32_close(got, want)
    assert ok, frac
