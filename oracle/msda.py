"""CPU checker of multi-scale deformable attention (test infrastructure; nothing in the shipped
package imports it).

``msda_forward`` restates the arithmetic of the reference's CUDA kernel
(mmcv/ops/csrc/common/cuda/ms_deform_attn_cuda_kernel.cuh:18-66 bilinear with per-corner validity,
:198-259 the walk over levels and points with the gate ``h_im > -1 && w_im > -1 && h_im < H &&
w_im < W`` where ``h_im = loc_h * H - 0.5``) with plain tensor operations, differentiable through
autograd, in whatever floating type it is given.  It is pinned against the outputs and gradients
of the reference's own pure-PyTorch implementation (``multi_scale_deformable_attn_pytorch``,
mmcv/ops/multi_scale_deform_attn.py:113-170, which goes through ``grid_sample``) in
``tests/golden/msda_cases.npz``.
"""
import torch


def msda_forward(value, spatial_shapes, sampling_locations, attention_weights):
    """value [B, S, M, D]; spatial_shapes [L, 2] (h, w); sampling_locations [B, Q, M, L, P, 2]
    (x, y); attention_weights [B, Q, M, L, P].  Returns [B, Q, M * D]."""
    B, S, M, D = value.shape
    _, Q, _, L, P, _ = sampling_locations.shape
    out = value.new_zeros((B, Q, M, D))
    start = 0
    b_idx = torch.arange(B).view(B, 1, 1, 1).expand(B, Q, M, P)
    m_idx = torch.arange(M).view(1, 1, M, 1).expand(B, Q, M, P)
    for lvl in range(L):
        H, W = int(spatial_shapes[lvl, 0]), int(spatial_shapes[lvl, 1])
        v = value[:, start:start + H * W].reshape(B, H, W, M, D)
        start += H * W
        loc = sampling_locations[:, :, :, lvl]            # [B, Q, M, P, 2]
        w_im = loc[..., 0] * W - 0.5
        h_im = loc[..., 1] * H - 0.5
        live = (h_im > -1) & (w_im > -1) & (h_im < H) & (w_im < W)
        h_low, w_low = torch.floor(h_im), torch.floor(w_im)
        lh, lw = h_im - h_low, w_im - w_low
        hh, hw = 1 - lh, 1 - lw
        h_low = torch.nan_to_num(h_low).long()
        w_low = torch.nan_to_num(w_low).long()
        acc = value.new_zeros((B, Q, M, P, D))
        for dy, dx, wt in ((0, 0, hh * hw), (0, 1, hh * lw), (1, 0, lh * hw), (1, 1, lh * lw)):
            y, x = h_low + dy, w_low + dx
            ok = live & (y >= 0) & (y <= H - 1) & (x >= 0) & (x <= W - 1)
            yc, xc = y.clamp(0, H - 1), x.clamp(0, W - 1)
            corner = v[b_idx, yc, xc, m_idx]               # [B, Q, M, P, D]
            corner = torch.where(ok.unsqueeze(-1), corner, torch.zeros_like(corner))
            wt = torch.where(ok, wt, torch.zeros_like(wt))
            acc = acc + wt.unsqueeze(-1) * corner
        out = out + (acc * attention_weights[:, :, :, lvl].unsqueeze(-1)).sum(3)
    return out.reshape(B, Q, M * D)
