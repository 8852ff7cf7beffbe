"""Independent formulation of the DFA3D operator -- TEST INFRASTRUCTURE ONLY.

DFA3D is, by construction, trilinear sampling of the outer product ``value (x) dist``:
per level build ``vol[b*H+h, c, z, y, x] = value[b,(y,x),h,c] * dist[b,(y,x),h,z]`` and sample it with
5-D ``torch.nn.functional.grid_sample(mode='bilinear', padding_mode='zeros', align_corners=False)`` at
``2*loc-1``; weight by the attention weights and sum over levels and points.  grid_sample's
un-normalisation ``((g+1)*S-1)/2 = loc*S-0.5`` is the kernels' pixel-centre convention
(DFA3D/dfa3D/ops/csrc/common/cuda/ms_depth_score_sample_cuda_kernel.cuh:133-135) and its zero
padding is the kernels' per-corner in-range tests (:52-88, wms_deform_attn_cuda_kernel.cuh:49-74).

It shares no code with ``oracle/dfa3d_oracle.c``; agreement of the two (forward and, through autograd,
all four input gradients) is one of the two pins of the oracle.  Memory-hungry (materialises the
volume): use on small cases only.
"""
import torch
import torch.nn.functional as F


def dfa3d_grid_sample(value, dist, shapes3, lsi, loc3, attn):
    """value (B,N,H,C), dist (B,N,H,D), loc3 (B,Q,H,L,P,3), attn (B,Q,H,L,P) -> (B,Q,H*C).
    Differentiable w.r.t. value, dist, loc3, attn."""
    B, N, H, C = value.shape
    D = dist.shape[-1]
    _, Q, _, L, P, _ = loc3.shape
    out = value.new_zeros(B * H, C, Q)
    for l in range(L):
        h, w, d = (int(x) for x in shapes3[l])
        assert d == D
        s = int(lsi[l])
        v = value[:, s:s + h * w].permute(0, 2, 3, 1).reshape(B * H, C, 1, h, w)
        p = dist[:, s:s + h * w].permute(0, 2, 3, 1).reshape(B * H, 1, D, h, w)
        vol = v * p                                                   # (B*H, C, D, h, w)
        grid = 2.0 * loc3[:, :, :, l] - 1.0                           # (B,Q,H,P,3) = (x,y,z)
        grid = grid.permute(0, 2, 1, 3, 4).reshape(B * H, Q, P, 1, 3)
        samp = F.grid_sample(vol, grid, mode="bilinear", padding_mode="zeros",
                             align_corners=False)                     # (B*H, C, Q, P, 1)
        a = attn[:, :, :, l].permute(0, 2, 1, 3).reshape(B * H, 1, Q, P)
        out = out + (samp[..., 0] * a).sum(-1)
    return out.view(B, H, C, Q).permute(0, 3, 1, 2).reshape(B, Q, H * C)


def dfa3d_grid_sample_grads(value, dist, shapes3, lsi, loc3, attn, grad_out):
    """Forward + autograd backward.  Returns (out, grad_value, grad_dist, grad_loc3, grad_attn)."""
    leaves = [t.detach().clone().requires_grad_(True) for t in (value, dist, loc3, attn)]
    out = dfa3d_grid_sample(leaves[0], leaves[1], shapes3, lsi, leaves[2], leaves[3])
    out.backward(grad_out)
    return (out.detach(),) + tuple(t.grad for t in leaves)


def msda_grid_sample(value, shapes2, lsi, loc2, attn):
    """Plain 2-D multi-scale deformable attention as per-level 4-D ``grid_sample`` -- the published
    formulation of the operator (mmcv's ``multi_scale_deformable_attn_pytorch``, which the reference
    calls as its CPU path at BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/
    temporal_self_attention.py:252 and decoder.py:336; mmcv itself is not part of the reference
    checkout).  value (B,N,H,C), loc2 (B,Q,H,L,P,2), attn (B,Q,H,L,P) -> (B,Q,H*C)."""
    B, N, H, C = value.shape
    _, Q, _, L, P, _ = loc2.shape
    out = value.new_zeros(B * H, C, Q)
    for l in range(L):
        h, w = int(shapes2[l][0]), int(shapes2[l][1])
        s = int(lsi[l])
        v = value[:, s:s + h * w].permute(0, 2, 3, 1).reshape(B * H, C, h, w)
        grid = (2.0 * loc2[:, :, :, l] - 1.0).permute(0, 2, 1, 3, 4).reshape(B * H, Q, P, 2)
        samp = F.grid_sample(v, grid, mode="bilinear", padding_mode="zeros", align_corners=False)
        a = attn[:, :, :, l].permute(0, 2, 1, 3).reshape(B * H, 1, Q, P)
        out = out + (samp * a).sum(-1)
    return out.view(B, H, C, Q).permute(0, 3, 1, 2).reshape(B, Q, H * C)
