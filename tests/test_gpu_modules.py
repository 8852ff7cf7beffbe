"""GPU test of the restated BEVFormer spatial cross-attention: the CUDA operator inside the module
against the same module with the operator replaced by the independent grid_sample formulation."""
import pytest
import torch

import grid_sample_form as G
from dfa3d_b200 import modules

pytestmark = pytest.mark.gpu
DEV = "cuda"


class _GridSampleOp:
    """Stand-in with the Function's call signature, built from differentiable torch ops."""

    @staticmethod
    def apply(value, dist, shapes3, lsi, loc, attn, im2col_step, return_depth_score=True):
        H = value.shape[2]
        dist_h = dist[:, :, None, :].expand(-1, -1, H, -1)
        out = G.dfa3d_grid_sample(value.double(), dist_h.double(), shapes3.tolist(), lsi.tolist(),
                                  loc.double(), attn.double()).to(value.dtype)
        ds = torch.zeros(*attn.shape, 4, dtype=value.dtype, device=value.device)
        return out, ds


def _inputs(seed, bs=1, cams=3, Q=50, Z=4, E=32, levels=((6, 10), (3, 5)), D=9):
    g = torch.Generator().manual_seed(seed)
    N = sum(h * w for h, w in levels)
    shapes = torch.tensor(levels, dtype=torch.int64)
    hw = shapes[:, 0] * shapes[:, 1]
    lsi = torch.cat([hw.new_zeros(1), hw.cumsum(0)[:-1]])
    d = dict(
        query=torch.randn(bs, Q, E, generator=g),
        value=torch.randn(cams, N, bs, E, generator=g),
        value_dpt_dist=torch.randn(cams, N, bs, D, generator=g).softmax(-1),
        reference_points_cam=torch.rand(cams, bs, Q, Z, 3, generator=g),
        bev_mask=torch.rand(cams, bs, Q, Z, generator=g) > 0.6,
        spatial_shapes=shapes, level_start_index=lsi)
    return {k: v.to(DEV) for k, v in d.items()}


def test_spatial_cross_attention_matches_grid_sample_form(lib_built, monkeypatch):
    torch.manual_seed(0)
    attn = modules.MSDeformableAttention3D_DFA3D(embed_dims=32, num_heads=2, num_levels=2, num_points=8)
    sca = modules.SpatialCrossAttention_DFA3D(embed_dims=32, num_cams=3, dropout=0.0,
                                              deformable_attention=attn).to(DEV)
    # non-trivial offsets / attention logits so that every input of the operator gets a gradient
    with torch.no_grad():
        for p in (attn.sampling_offsets.weight, attn.sampling_offsets_depth.weight,
                  attn.attention_weights.weight):
            p.normal_(0, 0.05)
    d = _inputs(3)
    q1 = d["query"].clone().requires_grad_(True)
    out1 = sca(q1, None, d["value"], d["value_dpt_dist"], d["reference_points_cam"], d["bev_mask"],
               d["spatial_shapes"], d["level_start_index"])
    w = torch.randn_like(out1)
    (out1 * w).sum().backward()
    g1 = {n: p.grad.clone() for n, p in sca.named_parameters()}
    gq1 = q1.grad.clone()
    sca.zero_grad()
    # reference path: the module's own tensor expressions + the independent grid_sample formulation
    attn.fuse_input_ops = False
    monkeypatch.setattr(modules, "MultiScale3DDeformableAttnFunction_fp32", _GridSampleOp)
    q2 = d["query"].clone().requires_grad_(True)
    out2 = sca(q2, None, d["value"], d["value_dpt_dist"], d["reference_points_cam"], d["bev_mask"],
               d["spatial_shapes"], d["level_start_index"])
    (out2 * w).sum().backward()
    torch.testing.assert_close(out1, out2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gq1, q2.grad, rtol=1e-3, atol=1e-5)
    for n, p in sca.named_parameters():
        torch.testing.assert_close(g1[n], p.grad, rtol=1e-3, atol=1e-4, msg=lambda m, n=n: f"{n}: {m}")


def test_module_paths_agree(lib_built):
    """The three ways the attention module can call the operator give the same output and gradients:
    offsets/logits fused into the kernels, assembled tensors without depth_score, and the reference's
    way (assembled tensors, depth_score materialised for weight_update)."""
    torch.manual_seed(2)
    d = _inputs(7, cams=2)
    res = []
    for fuse, wu in ((True, False), (False, False), (False, True)):
        torch.manual_seed(2)
        attn = modules.MSDeformableAttention3D_DFA3D(embed_dims=32, num_heads=2, num_levels=2,
                                                     num_points=8, fuse_input_ops=fuse,
                                                     compute_weight_update=wu).to(DEV)
        with torch.no_grad():
            for p in (attn.sampling_offsets.weight, attn.sampling_offsets_depth.weight,
                      attn.attention_weights.weight):
                p.normal_(0, 0.05)
        q = d["query"][:, :20].clone().requires_grad_(True)
        value = d["value"][0].permute(1, 0, 2).contiguous()          # (bs, N, E)
        dist = d["value_dpt_dist"][0].permute(1, 0, 2).contiguous()
        ref = d["reference_points_cam"][0][:, :20].contiguous()     # (bs, Q, Z, 3)
        out, wupd = attn(q, value, dist, ref, d["spatial_shapes"], d["level_start_index"])
        assert (wupd is not None) == wu
        out.pow(2).sum().backward()
        res.append((out.detach(), q.grad.clone(), {n: p.grad.clone() for n, p in attn.named_parameters()}))
    for other in res[1:]:
        torch.testing.assert_close(res[0][0], other[0], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(res[0][1], other[1], rtol=1e-4, atol=1e-6)
        for n in res[0][2]:
            torch.testing.assert_close(res[0][2][n], other[2][n], rtol=1e-4, atol=1e-5,
                                       msg=lambda m, n=n: f"{n}: {m}")


def test_encoder_stack_trains_one_step(lib_built):
    torch.manual_seed(1)
    stack = modules.SCAEncoderStack(num_layers=2, embed_dims=32, ffn_dims=64, num_cams=3, num_heads=2,
                                    num_levels=2, num_points=8, dropout=0.0).to(DEV)
    d = _inputs(5)
    kw = dict(key=None, value=d["value"], value_dpt_dist=d["value_dpt_dist"],
              reference_points_cam=d["reference_points_cam"], bev_mask=d["bev_mask"],
              spatial_shapes=d["spatial_shapes"], level_start_index=d["level_start_index"])
    opt = torch.optim.SGD(stack.parameters(), lr=1e-2)
    loss0 = stack(d["query"], **kw).pow(2).mean()
    loss0.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in stack.parameters())
    opt.step()
    loss1 = stack(d["query"], **kw).pow(2).mean()
    assert torch.isfinite(loss1) and loss1 != loss0
