"""GPU tests of the restated BEVFormer spatial cross-attention (row a9 of the scope): the CUDA operator
and the re-batching kernels inside the modules against

  * the same modules with the operator replaced by the independent grid_sample formulation, and
  * a loop restatement of the reference's SpatialCrossAttention_DFA3D.forward
    (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/spatial_cross_attention.py:700-751):
    per-camera index lists from nonzero(), zero-padded re-batching, per-camera attention, loop scatter.
"""
import numpy as np
import pytest
import torch

import dfa3d_oracle as O
import grid_sample_form as G
from dfa3d_b200 import modules

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _depth_score(dist, shapes3, lsi, loc):
    """depth_score from the CPU oracle (not differentiable, like the reference's fused Function)."""
    H = loc.shape[2]
    dist_h = dist[:, :, None, :].expand(-1, -1, H, -1).contiguous()
    ds = O.ms_depth_score_sample_forward(dist_h.detach().cpu().numpy().astype(np.float64),
                                         shapes3.cpu().numpy(), lsi.cpu().numpy(),
                                         loc.detach().cpu().numpy().astype(np.float64))
    return torch.from_numpy(ds).to(loc.dtype).to(loc.device)


class _GridSampleOp:
    """Stand-in with the dense Function's call signature, built from differentiable torch ops."""

    @staticmethod
    def apply(value, dist, shapes3, lsi, loc, attn, im2col_step, return_depth_score=True, dist_map=None):
        assert dist_map is None
        H = value.shape[2]
        dist_h = dist[:, :, None, :].expand(-1, -1, H, -1)
        out = G.dfa3d_grid_sample(value.double(), dist_h.double(), shapes3.tolist(), lsi.tolist(),
                                  loc.double(), attn.double()).to(value.dtype)
        ds = _depth_score(dist, shapes3, lsi, loc) if return_depth_score else None
        return out, ds


class _GridSampleRaggedOp:
    """Stand-in with the ragged Function's call signature: camera by camera through grid_sample."""

    @staticmethod
    def apply(value, dist, shapes3, lsi, loc, attn, query_offsets, max_queries, return_depth_score=True,
              dist_map=None):
        assert dist_map is None
        offs = query_offsets.tolist()
        outs, dss = [], []
        for b in range(value.shape[0]):
            r0, r1 = offs[b], offs[b + 1]
            if r1 == r0:
                continue
            o, ds = _GridSampleOp.apply(value[b:b + 1], dist[b:b + 1], shapes3, lsi, loc[None, r0:r1],
                                        attn[None, r0:r1], 64, return_depth_score)
            outs.append(o[0])
            dss.append(ds[0] if ds is not None else None)
        out = torch.cat(outs) if outs else value.new_zeros(0, value.shape[2] * value.shape[3])
        return out, (torch.cat(dss) if return_depth_score and dss else None)


def _inputs(seed, bs=1, cams=3, Q=50, Z=4, E=32, levels=((6, 10), (3, 5)), D=9, empty_camera=None):
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
    if empty_camera is not None:
        d["bev_mask"][empty_camera] = False
    return {k: v.to(DEV) for k, v in d.items()}


def _randomise(attn):
    """Non-trivial offsets / attention logits so that every input of the operator gets a gradient."""
    with torch.no_grad():
        for p in (attn.sampling_offsets.weight, attn.sampling_offsets_depth.weight,
                  attn.attention_weights.weight):
            p.normal_(0, 0.05)


def sca_loop_form(sca, query, value, value_dpt_dist, reference_points_cam, bev_mask, spatial_shapes,
                  level_start_index, query_pos=None):
    """SpatialCrossAttention_DFA3D.forward written like the reference (:700-751), calling the attention
    module on the zero-padded (bs*cams, max_len, ...) tensors."""
    inp_residual = query
    slots = torch.zeros_like(query)
    if query_pos is not None:
        query = query + query_pos
    bs, num_query, E = query.shape
    cams, Z = sca.num_cams, reference_points_cam.size(3)
    indexes = [mask_per_img[0].sum(-1).nonzero().squeeze(-1) for mask_per_img in bev_mask]
    max_len = max(len(each) for each in indexes)
    queries_rebatch = query.new_zeros([bs, cams, max_len, E])
    reference_points_rebatch = reference_points_cam.new_zeros([bs, cams, max_len, Z, 3])
    empty_queries_rebatch = query.new_zeros([bs, cams, max_len, sca.num_head, E])
    for j in range(bs):
        for i, reference_points_per_img in enumerate(reference_points_cam):
            ix = indexes[i]
            queries_rebatch[j, i, :len(ix)] = query[j, ix]
            reference_points_rebatch[j, i, :len(ix)] = reference_points_per_img[j, ix]
            if sca.use_empty:
                empty_queries_rebatch[j, i, :len(ix)] = sca.empty_query.weight.view(
                    sca.bev_h * sca.bev_w, sca.num_head, E)[ix]
    l = value.shape[1]
    value = value.permute(2, 0, 1, 3).reshape(bs * cams, l, E)
    value_dpt_dist = value_dpt_dist.permute(2, 0, 1, 3).reshape(bs * cams, l, value_dpt_dist.shape[-1])
    queries, update_weight = sca.deformable_attention(
        query=queries_rebatch.view(bs * cams, max_len, E), value=value, value_dpt_dist=value_dpt_dist,
        reference_points=reference_points_rebatch.view(bs * cams, max_len, Z, 3),
        spatial_shapes=spatial_shapes, level_start_index=level_start_index)
    queries = queries.view(bs, cams, max_len, E)
    if sca.use_empty:
        update_weight = update_weight.view(bs, cams, *update_weight.shape[1:])
        queries = queries + ((1 - update_weight) * empty_queries_rebatch).mean(dim=-2)
    for j in range(bs):
        for i, ix in enumerate(indexes):
            slots[j, ix] += queries[j, i, :len(ix)]
    count = (bev_mask.sum(-1) > 0).permute(1, 2, 0).sum(-1).clamp(min=1.0)
    slots = sca.output_proj(slots / count[..., None])
    return sca.dropout(slots) + inp_residual


@pytest.mark.parametrize("fuse", [True, False], ids=["offsets_fused", "tensors_assembled"])
def test_spatial_cross_attention_matches_grid_sample_form(lib_built, monkeypatch, fuse):
    """Packed-row path (plan + ragged operator) against the loop form with the grid_sample operator:
    output, query gradient and every parameter gradient.  One camera sees nothing."""
    torch.manual_seed(0)
    attn = modules.MSDeformableAttention3D_DFA3D(embed_dims=32, num_heads=2, num_levels=2, num_points=8,
                                                 fuse_input_ops=fuse)
    sca = modules.SpatialCrossAttention_DFA3D(embed_dims=32, num_cams=3, dropout=0.0,
                                              deformable_attention=attn).to(DEV)
    _randomise(attn)
    d = _inputs(3, bs=2, empty_camera=1)
    args = (d["value"], d["value_dpt_dist"], d["reference_points_cam"], d["bev_mask"], d["spatial_shapes"],
            d["level_start_index"])
    q1 = d["query"].clone().requires_grad_(True)
    out1 = sca(q1, None, *args)
    w = torch.randn_like(out1)
    (out1 * w).sum().backward()
    g1 = {n: p.grad.clone() for n, p in sca.named_parameters()}
    gq1 = q1.grad.clone()
    sca.zero_grad()
    # reference path: loop form + the module's own tensor expressions + the grid_sample operator
    attn.fuse_input_ops = False
    monkeypatch.setattr(modules, "MultiScale3DDeformableAttnFunction_fp32", _GridSampleOp)
    q2 = d["query"].clone().requires_grad_(True)
    out2 = sca_loop_form(sca, q2, *args)
    (out2 * w).sum().backward()
    torch.testing.assert_close(out1, out2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gq1, q2.grad, rtol=1e-3, atol=1e-5)
    for n, p in sca.named_parameters():
        torch.testing.assert_close(g1[n], p.grad, rtol=1e-3, atol=1e-4, msg=lambda m, n=n: f"{n}: {m}")


def test_weight_update_value_and_use_empty(lib_built):
    """weight_update is the attention-weighted mean corner depth score (:579): its value against the
    expression evaluated with the oracle's depth_score.  With use_empty=True (:721-722, :739-740) the
    module output against the loop form (batch of 2, a camera that sees nothing)."""
    torch.manual_seed(4)
    H, L, P, E = 2, 2, 8, 32
    attn = modules.MSDeformableAttention3D_DFA3D(embed_dims=E, num_heads=H, num_levels=L, num_points=P).to(DEV)
    _randomise(attn)
    d = _inputs(11, bs=2, Q=49, empty_camera=2)
    # --- weight_update value, dense call of the attention module
    q = d["query"][:, :20]
    value = d["value"][0].permute(1, 0, 2).contiguous()
    dist = d["value_dpt_dist"][0].permute(1, 0, 2).contiguous()
    ref = d["reference_points_cam"][0][:, :20].contiguous()
    with torch.no_grad():
        out, wupd = attn(q, value, dist, ref, d["spatial_shapes"], d["level_start_index"])
        D = dist.shape[-1]
        off_uv = attn.sampling_offsets(q).view(2, 20, H, L, P, 2)
        off_d = attn.sampling_offsets_depth(q).view(2, 20, H, L, P, 1)
        a = attn.attention_weights(q).view(2, 20, H, L * P).softmax(-1).view(2, 20, H, L, P)
        loc = modules.assemble_sampling_locations(ref, off_uv, off_d, d["spatial_shapes"], D)
        shapes3 = torch.cat([d["spatial_shapes"], torch.full_like(d["spatial_shapes"][:, :1], D)], -1)
        ds = _depth_score(dist, shapes3, d["level_start_index"], loc)
        expect = (ds.mean(-1) * a).flatten(-2).sum(-1, keepdim=True)
    assert wupd.shape == (2, 20, H, 1)
    torch.testing.assert_close(wupd, expect, rtol=1e-5, atol=1e-6)
    assert 0 < float(wupd.mean()) < 1
    # --- use_empty through the packed path against the loop form (forward; the fused Function gives
    # depth_score no gradient, in the reference as here)
    sca = modules.SpatialCrossAttention_DFA3D(embed_dims=E, num_cams=3, dropout=0.0, deformable_attention=attn,
                                              bev_h=7, bev_w=7, num_head=H, use_empty=True).to(DEV)
    assert attn.compute_weight_update
    args = (d["value"], d["value_dpt_dist"], d["reference_points_cam"], d["bev_mask"], d["spatial_shapes"],
            d["level_start_index"])
    with torch.no_grad():
        got = sca(d["query"], None, *args)
        want = sca_loop_form(sca, d["query"], *args)
        sca.use_empty = False
        plain = sca(d["query"], None, *args)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    assert (got - plain).abs().max() > 1e-3          # the empty embedding did contribute


def test_attention_module_options_match_grid_sample_form(lib_built, monkeypatch):
    """key_padding_mask, batch_first=False and query_pos, each against the grid_sample operator."""
    d = _inputs(13, bs=2, cams=1, Q=20)
    value = d["value"][0].permute(1, 0, 2).contiguous()            # (bs, N, E)
    dist = d["value_dpt_dist"][0].permute(1, 0, 2).contiguous()
    ref = d["reference_points_cam"][0].contiguous()                # (bs, Q, Z, 3)
    g = torch.Generator().manual_seed(5)
    pad = (torch.rand(2, value.shape[1], generator=g) < 0.3).to(DEV)
    pos = torch.randn(2, 20, 32, generator=g).to(DEV)

    def run(batch_first, use_grid_sample):
        torch.manual_seed(6)
        attn = modules.MSDeformableAttention3D_DFA3D(embed_dims=32, num_heads=2, num_levels=2, num_points=8,
                                                     batch_first=batch_first,
                                                     fuse_input_ops=not use_grid_sample,
                                                     compute_weight_update=False).to(DEV)
        _randomise(attn)
        q = d["query"].clone().requires_grad_(True)
        qq, vv, pp = (q, value, pos) if batch_first else (q.permute(1, 0, 2), value.permute(1, 0, 2),
                                                          pos.permute(1, 0, 2))
        out, _ = attn(qq, vv, dist, ref, d["spatial_shapes"], d["level_start_index"], query_pos=pp,
                      key_padding_mask=pad)
        assert out.shape == qq.shape
        out.pow(2).sum().backward()
        out = out if batch_first else out.permute(1, 0, 2)
        return out.detach(), q.grad.clone(), {n: p.grad.clone() for n, p in attn.named_parameters()}

    got_bf, got_sf = run(True, False), run(False, False)
    monkeypatch.setattr(modules, "MultiScale3DDeformableAttnFunction_fp32", _GridSampleOp)
    want = run(True, True)
    for got in (got_bf, got_sf):
        torch.testing.assert_close(got[0], want[0], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(got[1], want[1], rtol=1e-3, atol=1e-5)
        for n in want[2]:
            torch.testing.assert_close(got[2][n], want[2][n], rtol=1e-3, atol=1e-4,
                                       msg=lambda m, n=n: f"{n}: {m}")
    # the mask matters: without it the output differs
    torch.manual_seed(6)
    attn = modules.MSDeformableAttention3D_DFA3D(embed_dims=32, num_heads=2, num_levels=2, num_points=8,
                                                 compute_weight_update=False).to(DEV)
    _randomise(attn)
    with torch.no_grad():
        nomask, _ = attn(d["query"], value, dist, ref, d["spatial_shapes"], d["level_start_index"], query_pos=pos)
    assert (nomask - got_bf[0]).abs().max() > 1e-3


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
        _randomise(attn)
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


def test_encoder_stack_training_step_matches_grid_sample_form(lib_built, monkeypatch):
    """One SGD step of a 2-layer stack (cross-attention -> norm -> FFN -> norm, encoder.py:389-411):
    loss, every parameter's gradient and the updated parameters against the same stack with the
    grid_sample operator (ragged stand-in)."""
    d = _inputs(5)
    kw = dict(key=None, value=d["value"], value_dpt_dist=d["value_dpt_dist"],
              reference_points_cam=d["reference_points_cam"], bev_mask=d["bev_mask"],
              spatial_shapes=d["spatial_shapes"], level_start_index=d["level_start_index"])

    def one_step(use_grid_sample):
        torch.manual_seed(1)
        stack = modules.SCAEncoderStack(num_layers=2, embed_dims=32, ffn_dims=64, num_cams=3, num_heads=2,
                                        num_levels=2, num_points=8, dropout=0.0).to(DEV)
        for layer in stack.layers:
            _randomise(layer.cross_attn.deformable_attention)
            layer.cross_attn.deformable_attention.fuse_input_ops = not use_grid_sample
        opt = torch.optim.SGD(stack.parameters(), lr=1e-2)
        loss0 = stack(d["query"], **kw).pow(2).mean()
        loss0.backward()
        grads = {n: p.grad.clone() for n, p in stack.named_parameters()}
        opt.step()
        with torch.no_grad():
            loss1 = stack(d["query"], **kw).pow(2).mean()
        return loss0.item(), loss1.item(), grads, {n: p.detach().clone() for n, p in stack.named_parameters()}

    got = one_step(False)
    monkeypatch.setattr(modules, "MultiScale3DDeformableAttnRaggedFunction_fp32", _GridSampleRaggedOp)
    want = one_step(True)
    assert abs(got[0] - want[0]) <= 1e-4 * abs(want[0]) and abs(got[1] - want[1]) <= 1e-4 * abs(want[1])
    assert got[1] != got[0]
    for n in want[2]:
        assert torch.isfinite(got[2][n]).all()
        torch.testing.assert_close(got[2][n], want[2][n], rtol=2e-3, atol=1e-4, msg=lambda m, n=n: f"{n}: {m}")
        torch.testing.assert_close(got[3][n], want[3][n], rtol=1e-4, atol=1e-5, msg=lambda m, n=n: f"{n}: {m}")


def test_spatial_cross_attention_when_no_camera_sees_anything(lib_built):
    """Empty plan (zero packed rows): the layer reduces to output_proj(0) + residual, gradients flow to
    the residual path only, and nothing is launched with an empty grid."""
    torch.manual_seed(3)
    sca = modules.SpatialCrossAttention_DFA3D(embed_dims=32, num_cams=3, dropout=0.0,
                                              deformable_attention=modules.MSDeformableAttention3D_DFA3D(
                                                  embed_dims=32, num_heads=2, num_levels=2, num_points=8)).to(DEV)
    d = _inputs(9, bs=2)
    d["bev_mask"][:] = False
    q = d["query"].clone().requires_grad_(True)
    out = sca(q, None, d["value"], d["value_dpt_dist"], d["reference_points_cam"], d["bev_mask"],
              d["spatial_shapes"], d["level_start_index"])
    torch.testing.assert_close(out, q.detach() + sca.output_proj.bias.detach().expand_as(q))
    out.sum().backward()
    torch.testing.assert_close(q.grad, torch.ones_like(q))


class _MsdaGridSampleOp:
    """Stand-in with the 2-D Function's call signature: per-level 4-D grid_sample."""

    @staticmethod
    def apply(value, shapes2, lsi, loc, attn, im2col_step):
        return G.msda_grid_sample(value.double(), shapes2.tolist(), lsi.tolist(), loc.double(),
                                  attn.double()).to(value.dtype)


@pytest.mark.parametrize("with_prev,batch_first", [(True, True), (False, True), (True, False)])
def test_temporal_self_attention_matches_grid_sample_form(lib_built, monkeypatch, with_prev, batch_first):
    """TemporalSelfAttention (previous + current BEV, plain 2-D deformable attention on the depth-weighted
    kernels) against the same module with the 4-D grid_sample operator: output, query gradient, every
    parameter gradient (temporal_self_attention.py:130-272)."""
    bev_h, bev_w, E, H, P, bs = 8, 10, 32, 4, 4, 2
    Q = bev_h * bev_w
    g = torch.Generator().manual_seed(21)
    query = torch.randn(bs, Q, E, generator=g).to(DEV)
    prev = torch.randn(bs, Q, E, generator=g).to(DEV)
    pos = torch.randn(bs, Q, E, generator=g).to(DEV)
    refp = torch.rand(bs * 2, Q, 1, 2, generator=g).to(DEV) * 1.1 - 0.05
    shapes = torch.tensor([[bev_h, bev_w]], dtype=torch.int64, device=DEV)
    lsi = torch.zeros(1, dtype=torch.int64, device=DEV)

    def run():
        torch.manual_seed(5)
        tsa = modules.TemporalSelfAttention(embed_dims=E, num_heads=H, num_levels=1, num_points=P, dropout=0.0,
                                            batch_first=batch_first).to(DEV)
        with torch.no_grad():
            tsa.sampling_offsets.weight.normal_(0, 0.05)
            tsa.attention_weights.weight.normal_(0, 0.05)
        q = query.clone().requires_grad_(True)
        value = torch.stack([prev, q], 1).reshape(bs * 2, Q, E) if with_prev else None
        qq, pp = (q, pos) if batch_first else (q.permute(1, 0, 2), pos.permute(1, 0, 2))
        vv = value if (value is None or batch_first) else value.permute(1, 0, 2)
        out = tsa(qq, value=vv, query_pos=pp, reference_points=refp, spatial_shapes=shapes, level_start_index=lsi)
        assert out.shape == qq.shape
        out.pow(2).sum().backward()
        out = out if batch_first else out.permute(1, 0, 2)
        return out.detach(), q.grad.clone(), {n: p.grad.clone() for n, p in tsa.named_parameters()}

    got = run()
    monkeypatch.setattr(modules, "MultiScaleDeformableAttnFunction_fp32", _MsdaGridSampleOp)
    want = run()
    torch.testing.assert_close(got[0], want[0], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(got[1], want[1], rtol=1e-3, atol=1e-4)
    for n in want[2]:
        torch.testing.assert_close(got[2][n], want[2][n], rtol=1e-3, atol=1e-4, msg=lambda m, n=n: f"{n}: {m}")


def test_full_encoder_layer_is_the_composition_of_its_blocks(lib_built):
    """BEVFormerEncoderLayer = temporal self-attention -> norm -> spatial cross-attention -> norm -> FFN ->
    norm (encoder.py:363-411): its output equals the blocks applied by hand, and every parameter gets a
    finite gradient."""
    torch.manual_seed(7)
    bev_h, bev_w, E = 5, 10, 32
    layer = modules.BEVFormerEncoderLayer(embed_dims=E, ffn_dims=64, num_cams=3, num_heads=2, num_levels=2,
                                          num_points=8, bev_h=bev_h, bev_w=bev_w, dropout=0.0).to(DEV)
    _randomise(layer.cross_attn.deformable_attention)
    d = _inputs(17, bs=1, Q=bev_h * bev_w)
    kw = dict(key=None, value=d["value"], value_dpt_dist=d["value_dpt_dist"],
              reference_points_cam=d["reference_points_cam"], bev_mask=d["bev_mask"],
              spatial_shapes=d["spatial_shapes"], level_start_index=d["level_start_index"])
    g = torch.Generator().manual_seed(2)
    prev = torch.randn(2, bev_h * bev_w, E, generator=g).to(DEV)
    pos = torch.randn(1, bev_h * bev_w, E, generator=g).to(DEV)
    q = d["query"].clone().requires_grad_(True)
    out = layer(q, prev_bev=prev, bev_pos=pos, **kw)
    with torch.no_grad():
        ref2d = modules.bev_reference_points(bev_h, bev_w, dim="2d", bs=2, device=DEV)
        shapes = torch.tensor([[bev_h, bev_w]], dtype=torch.int64, device=DEV)
        x = layer.norm0(layer.self_attn(d["query"], value=prev, query_pos=pos, reference_points=ref2d,
                                        spatial_shapes=shapes, level_start_index=torch.zeros(1, dtype=torch.int64,
                                                                                             device=DEV)))
        x = layer.norm1(layer.cross_attn(x, **kw))
        want = layer.norm2(x + layer.ffn(x))
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-6)
    out.pow(2).mean().backward()
    assert torch.isfinite(q.grad).all() and q.grad.abs().sum() > 0
    for n, p in layer.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), n


@pytest.mark.parametrize("ref_dim", [2, 4])
def test_decoder_attention_matches_grid_sample_form(lib_built, monkeypatch, ref_dim):
    """CustomMSDeformableAttention (object queries -> BEV, decoder.py:231-345), with point and with box
    reference points, against the same module on the 4-D grid_sample operator."""
    E, H, L, P, bs, Q = 32, 4, 2, 4, 2, 37
    levels = ((8, 10), (4, 5))
    N = sum(h * w for h, w in levels)
    g = torch.Generator().manual_seed(33)
    query = torch.randn(Q, bs, E, generator=g).to(DEV)
    pos = torch.randn(Q, bs, E, generator=g).to(DEV)
    bev = torch.randn(N, bs, E, generator=g).to(DEV)
    refp = torch.rand(bs, Q, L, ref_dim, generator=g).to(DEV)
    shapes = torch.tensor(levels, dtype=torch.int64, device=DEV)
    lsi = torch.tensor([0, levels[0][0] * levels[0][1]], dtype=torch.int64, device=DEV)

    def run():
        torch.manual_seed(9)
        m = modules.CustomMSDeformableAttention(embed_dims=E, num_heads=H, num_levels=L, num_points=P,
                                                dropout=0.0).to(DEV)
        with torch.no_grad():
            m.sampling_offsets.weight.normal_(0, 0.05)
            m.attention_weights.weight.normal_(0, 0.05)
        q = query.clone().requires_grad_(True)
        v = bev.clone().requires_grad_(True)
        out = m(q, value=v, query_pos=pos, reference_points=refp, spatial_shapes=shapes, level_start_index=lsi)
        assert out.shape == q.shape
        out.pow(2).sum().backward()
        return out.detach(), q.grad.clone(), v.grad.clone(), {n: p.grad.clone() for n, p in m.named_parameters()}

    got = run()
    monkeypatch.setattr(modules, "MultiScaleDeformableAttnFunction_fp32", _MsdaGridSampleOp)
    want = run()
    torch.testing.assert_close(got[0], want[0], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(got[1], want[1], rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(got[2], want[2], rtol=1e-3, atol=1e-4)
    for n in want[3]:
        torch.testing.assert_close(got[3][n], want[3][n], rtol=1e-3, atol=1e-4, msg=lambda m_, n=n: f"{n}: {m_}")
