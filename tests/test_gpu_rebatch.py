"""GPU tests of the per-camera re-batching kernels and of the ragged (variable queries per camera)
operator entry points, against the loop form of the reference's spatial cross-attention
(BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/spatial_cross_attention.py:700-722, 741-748)
and against the dense entry points run camera by camera."""
import numpy as np
import pytest
import torch

from dfa3d_b200 import workloads as wl
from helpers import BWD, FWD, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def M(lib_built):
    import dfa3d_b200
    assert torch.cuda.is_available()
    return dfa3d_b200


def ragged_mask(cams, bs, Q, Z, seed, empty_camera=None):
    g = torch.Generator().manual_seed(seed)
    m = torch.rand(cams, bs, Q, Z, generator=g) < torch.linspace(0.05, 0.4, cams).view(cams, 1, 1, 1)
    if empty_camera is not None:
        m[empty_camera] = False
    return m


def loop_indexes(bev_mask):
    """The reference's per-camera lists (:703-706)."""
    return [mask_per_img[0].sum(-1).nonzero().squeeze(-1) for mask_per_img in bev_mask]


@pytest.mark.parametrize("cams,bs,Q,Z,empty", [(6, 2, 2500, 4, 3), (3, 1, 77, 1, None), (2, 3, 1, 2, 0),
                                               (6, 1, 40000, 4, None)])
def test_plan_matches_the_loop_form(M, cams, bs, Q, Z, empty):
    from dfa3d_b200.rebatch import RebatchPlan
    mask = ragged_mask(cams, bs, Q, Z, seed=cams * 100 + Q, empty_camera=empty)
    plan = RebatchPlan(mask.to(DEV))
    idx = loop_indexes(mask)
    lens = [len(i) for i in idx]
    assert plan.counts.tolist() == lens and plan.rows == sum(lens) and plan.max_queries == max(lens)
    off = np.concatenate([[0], np.cumsum(lens)])
    assert plan.offsets.tolist() == off.tolist()
    T = plan.rows
    assert plan.op_offsets.tolist() == [j * T + int(off[i]) for j in range(bs) for i in range(cams)] + [bs * T]
    assert plan.packed_query.tolist() == torch.cat(idx).tolist()
    assert plan.packed_camera.tolist() == sum(([i] * n for i, n in enumerate(lens)), [])
    row_of = torch.full((cams, Q), -1, dtype=torch.int64)
    for i, ix in enumerate(idx):
        row_of[i, ix] = torch.arange(len(ix)) + int(off[i])
    assert torch.equal(plan.row_of.cpu().long(), row_of)
    count = (mask.sum(-1) > 0).permute(1, 2, 0).sum(-1).clamp(min=1.0)
    assert torch.equal(plan.inv_count.cpu(), 1.0 / count)


@pytest.mark.parametrize("E", [256, 12, 7])
def test_gather_and_combine_match_the_loop_form(M, E):
    """Queries gathered per camera, per-camera results combined into BEV order, and both gradients."""
    from dfa3d_b200.rebatch import (CombineCamerasFunction, GatherQueriesFunction, GatherSharedRowsFunction,
                                    RebatchPlan, gather_per_camera)
    cams, bs, Q, Z = 5, 2, 300, 4
    mask = ragged_mask(cams, bs, Q, Z, seed=7, empty_camera=2)
    mask[:, 1] = ragged_mask(cams, 1, Q, Z, seed=8)[:, 0]      # batch element 1 sees differently
    plan = RebatchPlan(mask.to(DEV))
    idx = loop_indexes(mask)
    T, max_len = plan.rows, max(len(i) for i in idx)
    g = torch.Generator().manual_seed(1)
    query = torch.randn(bs, Q, E, generator=g)
    refpts = torch.randn(cams, bs, Q, Z, 3, generator=g)
    shared = torch.randn(Q, E, generator=g)
    weight = torch.randn(bs * T, E, generator=g)             # stands for what the attention does per row

    # ---- loop form (padded), as in the reference ----
    q_ref = query.clone().requires_grad_(True)
    s_ref = shared.clone().requires_grad_(True)
    queries_rebatch = q_ref.new_zeros(bs, cams, max_len, E)
    ref_rebatch = refpts.new_zeros(bs, cams, max_len, Z, 3)
    shared_rebatch = q_ref.new_zeros(bs, cams, max_len, E)
    pieces_q, pieces_r, pieces_s = [], [], []
    for j in range(bs):
        for i in range(cams):
            ix = idx[i]
            queries_rebatch = queries_rebatch.index_put(
                (torch.tensor(j), torch.tensor(i), torch.arange(len(ix))), q_ref[j, ix])
            ref_rebatch[j, i, :len(ix)] = refpts[i, j, ix]
            shared_rebatch = shared_rebatch.index_put(
                (torch.tensor(j), torch.tensor(i), torch.arange(len(ix))), s_ref[ix])
    slots = torch.zeros(bs, Q, E)
    out_rows = []
    for j in range(bs):
        for i in range(cams):
            ix = idx[i]
            rows = slice(j * T + int(plan.offsets[i]), j * T + int(plan.offsets[i]) + len(ix))
            per_cam = (queries_rebatch[j, i, :len(ix)] + shared_rebatch[j, i, :len(ix)]) * weight[rows]
            slots = slots.index_put((torch.tensor(j), ix), per_cam, accumulate=True)
            pieces_q.append(queries_rebatch[j, i, :len(ix)]); pieces_r.append(ref_rebatch[j, i, :len(ix)])
    count = (mask.sum(-1) > 0).permute(1, 2, 0).sum(-1).clamp(min=1.0)
    slots = slots / count[..., None]
    gslots = torch.randn(bs, Q, E, generator=g)
    slots.backward(gslots)

    # ---- kernels ----
    q = query.to(DEV).requires_grad_(True)
    s = shared.to(DEV).requires_grad_(True)
    packed_q = GatherQueriesFunction.apply(q, plan)
    packed_s = GatherSharedRowsFunction.apply(s, plan)
    packed_r = gather_per_camera(refpts.to(DEV), plan)
    assert torch.equal(packed_q.cpu(), torch.cat(pieces_q).detach())
    assert torch.equal(packed_r.cpu(), torch.cat(pieces_r))
    got = CombineCamerasFunction.apply((packed_q + packed_s) * weight.to(DEV), plan)
    assert_close("slots", got, slots.detach(), **FWD)
    got.backward(gslots.to(DEV))
    assert_close("grad_query", q.grad, q_ref.grad, **BWD)
    assert_close("grad_shared", s.grad, s_ref.grad, **BWD)


def _per_camera_problem(w, lens, seed):
    """Packed inputs for cameras with lens[b] queries each + the same data as a list of dense B=1 dicts."""
    g = torch.Generator().manual_seed(seed)
    d = wl.make_inputs(w.with_(B=len(lens), Q=max(max(lens), 1)), seed=seed)
    dense = []
    for b, n in enumerate(lens):
        dense.append({"value": d["value"][b:b + 1], "dist": d["dist"][b:b + 1], "loc": d["loc"][b:b + 1, :n],
                      "attn": d["attn"][b:b + 1, :n], "grad_out": d["grad_out"][b:b + 1, :n]})
    packed = {k: torch.cat([x[k][0] for x in dense]) for k in ("loc", "attn", "grad_out")}
    off = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    return d, dense, packed, off, g


@pytest.mark.parametrize("packed", [False, True], ids=["item_per_warp", "items_share_a_warp"])
@pytest.mark.parametrize("lens", [[5, 0, 9, 2], [33], [0, 0, 4]])
def test_ragged_fused_entry_points_match_dense_per_camera(M, lens, packed):
    from dfa3d_b200 import ext
    w = wl.WORKLOADS["odd"].with_(C=32)
    if packed:                                   # L*P = 8: the kernels in which a warp holds 4 items
        w = w.with_(levels=((9, 6), (4, 5)), P=4)
    d, dense, packed, off, _ = _per_camera_problem(w, lens, seed=5)
    t = {k: v.to(DEV) for k, v in d.items()}
    p = {k: v.to(DEV).contiguous() for k, v in packed.items()}
    off = off.to(DEV)
    out, ds = ext.dfa3d_fused_forward_ragged(t["value"], t["dist"], t["shapes"], t["lsi"], p["loc"], p["attn"],
                                             off, max(lens))
    gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
    gl = torch.empty_like(p["loc"]); ga = torch.empty_like(p["attn"])
    ext.dfa3d_fused_backward_ragged(t["value"], t["dist"], t["shapes"], t["lsi"], p["loc"], p["attn"], off,
                                    max(lens), p["grad_out"], gv, gd, gl, ga)
    r0 = 0
    for b, n in enumerate(lens):
        x = {k: v.to(DEV).contiguous() for k, v in dense[b].items()}
        o, s = ext.dfa3d_fused_forward(x["value"], x["dist"], t["shapes"], t["lsi"], x["loc"], x["attn"], 64)
        gv1 = torch.zeros_like(x["value"]); gd1 = torch.zeros_like(x["dist"])
        gl1 = torch.empty_like(x["loc"]); ga1 = torch.empty_like(x["attn"])
        ext.dfa3d_fused_backward(x["value"], x["dist"], t["shapes"], t["lsi"], x["loc"], x["attn"],
                                 x["grad_out"], gv1, gd1, gl1, ga1, 64)
        assert torch.equal(out[r0:r0 + n], o[0]) and torch.equal(ds[r0:r0 + n], s[0])
        assert torch.equal(gl[r0:r0 + n], gl1[0]) and torch.equal(ga[r0:r0 + n], ga1[0])
        assert_close("grad_value", gv[b:b + 1], gv1, **BWD)
        assert_close("grad_dist", gd[b:b + 1], gd1, **BWD)
        r0 += n


@pytest.mark.parametrize("packed", [False, True], ids=["item_per_warp", "items_share_a_warp"])
def test_ragged_offsets_entry_points_match_dense_per_camera(M, packed):
    from dfa3d_b200 import ext
    lens, Z = [7, 0, 12], 2
    w = wl.WORKLOADS["odd"].with_(C=32, P=4)
    if packed:                                   # L*P = 16: the kernels in which a warp holds 2 items
        w = w.with_(levels=((9, 6), (4, 5), (2, 2), (1, 1)))
    d, dense, packed, off, g = _per_camera_problem(w, lens, seed=9)
    R = sum(lens)
    ref = torch.rand(R, Z, 3, generator=g) * 1.2 - 0.1
    off_uv = torch.randn(R, w.H, w.L, w.P, 2, generator=g) * 1.5
    off_d = torch.randn(R, w.H, w.L, w.P, generator=g)
    logits = torch.randn(R, w.H, w.L * w.P, generator=g)
    t = {k: v.to(DEV) for k, v in d.items()}
    go = packed["grad_out"].to(DEV).contiguous()
    offd = off.to(DEV)
    args = [x.to(DEV) for x in (ref, off_uv, off_d, logits)]
    out = ext.dfa3d_attn3d_forward_ragged(t["value"], t["dist"], t["shapes"], t["lsi"], *args, offd, max(lens))
    gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
    guv, gdd, glg = torch.empty_like(args[1]), torch.empty_like(args[2]), torch.empty_like(args[3])
    ext.dfa3d_attn3d_backward_ragged(t["value"], t["dist"], t["shapes"], t["lsi"], *args, offd, max(lens), go,
                                     gv, gd, guv, gdd, glg)
    r0 = 0
    for b, n in enumerate(lens):
        if n == 0:
            assert not gv[b].any() and not gd[b].any()
            continue
        a1 = [x[r0:r0 + n][None].contiguous() for x in args]
        v1, d1 = t["value"][b:b + 1], t["dist"][b:b + 1]
        o = ext.dfa3d_attn3d_forward(v1, d1, t["shapes"], t["lsi"], *a1)
        gv1 = torch.zeros_like(v1); gd1 = torch.zeros_like(d1)
        g1 = [torch.empty_like(x) for x in a1[1:]]
        ext.dfa3d_attn3d_backward(v1, d1, t["shapes"], t["lsi"], *a1, go[r0:r0 + n][None].contiguous(), gv1, gd1,
                                  *g1)
        assert torch.equal(out[r0:r0 + n], o[0])
        assert torch.equal(guv[r0:r0 + n], g1[0][0]) and torch.equal(gdd[r0:r0 + n], g1[1][0])
        assert torch.equal(glg[r0:r0 + n], g1[2][0])
        assert_close("grad_value", gv[b:b + 1], gv1, **BWD)
        assert_close("grad_dist", gd[b:b + 1], gd1, **BWD)
        r0 += n
