"""GPU tests of the depth-distribution producer and of the operator's single-map (`dist_map`) option
against the tensor expressions of the reference: softmax / sigmoid over the channels and one
F.interpolate(mode="nearest") per level (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/dense_heads/
depth_head.py:265-276), flattened and concatenated channel-last (…/modules/transformer.py:368-391)."""
import pytest
import torch
import torch.nn.functional as F

from dfa3d_b200 import workloads as wl
from helpers import BWD, FWD, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def reference_dist(logits, levels, activation):
    """(B, D, h, w) logits -> (B, N, D), the reference's way."""
    p = logits.softmax(1) if activation == "softmax" else logits.sigmoid()
    per_level = [F.interpolate(p, size=tuple(hw), mode="nearest").flatten(2).permute(0, 2, 1) for hw in levels]
    return torch.cat(per_level, 1)


def level_tensors(levels):
    shapes = torch.tensor(levels, dtype=torch.int64)
    hw = shapes[:, 0] * shapes[:, 1]
    lsi = torch.cat([hw.new_zeros(1), hw.cumsum(0)[:-1]])
    return shapes.to(DEV), lsi.to(DEV), int(hw.sum())


CASES = {
    # map size, levels: equal size, exact halvings, non-integer ratios up and down, a 1x1 level
    "pyramid": ((12, 20), ((24, 40), (12, 20), (6, 10), (3, 5)), 64),
    "odd_ratios": ((13, 21), ((29, 50), (15, 25), (7, 11), (1, 1)), 118),
    "bevformer_like": ((58, 100), ((116, 200), (58, 100), (29, 50), (15, 25)), 64),
    "wide_map": ((5, 70), ((3, 33), (10, 140)), 7),
}


@pytest.mark.parametrize("activation", ["softmax", "sigmoid"])
@pytest.mark.parametrize("case", sorted(CASES))
def test_producer_matches_softmax_and_nearest_resize(lib_built, case, activation):
    from dfa3d_b200.dist_producer import depth_distribution
    (mh, mw), levels, D = CASES[case]
    g = torch.Generator().manual_seed(len(case))
    logits = (torch.randn(3, D, mh, mw, generator=g) * 3).to(DEV).requires_grad_(True)
    shapes, lsi, N = level_tensors(levels)
    ref_leaf = logits.detach().clone().requires_grad_(True)
    want = reference_dist(ref_leaf, levels, activation)
    got = depth_distribution(logits, shapes, lsi, N, activation=activation)
    assert got.shape == (3, N, D)
    assert_close("dist", got, want, rtol=2e-6, atol=1e-9)
    gd = torch.randn(3, N, D, generator=g).to(DEV)
    got.backward(gd)
    want.backward(gd)
    assert_close("grad_logits", logits.grad, ref_leaf.grad, rtol=1e-4, atol_frac=2e-6)
    # bf16 output: the fp32 result rounded once
    got16 = depth_distribution(logits.detach(), shapes, lsi, N, activation=activation, dtype=torch.bfloat16)
    assert got16.dtype == torch.bfloat16
    diff = (got16.float() - want.detach().bfloat16().float()).abs()
    assert (diff <= want.detach().abs() * 2 ** -7).all()          # at most one bf16 ulp apart
    goth = depth_distribution(logits.detach(), shapes, lsi, N, activation=activation, dtype=torch.float16)
    assert goth.dtype == torch.float16
    diff = (goth.float() - want.detach().half().float()).abs()
    assert (diff <= want.detach().abs() * 2 ** -10 + 2 ** -24).all()   # one fp16 ulp (subnormal step 2^-24)
    assert (diff > 0).float().mean() < 1e-3


def _resized_copies(dist_map_tensor, map_hw, levels):
    """(B, mh*mw, D) map -> (B, N, D): what the reference materialises for the operator."""
    B, _, D = dist_map_tensor.shape
    img = dist_map_tensor.view(B, map_hw[0], map_hw[1], D).permute(0, 3, 1, 2)
    return torch.cat([F.interpolate(img, size=tuple(hw), mode="nearest").flatten(2).permute(0, 2, 1)
                      for hw in levels], 1).contiguous()


@pytest.mark.parametrize("map_hw", [(9, 6), (5, 4), (20, 11)])
def test_single_map_option_equals_resized_copies(lib_built, map_hw):
    """The operator reading ONE dist map with nearest indexing gives bit-identical outputs to the
    operator fed with the per-level resized copies; grad_dist of the map is the sum of the copies'
    gradients (autograd of F.interpolate)."""
    import dfa3d_b200 as M
    from dfa3d_b200 import ext
    w = wl.WORKLOADS["odd"].with_(C=32)                   # levels (9,6), (4,5), (2,2)
    d = wl.make_inputs(w)
    t = {k: v.to(DEV) for k, v in d.items()}
    g = torch.Generator().manual_seed(3)
    dmap = torch.randn(w.B, map_hw[0] * map_hw[1], w.D, generator=g).softmax(-1).to(DEV)
    full_leaf = dmap.clone().requires_grad_(True)
    full = _resized_copies(full_leaf, map_hw, w.levels)
    # resized copies, the dense Function
    leaves = [t["value"].clone().requires_grad_(True), t["loc"].clone().requires_grad_(True),
              t["attn"].clone().requires_grad_(True)]
    out_f, ds_f = M.MultiScale3DDeformableAttnFunction.apply(leaves[0], full, t["shapes"], t["lsi"], leaves[1],
                                                            leaves[2], 64)
    out_f.backward(t["grad_out"])
    # single map
    mine = [t["value"].clone().requires_grad_(True), dmap.clone().requires_grad_(True),
            t["loc"].clone().requires_grad_(True), t["attn"].clone().requires_grad_(True)]
    out_m, ds_m = M.MultiScale3DDeformableAttnFunction.apply(mine[0], mine[1], t["shapes"], t["lsi"], mine[2],
                                                            mine[3], 64, True, map_hw)
    out_m.backward(t["grad_out"])
    assert torch.equal(out_m, out_f) and torch.equal(ds_m, ds_f)
    assert torch.equal(mine[2].grad, leaves[1].grad) and torch.equal(mine[3].grad, leaves[2].grad)
    assert_close("grad_value", mine[0].grad, leaves[0].grad, **BWD)
    assert_close("grad_dist_map", mine[1].grad, full_leaf.grad, **BWD)
    # the offsets/logits entry points and the two-stage depth sampling take the option too
    Z = 1
    ref = torch.rand(w.B, w.Q, Z, 3, generator=g).to(DEV)
    off_uv = (torch.randn(w.B, w.Q, w.H, w.L, w.P, 2, generator=g) * 1.5).to(DEV)
    off_d = torch.randn(w.B, w.Q, w.H, w.L, w.P, generator=g).to(DEV)
    logits = torch.randn(w.B, w.Q, w.H, w.L * w.P, generator=g).to(DEV)
    o1 = ext.dfa3d_attn3d_forward(t["value"], full.detach(), t["shapes"], t["lsi"], ref, off_uv, off_d, logits)
    o2 = ext.dfa3d_attn3d_forward(t["value"], dmap, t["shapes"], t["lsi"], ref, off_uv, off_d, logits,
                                  dist_map=map_hw)
    assert torch.equal(o1, o2)
    s1 = ext.ms_depth_score_sample_forward(full.detach(), t["shapes"], t["lsi"], t["loc"], 64)
    s2 = ext.ms_depth_score_sample_forward(dmap, t["shapes"], t["lsi"], t["loc"], 64, dist_map=map_hw)
    assert torch.equal(s1, s2)
    with pytest.raises(RuntimeError, match="inconsistent shapes"):
        ext.dfa3d_fused_forward(t["value"], dmap, t["shapes"], t["lsi"], t["loc"], t["attn"], 64,
                                dist_map=(map_hw[0] + 1, map_hw[1]))


def test_producer_feeds_the_operator_end_to_end(lib_built):
    """logits -> producer (single map, bf16) -> operator with dist_map: gradient reaches the logits."""
    import dfa3d_b200 as M
    from dfa3d_b200.dist_producer import depth_distribution
    w = wl.WORKLOADS["odd"].with_(C=32)
    d = wl.make_inputs(w)
    t = {k: v.to(DEV) for k, v in d.items()}
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(w.B, w.D, 9, 6, generator=g).to(DEV).requires_grad_(True)
    dist, hw = depth_distribution(logits, single_map=True)
    assert hw == (9, 6) and dist.shape == (w.B, 54, w.D)
    out, _ = M.MultiScale3DDeformableAttnFunction.apply(t["value"], dist, t["shapes"], t["lsi"], t["loc"],
                                                       t["attn"], 64, False, hw)
    out.backward(t["grad_out"])
    # the same through torch expressions and the dense operator
    leaf = logits.detach().clone().requires_grad_(True)
    full = reference_dist(leaf, w.levels, "softmax")
    out2, _ = M.MultiScale3DDeformableAttnFunction.apply(t["value"], full, t["shapes"], t["lsi"], t["loc"],
                                                        t["attn"], 64, False)
    out2.backward(t["grad_out"])
    assert_close("out", out, out2, **FWD)
    assert_close("grad_logits", logits.grad, leaf.grad, rtol=1e-4, atol_frac=1e-5)
