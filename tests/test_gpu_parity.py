"""GPU parity tests: the CUDA path (through the C ABI, via the reference-shaped Python API) against the
CPU oracle, the committed golden vectors and -- when its build travelled to the box -- the reference's
own CUDA op, on identical seeded inputs."""
import glob
import os

import numpy as np
import pytest
import torch

from dfa3d_b200 import workloads as wl
from helpers import BF16, BWD, FWD, assert_close, oracle_all

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DEV = "cuda"


@pytest.fixture(scope="module")
def M(lib_built):
    import dfa3d_b200
    assert torch.cuda.is_available()
    return dfa3d_b200


@pytest.fixture(scope="module")
def REF():
    import build_ref
    try:
        return build_ref.load()
    except ImportError as e:
        pytest.skip(f"reference op not available: {e}")


def run_fused(M, d, shared_dist, bf16=False, fn=None, storage=torch.bfloat16):
    """One-stage Function forward + backward on the GPU.  d: CPU dict with head-repeated dist."""
    fn = fn or M.MultiScale3DDeformableAttnFunction
    value, dist = d["value"], d["dist"]
    if shared_dist:
        dist = dist[:, :, 0].contiguous()
    value, dist = value.to(DEV), dist.to(DEV)
    loc = d["loc"].to(DEV).requires_grad_(True)
    attn = d["attn"].to(DEV).requires_grad_(True)
    shapes, lsi, go = d["shapes"].to(DEV), d["lsi"].to(DEV), d["grad_out"].to(DEV)
    if bf16:   # bf16 storage: gradients for value/dist are taken through the low-level entry points
        from dfa3d_b200 import ext
        vb, db = value.to(storage), dist.to(storage)
        out, ds = ext.dfa3d_fused_forward(vb, db, shapes, lsi, loc.detach(), attn.detach(), 64)
        gv = torch.zeros_like(value); gd = torch.zeros_like(dist)
        gl = torch.empty_like(loc); ga = torch.empty_like(attn)
        ext.dfa3d_fused_backward(vb, db, shapes, lsi, loc.detach(), attn.detach(), go, gv, gd, gl, ga, 64)
        return dict(out=out, ds=ds, grad_value=gv, grad_dist=gd, grad_loc=gl, grad_attn=ga)
    value.requires_grad_(True); dist.requires_grad_(True)
    out, ds = fn.apply(value, dist, shapes, lsi, loc, attn, 64)
    out.backward(go)
    return dict(out=out, ds=ds, grad_value=value.grad, grad_dist=dist.grad, grad_loc=loc.grad,
                grad_attn=attn.grad)


def check_against(got, ref, shared_dist, fwd=FWD, bwd=BWD):
    assert_close("out", got["out"], ref["out"], **fwd)
    assert_close("depth_score", got["ds"], ref["ds"], **fwd)
    gd = ref["grad_dist"].sum(2) if shared_dist else ref["grad_dist"]
    assert_close("grad_value", got["grad_value"], ref["grad_value"], **bwd)
    assert_close("grad_dist", got["grad_dist"], gd, **bwd)
    assert_close("grad_loc", got["grad_loc"], ref["grad_loc"], **bwd)
    assert_close("grad_attn", got["grad_attn"], ref["grad_attn"], **bwd)


@pytest.mark.parametrize("shared_dist", [False, True], ids=["dist_per_head", "dist_shared"])
@pytest.mark.parametrize("name", ["tiny", "odd", "cfg0"])
def test_fused_matches_oracle(M, name, shared_dist):
    d = wl.make_inputs(wl.WORKLOADS[name], head_repeat=True)
    got = run_fused(M, d, shared_dist)
    check_against(got, oracle_all(d, np.float32), shared_dist)
    # continuous outputs also against the fp64 oracle (depth_score slots and location gradients jump
    # at cell borders, where fp32 and fp64 coordinates may fall on different sides)
    o64 = oracle_all(d, np.float64)
    assert_close("out/f64", got["out"], o64["out"], **FWD)
    assert_close("grad_value/f64", got["grad_value"], o64["grad_value"], **BWD)
    assert_close("grad_attn/f64", got["grad_attn"], o64["grad_attn"], **BWD)


CHANNEL_CASES = {
    # vector kernels: C/4 in {2,4,8,16,32}; everything else takes the any-width kernel
    "C8": dict(C=8), "C16": dict(C=16), "C64": dict(C=64, H=2), "C12_generic": dict(C=12),
    "C20_generic": dict(C=20, H=3), "C128": dict(C=128, H=1), "C256_generic": dict(C=256, H=1),
    "LP45_two_chunks": dict(levels=((6, 5), (4, 4), (3, 3), (2, 3), (1, 1)), P=9),
    "LP32_exact": dict(levels=((6, 5), (4, 4), (3, 3), (2, 3)), P=8),
    "one_pixel_levels": dict(levels=((1, 1), (1, 2)), D=1),
    "D2": dict(D=2),
}


@pytest.mark.parametrize("case", sorted(CHANNEL_CASES))
def test_shape_coverage_matches_oracle(M, case):
    w = wl.WORKLOADS["tiny"].with_(name=case, seed=100 + len(case), Q=19, **CHANNEL_CASES[case])
    d = wl.make_inputs(w, head_repeat=True)
    ref = oracle_all(d, np.float32)
    for shared in (False, True):
        check_against(run_fused(M, d, shared), ref, shared)


@pytest.mark.parametrize("case", ["C16", "C32", "C64", "C24_generic"])
def test_bf16_storage_matches_oracle(M, case):
    """bf16 value/dist, fp32 accumulation and gradients: the oracle consumes the same bf16-rounded
    numbers in fp32, so the 1e-2 relative bound allowed for bf16 storage is met with a wide margin; the fp32-level
    tolerance is what is asserted."""
    C = int(case[1:3])
    w = wl.WORKLOADS["odd"].with_(name=case, C=C, value_dtype="bf16", seed=7)
    d = wl.make_inputs(w, head_repeat=True)
    ref = oracle_all(d, np.float32)
    for shared in (False, True):
        got = run_fused(M, d, shared, bf16=True)
        check_against(got, ref, shared)
        check_against(got, ref, shared, fwd=BF16, bwd=BF16)


@pytest.mark.parametrize("case", ["C16", "C32", "C64", "C128", "C24_generic"])
def test_fp16_storage_matches_oracle(M, case):
    """IEEE half value/dist (what the reference's *_fp16 Functions hand to the extension), fp32 arithmetic
    and gradients: the oracle consumes the same half-rounded numbers in fp32 and the fp32-level tolerance is
    asserted."""
    C = int(case[1:].split("_")[0])
    w = wl.WORKLOADS["odd"].with_(name=case, C=C, H=2 if C == 128 else 8, value_dtype="fp16", seed=8)
    d = wl.make_inputs(w, head_repeat=True)
    ref = oracle_all(d, np.float32)
    for shared in (False, True):
        check_against(run_fused(M, d, shared, bf16=True, storage=torch.float16), ref, shared)


def test_fp16_functions_like_the_reference_variants(M):
    """The *_fp16 Function variants (…attn_function.py:24,183,353) with half tensors throughout, as the
    reference's modules call them when value is half: outputs are half, equal to the fp32 oracle on the
    half-rounded inputs up to the output rounding; gradients arrive in the dtype of their inputs.  One-stage
    and two-stage."""
    w = wl.WORKLOADS["odd"].with_(C=32, seed=41)
    d = wl.make_inputs(w, head_repeat=True)
    h = {k: (v.half() if v.is_floating_point() else v) for k, v in d.items()}
    ref = oracle_all({k: (v.float() if v.is_floating_point() else v) for k, v in h.items()}, np.float32)
    shapes, lsi, go = d["shapes"].to(DEV), d["lsi"].to(DEV), h["grad_out"].to(DEV)
    HALF = dict(rtol=2e-3, atol=0.0, atol_frac=1e-3)        # half an ulp of fp16 = 2^-11

    def leaves():
        return [h[k].to(DEV).requires_grad_(True) for k in ("value", "dist", "loc", "attn")]

    value, dist, loc, attn = leaves()
    out, ds = M.MultiScale3DDeformableAttnFunction_fp16.apply(value, dist, shapes, lsi, loc, attn, 64)
    assert out.dtype == torch.float16 and ds.dtype == torch.float16
    out.backward(go)
    got1 = dict(out=out, ds=ds, grad_value=value.grad, grad_dist=dist.grad, grad_loc=loc.grad, grad_attn=attn.grad)
    value, dist, loc, attn = leaves()
    ds2 = M.MultiScaleDepthScoreSampleFunction_fp16.apply(dist, shapes, lsi, loc, 64)
    out2 = M.WeightedMultiScaleDeformableAttnFunction_fp16.apply(
        value, shapes[:, :2].contiguous(), lsi, loc[..., :2].contiguous(), attn, ds2, 64)
    assert out2.dtype == torch.float16 and ds2.dtype == torch.float16
    out2.backward(go)
    got2 = dict(out=out2, ds=ds2, grad_value=value.grad, grad_dist=dist.grad, grad_loc=loc.grad,
                grad_attn=attn.grad)
    for tag, got, tol in (("one-stage", got1, HALF), ("two-stage", got2, dict(rtol=8e-3, atol=0.0, atol_frac=4e-3))):
        for k in ("grad_value", "grad_dist", "grad_loc", "grad_attn"):
            assert got[k].dtype == torch.float16, (tag, k)
        # the two-stage path rounds depth_score to half between its stages
        for k in ("out", "ds", "grad_value", "grad_dist", "grad_attn"):
            assert_close(f"{tag}/{k}", got[k].float(), ref[k], **tol)


def test_fp16_functions_under_autocast(M):
    """Under autocast the *_fp16 variants cast float32 inputs to half themselves (custom_fwd cast_inputs), the
    *_fp32 ones cast half inputs to float32."""
    d = wl.make_inputs(wl.WORKLOADS["tiny"], head_repeat=True)
    t = {k: v.to(DEV) for k, v in d.items()}
    with torch.autocast("cuda", dtype=torch.float16):
        out16, _ = M.MultiScale3DDeformableAttnFunction_fp16.apply(t["value"], t["dist"], t["shapes"], t["lsi"],
                                                                   t["loc"], t["attn"], 64)
        out32, _ = M.MultiScale3DDeformableAttnFunction_fp32.apply(t["value"].half(), t["dist"].half(),
                                                                   t["shapes"], t["lsi"], t["loc"], t["attn"], 64)
    assert out16.dtype == torch.float16 and out32.dtype == torch.float32
    assert_close("autocast", out16.float(), out32, rtol=2e-2, atol=0.0, atol_frac=1e-2)


def test_fp16_needs_value_and_dist_in_half_together(M):
    from dfa3d_b200 import ext
    t = {k: v.to(DEV) for k, v in wl.make_inputs(wl.WORKLOADS["tiny"]).items()}
    with pytest.raises(RuntimeError, match="fp16 storage"):
        ext.dfa3d_fused_forward(t["value"].half(), t["dist"], t["shapes"], t["lsi"], t["loc"], t["attn"], 64)
    with pytest.raises(RuntimeError, match="fp16 storage"):
        ext.dfa3d_fused_forward(t["value"], t["dist"].half(), t["shapes"], t["lsi"], t["loc"], t["attn"], 64)


def test_fp16_storage_in_every_entry_point(M):
    """Each kernel instantiation that reads half storage -- caller-fused, ragged, single dist map, plain 2-D
    attention -- against the same call with float32 storage of the same (half-rounded) numbers: the arithmetic
    is float32 either way, so the results agree to the float32 tolerances."""
    from dfa3d_b200 import ext
    w = wl.WORKLOADS["odd"].with_(value_dtype="fp16", seed=52, C=32)
    d = wl.make_inputs(w)                                      # dist (B,N,D), shared by the heads
    t = {k: v.to(DEV) for k, v in d.items()}
    g = torch.Generator().manual_seed(52)
    Z = 5                                                      # anchors per pillar; divides P
    ref_pts = (torch.rand(w.B, w.Q, Z, 3, generator=g) * 1.2 - 0.1).to(DEV)
    off_uv = (torch.randn(w.B, w.Q, w.H, w.L, w.P, 2, generator=g) * 1.5).to(DEV)
    off_d = torch.randn(w.B, w.Q, w.H, w.L, w.P, generator=g).to(DEV)
    logits = torch.randn(w.B, w.Q, w.H, w.L * w.P, generator=g).to(DEV)
    # per-camera row offsets for the ragged calls: camera b keeps its first Q - b queries
    keep = [w.Q - b for b in range(w.B)]
    qoff = torch.tensor([0] + list(np.cumsum(keep)), dtype=torch.int32, device=DEV)
    rows = lambda x: torch.cat([x[b, :keep[b]] for b in range(w.B)]).contiguous()
    mh, mw = w.levels[1]
    dmap = torch.randn(w.B, mh * mw, w.D, generator=g).softmax(-1).half().float().to(DEV)

    def both(fn):
        """fn(value, dist) -> list of tensors, once with float32 and once with half storage."""
        a = fn(t["value"], t["dist"], dmap)
        b = fn(t["value"].half(), t["dist"].half(), dmap.half())
        assert len(a) == len(b)
        return zip(a, b)

    def fused(v, p, m):
        out, ds = ext.dfa3d_fused_forward(v, p, t["shapes"], t["lsi"], t["loc"], t["attn"], 64)
        outm, _ = ext.dfa3d_fused_forward(v, m, t["shapes"], t["lsi"], t["loc"], t["attn"], 64, dist_map=(mh, mw))
        gv = torch.zeros_like(t["value"]); gm = torch.zeros_like(dmap)
        gl = torch.empty_like(t["loc"]); ga = torch.empty_like(t["attn"])
        ext.dfa3d_fused_backward(v, m, t["shapes"], t["lsi"], t["loc"], t["attn"], t["grad_out"], gv, gm, gl, ga, 64,
                                 dist_map=(mh, mw))
        return [out, ds, outm, gv, gm, ga]

    def ragged(v, p, m):
        loc, attn, go = rows(t["loc"]), rows(t["attn"]), rows(t["grad_out"])
        out, ds = ext.dfa3d_fused_forward_ragged(v, p, t["shapes"], t["lsi"], loc, attn, qoff, w.Q)
        gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
        gl = torch.empty_like(loc); ga = torch.empty_like(attn)
        ext.dfa3d_fused_backward_ragged(v, p, t["shapes"], t["lsi"], loc, attn, qoff, w.Q, go, gv, gd, gl, ga)
        return [out, ds, gv, gd, ga]

    def caller_fused(v, p, m):
        out = ext.dfa3d_attn3d_forward(v, p, t["shapes"], t["lsi"], ref_pts, off_uv, off_d, logits)
        gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
        guv = torch.empty_like(off_uv); gdd = torch.empty_like(off_d); glg = torch.empty_like(logits)
        ext.dfa3d_attn3d_backward(v, p, t["shapes"], t["lsi"], ref_pts, off_uv, off_d, logits, t["grad_out"], gv, gd,
                                  guv, gdd, glg)
        return [out, gv, gd, guv, gdd, glg]

    def plain_2d(v, p, m):
        s2, l2 = t["shapes"][:, :2].contiguous(), t["loc"][..., :2].contiguous()
        out = ext.ms_deform_attn_forward(v, s2, t["lsi"], l2, t["attn"], 64)
        gv = torch.zeros_like(t["value"]); gl = torch.empty_like(l2); ga = torch.empty_like(t["attn"])
        ext.ms_deform_attn_backward(v, s2, t["lsi"], l2, t["attn"], t["grad_out"], gv, gl, ga, 64)
        return [out, gv, gl, ga]

    for fn in (fused, ragged, caller_fused, plain_2d):
        for i, (a, b) in enumerate(both(fn)):
            assert_close(f"{fn.__name__}[{i}]", b, a, **BWD)


def test_two_stage_api_matches_oracle(M):
    """MultiScaleDepthScoreSampleFunction -> WeightedMultiScaleDeformableAttnFunction with the
    gradient flowing through depth_score (unittest_DFA3D.py:11-22 drives the forward of this path)."""
    import dfa3d_oracle as O
    d = wl.make_inputs(wl.WORKLOADS["odd"], head_repeat=True)
    n = {k: v.numpy() for k, v in d.items()}
    dist = d["dist"].to(DEV).requires_grad_(True)
    value = d["value"].to(DEV).requires_grad_(True)
    loc = d["loc"].to(DEV).requires_grad_(True)
    attn = d["attn"].to(DEV).requires_grad_(True)
    shapes, lsi = d["shapes"].to(DEV), d["lsi"].to(DEV)
    ds = M.MultiScaleDepthScoreSampleFunction.apply(dist, shapes, lsi, loc, 64)
    ds.retain_grad()
    out = M.WeightedMultiScaleDeformableAttnFunction.apply(
        value, shapes[:, :2].contiguous(), lsi, loc[..., :2].contiguous(), attn, ds, 64)
    out.backward(d["grad_out"].to(DEV))
    o_ds = O.ms_depth_score_sample_forward(n["dist"], n["shapes"], n["lsi"], n["loc"])
    o_out = O.wms_deform_attn_forward(n["value"], n["shapes"][:, :2], n["lsi"], n["loc"][..., :2],
                                      n["attn"], o_ds)
    gv, gl2, ga, gds = O.wms_deform_attn_backward(n["value"], n["shapes"][:, :2], n["lsi"],
                                                  n["loc"][..., :2], n["attn"], o_ds, n["grad_out"])
    gd, gl3 = O.ms_depth_score_sample_backward(n["dist"], n["shapes"], n["lsi"], n["loc"], gds)
    gl3[..., :2] += gl2
    assert_close("depth_score", ds, o_ds, **FWD)
    assert_close("out", out, o_out, **FWD)
    assert_close("grad_depth_score", ds.grad, gds, **BWD)
    assert_close("grad_value", value.grad, gv, **BWD)
    assert_close("grad_dist", dist.grad, gd, **BWD)
    assert_close("grad_loc", loc.grad, gl3, **BWD)
    assert_close("grad_attn", attn.grad, ga, **BWD)


def test_depth_range_failure_semantics(M):
    """z outside the depth range: depth_score 0, output 0, yet the two-stage attention backward still
    reports grad_depth_score (wms_deform_attn_cuda_kernel.cuh:119 is not gated by the 3-D test)."""
    w = wl.WORKLOADS["tiny"]
    d = wl.make_inputs(w, head_repeat=True)
    d["loc"][..., 2] = 1.7
    got = run_fused(M, d, False)
    assert not got["out"].any() and not got["ds"].any() and not got["grad_value"].any()
    assert not got["grad_loc"].any()
    from dfa3d_b200 import ext
    t = {k: v.to(DEV) for k, v in d.items()}
    ds = torch.zeros(*t["attn"].shape, 4, device=DEV)
    gv = torch.zeros_like(t["value"]); gl = torch.empty_like(t["loc"][..., :2].contiguous())
    ga = torch.empty_like(t["attn"]); gds = torch.empty_like(ds)
    ext.wms_deform_attn_backward(t["value"], t["shapes"][:, :2].contiguous(), t["lsi"],
                                 t["loc"][..., :2].contiguous(), t["attn"], ds, t["grad_out"], gv, gl,
                                 ga, gds, 64)
    assert gds.abs().sum() > 0 and not gv.any()


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "*_ref_cuda_f32.npz"))) or [None])
def test_matches_reference_cuda_golden(M, path):
    if path is None:
        pytest.skip("no reference-CUDA golden fixture committed yet")
    z = np.load(path)
    name = os.path.basename(path).split("_ref_cuda")[0]
    if "in_value" in z.files:
        d = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    else:
        d = wl.make_inputs(wl.WORKLOADS[name], head_repeat=True)
    got = run_fused(M, d, False)
    ref = {k: z[k] for k in ("out", "ds", "grad_value", "grad_dist", "grad_loc", "grad_attn")}
    check_against(got, ref, False)


@pytest.mark.parametrize("name", ["cfg0", "cfg1", "cfg2", "cfg4op"])
def test_matches_reference_op_live(M, REF, name):
    """The reference's unmodified CUDA op (built for sm_100a), same tensors, same GPU.  cfg4op has
    D = 118 depth bins: not a multiple of 4, so the unaligned branches of the depth-pair loads and
    reductions run at full size here."""
    w = wl.WORKLOADS[name]
    d = wl.make_inputs(w, head_repeat=False)
    t = {k: v.to(DEV) for k, v in d.items()}
    dist_h = t["dist"].view(w.B, w.N, 1, w.D).repeat(1, 1, w.H, 1)
    leaves = [t["value"].clone().requires_grad_(True), dist_h.requires_grad_(True),
              t["loc"].clone().requires_grad_(True), t["attn"].clone().requires_grad_(True)]
    r_out, r_ds = REF.MultiScale3DDeformableAttnFunction_fp32.apply(
        leaves[0], leaves[1], t["shapes"], t["lsi"], leaves[2], leaves[3], 64)
    r_out.backward(t["grad_out"])
    mine = [t["value"].clone().requires_grad_(True), t["dist"].clone().requires_grad_(True),
            t["loc"].clone().requires_grad_(True), t["attn"].clone().requires_grad_(True)]
    out, ds = M.MultiScale3DDeformableAttnFunction_fp32.apply(
        mine[0], mine[1], t["shapes"], t["lsi"], mine[2], mine[3], 64)
    out.backward(t["grad_out"])
    assert_close("out", out, r_out, **FWD)
    assert_close("depth_score", ds, r_ds, **FWD)
    assert_close("grad_value", mine[0].grad, leaves[0].grad, **BWD)
    assert_close("grad_dist", mine[1].grad, leaves[1].grad.sum(2), **BWD)
    assert_close("grad_loc", mine[2].grad, leaves[2].grad, **BWD)
    assert_close("grad_attn", mine[3].grad, leaves[3].grad, **BWD)


@pytest.mark.parametrize("name", ["cfg0", "cfg1"])
def test_two_stage_api_matches_reference_op_live(M, REF, name):
    """MultiScaleDepthScoreSampleFunction -> WeightedMultiScaleDeformableAttnFunction against the
    reference's own two Functions (DFA3D/dfa3D/ops/multi_scale_3D_deform_attn.py:22-145) with the
    gradient flowing through depth_score, at C = 32 (the vector kernels in "depth score given" mode)."""
    w = wl.WORKLOADS[name]
    d = wl.make_inputs(w, head_repeat=True)
    t = {k: v.to(DEV) for k, v in d.items()}
    shapes2, go = t["shapes"][:, :2].contiguous(), t["grad_out"]

    def two_stage(ns):
        dist = t["dist"].clone().requires_grad_(True)
        value = t["value"].clone().requires_grad_(True)
        loc = t["loc"].clone().requires_grad_(True)
        attn = t["attn"].clone().requires_grad_(True)
        ds = ns.MultiScaleDepthScoreSampleFunction.apply(dist, t["shapes"], t["lsi"], loc, 64)
        ds.retain_grad()
        out = ns.WeightedMultiScaleDeformableAttnFunction.apply(
            value, shapes2, t["lsi"], loc[..., :2].contiguous(), attn, ds, 64)
        out.backward(go)
        return dict(ds=ds, out=out, grad_ds=ds.grad, grad_value=value.grad, grad_dist=dist.grad,
                    grad_loc=loc.grad, grad_attn=attn.grad)

    ref, got = two_stage(REF), two_stage(M)
    assert_close("depth_score", got["ds"], ref["ds"], **FWD)
    assert_close("out", got["out"], ref["out"], **FWD)
    for k in ("grad_ds", "grad_value", "grad_dist", "grad_loc", "grad_attn"):
        assert_close(k, got[k], ref[k], **BWD)


def test_two_stage_grad_depth_score_matches_reference_cuda_golden(M):
    """grad_depth_score of the attention backward against the value the reference's CUDA op produced
    for cfg0 (stored in the golden file by tests/golden/make_golden.py)."""
    z = np.load(os.path.join(GOLD, "cfg0_ref_cuda_f32.npz"))
    d = wl.make_inputs(wl.WORKLOADS["cfg0"], head_repeat=True)
    t = {k: v.to(DEV) for k, v in d.items()}
    ds = torch.from_numpy(z["ds"]).to(DEV).requires_grad_(True)
    value = t["value"].clone().requires_grad_(True)
    out = M.WeightedMultiScaleDeformableAttnFunction.apply(
        value, t["shapes"][:, :2].contiguous(), t["lsi"], t["loc"][..., :2].contiguous(), t["attn"], ds, 64)
    out.backward(t["grad_out"])
    assert_close("out", out, z["out"], **FWD)
    assert_close("grad_ds", ds.grad, z["grad_ds"], **BWD)
    assert_close("grad_value", value.grad, z["grad_value"], **BWD)


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "cfg4op"])
def test_benchmark_shape_camera_matches_oracle(M, name, record_property):
    """Element-wise check at the benchmark shapes: one camera of cfg2 (fp32), cfg3 (bf16 storage of
    value and dist; the oracle consumes the same bf16-rounded numbers in fp32) and cfg4op (D = 118),
    all six outputs against the C oracle.  bf16 storage is held to the 1e-2 relative bound it is
    allowed and, like fp32, to the fp32 tolerances; the number of elements outside the fp32 tolerances
    is recorded."""
    from dfa3d_b200 import ext
    from helpers import count_out_of_tolerance
    w = wl.WORKLOADS[name].with_(B=1)
    bf16 = w.value_dtype == "bf16"
    d = wl.make_inputs(w, head_repeat=True)
    ref = oracle_all(d, np.float32)
    t = {k: v.to(DEV) for k, v in d.items()}
    value = t["value"].bfloat16() if bf16 else t["value"]
    for shared in (True, False):
        dist32 = t["dist"][:, :, 0].contiguous() if shared else t["dist"]
        dist = dist32.bfloat16() if bf16 else dist32
        out, ds = ext.dfa3d_fused_forward(value, dist, t["shapes"], t["lsi"], t["loc"], t["attn"], 64)
        gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(dist32)
        gl = torch.empty_like(t["loc"]); ga = torch.empty_like(t["attn"])
        ext.dfa3d_fused_backward(value, dist, t["shapes"], t["lsi"], t["loc"], t["attn"], t["grad_out"], gv,
                                 gd, gl, ga, 64)
        got = dict(out=out, ds=ds, grad_value=gv, grad_dist=gd, grad_loc=gl, grad_attn=ga)
        if bf16:
            check_against(got, ref, shared, fwd=BF16, bwd=BF16)
        misses = {}
        for k, tol in (("out", FWD), ("ds", FWD), ("grad_value", BWD), ("grad_dist", BWD),
                       ("grad_loc", BWD), ("grad_attn", BWD)):
            r = ref[k].sum(2) if (k == "grad_dist" and shared) else ref[k]
            misses[k] = count_out_of_tolerance(got[k], r, **tol)
        record_property(f"fp32_tolerance_misses_{'shared' if shared else 'per_head'}", misses)
        print(f"{name} ({'shared' if shared else 'per-head'} dist): elements outside the fp32 tolerances: {misses}")
        check_against(got, ref, shared)


def test_bf16_leaves_through_autograd(M):
    """The one-stage Function called with bfloat16 value / value_dpt_dist LEAVES, as a user would.  The
    kernels produce float32 gradients; autograd hands a leaf a gradient of the leaf's own dtype, so
    value.grad and value_dpt_dist.grad arrive rounded to bfloat16 (the float32 gradients are available
    through ext.dfa3d_fused_backward).  Locations and attention weights are float32 leaves and get
    float32 gradients."""
    w = wl.WORKLOADS["odd"].with_(C=32, value_dtype="bf16", seed=31)
    d = wl.make_inputs(w, head_repeat=True)
    ref = oracle_all(d, np.float32)
    value = d["value"].to(DEV).bfloat16().requires_grad_(True)
    dist = d["dist"].to(DEV).bfloat16().requires_grad_(True)
    loc = d["loc"].to(DEV).requires_grad_(True)
    attn = d["attn"].to(DEV).requires_grad_(True)
    out, ds = M.MultiScale3DDeformableAttnFunction.apply(value, dist, d["shapes"].to(DEV), d["lsi"].to(DEV),
                                                         loc, attn, 64)
    out.backward(d["grad_out"].to(DEV))
    assert out.dtype == torch.float32 and ds.dtype == torch.float32
    assert value.grad.dtype == torch.bfloat16 and dist.grad.dtype == torch.bfloat16
    assert loc.grad.dtype == torch.float32 and attn.grad.dtype == torch.float32
    assert_close("out", out, ref["out"], **FWD)
    assert_close("grad_loc", loc.grad, ref["grad_loc"], **BWD)
    assert_close("grad_attn", attn.grad, ref["grad_attn"], **BWD)
    # bf16 rounding of the gradient: half an ulp = 2^-9 relative
    assert_close("grad_value", value.grad.float(), ref["grad_value"], rtol=4e-3, atol_frac=1e-5)
    assert_close("grad_dist", dist.grad.float(), ref["grad_dist"], rtol=4e-3, atol_frac=1e-5)


@pytest.mark.parametrize("name,bf16", [("cfg2", False), ("cfg3", True), ("cfg4op", False)])
def test_full_size_properties(M, name, bf16):
    """Size-independent checks at the benchmark shapes: the operator is linear in value, in dist and in
    the attention weights, so <grad_out, out> must equal <grad_x, x> for each of them; the forward is
    run-to-run bit-identical; ~15 % of the points leave the image."""
    from dfa3d_b200 import ext
    w = wl.WORKLOADS[name]
    d = wl.make_inputs(w, head_repeat=False)
    frac = ((d["loc"][..., :2] < 0) | (d["loc"][..., :2] > 1)).any(-1).float().mean().item()
    assert abs(frac - 0.15) < 0.005, frac
    t = {k: v.to(DEV) for k, v in d.items()}
    value = t["value"].bfloat16() if bf16 else t["value"]
    dist = t["dist"].bfloat16() if bf16 else t["dist"]
    out, _ = ext.dfa3d_fused_forward(value, dist, t["shapes"], t["lsi"], t["loc"], t["attn"], 64,
                                     need_depth_score=False)
    out2, _ = ext.dfa3d_fused_forward(value, dist, t["shapes"], t["lsi"], t["loc"], t["attn"], 64,
                                      need_depth_score=False)
    assert torch.equal(out, out2)
    gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
    gl = torch.empty_like(t["loc"]); ga = torch.empty_like(t["attn"])
    ext.dfa3d_fused_backward(value, dist, t["shapes"], t["lsi"], t["loc"], t["attn"], t["grad_out"], gv,
                             gd, gl, ga, 64)
    lhs = (t["grad_out"].double() * out.double()).sum().item()
    for nm, g, x in (("value", gv, value), ("dist", gd, dist), ("attn", ga, t["attn"])):
        rhs = (g.double() * x.double()).sum().item()
        assert abs(lhs - rhs) <= 1e-4 * abs(lhs), (nm, lhs, rhs)
    # linearity in the attention weights
    out3, _ = ext.dfa3d_fused_forward(value, dist, t["shapes"], t["lsi"], t["loc"], t["attn"] * 2.0, 64,
                                      need_depth_score=False)
    assert torch.equal(out3, out * 2.0)
    assert torch.isfinite(gl).all()


def test_empty_queries_and_error_behaviour(M):
    from dfa3d_b200 import ext
    w = wl.WORKLOADS["tiny"]
    d = {k: v.to(DEV) for k, v in wl.make_inputs(w).items()}
    out, ds = ext.dfa3d_fused_forward(d["value"], d["dist"], d["shapes"], d["lsi"], d["loc"][:, :0],
                                      d["attn"][:, :0], 64)
    assert out.shape == (w.B, 0, w.H * w.C) and ds.shape[1] == 0
    with pytest.raises(RuntimeError, match="contiguous"):
        ext.dfa3d_fused_forward(d["value"].transpose(0, 1), d["dist"], d["shapes"], d["lsi"], d["loc"],
                                d["attn"], 64)
    with pytest.raises(RuntimeError, match="must divide im2col_step"):
        M.MultiScale3DDeformableAttnFunction.apply(
            d["value"].repeat(3, 1, 1, 1)[:3], d["dist"].repeat(3, 1, 1)[:3], d["shapes"], d["lsi"],
            d["loc"].repeat(3, 1, 1, 1, 1, 1)[:3], d["attn"].repeat(3, 1, 1, 1, 1)[:3], 2)
    with pytest.raises(RuntimeError, match="inconsistent shapes"):
        ext.dfa3d_fused_forward(d["value"], d["dist"], d["shapes"][:1], d["lsi"], d["loc"], d["attn"], 64)
    # a gradient flowing into the returned depth_score is refused like in the reference
    v = d["value"].clone().requires_grad_(True)
    out, ds = M.MultiScale3DDeformableAttnFunction.apply(v, d["dist"], d["shapes"], d["lsi"], d["loc"],
                                                         d["attn"], 64)
    with pytest.raises(NotImplementedError):
        (out.sum() + ds.sum()).backward()


def test_non_default_stream_and_inconsistent_level_table(M):
    from dfa3d_b200 import ext
    w = wl.WORKLOADS["odd"]
    d = {k: v.to(DEV) for k, v in wl.make_inputs(w).items()}
    ref, _ = ext.dfa3d_fused_forward(d["value"], d["dist"], d["shapes"], d["lsi"], d["loc"], d["attn"], 64)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        got, _ = ext.dfa3d_fused_forward(d["value"], d["dist"], d["shapes"], d["lsi"], d["loc"],
                                         d["attn"], 64)
    s.synchronize()
    assert torch.equal(ref, got)
    # a level table that points past the value tensor must not touch memory outside it
    bad = d["shapes"].clone(); bad[:, :2] *= 3
    out, _ = ext.dfa3d_fused_forward(d["value"], d["dist"], bad, d["lsi"], d["loc"], d["attn"], 64)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()


def test_host_pipeline_matches_device_path(M):
    """Pinned host buffers streamed per camera give the same numbers as the device-resident calls."""
    from dfa3d_b200 import ext, HostPipeline
    w = wl.WORKLOADS["odd"].with_(B=5)
    d = wl.make_inputs(w)
    t = {k: v.to(DEV) for k, v in d.items()}
    out, _ = ext.dfa3d_fused_forward(t["value"], t["dist"], t["shapes"], t["lsi"], t["loc"], t["attn"], 64,
                                     need_depth_score=False)
    gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
    gl = torch.empty_like(t["loc"]); ga = torch.empty_like(t["attn"])
    ext.dfa3d_fused_backward(t["value"], t["dist"], t["shapes"], t["lsi"], t["loc"], t["attn"],
                             t["grad_out"], gv, gd, gl, ga, 64)
    host_in = {k: d[k].pin_memory() for k in ("value", "dist", "loc", "attn", "grad_out")}
    host_out = {"out": torch.empty_like(d["grad_out"]).pin_memory(),
                "grad_value": torch.empty_like(d["value"]).pin_memory(),
                "grad_dist": torch.empty_like(d["dist"]).pin_memory(),
                "grad_loc": torch.empty_like(d["loc"]).pin_memory(),
                "grad_attn": torch.empty_like(d["attn"]).pin_memory()}
    pipe = HostPipeline(d["shapes"], d["lsi"], DEV, cameras_per_chunk=2, slots=2)
    for _ in range(2):                       # second run reuses the slots
        pipe.run(host_in, host_out)
        torch.cuda.synchronize()
        assert torch.equal(host_out["out"], out.cpu())
        assert torch.equal(host_out["grad_loc"], gl.cpu()) and torch.equal(host_out["grad_attn"], ga.cpu())
        assert_close("grad_value", host_out["grad_value"], gv, **BWD)     # atomics: order may differ
        assert_close("grad_dist", host_out["grad_dist"], gd, **BWD)
    # consecutive batches overlapping (join=False), joined once at the end; and the copies-only mode
    for v in host_out.values():
        v.fill_(float("nan"))
    for i in range(3):
        pipe.run(host_in, host_out, join=(i == 2))
    torch.cuda.synchronize()
    assert torch.equal(host_out["out"], out.cpu()) and torch.equal(host_out["grad_loc"], gl.cpu())
    assert_close("grad_value", host_out["grad_value"], gv, **BWD)
    pipe.run(host_in, host_out, join=False)
    pipe.join()
    torch.cuda.synchronize()
    assert torch.equal(host_out["grad_attn"], ga.cpu())
    with pytest.raises(RuntimeError, match="pinned"):
        pipe.run({k: v.clone() for k, v in d.items()}, host_out)


def test_mixed_storage_types_match_oracle(M):
    """fp32 value with bf16 dist and the reverse: each tensor's storage type is independent."""
    from dfa3d_b200 import ext
    w = wl.WORKLOADS["odd"].with_(value_dtype="bf16", seed=21, C=32)
    d = wl.make_inputs(w, head_repeat=True)
    ref = oracle_all(d, np.float32)
    t = {k: v.to(DEV) for k, v in d.items()}
    for vb, db in ((False, True), (True, False)):
        value = t["value"].bfloat16() if vb else t["value"]
        dist = t["dist"].bfloat16() if db else t["dist"]
        out, ds = ext.dfa3d_fused_forward(value, dist, t["shapes"], t["lsi"], t["loc"], t["attn"], 64)
        gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
        gl = torch.empty_like(t["loc"]); ga = torch.empty_like(t["attn"])
        ext.dfa3d_fused_backward(value, dist, t["shapes"], t["lsi"], t["loc"], t["attn"], t["grad_out"], gv,
                                 gd, gl, ga, 64)
        check_against(dict(out=out, ds=ds, grad_value=gv, grad_dist=gd, grad_loc=gl, grad_attn=ga), ref,
                      False)


def test_more_cameras_than_one_launch_covers(M):
    """The camera index is the grid's y dimension (limit 65535): larger batches take several launches."""
    from dfa3d_b200 import ext
    B = 65535 + 3
    w = wl.WORKLOADS["tiny"].with_(B=B, levels=((2, 2),), Q=1, H=1, C=8, P=2, D=2, seed=5)
    d = wl.make_inputs(w, head_repeat=True)
    t = {k: v.to(DEV) for k, v in d.items()}
    out, _ = ext.dfa3d_fused_forward(t["value"], t["dist"], t["shapes"], t["lsi"], t["loc"], t["attn"], B)
    gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
    gl = torch.empty_like(t["loc"]); ga = torch.empty_like(t["attn"])
    ext.dfa3d_fused_backward(t["value"], t["dist"], t["shapes"], t["lsi"], t["loc"], t["attn"],
                             t["grad_out"], gv, gd, gl, ga, B)
    # the last cameras (second launch) against the oracle on just those cameras
    tail = {k: (v[-5:].contiguous() if k not in ("shapes", "lsi") else v) for k, v in d.items()}
    ref = oracle_all(tail, np.float32)
    assert_close("out", out[-5:], ref["out"], **FWD)
    assert_close("grad_value", gv[-5:], ref["grad_value"], **BWD)
    assert_close("grad_loc", gl[-5:], ref["grad_loc"], **BWD)
    assert_close("grad_dist", gd[-5:], ref["grad_dist"], **BWD)


ATTN3D_CASES = {
    "LP8_Z2": dict(levels=((5, 7), (3, 4)), P=4, Z=2),
    "LP32_Z4": dict(levels=((6, 5), (4, 4), (3, 3), (2, 3)), P=8, Z=4),
    "LP45_Z3_two_chunks": dict(levels=((6, 5), (4, 4), (3, 3), (2, 3), (1, 1)), P=9, Z=3),
    "C12_generic_Z1": dict(levels=((5, 7), (3, 4)), P=3, Z=1, C=12),
    # several items per warp (L*P = 4 / 8 / 16 with 16 / 32 / 64 channels)
    "packed_LP4_C32_Z2": dict(levels=((5, 7),), P=4, Z=2, C=32, H=3),
    "packed_LP8_C16_Z4": dict(levels=((5, 7),), P=8, Z=4, C=16, H=5),
    "packed_LP16_C64_Z4": dict(levels=((5, 7), (3, 4)), P=8, Z=4, C=64, H=1),
}


@pytest.mark.parametrize("case", sorted(ATTN3D_CASES))
@pytest.mark.parametrize("shared_dist", [False, True], ids=["dist_per_head", "dist_shared"])
def test_offsets_and_logits_entry_points_match_oracle(M, case, shared_dist):
    """Caller-fused path: reference points + raw offsets + raw logits in, softmax and location assembly
    inside the kernels; against the oracle's composition of the same tensor expressions."""
    import dfa3d_oracle as O
    kw = dict(ATTN3D_CASES[case]); Z = kw.pop("Z")
    w = wl.WORKLOADS["tiny"].with_(name=case, seed=40 + Z, Q=11, **kw)
    d = wl.make_inputs(w, head_repeat=True)
    g = torch.Generator().manual_seed(w.seed)
    ref_pts = torch.rand(w.B, w.Q, Z, 3, generator=g) * 1.2 - 0.1
    off_uv = torch.randn(w.B, w.Q, w.H, w.L, w.P, 2, generator=g) * 1.5
    off_d = torch.randn(w.B, w.Q, w.H, w.L, w.P, generator=g)
    logits = torch.randn(w.B, w.Q, w.H, w.L * w.P, generator=g)
    n = {k: v.numpy() for k, v in d.items()}
    o_out = O.attn3d_forward(n["value"], n["dist"], n["shapes"], n["lsi"], ref_pts.numpy(), off_uv.numpy(),
                             off_d.numpy(), logits.numpy())
    o_g = O.attn3d_backward(n["value"], n["dist"], n["shapes"], n["lsi"], ref_pts.numpy(), off_uv.numpy(),
                            off_d.numpy(), logits.numpy(), n["grad_out"])
    dist = d["dist"][:, :, 0].contiguous() if shared_dist else d["dist"]
    leaves = [t.to(DEV).requires_grad_(True) for t in (d["value"], dist, off_uv, off_d, logits)]
    out = M.DeformableAttn3DFromOffsetsFunction.apply(
        leaves[0], leaves[1], d["shapes"].to(DEV), d["lsi"].to(DEV), ref_pts.to(DEV), leaves[2], leaves[3],
        leaves[4])
    out.backward(d["grad_out"].to(DEV))
    assert_close("out", out, o_out, **FWD)
    assert_close("grad_value", leaves[0].grad, o_g[0], **BWD)
    assert_close("grad_dist", leaves[1].grad, o_g[1].sum(2) if shared_dist else o_g[1], **BWD)
    assert_close("grad_offsets_uv", leaves[2].grad, o_g[2], **BWD)
    assert_close("grad_offsets_depth", leaves[3].grad, o_g[3], **BWD)
    assert_close("grad_logits", leaves[4].grad, o_g[4], **BWD)


def test_fp32_variant_casts_under_autocast(M):
    """The `_fp32` Functions run in float32 inside an autocast region, like the reference's
    custom_fwd(cast_inputs=torch.float32) variants."""
    d = {k: v.to(DEV) for k, v in wl.make_inputs(wl.WORKLOADS["tiny"]).items()}
    ref, _ = M.MultiScale3DDeformableAttnFunction.apply(d["value"], d["dist"], d["shapes"], d["lsi"],
                                                        d["loc"], d["attn"], 64)
    v = d["value"].clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.float16):
        out, ds = M.MultiScale3DDeformableAttnFunction_fp32.apply(
            v.half(), d["dist"].half(), d["shapes"], d["lsi"], d["loc"], d["attn"], 64)
        assert out.dtype == torch.float32 and ds.dtype == torch.float32
    out.sum().backward()
    assert v.grad is not None and torch.isfinite(v.grad).all()
    # inputs went through fp16 once: same result as feeding the fp16-rounded values in fp32
    ref16, _ = M.MultiScale3DDeformableAttnFunction.apply(d["value"].half().float(), d["dist"].half().float(),
                                                          d["shapes"], d["lsi"], d["loc"], d["attn"], 64)
    assert torch.equal(out, ref16) and not torch.equal(ref, ref16)


@pytest.mark.parametrize("name", ["tiny", "odd", "cfg0"])
def test_plain_2d_deformable_attention_matches_oracle(M, name):
    """MultiScaleDeformableAttnFunction (the operator of BEVFormer's temporal self-attention and
    decoder) on the depth-weighted kernels with depth scores 1."""
    import dfa3d_oracle as O
    d = wl.make_inputs(wl.WORKLOADS[name])
    n = {k: v.numpy() for k, v in d.items()}
    shapes2 = n["shapes"][:, :2]
    loc2 = np.ascontiguousarray(n["loc"][..., :2])
    o = O.ms_deform_attn_forward(n["value"], shapes2, n["lsi"], loc2, n["attn"])
    gv, gl, ga = O.ms_deform_attn_backward(n["value"], shapes2, n["lsi"], loc2, n["attn"], n["grad_out"])
    value = d["value"].to(DEV).requires_grad_(True)
    loc = d["loc"][..., :2].contiguous().to(DEV).requires_grad_(True)
    attn = d["attn"].to(DEV).requires_grad_(True)
    out = M.MultiScaleDeformableAttnFunction_fp32.apply(
        value, d["shapes"][:, :2].contiguous().to(DEV), d["lsi"].to(DEV), loc, attn, 64)
    out.backward(d["grad_out"].to(DEV))
    assert_close("out", out, o, **FWD)
    assert_close("grad_value", value.grad, gv, **BWD)
    assert_close("grad_loc", loc.grad, gl, **BWD)
    assert_close("grad_attn", attn.grad, ga, **BWD)


PACKED_CASES = {
    # L*P in {4, 8, 16} with 16 / 32 / 64 float channels: several items share a warp
    "LP4_C32": dict(levels=((9, 7),), P=4, C=32, H=3, Q=37),
    "LP4_C16": dict(levels=((9, 7),), P=4, C=16, H=5, Q=13),
    "LP4_C64": dict(levels=((6, 5),), P=4, C=64, H=2, Q=21),
    "LP8_C32": dict(levels=((9, 7), (4, 3)), P=4, C=32, H=3, Q=19),
    "LP8_C16_one_level": dict(levels=((8, 8),), P=8, C=16, H=1, Q=50),
    "LP16_C32": dict(levels=((9, 7), (4, 3), (2, 2), (1, 1)), P=4, C=32, H=3, Q=11),
    "LP16_C16": dict(levels=((9, 7), (4, 3)), P=8, C=16, H=2, Q=9),
    "LP16_C64": dict(levels=((9, 7), (4, 3)), P=8, C=64, H=1, Q=7),
    "LP4_single_item": dict(levels=((3, 3),), P=4, C=32, H=1, Q=1),
}


@pytest.mark.parametrize("case", sorted(PACKED_CASES))
def test_few_points_per_item_match_oracle(M, case):
    """Items of 4, 8 or 16 points (temporal self-attention, decoder, single-level models) take kernels in
    which a warp holds several items: one-stage operator, two-stage attention with a given depth score and
    the plain 2-D operator against the oracle, item counts that do not fill the last warp."""
    import dfa3d_oracle as O
    w = wl.WORKLOADS["odd"].with_(name=case, seed=60 + len(case), D=6, **PACKED_CASES[case])
    d = wl.make_inputs(w, head_repeat=True)
    ref = oracle_all(d, np.float32)
    for shared in (False, True):
        check_against(run_fused(M, d, shared), ref, shared)
    n = {k: v.numpy() for k, v in d.items()}
    shapes2, loc2 = n["shapes"][:, :2], np.ascontiguousarray(n["loc"][..., :2])
    # two-stage attention: depth scores given
    o_out = O.wms_deform_attn_forward(n["value"], shapes2, n["lsi"], loc2, n["attn"], ref["ds"])
    gv, gl2, ga, gds = O.wms_deform_attn_backward(n["value"], shapes2, n["lsi"], loc2, n["attn"], ref["ds"],
                                                  n["grad_out"])
    t = {k: v.to(DEV) for k, v in d.items()}
    value, attn = t["value"].clone().requires_grad_(True), t["attn"].clone().requires_grad_(True)
    loc = t["loc"][..., :2].contiguous().requires_grad_(True)
    ds = torch.from_numpy(ref["ds"]).to(DEV).requires_grad_(True)
    s2 = t["shapes"][:, :2].contiguous()
    out = M.WeightedMultiScaleDeformableAttnFunction.apply(value, s2, t["lsi"], loc, attn, ds, 64)
    out.backward(t["grad_out"])
    for name, got, want in (("out", out, o_out), ("grad_value", value.grad, gv), ("grad_loc", loc.grad, gl2),
                            ("grad_attn", attn.grad, ga), ("grad_ds", ds.grad, gds)):
        assert_close("two-stage/" + name, got, want, **(FWD if name == "out" else BWD))
    # plain 2-D operator
    o = O.ms_deform_attn_forward(n["value"], shapes2, n["lsi"], loc2, n["attn"])
    gv, gl, ga = O.ms_deform_attn_backward(n["value"], shapes2, n["lsi"], loc2, n["attn"], n["grad_out"])
    value, attn = t["value"].clone().requires_grad_(True), t["attn"].clone().requires_grad_(True)
    loc = t["loc"][..., :2].contiguous().requires_grad_(True)
    out = M.MultiScaleDeformableAttnFunction.apply(value, s2, t["lsi"], loc, attn, 64)
    out.backward(t["grad_out"])
    for name, got, want in (("out", out, o), ("grad_value", value.grad, gv), ("grad_loc", loc.grad, gl),
                            ("grad_attn", attn.grad, ga)):
        assert_close("2d/" + name, got, want, **(FWD if name == "out" else BWD))


def test_random_small_item_shapes_match_oracle(M):
    """Seeded random problems with 4 / 8 / 16 points per item (levels, heads, channels, cameras, query counts
    drawn at random): one-stage operator with per-head and shared dist, and the caller-fused entry points,
    against the oracle; ragged cameras bit-equal to the dense call on per-query outputs."""
    import random
    import dfa3d_oracle as O
    from dfa3d_b200 import ext
    rnd = random.Random(5)
    for it in range(16):
        LP = rnd.choice([4, 8, 16])
        L = rnd.choice([x for x in (1, 2, 4) if LP % x == 0])
        P = LP // L
        Z = rnd.choice([z for z in (1, 2, 4) if P % z == 0])
        w = wl.Workload(f"rnd{it}", B=rnd.randint(1, 3), levels=tuple((rnd.randint(1, 10), rnd.randint(1, 10))
                                                                     for _ in range(L)),
                        D=rnd.randint(1, 9), Q=rnd.randint(1, 90), P=P, H=rnd.randint(1, 7),
                        C=rnd.choice([16, 32, 64]), seed=200 + it, oob=True)
        d = wl.make_inputs(w, head_repeat=True)
        ref = oracle_all(d, np.float32)
        for shared in (False, True):
            check_against(run_fused(M, d, shared), ref, shared)
        g = torch.Generator().manual_seed(it)
        ref_pts = torch.rand(w.B, w.Q, Z, 3, generator=g) * 1.2 - 0.1
        off_uv = torch.randn(w.B, w.Q, w.H, w.L, w.P, 2, generator=g) * 1.5
        off_d = torch.randn(w.B, w.Q, w.H, w.L, w.P, generator=g)
        logits = torch.randn(w.B, w.Q, w.H, w.L * w.P, generator=g)
        n = {k: v.numpy() for k, v in d.items()}
        t = {k: v.to(DEV) for k, v in d.items()}
        o_out = O.attn3d_forward(n["value"], n["dist"], n["shapes"], n["lsi"], ref_pts.numpy(), off_uv.numpy(),
                                 off_d.numpy(), logits.numpy())
        o_g = O.attn3d_backward(n["value"], n["dist"], n["shapes"], n["lsi"], ref_pts.numpy(), off_uv.numpy(),
                                off_d.numpy(), logits.numpy(), n["grad_out"])
        a = [x.to(DEV) for x in (ref_pts, off_uv, off_d, logits)]
        out = ext.dfa3d_attn3d_forward(t["value"], t["dist"], t["shapes"], t["lsi"], *a)
        gv = torch.zeros_like(t["value"]); gd = torch.zeros_like(t["dist"])
        gs = [torch.empty_like(x) for x in a[1:]]
        ext.dfa3d_attn3d_backward(t["value"], t["dist"], t["shapes"], t["lsi"], *a, t["grad_out"], gv, gd, *gs)
        assert_close(f"{w.name}/out", out, o_out, **FWD)
        for nm, got, want in zip(("grad_value", "grad_dist", "grad_off_uv", "grad_off_d", "grad_logits"),
                                 (gv, gd, *gs), o_g):
            assert_close(f"{w.name}/{nm}", got, want, **BWD)
        lens = [rnd.randint(0, w.Q) for _ in range(w.B)]
        if sum(lens) == 0:
            continue
        off = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
        rows = lambda x: torch.cat([x[b, :lens[b]] for b in range(w.B)]).contiguous()
        ro, rds = ext.dfa3d_fused_forward_ragged(t["value"], t["dist"], t["shapes"], t["lsi"], rows(t["loc"]),
                                                 rows(t["attn"]), off, max(lens))
        do, dds = ext.dfa3d_fused_forward(t["value"], t["dist"], t["shapes"], t["lsi"], t["loc"], t["attn"], 64)
        assert torch.equal(ro, rows(do)) and torch.equal(rds, rows(dds)), w


def test_temporal_self_attention_shape_at_full_size(M):
    """The plain 2-D operator at the temporal self-attention shape (200 x 200 BEV, 40 000 queries, 8 heads x 32
    channels, 1 level x 4 points: 8 items per warp): three slices of 256 queries -- first, middle, last --
    against the oracle run on those queries alone (outputs and per-query gradients), and grad_value against
    the oracle when only those queries carry an output gradient."""
    import dfa3d_oracle as O
    from dfa3d_b200 import ext
    g = torch.Generator().manual_seed(77)
    side, Q, H, C, P = 200, 40000, 8, 32, 4
    shapes = torch.tensor([[side, side]], dtype=torch.int64)
    lsi = torch.zeros(1, dtype=torch.int64)
    value = torch.randn(1, side * side, H, C, generator=g)
    loc = torch.rand(1, Q, H, 1, P, 2, generator=g) * 1.06 - 0.03
    attn = torch.rand(1, Q, H, 1, P, generator=g)
    picks = [slice(0, 256), slice(20000 - 128, 20000 + 128), slice(Q - 256, Q)]
    go = torch.zeros(1, Q, H * C)
    for sl in picks:
        go[:, sl] = torch.randn(1, 256, H * C, generator=g)
    dv, dl, da, dg = (t.to(DEV) for t in (value, loc, attn, go))
    out = ext.ms_deform_attn_forward(dv, shapes.to(DEV), lsi.to(DEV), dl, da, 64)
    gv = torch.zeros_like(dv); gl = torch.empty_like(dl); ga = torch.empty_like(da)
    ext.ms_deform_attn_backward(dv, shapes.to(DEV), lsi.to(DEV), dl, da, dg, gv, gl, ga, 64)
    want_gv = np.zeros(value.shape, dtype=np.float32)
    for sl in picks:
        l1, a1, g1 = (np.ascontiguousarray(t[:, sl].numpy()) for t in (loc, attn, go))
        o = O.ms_deform_attn_forward(value.numpy(), shapes.numpy(), lsi.numpy(), l1, a1)
        ogv, ogl, oga = O.ms_deform_attn_backward(value.numpy(), shapes.numpy(), lsi.numpy(), l1, a1, g1)
        assert_close("out", out[:, sl], o, **FWD)
        assert_close("grad_loc", gl[:, sl], ogl, **BWD)
        assert_close("grad_attn", ga[:, sl], oga, **BWD)
        want_gv += ogv
    assert_close("grad_value", gv, want_gv, **BWD)


def test_forward_backward_capture_into_a_cuda_graph(M):
    """The C-ABI calls only launch on the given stream (no allocation, no synchronisation), so a step
    on preallocated tensors can be captured once and replayed -- what a launch-bound small problem
    wants."""
    from dfa3d_b200 import ext
    d = {k: v.to(DEV) for k, v in wl.make_inputs(wl.WORKLOADS["cfg0"]).items()}
    out = torch.empty(d["grad_out"].shape, device=DEV)
    gv = torch.zeros_like(d["value"]); gd = torch.zeros_like(d["dist"])
    gl = torch.empty_like(d["loc"]); ga = torch.empty_like(d["attn"])

    def step():
        ext.dfa3d_fused_forward(d["value"], d["dist"], d["shapes"], d["lsi"], d["loc"], d["attn"], 64,
                                need_depth_score=False, out=out)
        gv.zero_(); gd.zero_()
        ext.dfa3d_fused_backward(d["value"], d["dist"], d["shapes"], d["lsi"], d["loc"], d["attn"],
                                 d["grad_out"], gv, gd, gl, ga, 64)

    step()
    torch.cuda.synchronize()
    ref = [t.clone() for t in (out, gv, gd, gl, ga)]
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step()                                   # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for t in (out, gv, gd, gl, ga):
        t.fill_(float("nan"))
    d["attn"].mul_(1.0)                          # inputs stay where they are: replay reads them in place
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, ref[0]) and torch.equal(gl, ref[3]) and torch.equal(ga, ref[4])
    assert_close("grad_value", gv, ref[1], **BWD)
    assert_close("grad_dist", gd, ref[2], **BWD)
