"""Double precision on the GPU (the reference instantiates its kernels for float and double,
DFA3D/dfa3D/ops/csrc/cuda/wms_deform_attn_cuda.cu:267,344): the *_f64 entry points through the same
Functions, against the fp64 oracle, the reference's own op run in double, and finite differences."""
import numpy as np
import pytest
import torch

from dfa3d_b200 import workloads as wl
from helpers import assert_close, oracle_all

pytestmark = pytest.mark.gpu
DEV = "cuda"
F64 = dict(rtol=1e-10, atol=1e-12)


@pytest.fixture(scope="module")
def M(lib_built):
    import dfa3d_b200
    assert torch.cuda.is_available()
    return dfa3d_b200


def _leaves(d, shared_dist):
    dist = d["dist"][:, :, 0].contiguous() if shared_dist else d["dist"]
    return [t.double().to(DEV).requires_grad_(True) for t in (d["value"], dist, d["loc"], d["attn"])]


@pytest.mark.parametrize("shared_dist", [False, True], ids=["dist_per_head", "dist_shared"])
@pytest.mark.parametrize("name", ["tiny", "odd", "cfg0"])
def test_one_stage_function_in_double_matches_fp64_oracle(M, name, shared_dist):
    d = wl.make_inputs(wl.WORKLOADS[name], head_repeat=True)
    ref = oracle_all(d, np.float64)
    value, dist, loc, attn = _leaves(d, shared_dist)
    out, ds = M.MultiScale3DDeformableAttnFunction.apply(value, dist, d["shapes"].to(DEV), d["lsi"].to(DEV), loc,
                                                         attn, 64)
    assert out.dtype == torch.float64 and ds.dtype == torch.float64
    out.backward(d["grad_out"].double().to(DEV))
    assert value.grad.dtype == torch.float64
    assert_close("out", out, ref["out"], **F64)
    assert_close("depth_score", ds, ref["ds"], **F64)
    assert_close("grad_value", value.grad, ref["grad_value"], **F64)
    assert_close("grad_dist", dist.grad, ref["grad_dist"].sum(2) if shared_dist else ref["grad_dist"], **F64)
    assert_close("grad_loc", loc.grad, ref["grad_loc"], **F64)
    assert_close("grad_attn", attn.grad, ref["grad_attn"], **F64)


def test_two_stage_functions_in_double_match_fp64_oracle(M):
    import dfa3d_oracle as O
    d = wl.make_inputs(wl.WORKLOADS["odd"], head_repeat=True)
    n = {k: (v.numpy().astype(np.float64) if v.is_floating_point() else v.numpy()) for k, v in d.items()}
    value, dist, loc, attn = _leaves(d, False)
    shapes, lsi = d["shapes"].to(DEV), d["lsi"].to(DEV)
    ds = M.MultiScaleDepthScoreSampleFunction.apply(dist, shapes, lsi, loc, 64)
    ds.retain_grad()
    out = M.WeightedMultiScaleDeformableAttnFunction.apply(value, shapes[:, :2].contiguous(), lsi,
                                                           loc[..., :2].contiguous(), attn, ds, 64)
    out.backward(d["grad_out"].double().to(DEV))
    o_ds = O.ms_depth_score_sample_forward(n["dist"], n["shapes"], n["lsi"], n["loc"])
    o_out = O.wms_deform_attn_forward(n["value"], n["shapes"][:, :2], n["lsi"], n["loc"][..., :2], n["attn"], o_ds)
    gv, gl2, ga, gds = O.wms_deform_attn_backward(n["value"], n["shapes"][:, :2], n["lsi"], n["loc"][..., :2],
                                                  n["attn"], o_ds, n["grad_out"])
    gd, gl3 = O.ms_depth_score_sample_backward(n["dist"], n["shapes"], n["lsi"], n["loc"], gds)
    gl3[..., :2] += gl2
    for name, got, want in (("depth_score", ds, o_ds), ("out", out, o_out), ("grad_ds", ds.grad, gds),
                            ("grad_value", value.grad, gv), ("grad_dist", dist.grad, gd),
                            ("grad_loc", loc.grad, gl3), ("grad_attn", attn.grad, ga)):
        assert_close(name, got, want, **F64)


def test_double_matches_the_reference_op_run_in_double(M):
    """The reference's unmodified CUDA op with double tensors (its own AT_DISPATCH double branch)."""
    import build_ref
    try:
        REF = build_ref.load()
    except ImportError as e:
        pytest.skip(f"reference op not available: {e}")
    d = wl.make_inputs(wl.WORKLOADS["cfg0"], head_repeat=True)
    shapes, lsi, go = d["shapes"].to(DEV), d["lsi"].to(DEV), d["grad_out"].double().to(DEV)
    mine, theirs = _leaves(d, False), _leaves(d, False)
    out, ds = M.MultiScale3DDeformableAttnFunction.apply(mine[0], mine[1], shapes, lsi, mine[2], mine[3], 64)
    out.backward(go)
    # the reference's one-stage Function casts to float32; its two-stage Functions keep the caller's dtype
    r_ds = REF.MultiScaleDepthScoreSampleFunction.apply(theirs[1], shapes, lsi, theirs[2], 64)
    r_out = REF.WeightedMultiScaleDeformableAttnFunction.apply(
        theirs[0], shapes[:, :2].contiguous(), lsi, theirs[2][..., :2].contiguous(), theirs[3], r_ds, 64)
    assert r_out.dtype == torch.float64
    r_out.backward(go)
    assert_close("out", out, r_out, **F64)
    assert_close("depth_score", ds, r_ds, **F64)
    for name, a, b in zip(("grad_value", "grad_dist", "grad_loc", "grad_attn"), mine, theirs):
        assert_close(name, a.grad, b.grad, rtol=1e-9, atol=1e-12)


def test_finite_differences_agree_with_the_analytic_gradients(M):
    """torch.autograd.gradcheck of the one-stage and of the two-stage path in double.  Locations are kept
    away from cell borders (the operator is piecewise smooth in them)."""
    w = wl.WORKLOADS["tiny"].with_(Q=3, oob=False)
    d = wl.make_inputs(w, head_repeat=True)
    shapes, lsi = d["shapes"].to(DEV), d["lsi"].to(DEV)
    # snap every coordinate to 0.3 of a cell so that +-1e-6 never crosses a cell border
    size = torch.tensor([[ww, h, w.D] for h, ww in w.levels], dtype=torch.float64)      # (L, 3) = (W, H, D)
    loc = d["loc"].double()
    cell = torch.floor(loc * size[None, None, None, :, None, :] - 0.5)
    loc = (cell + 0.5 + 0.3) / size[None, None, None, :, None, :]
    value, dist, _, attn = _leaves(d, True)
    loc = loc.to(DEV).requires_grad_(True)

    def one_stage(v, p, x, a):
        return M.MultiScale3DDeformableAttnFunction.apply(v, p, shapes, lsi, x, a, 64, False)[0]

    def two_stage(v, p, x, a):
        p4 = p[:, :, None, :].expand(-1, -1, w.H, -1).contiguous()
        ds = M.MultiScaleDepthScoreSampleFunction.apply(p4, shapes, lsi, x, 64)
        return M.WeightedMultiScaleDeformableAttnFunction.apply(v, shapes[:, :2].contiguous(), lsi,
                                                                x[..., :2].contiguous(), a, ds, 64)

    for fn in (one_stage, two_stage):
        assert torch.autograd.gradcheck(fn, (value, dist, loc, attn), eps=1e-6, atol=1e-6, rtol=1e-4,
                                        nondet_tol=1e-9, fast_mode=False)


def test_double_argument_checks(M):
    from dfa3d_b200 import ext
    d = {k: v.to(DEV) for k, v in wl.make_inputs(wl.WORKLOADS["tiny"]).items()}
    v64, p64 = d["value"].double(), d["dist"].double()
    with pytest.raises(RuntimeError, match="dtype"):          # mixed precision within one call
        ext.dfa3d_fused_forward(v64, p64, d["shapes"], d["lsi"], d["loc"], d["attn"].double(), 64)
    with pytest.raises(RuntimeError, match="double precision"):
        ext.dfa3d_fused_forward(v64, p64, d["shapes"], d["lsi"], d["loc"].double(), d["attn"].double(), 64,
                                dist_map=(2, 2))
