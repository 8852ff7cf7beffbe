"""CPU tests of the oracle: pins against the committed golden vectors, hand-computable cases,
finite differences.  No GPU needed."""
import glob
import os

import numpy as np
import pytest
import torch

import dfa3d_oracle as O
from dfa3d_b200 import workloads as wl
from helpers import BWD, FWD, assert_close, oracle_all

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    z = np.load(os.path.join(GOLD, name), allow_pickle=False)
    return {k: z[k] for k in z.files}


def _inputs_from(z):
    return {k[3:]: torch.from_numpy(z[k]) for k in z if k.startswith("in_")}


@pytest.mark.parametrize("name", ["tiny", "odd"])
def test_oracle_f64_matches_grid_sample_golden(name):
    z = _load(f"{name}_grid_sample_f64.npz")
    d = _inputs_from(z)
    o = oracle_all(d, np.float64)
    for k in ("out", "grad_value", "grad_dist", "grad_loc", "grad_attn"):
        assert_close(k, o[k], z[k], rtol=1e-11, atol=1e-13)


@pytest.mark.parametrize("name", ["tiny", "odd"])
def test_oracle_f32_close_to_f64(name):
    z = _load(f"{name}_grid_sample_f64.npz")
    d = _inputs_from(z)
    o = oracle_all(d, np.float32)
    assert o["out"].dtype == np.float32
    assert_close("out", o["out"], z["out"], **FWD)
    for k in ("grad_value", "grad_dist", "grad_loc", "grad_attn"):
        assert_close(k, o[k], z[k], **BWD)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "*_ref_cuda_f32.npz"))) or [None])
def test_oracle_matches_reference_cuda_golden(path):
    """Outputs of the reference's own CUDA op (fp32, generated on a B200 by make_golden.py)."""
    if path is None:
        pytest.skip("no reference-CUDA golden fixture committed yet")
    z = _load(path)
    name = os.path.basename(path).split("_ref_cuda")[0]
    if any(k.startswith("in_") for k in z):
        d = _inputs_from(z)
    else:
        d = wl.make_inputs(wl.WORKLOADS[name], head_repeat=True)
        from make_golden import input_digest  # same generator, same bits
        assert input_digest(d) == str(z["input_sha256"]), "workload generator drifted from the fixture"
    o = oracle_all(d, np.float64)
    assert_close("out", z["out"], o["out"], **FWD)
    assert_close("ds", z["ds"], o["ds"], **FWD)
    for k in ("grad_value", "grad_dist", "grad_loc", "grad_attn"):
        assert_close(k, z[k], o[k], **BWD)
    # two-stage: gradient with respect to a given depth_score
    n = {k: v.numpy().astype(np.float64) if v.is_floating_point() else v.numpy() for k, v in d.items()}
    _, _, _, gds = O.wms_deform_attn_backward(n["value"], n["shapes"][:, :2], n["lsi"], n["loc"][..., :2],
                                              n["attn"], o["ds"], n["grad_out"])
    assert_close("grad_ds", z["grad_ds"], gds, **BWD)


def _micro(value, dist, loc, attn, hw=(1, 1), D=1):
    """One camera, one head, one level, one query, one point."""
    h, w = hw
    value = np.asarray(value, np.float64).reshape(1, h * w, 1, -1)
    dist = np.asarray(dist, np.float64).reshape(1, h * w, 1, D)
    loc = np.asarray(loc, np.float64).reshape(1, 1, 1, 1, 1, 3)
    attn = np.asarray(attn, np.float64).reshape(1, 1, 1, 1, 1)
    shapes = np.array([[h, w, D]], np.int64)
    lsi = np.array([0], np.int64)
    return O.dfa3d_forward(value, dist, shapes, lsi, loc, attn)


def test_micro_centre_of_single_pixel():
    # loc 0.5 -> pixel coordinate 0: only corner 0 and depth bin 0 contribute, all weights 1
    out, ds = _micro([2.0, -3.0], [0.25], [0.5, 0.5, 0.5], 0.5)
    np.testing.assert_allclose(ds.ravel(), [0.25, 0, 0, 0])
    np.testing.assert_allclose(out.ravel(), [0.5 * 0.25 * 2.0, 0.5 * 0.25 * -3.0])


def test_micro_left_of_single_pixel_uses_corner_1():
    # x = 0.25 -> w_im = -0.25: x0 = -1 (outside), x1 = 0 with weight lw = 0.75
    out, ds = _micro([4.0], [1.0], [0.25, 0.5, 0.5], 1.0)
    np.testing.assert_allclose(ds.ravel(), [0, 1.0, 0, 0])
    np.testing.assert_allclose(out.ravel(), [0.75 * 4.0])


def test_micro_corner_order_bottom_right_is_slot_2():
    # 2x2 map, point at pixel coordinate (x=0.5, y=0.5): all four corners with weight 0.25;
    # dist differs per pixel so the slot order shows: 0=TL 1=TR 2=BR 3=BL
    dist = [0.1, 0.2, 0.3, 0.4]      # pixels (0,0) (0,1) (1,0) (1,1), D = 1
    out, ds = _micro([1, 1, 1, 1], dist, [0.5, 0.5, 0.5], 1.0, hw=(2, 2))
    np.testing.assert_allclose(ds.ravel(), [0.1, 0.2, 0.4, 0.3])
    np.testing.assert_allclose(out.ravel(), [0.25 * (0.1 + 0.2 + 0.3 + 0.4)])


def test_micro_strict_range_tests():
    # w_im == -1 exactly (x = -0.5 on a 1-wide map) is outside; just inside contributes
    out, _ = _micro([1.0], [1.0], [-0.5, 0.5, 0.5], 1.0)
    assert out.ravel()[0] == 0.0
    out, _ = _micro([1.0], [1.0], [-0.499, 0.5, 0.5], 1.0)
    assert out.ravel()[0] > 0.0
    # depth coordinate out of range zeroes the depth score but the 2-D part is still "in range"
    out, ds = _micro([1.0], [1.0], [0.5, 0.5, 1.6], 1.0)
    assert out.ravel()[0] == 0.0 and not ds.any()


def test_micro_depth_interpolation():
    # D = 2, z = 0.5 -> d_im = 0.5: half of bin 0, half of bin 1
    out, ds = _micro([1.0], [0.2, 0.6], [0.5, 0.5, 0.5], 1.0, D=2)
    np.testing.assert_allclose(ds.ravel()[0], 0.4)
    # z = 0.1 -> d_im = -0.3: bin -1 is outside, bin 0 with weight 0.7
    out, ds = _micro([1.0], [0.2, 0.6], [0.5, 0.5, 0.1], 1.0, D=2)
    np.testing.assert_allclose(ds.ravel()[0], 0.7 * 0.2)


def test_depth_failure_keeps_grad_depth_score():
    """A point whose depth coordinate is out of range has depth_score 0, yet the attention backward
    still reports a gradient for that depth_score (the depth backward then drops it)."""
    value = np.ones((1, 1, 1, 1)); shapes2 = np.array([[1, 1]], np.int64); lsi = np.zeros(1, np.int64)
    loc2 = np.full((1, 1, 1, 1, 1, 2), 0.5); attn = np.ones((1, 1, 1, 1, 1)); ds = np.zeros((1, 1, 1, 1, 1, 4))
    go = np.ones((1, 1, 1))
    gv, gl, ga, gds = O.wms_deform_attn_backward(value, shapes2, lsi, loc2, attn, ds, go)
    assert gds.ravel()[0] == 1.0 and gv.ravel()[0] == 0.0 and ga.ravel()[0] == 0.0


def test_finite_differences_fp64():
    w = wl.WORKLOADS["tiny"]
    d = wl.make_inputs(w, head_repeat=True)
    n = {k: v.numpy().astype(np.float64) if v.is_floating_point() else v.numpy() for k, v in d.items()}
    g = dict(zip(("value", "dist", "loc", "attn"),
                 O.dfa3d_backward(n["value"], n["dist"], n["shapes"], n["lsi"], n["loc"], n["attn"],
                                  n["grad_out"])))
    rng = np.random.default_rng(0)

    def f(**over):
        a = dict(n); a.update(over)
        out, _ = O.dfa3d_forward(a["value"], a["dist"], a["shapes"], a["lsi"], a["loc"], a["attn"])
        return float((out * n["grad_out"]).sum())

    for key, eps in (("value", 1e-6), ("dist", 1e-6), ("attn", 1e-6), ("loc", 1e-9)):
        v = rng.standard_normal(n[key].shape)
        num = (f(**{key: n[key] + eps * v}) - f(**{key: n[key] - eps * v})) / (2 * eps)
        ana = float((g[key] * v).sum())
        assert abs(num - ana) <= 1e-5 * max(1.0, abs(ana)), (key, num, ana)


def test_empty_and_ragged_shapes():
    shapes = np.array([[2, 3, 4]], np.int64); lsi = np.zeros(1, np.int64)
    value = np.zeros((1, 6, 2, 4)); dist = np.zeros((1, 6, 2, 4))
    loc = np.zeros((1, 0, 2, 1, 5, 3)); attn = np.zeros((1, 0, 2, 1, 5))
    out, ds = O.dfa3d_forward(value, dist, shapes, lsi, loc, attn)
    assert out.shape == (1, 0, 8) and ds.shape == (1, 0, 2, 1, 5, 4)


def test_attn3d_composition_matches_torch_autograd_fp64():
    """Oracle of the caller-fused entry points (offsets + logits in) against PyTorch autograd through
    the module's own tensor expressions and the independent grid_sample formulation."""
    import grid_sample_form as G
    from dfa3d_b200 import modules
    g = torch.Generator().manual_seed(3)
    B, Q, H, C, D, Z, P = 2, 5, 2, 4, 6, 2, 4
    levels = ((5, 7), (3, 4))
    L = len(levels); N = sum(h * w for h, w in levels)
    shapes3 = torch.tensor([[h, w, D] for h, w in levels]); lsi = torch.tensor([0, 35])
    value = torch.randn(B, N, H, C, generator=g, dtype=torch.float64)
    dist = torch.randn(B, N, H, D, generator=g, dtype=torch.float64).softmax(-1)
    ref = torch.rand(B, Q, Z, 3, generator=g, dtype=torch.float64)
    off_uv = torch.randn(B, Q, H, L, P, 2, generator=g, dtype=torch.float64, requires_grad=True)
    off_d = torch.randn(B, Q, H, L, P, 1, generator=g, dtype=torch.float64, requires_grad=True)
    logits = torch.randn(B, Q, H, L * P, generator=g, dtype=torch.float64, requires_grad=True)
    go = torch.randn(B, Q, H * C, generator=g, dtype=torch.float64)
    loc = modules.assemble_sampling_locations(ref, off_uv, off_d, shapes3[:, :2], D)
    attn = logits.softmax(-1).view(B, Q, H, L, P)
    out = G.dfa3d_grid_sample(value, dist, shapes3.tolist(), lsi.tolist(), loc, attn)
    out.backward(go)
    n = lambda t: t.detach().numpy()
    o_out = O.attn3d_forward(n(value), n(dist), n(shapes3), n(lsi), n(ref), n(off_uv), n(off_d)[..., 0],
                             n(logits))
    gv, gd, guv, gdd, glg = O.attn3d_backward(n(value), n(dist), n(shapes3), n(lsi), n(ref), n(off_uv),
                                              n(off_d)[..., 0], n(logits), n(go))
    assert_close("out", o_out, n(out), rtol=1e-11, atol=1e-13)
    assert_close("grad_off_uv", guv, n(off_uv.grad), rtol=1e-10, atol=1e-12)
    assert_close("grad_off_d", gdd, n(off_d.grad)[..., 0], rtol=1e-10, atol=1e-12)
    assert_close("grad_logits", glg, n(logits.grad), rtol=1e-10, atol=1e-12)


def test_plain_2d_attention_oracle_matches_grid_sample_fp64():
    import grid_sample_form as G
    d = wl.make_inputs(wl.WORKLOADS["odd"])
    dd = {k: (v.double() if v.is_floating_point() else v) for k, v in d.items()}
    value = dd["value"].clone().requires_grad_(True)
    loc2 = dd["loc"][..., :2].clone().requires_grad_(True)
    attn = dd["attn"].clone().requires_grad_(True)
    out = G.msda_grid_sample(value, dd["shapes"][:, :2].tolist(), dd["lsi"].tolist(), loc2, attn)
    out.backward(dd["grad_out"])
    n = lambda t: t.detach().numpy()
    o = O.ms_deform_attn_forward(n(value), n(dd["shapes"][:, :2]), n(dd["lsi"]), n(loc2), n(attn))
    gv, gl, ga = O.ms_deform_attn_backward(n(value), n(dd["shapes"][:, :2]), n(dd["lsi"]), n(loc2), n(attn),
                                           n(dd["grad_out"]))
    assert_close("out", o, n(out), rtol=1e-11, atol=1e-13)
    assert_close("grad_value", gv, n(value.grad), rtol=1e-10, atol=1e-12)
    assert_close("grad_loc", gl, n(loc2.grad), rtol=1e-10, atol=1e-11)
    assert_close("grad_attn", ga, n(attn.grad), rtol=1e-10, atol=1e-12)
