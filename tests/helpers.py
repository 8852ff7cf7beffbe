"""Shared helpers of the parity tests."""
import os

import numpy as np
import torch

# Acceptance tolerances of this operator: forward within 1e-5 relative / 1e-6 absolute in fp32;
# backward within 1e-4 relative (atomic reordering); bf16 storage within 1e-2 relative.  Gradients are
# sums with cancellation, so "relative" is taken against the tensor's scale as well as the element:
#     |got - ref| <= rtol * |ref| + atol,   atol = atol_frac * max|ref|
FWD = dict(rtol=1e-5, atol=1e-6, atol_frac=0.0)
BWD = dict(rtol=1e-4, atol=0.0, atol_frac=1e-5)
BF16 = dict(rtol=1e-2, atol=0.0, atol_frac=1e-3)


def to_np(t):
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().double().numpy()
    return np.asarray(t, dtype=np.float64)


# Filled by assert_close when the environment variable DFA3D_TOL_STATS names a file: per comparison,
# how many elements pass only thanks to the absolute term of the tolerance (written at session end by
# conftest.py).  Lets the share of elements that lean on `atol_frac * max|ref|` be stated with numbers.
TOL_STATS = []


def count_out_of_tolerance(got, ref, rtol, atol=0.0, atol_frac=0.0):
    """Number of elements with |got - ref| > rtol*|ref| + atol + atol_frac*max|ref|."""
    got, ref = to_np(got), to_np(ref)
    tol = rtol * np.abs(ref) + atol + atol_frac * (np.abs(ref).max() if ref.size else 0.0)
    return int((np.abs(got - ref) > tol).sum())


def assert_close(name, got, ref, rtol, atol=0.0, atol_frac=0.0):
    got, ref = to_np(got), to_np(ref)
    assert got.shape == ref.shape, f"{name}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{name}: non-finite values"
    tol = rtol * np.abs(ref) + atol + atol_frac * (np.abs(ref).max() if ref.size else 0.0)
    err = np.abs(got - ref)
    bad = err > tol
    if os.environ.get("DFA3D_TOL_STATS"):
        TOL_STATS.append({"test": os.environ.get("PYTEST_CURRENT_TEST", ""), "tensor": name,
                          "elements": int(err.size), "beyond_relative_term": int((err > rtol * np.abs(ref)).sum()),
                          "failed": int(bad.sum()), "rtol": rtol, "atol": atol, "atol_frac": atol_frac,
                          "max_abs_ref": float(np.abs(ref).max()) if ref.size else 0.0,
                          "max_abs_err": float(err.max()) if err.size else 0.0})
    if bad.any():
        i = np.unravel_index(np.argmax(err - tol), err.shape)
        raise AssertionError(
            f"{name}: {bad.sum()} of {bad.size} elements out of tolerance; worst at {i}: "
            f"got {got[i]!r} ref {ref[i]!r} err {err[i]:.3e} tol {tol[i]:.3e}; max|ref| {np.abs(ref).max():.3e}")


def oracle_all(d, dtype=np.float64):
    """Run the CPU oracle (one-stage composition) on a workload dict made with head_repeat=True.
    Returns dict(out, ds, grad_value, grad_dist, grad_loc, grad_attn) as numpy arrays."""
    import dfa3d_oracle as O
    n = {k: (v.numpy().astype(dtype) if v.is_floating_point() else v.numpy()) for k, v in d.items()}
    out, ds = O.dfa3d_forward(n["value"], n["dist"], n["shapes"], n["lsi"], n["loc"], n["attn"])
    gv, gd, gl, ga = O.dfa3d_backward(n["value"], n["dist"], n["shapes"], n["lsi"], n["loc"], n["attn"],
                                      n["grad_out"], depth_score=ds)
    return dict(out=out, ds=ds, grad_value=gv, grad_dist=gd, grad_loc=gl, grad_attn=ga)
