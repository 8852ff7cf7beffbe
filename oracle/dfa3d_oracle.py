"""numpy/ctypes front end of the CPU oracle (``oracle/dfa3d_oracle.c``) -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` may
import this module.  The shipped package never does: it has no CPU path at all.

The four low-level functions mirror the reference's extension entry points
(DFA3D/dfa3D/ops/csrc/pybind.cpp:42-66); the three composed functions mirror its autograd Functions:
  * two-stage: DFA3D/dfa3D/ops/multi_scale_3D_deform_attn.py:22-66 and :67-145
  * one-stage: BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/
               multi_scale_3ddeformable_attn_function.py:276-352 (the copy whose backward is correct)
Arrays are numpy, float32 or float64 (all floating inputs of one call share a dtype); shapes follow
the reference: value (B,N,H,C), dist (B,N,H,D), loc (B,Q,H,L,P,2|3), attn (B,Q,H,L,P),
depth_score (B,Q,H,L,P,4), spatial shapes (L,2|3) and level_start_index (L) int64.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libdfa3d_oracle.so")
_lib = None


def build(force=False):
    """Compile the C oracle with the committed Makefile (gcc + OpenMP)."""
    src_m = max(os.path.getmtime(os.path.join(_HERE, f))
                for f in ("dfa3d_oracle.c", "dfa3d_oracle_body.inc", "Makefile"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_m:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _suffix(dtype):
    if dtype == np.float32:
        return "_f32"
    if dtype == np.float64:
        return "_f64"
    raise TypeError(f"oracle supports float32/float64, got {dtype}")


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype=None):
    return np.ascontiguousarray(a, dtype=dtype)


def _i64(a):
    return np.ascontiguousarray(np.asarray(a), dtype=np.int64)


def _call(name, dtype, *args):
    fn = getattr(lib(), name + _suffix(dtype))
    fn.restype = None
    conv = [ctypes.c_int(int(a)) if isinstance(a, (int, np.integer)) else a for a in args]
    fn(*conv)


# ----------------------------------------------------------------------------------------------
# low level: the four extension entry points (pybind.cpp:42-66)
# ----------------------------------------------------------------------------------------------
def ms_depth_score_sample_forward(dist, shapes3, lsi, loc3):
    """ms_depth_score_sample_cuda.cu:49-111 + kernel.  Returns depth_score (B,Q,H,L,P,4)."""
    dist = _c(dist); dt = dist.dtype
    loc3 = _c(loc3, dt); shapes3 = _i64(shapes3); lsi = _i64(lsi)
    B, N, H, CD = dist.shape
    _, Q, _, L, P, three = loc3.shape
    assert three == 3 and shapes3.shape == (L, 3)
    ds = np.empty((B, Q, H, L, P, 4), dtype=dt)
    _call("dfa3d_oracle_depth_forward", dt, _p(dist), _p(shapes3), _p(lsi), _p(loc3),
          B, N, H, CD, L, Q, P, _p(ds))
    return ds


def ms_depth_score_sample_backward(dist, shapes3, lsi, loc3, grad_ds):
    """ms_depth_score_sample_cuda.cu:137-202 + kernel.  Returns (grad_dist, grad_loc3)."""
    dist = _c(dist); dt = dist.dtype
    loc3 = _c(loc3, dt); grad_ds = _c(grad_ds, dt); shapes3 = _i64(shapes3); lsi = _i64(lsi)
    B, N, H, CD = dist.shape
    _, Q, _, L, P, _ = loc3.shape
    grad_dist = np.zeros_like(dist)
    grad_loc3 = np.empty_like(loc3)
    _call("dfa3d_oracle_depth_backward", dt, _p(dist), _p(shapes3), _p(lsi), _p(loc3), _p(grad_ds),
          B, N, H, CD, L, Q, P, _p(grad_dist), _p(grad_loc3))
    return grad_dist, grad_loc3


def wms_deform_attn_forward(value, shapes2, lsi, loc2, attn, ds):
    """wms_deform_attn_cuda.cu:213-288 + kernel.  Returns output (B,Q,H*C)."""
    value = _c(value); dt = value.dtype
    loc2 = _c(loc2, dt); attn = _c(attn, dt); ds = _c(ds, dt); shapes2 = _i64(shapes2); lsi = _i64(lsi)
    B, N, H, C = value.shape
    _, Q, _, L, P, two = loc2.shape
    assert two == 2 and shapes2.shape == (L, 2)
    out = np.empty((B, Q, H * C), dtype=dt)
    _call("dfa3d_oracle_wms_forward", dt, _p(value), _p(shapes2), _p(lsi), _p(loc2), _p(attn), _p(ds),
          B, N, H, C, L, Q, P, _p(out))
    return out


def wms_deform_attn_backward(value, shapes2, lsi, loc2, attn, ds, grad_out):
    """wms_deform_attn_cuda.cu:291-370 + kernel.
    Returns (grad_value, grad_loc2, grad_attn, grad_depth_score)."""
    value = _c(value); dt = value.dtype
    loc2 = _c(loc2, dt); attn = _c(attn, dt); ds = _c(ds, dt); grad_out = _c(grad_out, dt)
    shapes2 = _i64(shapes2); lsi = _i64(lsi)
    B, N, H, C = value.shape
    _, Q, _, L, P, _ = loc2.shape
    grad_value = np.zeros_like(value)
    grad_loc2 = np.empty_like(loc2)
    grad_attn = np.empty_like(attn)
    grad_ds = np.empty_like(ds)
    _call("dfa3d_oracle_wms_backward", dt, _p(value), _p(shapes2), _p(lsi), _p(loc2), _p(attn), _p(ds),
          _p(grad_out), B, N, H, C, L, Q, P, _p(grad_value), _p(grad_loc2), _p(grad_attn), _p(grad_ds))
    return grad_value, grad_loc2, grad_attn, grad_ds


# ----------------------------------------------------------------------------------------------
# composed: the one-stage Function (…/multi_scale_3ddeformable_attn_function.py:276-352)
# ----------------------------------------------------------------------------------------------
def dfa3d_forward(value, dist, shapes3, lsi, loc3, attn):
    """forward :279-305 -> (output (B,Q,H*C), depth_score (B,Q,H,L,P,4))."""
    shapes3 = _i64(shapes3)
    ds = ms_depth_score_sample_forward(dist, shapes3, lsi, loc3)
    out = wms_deform_attn_forward(value, shapes3[:, :2], lsi, np.asarray(loc3)[..., :2], attn, ds)
    return out, ds


def dfa3d_backward(value, dist, shapes3, lsi, loc3, attn, grad_out, depth_score=None):
    """backward :306-352 -> (grad_value, grad_dist, grad_loc3, grad_attn).

    grad_loc3[..., :2] comes from the attention kernel, grad_loc3[..., 2] from the depth kernel
    (:350); grad_depth_score is internal."""
    shapes3 = _i64(shapes3)
    loc3 = np.asarray(loc3)
    if depth_score is None:
        depth_score = ms_depth_score_sample_forward(dist, shapes3, lsi, loc3)
    grad_value, grad_loc2, grad_attn, grad_ds = wms_deform_attn_backward(
        value, shapes3[:, :2], lsi, loc3[..., :2], attn, depth_score, grad_out)
    grad_dist, grad_loc3 = ms_depth_score_sample_backward(dist, shapes3, lsi, loc3, grad_ds)
    grad_loc3[..., :2] += grad_loc2
    return grad_value, grad_dist, grad_loc3, grad_attn


# ----------------------------------------------------------------------------------------------
# the attention module's tensor code around the operator
# (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/spatial_cross_attention.py:503-538)
# ----------------------------------------------------------------------------------------------
def _assemble(ref, off_uv, off_d, shapes3, dtype):
    """:513-538 -> (loc (B,Q,H,L,P,3), normalizer (L,3) = (w, h, D))."""
    shapes3 = _i64(shapes3)
    B, Q, H, L, P, _ = off_uv.shape
    Z = ref.shape[2]
    norm = np.stack([shapes3[:, 1], shapes3[:, 0], shapes3[:, 2]], -1).astype(dtype)
    off = np.concatenate([off_uv, off_d.reshape(B, Q, H, L, P, 1)], -1) / norm[None, None, None, :, None, :]
    loc = ref[:, :, None, None, None, :, :] + off.reshape(B, Q, H, L, P // Z, Z, 3)
    return np.ascontiguousarray(loc.reshape(B, Q, H, L, P, 3), dtype=dtype), norm


def _softmax(logits):
    """:503-511, over the flattened levels x points."""
    e = np.exp(logits - logits.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def attn3d_forward(value, dist, shapes3, lsi, ref, off_uv, off_d, logits):
    """Reference points (B,Q,Z,3) + raw offsets (B,Q,H,L,P,2|1) + raw logits (B,Q,H,L*P) -> output."""
    dt = np.asarray(value).dtype
    B, Q, H, L, P, _ = off_uv.shape
    loc, _ = _assemble(np.asarray(ref, dt), np.asarray(off_uv, dt), np.asarray(off_d, dt), shapes3, dt)
    attn = _softmax(np.asarray(logits, dt).reshape(B, Q, H, L * P)).reshape(B, Q, H, L, P).astype(dt)
    out, _ = dfa3d_forward(value, dist, shapes3, lsi, loc, attn)
    return out


def attn3d_backward(value, dist, shapes3, lsi, ref, off_uv, off_d, logits, grad_out):
    """Chain rule of the division, the addition and the softmax around dfa3d_backward.
    Returns (grad_value, grad_dist, grad_off_uv, grad_off_d, grad_logits)."""
    dt = np.asarray(value).dtype
    B, Q, H, L, P, _ = off_uv.shape
    loc, norm = _assemble(np.asarray(ref, dt), np.asarray(off_uv, dt), np.asarray(off_d, dt), shapes3, dt)
    attn = _softmax(np.asarray(logits, dt).reshape(B, Q, H, L * P)).astype(dt)
    gv, gd, gl, ga = dfa3d_backward(value, dist, shapes3, lsi, loc, attn.reshape(B, Q, H, L, P), grad_out)
    g_off = gl / norm[None, None, None, :, None, :]
    ga = ga.reshape(B, Q, H, L * P)
    g_logits = attn * (ga - (attn * ga).sum(-1, keepdims=True))
    return gv, gd, g_off[..., :2].copy(), g_off[..., 2].copy(), g_logits


# ----------------------------------------------------------------------------------------------
# plain 2-D multi-scale deformable attention = the depth-weighted operator with depth scores 1
# (call sites: …/bevformer/modules/multi_scale_deformable_attn_function.py:116-122, :147-158)
# ----------------------------------------------------------------------------------------------
def ms_deform_attn_forward(value, shapes2, lsi, loc2, attn):
    value = _c(value)
    ones = np.ones(tuple(np.asarray(attn).shape) + (4,), dtype=value.dtype)
    return wms_deform_attn_forward(value, shapes2, lsi, loc2, attn, ones)


def ms_deform_attn_backward(value, shapes2, lsi, loc2, attn, grad_out):
    """Returns (grad_value, grad_loc2, grad_attn)."""
    value = _c(value)
    ones = np.ones(tuple(np.asarray(attn).shape) + (4,), dtype=value.dtype)
    gv, gl, ga, _ = wms_deform_attn_backward(value, shapes2, lsi, loc2, attn, ones, grad_out)
    return gv, gl, ga
