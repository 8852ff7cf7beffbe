"""Drop-in for the reference's compiled extension module ``dfa3D._ext``.

The four functions have the names, keyword arguments, return values and in-place conventions of the
reference's pybind module (DFA3D/dfa3D/ops/csrc/pybind.cpp:42-66); two more expose the one-launch
fused forward / backward.  All of them validate their tensors like the reference's launchers
(contiguous, CUDA, ``batch % min(batch, im2col_step) == 0`` -- DFA3D/dfa3D/ops/csrc/cuda/
wms_deform_attn_cuda.cu:220-253) and then call the C ABI on the current CUDA stream.

Narrowing with respect to the reference: tensors are float32 (the reference also instantiates
float64), plus bfloat16 storage for ``value`` / ``dist`` which the reference lacks.
"""
import torch

from . import _lib


def _chk(t, name, dtypes=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} tensor has to be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise RuntimeError(f"{name} has dtype {t.dtype}; supported: {dtypes}")


def _same_device(*ts):
    dev = ts[0].device
    for t in ts[1:]:
        if t is not None and t.device != dev:
            raise RuntimeError(f"all tensors must be on one device, got {dev} and {t.device}")


def _step_check(batch, im2col_step):
    # the reference asserts this although only its chunk loop needs it; kept for identical errors
    if batch > 0:
        step = min(batch, int(im2col_step))
        if step <= 0 or batch % step != 0:
            raise RuntimeError(f"batch({batch}) must divide im2col_step({step})")


_F32 = (torch.float32,)
_F64 = (torch.float64,)
_VAL = (torch.float32, torch.bfloat16, torch.float16)
_I64 = (torch.int64,)


def _dt(t):
    if t.dtype == torch.float64:
        return _lib.DTYPE_F64
    if t.dtype == torch.float16:
        return _lib.DTYPE_F16
    return _lib.DTYPE_BF16 if t.dtype == torch.bfloat16 else _lib.DTYPE_F32


def _types(t, dist_map=None):
    """(dtypes allowed for value/dist, dtypes allowed for everything else, output dtype, entry-point
    suffix) chosen by the scalar type of the call's main tensor."""
    if t.dtype == torch.float64:
        if dist_map is not None:
            raise RuntimeError("dist_map is not available in double precision")
        return _F64, _F64, torch.float64, "_f64"
    return _VAL, _F32, torch.float32, ""


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _map(dist_map):
    """dist_map: None, or (h, w) of the single map all levels read with nearest indexing."""
    if dist_map is None:
        return 0, 0
    mh, mw = int(dist_map[0]), int(dist_map[1])
    if mh <= 0 or mw <= 0:
        raise RuntimeError(f"dist_map must be two positive sizes, got {dist_map}")
    return mh, mw


def _dist_rows_ok(Nd, N, dist_map):
    mh, mw = _map(dist_map)
    return Nd == (mh * mw if mh else N)


def _dist_problem(dist, H):
    """dist is (B,N,H,D), or (B,N,D) shared by all heads.  Returns (B, N, D, head_stride)."""
    if dist.dim() == 4:
        B, N, Hd, D = dist.shape
        if Hd != H:
            raise RuntimeError(f"dist has {Hd} heads, expected {H}")
        return B, N, D, D
    if dist.dim() == 3:
        B, N, D = dist.shape
        return B, N, D, 0
    raise RuntimeError("dist must be (B,N,H,D) or (B,N,D)")


def _level_table(shapes, lsi, L, width):
    """spatial_shapes must be (L, width) and level_start_index must hold L entries: the kernels read
    entry l of both for every level l < L."""
    if tuple(shapes.shape) != (L, width) or lsi.numel() != L:
        raise RuntimeError(f"inconsistent shapes: spatial_shapes must be ({L},{width}) and "
                           f"level_start_index must have {L} entries, got {tuple(shapes.shape)} and "
                           f"{lsi.numel()}")


def _level_pixels(n_dist_rows, dist_map, shapes):
    """N of the problem descriptor for the depth-only entry points: the rows of dist, or -- with a single
    map -- the pixels of all levels (corner pixels are bounded by it)."""
    if dist_map is None:
        return n_dist_rows
    mh, mw = _map(dist_map)
    if n_dist_rows != mh * mw:
        raise RuntimeError(f"value has {n_dist_rows} rows per camera, dist_map {mh}x{mw} needs {mh * mw}")
    return int((shapes[:, 0] * shapes[:, 1]).sum())     # one read-back; depth-only API with a map


def _loc_dims(loc, last):
    if loc.dim() != 6 or loc.shape[-1] != last:
        raise RuntimeError(f"sampling_locations must be (B,Q,H,L,P,{last}), got {tuple(loc.shape)}")
    return loc.shape[:5]


# ------------------------------------------------------------------------------------------------
def ms_depth_score_sample_forward(value, value_spatial_shapes, value_level_start_index,
                                  sampling_locations, im2col_step, dist_map=None):
    """`value` is the depth distribution (B,N,H,D) [or (B,N,D)]; returns depth_score (B,Q,H,L,P,4).
    dist_map=(h, w): `value` is one h x w map per camera that every level reads with nearest indexing."""
    dist = value
    VAL, F, odt, sfx = _types(dist, dist_map)
    _chk(dist, "value", VAL); _chk(value_spatial_shapes, "spatial_shapes", _I64)
    _chk(value_level_start_index, "level_start_index", _I64)
    _chk(sampling_locations, "sampling_loc", F)
    _same_device(dist, value_spatial_shapes, value_level_start_index, sampling_locations)
    B, Q, H, L, P = _loc_dims(sampling_locations, 3)
    Bd, N, D, hs = _dist_problem(dist, H)
    if Bd != B or tuple(value_spatial_shapes.shape) != (L, 3):
        raise RuntimeError("inconsistent shapes between value, spatial_shapes (L,3) and sampling_loc")
    _level_table(value_spatial_shapes, value_level_start_index, L, 3)
    _step_check(B, im2col_step)
    out = torch.empty((B, Q, H, L, P, 4), dtype=odt, device=dist.device)
    N = _level_pixels(N, dist_map, value_spatial_shapes)
    pr = _lib.Problem(B, N, H, 0, D, L, Q, P, _lib.DTYPE_F32, _dt(dist), hs, *_map(dist_map))
    with torch.cuda.device(dist.device):
        _lib.call("dfa3d_depth_score_forward" + sfx, pr, _ptr(dist), _ptr(value_spatial_shapes),
                  _ptr(value_level_start_index), _ptr(sampling_locations), _ptr(out), _stream(dist))
    return out


def ms_depth_score_sample_backward(value, value_spatial_shapes, value_level_start_index,
                                   sampling_locations, grad_output, grad_value, grad_sampling_loc,
                                   im2col_step, dist_map=None):
    """Accumulates into grad_value (layout of `value`, float32, caller-zeroed) and overwrites
    grad_sampling_loc (B,Q,H,L,P,3) with (0, 0, dL/dz)."""
    dist = value
    VAL, F, odt, sfx = _types(dist, dist_map)
    _chk(dist, "value", VAL); _chk(value_spatial_shapes, "spatial_shapes", _I64)
    _chk(value_level_start_index, "level_start_index", _I64)
    _chk(sampling_locations, "sampling_loc", F); _chk(grad_output, "grad_output", F)
    _chk(grad_value, "grad_value", F); _chk(grad_sampling_loc, "grad_sampling_loc", F)
    _same_device(dist, value_spatial_shapes, value_level_start_index, sampling_locations, grad_output,
                 grad_value, grad_sampling_loc)
    B, Q, H, L, P = _loc_dims(sampling_locations, 3)
    Bd, N, D, hs = _dist_problem(dist, H)
    if grad_value.shape != dist.shape or grad_sampling_loc.shape != sampling_locations.shape \
            or tuple(grad_output.shape) != (B, Q, H, L, P, 4):
        raise RuntimeError("gradient tensors do not match their forward tensors")
    if Bd != B:
        raise RuntimeError("inconsistent shapes between value and sampling_loc")
    _level_table(value_spatial_shapes, value_level_start_index, L, 3)
    _step_check(B, im2col_step)
    N = _level_pixels(N, dist_map, value_spatial_shapes)
    pr = _lib.Problem(B, N, H, 0, D, L, Q, P, _lib.DTYPE_F32, _dt(dist), hs, *_map(dist_map))
    with torch.cuda.device(dist.device):
        _lib.call("dfa3d_depth_score_backward" + sfx, pr, _ptr(dist), _ptr(value_spatial_shapes),
                  _ptr(value_level_start_index), _ptr(sampling_locations), _ptr(grad_output),
                  _ptr(grad_value), _ptr(grad_sampling_loc), _stream(dist))


def wms_deform_attn_forward(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                            attention_weights, depth_scores, im2col_step):
    """Returns output (B,Q,H*C), float32 (float64 for float64 inputs)."""
    VAL, F, odt, sfx = _types(value)
    _chk(value, "value", VAL); _chk(value_spatial_shapes, "spatial_shapes", _I64)
    _chk(value_level_start_index, "level_start_index", _I64)
    _chk(sampling_locations, "sampling_loc", F); _chk(attention_weights, "attn_weight", F)
    _chk(depth_scores, "depth_score", F)
    _same_device(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                 attention_weights, depth_scores)
    B, N, H, C = value.shape
    Bq, Q, Hq, L, P = _loc_dims(sampling_locations, 2)
    if (Bq, Hq) != (B, H) or tuple(value_spatial_shapes.shape) != (L, 2) \
            or tuple(attention_weights.shape) != (B, Q, H, L, P) \
            or tuple(depth_scores.shape) != (B, Q, H, L, P, 4):
        raise RuntimeError("inconsistent shapes between value, spatial_shapes (L,2), sampling_loc, "
                           "attn_weight and depth_score")
    _level_table(value_spatial_shapes, value_level_start_index, L, 2)
    _step_check(B, im2col_step)
    out = torch.empty((B, Q, H * C), dtype=odt, device=value.device)
    pr = _lib.Problem(B, N, H, C, 1, L, Q, P, _dt(value), _lib.DTYPE_F32, 0)
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_wms_attn_forward" + sfx, pr, _ptr(value), _ptr(value_spatial_shapes),
                  _ptr(value_level_start_index), _ptr(sampling_locations), _ptr(attention_weights),
                  _ptr(depth_scores), _ptr(out), _stream(value))
    return out


def wms_deform_attn_backward(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                             attention_weights, depth_scores, grad_output, grad_value,
                             grad_sampling_loc, grad_attn_weight, grad_depth_score, im2col_step):
    """Accumulates into grad_value (float32, caller-zeroed); overwrites the other three."""
    VAL, F, odt, sfx = _types(value)
    _chk(value, "value", VAL); _chk(value_spatial_shapes, "spatial_shapes", _I64)
    _chk(value_level_start_index, "level_start_index", _I64)
    _chk(sampling_locations, "sampling_loc", F); _chk(attention_weights, "attn_weight", F)
    _chk(depth_scores, "depth_score", F); _chk(grad_output, "grad_output", F)
    _chk(grad_value, "grad_value", F); _chk(grad_sampling_loc, "grad_sampling_loc", F)
    _chk(grad_attn_weight, "grad_attn_weight", F); _chk(grad_depth_score, "grad_depth_score", F)
    _same_device(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                 attention_weights, depth_scores, grad_output, grad_value, grad_sampling_loc,
                 grad_attn_weight, grad_depth_score)
    B, N, H, C = value.shape
    Bq, Q, Hq, L, P = _loc_dims(sampling_locations, 2)
    if (Bq, Hq) != (B, H) or tuple(value_spatial_shapes.shape) != (L, 2) \
            or grad_output.numel() != B * Q * H * C or grad_value.shape != value.shape \
            or grad_sampling_loc.shape != sampling_locations.shape \
            or grad_attn_weight.shape != attention_weights.shape \
            or grad_depth_score.shape != depth_scores.shape:
        raise RuntimeError("inconsistent shapes in wms_deform_attn_backward")
    _level_table(value_spatial_shapes, value_level_start_index, L, 2)
    _step_check(B, im2col_step)
    pr = _lib.Problem(B, N, H, C, 1, L, Q, P, _dt(value), _lib.DTYPE_F32, 0)
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_wms_attn_backward" + sfx, pr, _ptr(value), _ptr(value_spatial_shapes),
                  _ptr(value_level_start_index), _ptr(sampling_locations), _ptr(attention_weights),
                  _ptr(depth_scores), _ptr(grad_output), _ptr(grad_value), _ptr(grad_sampling_loc),
                  _ptr(grad_attn_weight), _ptr(grad_depth_score), _stream(value))


# ------------------------------------------------------------------------------------------------
# plain 2-D multi-scale deformable attention, with the names and signatures of the mmcv extension that
# BEVFormer_DFA3D's temporal self-attention and decoder call
# (…/bevformer/modules/multi_scale_deformable_attn_function.py:10-12, :40-46, :74-85)
# ------------------------------------------------------------------------------------------------
def ms_deform_attn_forward(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                           attention_weights, im2col_step):
    """value (B,N,H,C); shapes (L,2); locations (B,Q,H,L,P,2); weights (B,Q,H,L,P) -> (B,Q,H*C)."""
    _chk(value, "value", _VAL); _chk(value_spatial_shapes, "spatial_shapes", _I64)
    _chk(value_level_start_index, "level_start_index", _I64)
    _chk(sampling_locations, "sampling_loc", _F32); _chk(attention_weights, "attn_weight", _F32)
    _same_device(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                 attention_weights)
    B, N, H, C = value.shape
    Bq, Q, Hq, L, P = _loc_dims(sampling_locations, 2)
    if (Bq, Hq) != (B, H) or tuple(value_spatial_shapes.shape) != (L, 2) \
            or tuple(attention_weights.shape) != (B, Q, H, L, P):
        raise RuntimeError("inconsistent shapes between value, spatial_shapes (L,2), sampling_loc and "
                           "attn_weight")
    _level_table(value_spatial_shapes, value_level_start_index, L, 2)
    _step_check(B, im2col_step)
    out = torch.empty((B, Q, H * C), dtype=torch.float32, device=value.device)
    pr = _lib.Problem(B, N, H, C, 1, L, Q, P, _dt(value), _lib.DTYPE_F32, 0)
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_msda_forward", pr, _ptr(value), _ptr(value_spatial_shapes),
                  _ptr(value_level_start_index), _ptr(sampling_locations), _ptr(attention_weights),
                  _ptr(out), _stream(value))
    return out


def ms_deform_attn_backward(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                            attention_weights, grad_output, grad_value, grad_sampling_loc,
                            grad_attn_weight, im2col_step):
    """Accumulates into grad_value (float32, caller-zeroed); overwrites the other two."""
    _chk(value, "value", _VAL); _chk(value_spatial_shapes, "spatial_shapes", _I64)
    _chk(value_level_start_index, "level_start_index", _I64)
    _chk(sampling_locations, "sampling_loc", _F32); _chk(attention_weights, "attn_weight", _F32)
    _chk(grad_output, "grad_output", _F32); _chk(grad_value, "grad_value", _F32)
    _chk(grad_sampling_loc, "grad_sampling_loc", _F32); _chk(grad_attn_weight, "grad_attn_weight", _F32)
    _same_device(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                 attention_weights, grad_output, grad_value, grad_sampling_loc, grad_attn_weight)
    B, N, H, C = value.shape
    Bq, Q, Hq, L, P = _loc_dims(sampling_locations, 2)
    if (Bq, Hq) != (B, H) or tuple(value_spatial_shapes.shape) != (L, 2) \
            or grad_output.numel() != B * Q * H * C or grad_value.shape != value.shape \
            or grad_sampling_loc.shape != sampling_locations.shape \
            or grad_attn_weight.shape != attention_weights.shape:
        raise RuntimeError("inconsistent shapes in ms_deform_attn_backward")
    _level_table(value_spatial_shapes, value_level_start_index, L, 2)
    _step_check(B, im2col_step)
    pr = _lib.Problem(B, N, H, C, 1, L, Q, P, _dt(value), _lib.DTYPE_F32, 0)
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_msda_backward", pr, _ptr(value), _ptr(value_spatial_shapes),
                  _ptr(value_level_start_index), _ptr(sampling_locations), _ptr(attention_weights),
                  _ptr(grad_output), _ptr(grad_value), _ptr(grad_sampling_loc), _ptr(grad_attn_weight),
                  _stream(value))


# ------------------------------------------------------------------------------------------------
# one-launch fused entry points (no counterpart in the reference's extension; they serve the
# one-stage autograd Function)
# ------------------------------------------------------------------------------------------------
def _fused_problem(value, dist, shapes3, lsi, loc3, attn, dist_map=None):
    VAL, F, _, _ = _types(value, dist_map)
    _chk(value, "value", VAL); _chk(dist, "value_dpt_dist", VAL)
    _chk(shapes3, "spatial_shapes", _I64); _chk(lsi, "level_start_index", _I64)
    _chk(loc3, "sampling_loc", F); _chk(attn, "attn_weight", F)
    _same_device(value, dist, shapes3, lsi, loc3, attn)
    B, N, H, C = value.shape
    Bq, Q, Hq, L, P = _loc_dims(loc3, 3)
    Bd, Nd, D, hs = _dist_problem(dist, H)
    if (Bq, Hq) != (B, H) or Bd != B or not _dist_rows_ok(Nd, N, dist_map) or tuple(shapes3.shape) != (L, 3) \
            or tuple(attn.shape) != (B, Q, H, L, P):
        raise RuntimeError("inconsistent shapes between value, value_dpt_dist, spatial_shapes (L,3), "
                           "sampling_loc and attn_weight")
    _level_table(shapes3, lsi, L, 3)
    return (_lib.Problem(B, N, H, C, D, L, Q, P, _dt(value), _dt(dist), hs, *_map(dist_map)),
            (B, Q, H, L, P, C))


def dfa3d_fused_forward(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                        sampling_locations, attention_weights, im2col_step, need_depth_score=True,
                        out=None, dist_map=None):
    """Returns (output (B,Q,H*C), depth_score (B,Q,H,L,P,4) or None).  `out`, if given, is a
    preallocated float32 (B,Q,H*C) tensor that receives the output (every element is written).
    dist_map=(h, w): value_dpt_dist is ONE h x w map per camera, (B, h*w, D) [or (B, h*w, H, D)], read by
    every level with nearest-neighbour indexing instead of one resized copy per level."""
    pr, (B, Q, H, L, P, C) = _fused_problem(value, value_dpt_dist, value_spatial_shapes,
                                            value_level_start_index, sampling_locations,
                                            attention_weights, dist_map)
    _step_check(B, im2col_step)
    dev = value.device
    _, F, odt, sfx = _types(value, dist_map)
    if out is None:
        out = torch.empty((B, Q, H * C), dtype=odt, device=dev)
    else:
        _chk(out, "out", F)
        _same_device(value, out)
        if out.numel() != B * Q * H * C:
            raise RuntimeError("out has the wrong number of elements")
    ds = torch.empty((B, Q, H, L, P, 4), dtype=odt, device=dev) if need_depth_score else None
    with torch.cuda.device(dev):
        _lib.call("dfa3d_fused_forward" + sfx, pr, _ptr(value), _ptr(value_dpt_dist),
                  _ptr(value_spatial_shapes), _ptr(value_level_start_index),
                  _ptr(sampling_locations), _ptr(attention_weights), _ptr(out), _ptr(ds),
                  _stream(value))
    return out, ds


def dfa3d_fused_backward(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                         sampling_locations, attention_weights, grad_output, grad_value,
                         grad_value_dpt_dist, grad_sampling_loc, grad_attn_weight, im2col_step,
                         dist_map=None):
    """Accumulates into grad_value and grad_value_dpt_dist (float32, caller-zeroed); overwrites
    grad_sampling_loc (B,Q,H,L,P,3) and grad_attn_weight."""
    pr, (B, Q, H, L, P, C) = _fused_problem(value, value_dpt_dist, value_spatial_shapes,
                                            value_level_start_index, sampling_locations,
                                            attention_weights, dist_map)
    _, F, _, sfx = _types(value, dist_map)
    for t, n in ((grad_output, "grad_output"), (grad_value, "grad_value"),
                 (grad_value_dpt_dist, "grad_value_dpt_dist"), (grad_sampling_loc, "grad_sampling_loc"),
                 (grad_attn_weight, "grad_attn_weight")):
        _chk(t, n, F)
    _same_device(value, grad_output, grad_value, grad_value_dpt_dist, grad_sampling_loc,
                 grad_attn_weight)
    if grad_output.numel() != B * Q * H * C or grad_value.shape != value.shape \
            or grad_value_dpt_dist.shape != value_dpt_dist.shape \
            or grad_sampling_loc.shape != sampling_locations.shape \
            or grad_attn_weight.shape != attention_weights.shape:
        raise RuntimeError("inconsistent shapes in dfa3d_fused_backward")
    _step_check(B, im2col_step)
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_fused_backward" + sfx, pr, _ptr(value), _ptr(value_dpt_dist),
                  _ptr(value_spatial_shapes), _ptr(value_level_start_index),
                  _ptr(sampling_locations), _ptr(attention_weights), _ptr(grad_output),
                  _ptr(grad_value), _ptr(grad_value_dpt_dist), _ptr(grad_sampling_loc),
                  _ptr(grad_attn_weight), _stream(value))


# ------------------------------------------------------------------------------------------------
# caller-fused entry points: the location assembly and the softmax of the attention module happen
# inside the kernels (BEVFormer_DFA3D/.../spatial_cross_attention.py:503-538)
# ------------------------------------------------------------------------------------------------
def _attn3d_problem(value, dist, shapes3, lsi, ref, off_uv, off_d, logits, dist_map=None):
    _chk(value, "value", _VAL); _chk(dist, "value_dpt_dist", _VAL)
    _chk(shapes3, "spatial_shapes", _I64); _chk(lsi, "level_start_index", _I64)
    for t, n in ((ref, "reference_points"), (off_uv, "sampling_offsets_uv"),
                 (off_d, "sampling_offsets_depth"), (logits, "attention_logits")):
        _chk(t, n, _F32)
    _same_device(value, dist, shapes3, lsi, ref, off_uv, off_d, logits)
    B, N, H, C = value.shape
    if off_uv.dim() != 6 or off_uv.shape[-1] != 2:
        raise RuntimeError(f"sampling_offsets_uv must be (B,Q,H,L,P,2), got {tuple(off_uv.shape)}")
    Bq, Q, Hq, L, P, _ = off_uv.shape
    Bd, Nd, D, hs = _dist_problem(dist, H)
    if ref.dim() != 4 or ref.shape[-1] != 3 or tuple(ref.shape[:2]) != (B, Q):
        raise RuntimeError(f"reference_points must be (B,Q,Z,3), got {tuple(ref.shape)}")
    Z = ref.shape[2]
    if Z <= 0 or P % Z != 0:
        raise RuntimeError(f"the number of anchors ({Z}) must divide the points per level ({P})")
    if (Bq, Hq) != (B, H) or Bd != B or not _dist_rows_ok(Nd, N, dist_map) or tuple(shapes3.shape) != (L, 3) \
            or off_d.numel() != B * Q * H * L * P or logits.numel() != B * Q * H * L * P:
        raise RuntimeError("inconsistent shapes between value, value_dpt_dist, spatial_shapes (L,3), "
                           "offsets and logits")
    _level_table(shapes3, lsi, L, 3)
    return _lib.Problem(B, N, H, C, D, L, Q, P, _dt(value), _dt(dist), hs, *_map(dist_map)), Z, (B, Q, H, C)


def dfa3d_attn3d_forward(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                         reference_points, sampling_offsets_uv, sampling_offsets_depth,
                         attention_logits, out=None, dist_map=None):
    """value (B,N,H,C); value_dpt_dist (B,N,D)|(B,N,H,D); reference_points (B,Q,Z,3);
    sampling_offsets_uv (B,Q,H,L,P,2) in pixels; sampling_offsets_depth (B,Q,H,L,P) in bins;
    attention_logits (B,Q,H,L*P) before the softmax.  Returns output (B,Q,H*C)."""
    pr, Z, (B, Q, H, C) = _attn3d_problem(value, value_dpt_dist, value_spatial_shapes,
                                          value_level_start_index, reference_points,
                                          sampling_offsets_uv, sampling_offsets_depth, attention_logits,
                                          dist_map)
    if out is None:
        out = torch.empty((B, Q, H * C), dtype=torch.float32, device=value.device)
    else:
        _chk(out, "out", _F32)
        _same_device(value, out)
        if out.numel() != B * Q * H * C:
            raise RuntimeError("out has the wrong number of elements")
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_attn3d_forward", pr, Z, _ptr(value), _ptr(value_dpt_dist),
                  _ptr(value_spatial_shapes), _ptr(value_level_start_index), _ptr(reference_points),
                  _ptr(sampling_offsets_uv), _ptr(sampling_offsets_depth), _ptr(attention_logits),
                  _ptr(out), _stream(value))
    return out


def dfa3d_attn3d_backward(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                          reference_points, sampling_offsets_uv, sampling_offsets_depth,
                          attention_logits, grad_output, grad_value, grad_value_dpt_dist,
                          grad_offsets_uv, grad_offsets_depth, grad_logits, dist_map=None):
    """Accumulates into grad_value / grad_value_dpt_dist (float32, caller-zeroed); overwrites the
    gradients of the offsets and of the logits."""
    pr, Z, (B, Q, H, C) = _attn3d_problem(value, value_dpt_dist, value_spatial_shapes,
                                          value_level_start_index, reference_points,
                                          sampling_offsets_uv, sampling_offsets_depth, attention_logits,
                                          dist_map)
    for t, n in ((grad_output, "grad_output"), (grad_value, "grad_value"),
                 (grad_value_dpt_dist, "grad_value_dpt_dist"), (grad_offsets_uv, "grad_offsets_uv"),
                 (grad_offsets_depth, "grad_offsets_depth"), (grad_logits, "grad_logits")):
        _chk(t, n, _F32)
    _same_device(value, grad_output, grad_value, grad_value_dpt_dist, grad_offsets_uv, grad_offsets_depth,
                 grad_logits)
    if grad_output.numel() != B * Q * H * C or grad_value.shape != value.shape \
            or grad_value_dpt_dist.shape != value_dpt_dist.shape \
            or grad_offsets_uv.shape != sampling_offsets_uv.shape \
            or grad_offsets_depth.numel() != sampling_offsets_depth.numel() \
            or grad_logits.numel() != attention_logits.numel():
        raise RuntimeError("inconsistent shapes in dfa3d_attn3d_backward")
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_attn3d_backward", pr, Z, _ptr(value), _ptr(value_dpt_dist),
                  _ptr(value_spatial_shapes), _ptr(value_level_start_index), _ptr(reference_points),
                  _ptr(sampling_offsets_uv), _ptr(sampling_offsets_depth), _ptr(attention_logits),
                  _ptr(grad_output), _ptr(grad_value), _ptr(grad_value_dpt_dist), _ptr(grad_offsets_uv),
                  _ptr(grad_offsets_depth), _ptr(grad_logits), _stream(value))


# ------------------------------------------------------------------------------------------------
# ragged variants: cameras with different numbers of queries share one launch.  Per-query tensors are
# packed rows without a batch dimension; query_offsets (B+1 int32, CUDA) says which rows belong to
# which camera; max_queries bounds the queries of any one camera (it sizes the launch).
# ------------------------------------------------------------------------------------------------
_I32 = (torch.int32,)


def _ragged_common(value, dist, shapes3, lsi, query_offsets, max_queries, rows, per_row, names,
                   dist_map=None):
    """Checks shared by the ragged entry points.  `per_row`: tensors whose first dimension is the packed
    row count `rows`.  Returns the problem descriptor with Q = max_queries."""
    _chk(value, "value", _VAL); _chk(dist, "value_dpt_dist", _VAL)
    _chk(shapes3, "spatial_shapes", _I64); _chk(lsi, "level_start_index", _I64)
    _chk(query_offsets, "query_offsets", _I32)
    for t, n in zip(per_row, names):
        _chk(t, n, _F32)
        if t.shape[0] != rows:
            raise RuntimeError(f"{n} must have {rows} packed rows, got {t.shape[0]}")
    _same_device(value, dist, shapes3, lsi, query_offsets, *per_row)
    B, N, H, C = value.shape
    Bd, Nd, D, hs = _dist_problem(dist, H)
    if Bd != B or not _dist_rows_ok(Nd, N, dist_map) or query_offsets.numel() != B + 1:
        raise RuntimeError("inconsistent shapes between value, value_dpt_dist and query_offsets (B+1)")
    if int(max_queries) < 0:
        raise RuntimeError("max_queries must be >= 0")
    return B, N, H, C, D, hs


def dfa3d_fused_forward_ragged(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                               sampling_locations, attention_weights, query_offsets, max_queries,
                               need_depth_score=True, dist_map=None):
    """sampling_locations (R,H,L,P,3), attention_weights (R,H,L,P) -> (output (R,H*C), depth_score
    (R,H,L,P,4) or None)."""
    if sampling_locations.dim() != 5 or sampling_locations.shape[-1] != 3:
        raise RuntimeError("sampling_locations must be (R,H,L,P,3)")
    R, Hq, L, P, _ = sampling_locations.shape
    B, N, H, C, D, hs = _ragged_common(value, value_dpt_dist, value_spatial_shapes,
                                       value_level_start_index, query_offsets, max_queries, R,
                                       (sampling_locations, attention_weights),
                                       ("sampling_loc", "attn_weight"), dist_map)
    if Hq != H or tuple(attention_weights.shape) != (R, H, L, P):
        raise RuntimeError("inconsistent shapes between value, sampling_loc and attn_weight")
    _level_table(value_spatial_shapes, value_level_start_index, L, 3)
    dev = value.device
    out = torch.empty((R, H * C), dtype=torch.float32, device=dev)
    ds = torch.empty((R, H, L, P, 4), dtype=torch.float32, device=dev) if need_depth_score else None
    pr = _lib.Problem(B, N, H, C, D, L, int(max_queries), P, _dt(value), _dt(value_dpt_dist), hs,
                      *_map(dist_map))
    with torch.cuda.device(dev):
        _lib.call("dfa3d_fused_forward_ragged", pr, _ptr(query_offsets), _ptr(value), _ptr(value_dpt_dist),
                  _ptr(value_spatial_shapes), _ptr(value_level_start_index), _ptr(sampling_locations),
                  _ptr(attention_weights), _ptr(out), _ptr(ds), _stream(value))
    return out, ds


def dfa3d_fused_backward_ragged(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                                sampling_locations, attention_weights, query_offsets, max_queries,
                                grad_output, grad_value, grad_value_dpt_dist, grad_sampling_loc,
                                grad_attn_weight, dist_map=None):
    """Accumulates into grad_value / grad_value_dpt_dist (float32, caller-zeroed); overwrites
    grad_sampling_loc (R,H,L,P,3) and grad_attn_weight (R,H,L,P)."""
    R, Hq, L, P, _ = sampling_locations.shape
    B, N, H, C, D, hs = _ragged_common(
        value, value_dpt_dist, value_spatial_shapes, value_level_start_index, query_offsets, max_queries,
        R, (sampling_locations, attention_weights, grad_output, grad_sampling_loc, grad_attn_weight),
        ("sampling_loc", "attn_weight", "grad_output", "grad_sampling_loc", "grad_attn_weight"), dist_map)
    _chk(grad_value, "grad_value", _F32); _chk(grad_value_dpt_dist, "grad_value_dpt_dist", _F32)
    _same_device(value, grad_value, grad_value_dpt_dist)
    if Hq != H or grad_output.numel() != R * H * C or grad_value.shape != value.shape \
            or grad_value_dpt_dist.shape != value_dpt_dist.shape \
            or grad_sampling_loc.shape != sampling_locations.shape \
            or grad_attn_weight.shape != attention_weights.shape:
        raise RuntimeError("inconsistent shapes in dfa3d_fused_backward_ragged")
    _level_table(value_spatial_shapes, value_level_start_index, L, 3)
    pr = _lib.Problem(B, N, H, C, D, L, int(max_queries), P, _dt(value), _dt(value_dpt_dist), hs,
                      *_map(dist_map))
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_fused_backward_ragged", pr, _ptr(query_offsets), _ptr(value),
                  _ptr(value_dpt_dist), _ptr(value_spatial_shapes), _ptr(value_level_start_index),
                  _ptr(sampling_locations), _ptr(attention_weights), _ptr(grad_output), _ptr(grad_value),
                  _ptr(grad_value_dpt_dist), _ptr(grad_sampling_loc), _ptr(grad_attn_weight),
                  _stream(value))


def _attn3d_ragged_problem(value, dist, shapes3, lsi, ref, off_uv, off_d, logits, query_offsets,
                           max_queries, extra=(), extra_names=(), dist_map=None):
    if off_uv.dim() != 5 or off_uv.shape[-1] != 2:
        raise RuntimeError(f"sampling_offsets_uv must be (R,H,L,P,2), got {tuple(off_uv.shape)}")
    R, Hq, L, P, _ = off_uv.shape
    B, N, H, C, D, hs = _ragged_common(
        value, dist, shapes3, lsi, query_offsets, max_queries, R,
        (ref, off_uv, off_d, logits) + tuple(extra),
        ("reference_points", "sampling_offsets_uv", "sampling_offsets_depth", "attention_logits")
        + tuple(extra_names), dist_map)
    if ref.dim() != 3 or ref.shape[-1] != 3:
        raise RuntimeError(f"reference_points must be (R,Z,3), got {tuple(ref.shape)}")
    Z = ref.shape[1]
    if Z <= 0 or P % Z != 0:
        raise RuntimeError(f"the number of anchors ({Z}) must divide the points per level ({P})")
    if Hq != H or off_d.numel() != R * H * L * P or logits.numel() != R * H * L * P:
        raise RuntimeError("inconsistent shapes between value, offsets and logits")
    _level_table(shapes3, lsi, L, 3)
    pr = _lib.Problem(B, N, H, C, D, L, int(max_queries), P, _dt(value), _dt(dist), hs, *_map(dist_map))
    return pr, Z, (R, H, C)


def dfa3d_attn3d_forward_ragged(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                                reference_points, sampling_offsets_uv, sampling_offsets_depth,
                                attention_logits, query_offsets, max_queries, dist_map=None):
    """reference_points (R,Z,3); sampling_offsets_uv (R,H,L,P,2); sampling_offsets_depth (R,H,L,P);
    attention_logits (R,H,L*P).  Returns output (R,H*C)."""
    pr, Z, (R, H, C) = _attn3d_ragged_problem(
        value, value_dpt_dist, value_spatial_shapes, value_level_start_index, reference_points,
        sampling_offsets_uv, sampling_offsets_depth, attention_logits, query_offsets, max_queries,
        dist_map=dist_map)
    out = torch.empty((R, H * C), dtype=torch.float32, device=value.device)
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_attn3d_forward_ragged", pr, Z, _ptr(query_offsets), _ptr(value),
                  _ptr(value_dpt_dist), _ptr(value_spatial_shapes), _ptr(value_level_start_index),
                  _ptr(reference_points), _ptr(sampling_offsets_uv), _ptr(sampling_offsets_depth),
                  _ptr(attention_logits), _ptr(out), _stream(value))
    return out


def dfa3d_attn3d_backward_ragged(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                                 reference_points, sampling_offsets_uv, sampling_offsets_depth,
                                 attention_logits, query_offsets, max_queries, grad_output, grad_value,
                                 grad_value_dpt_dist, grad_offsets_uv, grad_offsets_depth, grad_logits,
                                 dist_map=None):
    """Accumulates into grad_value / grad_value_dpt_dist (float32, caller-zeroed); overwrites the
    gradients of the offsets and of the logits (packed rows)."""
    pr, Z, (R, H, C) = _attn3d_ragged_problem(
        value, value_dpt_dist, value_spatial_shapes, value_level_start_index, reference_points,
        sampling_offsets_uv, sampling_offsets_depth, attention_logits, query_offsets, max_queries,
        (grad_output, grad_offsets_uv, grad_offsets_depth, grad_logits),
        ("grad_output", "grad_offsets_uv", "grad_offsets_depth", "grad_logits"), dist_map)
    _chk(grad_value, "grad_value", _F32); _chk(grad_value_dpt_dist, "grad_value_dpt_dist", _F32)
    _same_device(value, grad_value, grad_value_dpt_dist)
    if grad_output.numel() != R * H * C or grad_value.shape != value.shape \
            or grad_value_dpt_dist.shape != value_dpt_dist.shape \
            or grad_offsets_uv.shape != sampling_offsets_uv.shape \
            or grad_offsets_depth.numel() != sampling_offsets_depth.numel() \
            or grad_logits.numel() != attention_logits.numel():
        raise RuntimeError("inconsistent shapes in dfa3d_attn3d_backward_ragged")
    with torch.cuda.device(value.device):
        _lib.call("dfa3d_attn3d_backward_ragged", pr, Z, _ptr(query_offsets), _ptr(value),
                  _ptr(value_dpt_dist), _ptr(value_spatial_shapes), _ptr(value_level_start_index),
                  _ptr(reference_points), _ptr(sampling_offsets_uv), _ptr(sampling_offsets_depth),
                  _ptr(attention_logits), _ptr(grad_output), _ptr(grad_value), _ptr(grad_value_dpt_dist),
                  _ptr(grad_offsets_uv), _ptr(grad_offsets_depth), _ptr(grad_logits), _stream(value))
