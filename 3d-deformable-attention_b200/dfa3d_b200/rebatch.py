"""Per-camera re-batching of BEV queries on the device.

BEVFormer's spatial cross-attention lets every camera attend only from the BEV queries it sees.  The
reference finds them with ``nonzero()`` per camera (a host synchronisation each), copies queries and
reference points into tensors padded to the longest list with Python double loops, and adds the results
back with more loops (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/
spatial_cross_attention.py:700-722, :741-748).  Here a ``RebatchPlan`` holds the lists as device index
tensors built by one call (``dfa3d_rebatch_plan``), the rows are PACKED (exactly the visible
(camera, query) pairs, no padding) and moved by two kernels, and the operator takes the plan's
per-camera row offsets so that cameras of different length share one launch.

A plan depends only on ``bev_mask``, which is geometry: build it once per frame and hand it to every
encoder layer.  Building reads one integer back (the packed row count, needed to size tensors); nothing
after that synchronises.
"""
import torch
from torch.autograd.function import Function, once_differentiable

from . import _lib


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


class RebatchPlan:
    """Index tensors of one ``bev_mask`` (num_cams, bs, Q, Z).

    counts (cams), offsets (cams+1), op_offsets (bs*cams+1) int32; packed_query / packed_camera (T)
    int32; row_of (cams, Q) int32 (-1 = not seen); inv_count (bs, Q) float32; ``rows`` = T = packed rows
    of one batch element, ``max_queries`` = longest camera list (both Python ints).
    """

    def __init__(self, bev_mask):
        if bev_mask.dim() != 4:
            raise RuntimeError("bev_mask must be (num_cams, bs, Q, Z)")
        if not bev_mask.is_cuda:
            raise RuntimeError("bev_mask must be a CUDA tensor")
        cams, bs, Q, Z = bev_mask.shape
        mask = bev_mask.contiguous()
        mask = mask.view(torch.uint8) if mask.dtype == torch.bool else (mask != 0).view(torch.uint8)
        dev = mask.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.cams, self.bs, self.Q, self.Z = cams, bs, Q, Z
        self.counts = torch.empty(cams, **i32)
        self.offsets = torch.empty(cams + 1, **i32)
        self.op_offsets = torch.empty(bs * cams + 1, **i32)
        packed_query = torch.empty(max(1, cams * Q), **i32)
        packed_camera = torch.empty(max(1, cams * Q), **i32)
        self.row_of = torch.empty((cams, Q), **i32)
        self.inv_count = torch.empty((bs, Q), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.call_plain("dfa3d_rebatch_plan", mask.data_ptr(), cams, bs, Q, Z, self.counts.data_ptr(),
                            self.offsets.data_ptr(), self.op_offsets.data_ptr(), packed_query.data_ptr(),
                            packed_camera.data_ptr(), self.row_of.data_ptr(), self.inv_count.data_ptr(),
                            _stream(mask))
        counts = self.counts.tolist()            # the one read-back: sizes of the packed tensors
        self.rows = int(sum(counts))
        self.max_queries = int(max(counts)) if counts else 0
        self.packed_query = packed_query[:self.rows]
        self.packed_camera = packed_camera[:self.rows]
        self._pq, self._pc = packed_query, packed_camera     # keep the full buffers alive

    @property
    def device(self):
        return self.counts.device


def _gather(plan, src, width, cam_stride, batch_stride, scale):
    dst = torch.empty((plan.bs * plan.rows, width), dtype=torch.float32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.call_plain("dfa3d_rebatch_gather", src.data_ptr(), plan._pq.data_ptr(), plan._pc.data_ptr(),
                        plan.offsets.data_ptr(), plan.cams, plan.bs, plan.Q, width, cam_stride, batch_stride,
                        None if scale is None else scale.data_ptr(), dst.data_ptr(), plan.bs * plan.rows,
                        _stream(src))
    return dst


def _combine(plan, packed, width, scale):
    dst = torch.empty((plan.bs, plan.Q, width), dtype=torch.float32, device=packed.device)
    # an empty plan has no packed rows and PyTorch gives an empty tensor no storage: hand the library some
    # valid address instead of null (with no rows, row_of is all -1 and nothing is read through it)
    src_ptr = packed.data_ptr() if packed.numel() else plan.inv_count.data_ptr()
    with torch.cuda.device(packed.device):
        _lib.call_plain("dfa3d_rebatch_combine", src_ptr, plan.row_of.data_ptr(),
                        plan.offsets.data_ptr(), plan.cams, plan.bs, plan.Q, width,
                        None if scale is None else scale.data_ptr(), dst.data_ptr(), _stream(packed))
    return dst


def _check(t, name):
    if not t.is_cuda or t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be a float32 CUDA tensor")
    return t.contiguous()


class GatherQueriesFunction(Function):
    """(bs, Q, W) in BEV order -> (bs*T, W) packed rows: row j*T + p holds query packed_query[p] of
    batch element j (spatial_cross_attention.py:714-717).  Backward: sum over the cameras of a query."""

    @staticmethod
    def forward(ctx, src, plan):
        src = _check(src, "src")
        if tuple(src.shape[:2]) != (plan.bs, plan.Q):
            raise RuntimeError(f"src must be (bs={plan.bs}, Q={plan.Q}, W), got {tuple(src.shape)}")
        ctx.plan, ctx.width = plan, src.shape[2]
        return _gather(plan, src, src.shape[2], 0, plan.Q, None)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        return _combine(ctx.plan, _check(grad, "grad"), ctx.width, None), None


class GatherSharedRowsFunction(Function):
    """(Q, W) rows shared by all batch elements and cameras -> (bs*T, W) packed rows (the empty-query
    embedding, spatial_cross_attention.py:721-722).  Backward: sum over cameras and batch elements."""

    @staticmethod
    def forward(ctx, src, plan):
        src = _check(src, "src")
        if src.shape[0] != plan.Q or src.dim() != 2:
            raise RuntimeError(f"src must be (Q={plan.Q}, W), got {tuple(src.shape)}")
        ctx.plan, ctx.width = plan, src.shape[1]
        return _gather(plan, src, src.shape[1], 0, 0, None)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        return _combine(ctx.plan, _check(grad, "grad"), ctx.width, None).sum(0), None


def gather_per_camera(src, plan):
    """(cams, bs, Q, ...) per-camera rows (the projected reference points, spatial_cross_attention.py:
    718-719) -> (bs*T, ...) packed rows.  No gradient (the reference points come from fixed geometry)."""
    src = _check(src.detach(), "src")
    if tuple(src.shape[:3]) != (plan.cams, plan.bs, plan.Q):
        raise RuntimeError(f"src must be (cams, bs, Q, ...), got {tuple(src.shape)}")
    width = 1
    for s in src.shape[3:]:
        width *= s
    out = _gather(plan, src, width, plan.bs * plan.Q, plan.Q, None)
    return out.view((plan.bs * plan.rows,) + tuple(src.shape[3:]))


class CombineCamerasFunction(Function):
    """(bs*T, W) packed per-camera results -> (bs, Q, W): sum over the cameras that see a query, divided
    by their number (at least 1), zeros where no camera sees it (spatial_cross_attention.py:741-748).
    Backward: each packed row receives its query's gradient times the same factor."""

    @staticmethod
    def forward(ctx, packed, plan):
        packed = _check(packed, "packed")
        if packed.dim() != 2 or packed.shape[0] != plan.bs * plan.rows:
            raise RuntimeError(f"packed must be (bs*T={plan.bs * plan.rows}, W), got {tuple(packed.shape)}")
        ctx.plan, ctx.width = plan, packed.shape[1]
        return _combine(plan, packed, packed.shape[1], plan.inv_count)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        plan = ctx.plan
        return _gather(plan, _check(grad, "grad"), ctx.width, 0, plan.Q, plan.inv_count), None
