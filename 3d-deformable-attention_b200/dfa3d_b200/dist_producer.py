"""Depth distribution straight from the depth network's logits, in the operator's layout.

``depth_distribution(logits, spatial_shapes, level_start_index)`` does in one kernel what the reference
does in four passes: softmax (or sigmoid) over the D channels of the (B, D, h, w) logits, one
``F.interpolate(mode="nearest")`` per feature level, and the flatten / permute / cat into (B, N, D)
(BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/dense_heads/depth_head.py:265-276,
…/modules/transformer.py:368-391, …/modules/spatial_cross_attention.py:727-728).  The result can be
float32 or bfloat16; its backward is one kernel as well.  With ``single_map=True`` only the softmaxed
map itself is written, channel-last, for the operator's ``dist_map`` option (every level then reads
that one map with nearest indexing and no resized copy is made at all).
"""
import torch
from torch.autograd.function import Function, once_differentiable

from . import _lib


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _check(logits, shapes, lsi):
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 4:
        raise RuntimeError("logits must be a float32 CUDA tensor (B, D, h, w)")
    if shapes.dtype != torch.int64 or lsi.dtype != torch.int64 or shapes.dim() != 2 \
            or shapes.shape[1] not in (2, 3) or lsi.numel() != shapes.shape[0]:
        raise RuntimeError("spatial_shapes must be int64 (L, 2|3) and level_start_index int64 (L)")
    if shapes.device != logits.device or lsi.device != logits.device:
        raise RuntimeError("all tensors must be on one device")
    return logits.contiguous(), shapes.contiguous(), lsi.contiguous()


_DTYPES = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16}


class DepthDistributionFunction(Function):
    @staticmethod
    def forward(ctx, logits, spatial_shapes, level_start_index, num_pixels, activation="softmax",
                dtype=torch.float32):
        """logits (B, D, h, w) float32; spatial_shapes (L, 2|3) / level_start_index (L) int64 on the
        device; num_pixels = N = sum of the levels' pixels.  Returns dist (B, N, D) of `dtype`."""
        logits, shapes, lsi = _check(logits, spatial_shapes, level_start_index)
        if activation not in ("softmax", "sigmoid"):
            raise ValueError("activation must be 'softmax' or 'sigmoid'")
        if dtype not in _DTYPES:
            raise ValueError("dtype must be torch.float32, torch.bfloat16 or torch.float16")
        B, D, h, w = logits.shape
        act = _lib.ACT_SOFTMAX if activation == "softmax" else _lib.ACT_SIGMOID
        dist = torch.empty((B, int(num_pixels), D), dtype=dtype, device=logits.device)
        with torch.cuda.device(logits.device):
            _lib.call_plain("dfa3d_dist_from_logits", logits.data_ptr(), B, D, h, w, shapes.data_ptr(),
                            shapes.shape[1], lsi.data_ptr(), shapes.shape[0], int(num_pixels), act,
                            _DTYPES[dtype],
                            dist.data_ptr(), _stream(logits))
        ctx.save_for_backward(logits, shapes, lsi)
        ctx.act, ctx.N = act, int(num_pixels)
        return dist

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_dist):
        logits, shapes, lsi = ctx.saved_tensors
        B, D, h, w = logits.shape
        grad_dist = grad_dist.float().contiguous()
        grad_logits = torch.empty_like(logits)
        with torch.cuda.device(logits.device):
            _lib.call_plain("dfa3d_dist_from_logits_backward", logits.data_ptr(), B, D, h, w,
                            shapes.data_ptr(), shapes.shape[1], lsi.data_ptr(), shapes.shape[0], ctx.N,
                            ctx.act, grad_dist.data_ptr(), grad_logits.data_ptr(), _stream(logits))
        return grad_logits, None, None, None, None, None


def depth_distribution(logits, spatial_shapes=None, level_start_index=None, num_pixels=None,
                       activation="softmax", dtype=torch.float32, single_map=False):
    """dist (B, N, D) for all levels, or -- single_map=True -- the (B, h*w, D) map alone together with
    its (h, w), to be passed to the operator as ``dist_map``."""
    if single_map:
        B, D, h, w = logits.shape
        shapes = torch.tensor([[h, w]], dtype=torch.int64, device=logits.device)
        lsi = torch.zeros(1, dtype=torch.int64, device=logits.device)
        return DepthDistributionFunction.apply(logits, shapes, lsi, h * w, activation, dtype), (h, w)
    if num_pixels is None:
        num_pixels = int((spatial_shapes[:, 0] * spatial_shapes[:, 1]).sum())
    return DepthDistributionFunction.apply(logits, spatial_shapes, level_start_index, num_pixels,
                                           activation, dtype)
