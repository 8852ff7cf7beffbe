"""Autograd Functions with the names, argument order and return conventions of the reference.

  * MultiScaleDepthScoreSampleFunction, WeightedMultiScaleDeformableAttnFunction (two-stage API):
    DFA3D/dfa3D/ops/multi_scale_3D_deform_attn.py:22-66 and :67-145.
  * MultiScale3DDeformableAttnFunction (one-stage): semantics of the BEVFormer-side copy
    BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/
    multi_scale_3ddeformable_attn_function.py:276-352 (forward returns (output, depth_score); backward
    returns gradients for value, value_dpt_dist, sampling_locations (x, y and z) and
    attention_weights).  The package-level copy at multi_scale_3D_deform_attn.py:146-221 cannot run
    its backward (it returns 8 gradients for 7 inputs and drops the x/y location gradient), so the
    working copy is the one reproduced.
  * `_fp32` aliases cast inputs to float32 under autocast like the reference's
    ``custom_fwd(cast_inputs=torch.float32)`` variants.

  * `_fp16` aliases are the reference's ``custom_fwd(cast_inputs=torch.float16)`` variants
    (…attn_function.py:24,183,353; multi_scale_deformable_attn_function.py:15), which the reference's
    modules pick when ``value`` is half (spatial_cross_attention.py:556-560).  The reference's kernels are
    instantiated for float and double only, so there those classes stop with "not implemented for
    'Half'"; here value / value_dpt_dist stay half in memory and are read as such by the kernels, the small
    tensors are widened to float32, arithmetic is float32 and the outputs come back as half.

Differences, all additive: ``value_dpt_dist`` may also be (B,N,D), shared by all heads (the reference
needs it repeated per head); ``value`` / ``value_dpt_dist`` may be bfloat16; the one-stage Function
takes an optional trailing ``return_depth_score`` flag; the one-stage backward is a single kernel
that recomputes the depth scores instead of re-reading them.
"""
import torch
from torch.autograd.function import Function, once_differentiable

from . import ext as ext_module


def _grad_dtype(t):
    """Gradients are float32 (also for bfloat16 / float16 storage) unless the call is in double precision."""
    return torch.float64 if t.dtype == torch.float64 else torch.float32


class MultiScaleDepthScoreSampleFunction(Function):
    @staticmethod
    def forward(ctx, value, value_spatial_shapes, value_level_start_index, sampling_locations,
                im2col_step):
        """value: depth distribution (B,N,H,D); spatial shapes (L,3); locations (B,Q,H,L,P,3).
        Returns depth_score (B,Q,H,L,P,4)."""
        ctx.im2col_step = im2col_step
        output = ext_module.ms_depth_score_sample_forward(
            value, value_spatial_shapes, value_level_start_index, sampling_locations,
            im2col_step=ctx.im2col_step)
        ctx.save_for_backward(value, value_spatial_shapes, value_level_start_index, sampling_locations)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, shapes, lsi, loc = ctx.saved_tensors
        grad_value = torch.zeros(value.shape, dtype=_grad_dtype(value), device=value.device)
        grad_sampling_loc = torch.empty_like(loc)     # every element is written by the kernel
        ext_module.ms_depth_score_sample_backward(
            value, shapes, lsi, loc, grad_output.contiguous(), grad_value, grad_sampling_loc,
            im2col_step=ctx.im2col_step)
        return grad_value, None, None, grad_sampling_loc, None


class WeightedMultiScaleDeformableAttnFunction(Function):
    @staticmethod
    def forward(ctx, value, value_spatial_shapes, value_level_start_index, sampling_locations,
                attention_weights, depth_score, im2col_step):
        """value (B,N,H,C); spatial shapes (L,2); locations (B,Q,H,L,P,2); attention (B,Q,H,L,P);
        depth_score (B,Q,H,L,P,4).  Returns (B,Q,H*C)."""
        ctx.im2col_step = im2col_step
        output = ext_module.wms_deform_attn_forward(
            value, value_spatial_shapes, value_level_start_index, sampling_locations,
            attention_weights, depth_score, im2col_step=ctx.im2col_step)
        ctx.save_for_backward(value, value_spatial_shapes, value_level_start_index,
                              sampling_locations, attention_weights, depth_score)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, shapes, lsi, loc, attn, depth_score = ctx.saved_tensors
        grad_value = torch.zeros(value.shape, dtype=_grad_dtype(value), device=value.device)
        grad_sampling_loc = torch.empty_like(loc)
        grad_attn_weight = torch.empty_like(attn)
        grad_depth_score = torch.empty_like(depth_score)
        ext_module.wms_deform_attn_backward(
            value, shapes, lsi, loc, attn, depth_score, grad_output.contiguous(), grad_value,
            grad_sampling_loc, grad_attn_weight, grad_depth_score, im2col_step=ctx.im2col_step)
        return grad_value, None, None, grad_sampling_loc, grad_attn_weight, grad_depth_score, None


class MultiScale3DDeformableAttnFunction(Function):
    @staticmethod
    def forward(ctx, value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                sampling_locations, attention_weights, im2col_step, return_depth_score=True,
                dist_map=None):
        """value (B,N,H,C); value_dpt_dist (B,N,H,D) or (B,N,D); spatial shapes (L,3);
        locations (B,Q,H,L,P,3); attention (B,Q,H,L,P).  Returns (output (B,Q,H*C), depth_score).
        dist_map=(h, w): value_dpt_dist is one h x w map per camera, (B,h*w,D) or (B,h*w,H,D), that all
        levels read with nearest indexing (the reference resizes it to every level first,
        depth_head.py:273-276)."""
        ctx.im2col_step = im2col_step
        ctx.dist_map = dist_map
        ctx.set_materialize_grads(False)
        output, depth_score = ext_module.dfa3d_fused_forward(
            value, value_dpt_dist, value_spatial_shapes, value_level_start_index, sampling_locations,
            attention_weights, im2col_step=ctx.im2col_step, need_depth_score=return_depth_score,
            dist_map=dist_map)
        ctx.save_for_backward(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                              sampling_locations, attention_weights)
        return output, depth_score

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output, grad_depth_score_=None):
        # As in the reference (…attn_function.py:315-316) a gradient flowing into the returned
        # depth_score is not supported.  Gradients are not materialised, so the usual case (nothing
        # consumes depth_score's gradient) arrives as None and costs no device synchronisation.
        if grad_depth_score_ is not None and grad_depth_score_.sum() != 0.0:
            raise NotImplementedError
        value, dist, shapes, lsi, loc, attn = ctx.saved_tensors
        if grad_output is None:
            return (None,) * 9
        grad_value = torch.zeros(value.shape, dtype=_grad_dtype(value), device=value.device)
        grad_dist = torch.zeros(dist.shape, dtype=_grad_dtype(value), device=dist.device)
        grad_sampling_loc = torch.empty_like(loc)
        grad_attn_weight = torch.empty_like(attn)
        ext_module.dfa3d_fused_backward(
            value, dist, shapes, lsi, loc, attn, grad_output.contiguous(), grad_value, grad_dist,
            grad_sampling_loc, grad_attn_weight, im2col_step=ctx.im2col_step, dist_map=ctx.dist_map)
        return grad_value, grad_dist, None, None, grad_sampling_loc, grad_attn_weight, None, None, None


class MultiScaleDeformableAttnFunction(Function):
    """Plain 2-D multi-scale deformable attention with the call signature BEVFormer_DFA3D uses for its
    temporal self-attention and decoder (…/bevformer/modules/multi_scale_deformable_attn_function.py:
    MultiScaleDeformableAttnFunction_fp32.forward :97-131, backward :133-163; there the kernels come
    from the third-party mmcv extension).  Here it is the depth-weighted operator with all depth
    scores 1, on the same kernels."""

    @staticmethod
    def forward(ctx, value, value_spatial_shapes, value_level_start_index, sampling_locations,
                attention_weights, im2col_step):
        ctx.im2col_step = im2col_step
        output = ext_module.ms_deform_attn_forward(
            value, value_spatial_shapes, value_level_start_index, sampling_locations, attention_weights,
            im2col_step=ctx.im2col_step)
        ctx.save_for_backward(value, value_spatial_shapes, value_level_start_index, sampling_locations,
                              attention_weights)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, shapes, lsi, loc, attn = ctx.saved_tensors
        grad_value = torch.zeros(value.shape, dtype=torch.float32, device=value.device)
        grad_sampling_loc = torch.empty_like(loc)
        grad_attn_weight = torch.empty_like(attn)
        ext_module.ms_deform_attn_backward(
            value, shapes, lsi, loc, attn, grad_output.contiguous(), grad_value, grad_sampling_loc,
            grad_attn_weight, im2col_step=ctx.im2col_step)
        return grad_value, None, None, grad_sampling_loc, grad_attn_weight, None


class DeformableAttn3DFromOffsetsFunction(Function):
    """The one-stage operator fed with what the attention module's Linear layers produce: reference
    points, raw sampling offsets (pixels / depth bins) and raw attention logits.  The division by the
    level sizes, the addition of the reference points and the softmax over levels x points
    (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/spatial_cross_attention.py:503-538) run
    in the kernels' prologue, so neither the (B,Q,H,L,P,3) location tensor nor the attention weights
    nor their gradients are ever materialised.  No counterpart in the reference: it calls its Function
    with the assembled tensors.  The reference points receive no gradient."""

    @staticmethod
    def forward(ctx, value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                reference_points, sampling_offsets_uv, sampling_offsets_depth, attention_logits,
                dist_map=None):
        ctx.dist_map = dist_map
        output = ext_module.dfa3d_attn3d_forward(
            value, value_dpt_dist, value_spatial_shapes, value_level_start_index, reference_points,
            sampling_offsets_uv, sampling_offsets_depth, attention_logits, dist_map=dist_map)
        ctx.save_for_backward(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                              reference_points, sampling_offsets_uv, sampling_offsets_depth,
                              attention_logits)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, dist, shapes, lsi, ref, off_uv, off_d, logits = ctx.saved_tensors
        grad_value = torch.zeros(value.shape, dtype=torch.float32, device=value.device)
        grad_dist = torch.zeros(dist.shape, dtype=torch.float32, device=dist.device)
        grad_uv = torch.empty_like(off_uv)
        grad_d = torch.empty_like(off_d)
        grad_logits = torch.empty_like(logits)
        ext_module.dfa3d_attn3d_backward(value, dist, shapes, lsi, ref, off_uv, off_d, logits,
                                         grad_output.contiguous(), grad_value, grad_dist, grad_uv, grad_d,
                                         grad_logits, dist_map=ctx.dist_map)
        return grad_value, grad_dist, None, None, None, grad_uv, grad_d, grad_logits, None


class MultiScale3DDeformableAttnRaggedFunction(Function):
    """The one-stage operator for cameras with different numbers of queries: sampling_locations
    (R,H,L,P,3) and attention_weights (R,H,L,P) are packed rows, camera b owning rows
    [query_offsets[b], query_offsets[b+1]); max_queries bounds the rows of one camera.  Returns
    (output (R,H*C), depth_score (R,H,L,P,4) or None).  The reference pads every camera to the longest
    list instead (spatial_cross_attention.py:707-722) and calls the dense Function."""

    @staticmethod
    def forward(ctx, value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                sampling_locations, attention_weights, query_offsets, max_queries,
                return_depth_score=True, dist_map=None):
        ctx.max_queries = int(max_queries)
        ctx.dist_map = dist_map
        ctx.set_materialize_grads(False)
        output, depth_score = ext_module.dfa3d_fused_forward_ragged(
            value, value_dpt_dist, value_spatial_shapes, value_level_start_index, sampling_locations,
            attention_weights, query_offsets, ctx.max_queries, need_depth_score=return_depth_score,
            dist_map=dist_map)
        ctx.save_for_backward(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                              sampling_locations, attention_weights, query_offsets)
        return output, depth_score

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output, grad_depth_score_=None):
        if grad_depth_score_ is not None and grad_depth_score_.sum() != 0.0:
            raise NotImplementedError      # as the dense Function: depth_score carries no gradient
        value, dist, shapes, lsi, loc, attn, q_off = ctx.saved_tensors
        if grad_output is None:
            return (None,) * 10
        grad_value = torch.zeros(value.shape, dtype=torch.float32, device=value.device)
        grad_dist = torch.zeros(dist.shape, dtype=torch.float32, device=dist.device)
        grad_sampling_loc = torch.empty_like(loc)
        grad_attn_weight = torch.empty_like(attn)
        ext_module.dfa3d_fused_backward_ragged(
            value, dist, shapes, lsi, loc, attn, q_off, ctx.max_queries, grad_output.contiguous(),
            grad_value, grad_dist, grad_sampling_loc, grad_attn_weight, dist_map=ctx.dist_map)
        return (grad_value, grad_dist, None, None, grad_sampling_loc, grad_attn_weight, None, None, None,
                None)


class DeformableAttn3DFromOffsetsRaggedFunction(Function):
    """DeformableAttn3DFromOffsetsFunction on packed rows: reference_points (R,Z,3),
    sampling_offsets_uv (R,H,L,P,2), sampling_offsets_depth (R,H,L,P), attention_logits (R,H,L*P);
    camera b owns rows [query_offsets[b], query_offsets[b+1]).  Returns output (R,H*C)."""

    @staticmethod
    def forward(ctx, value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                reference_points, sampling_offsets_uv, sampling_offsets_depth, attention_logits,
                query_offsets, max_queries, dist_map=None):
        ctx.max_queries = int(max_queries)
        ctx.dist_map = dist_map
        output = ext_module.dfa3d_attn3d_forward_ragged(
            value, value_dpt_dist, value_spatial_shapes, value_level_start_index, reference_points,
            sampling_offsets_uv, sampling_offsets_depth, attention_logits, query_offsets, ctx.max_queries,
            dist_map=dist_map)
        ctx.save_for_backward(value, value_dpt_dist, value_spatial_shapes, value_level_start_index,
                              reference_points, sampling_offsets_uv, sampling_offsets_depth,
                              attention_logits, query_offsets)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, dist, shapes, lsi, ref, off_uv, off_d, logits, q_off = ctx.saved_tensors
        grad_value = torch.zeros(value.shape, dtype=torch.float32, device=value.device)
        grad_dist = torch.zeros(dist.shape, dtype=torch.float32, device=dist.device)
        grad_uv = torch.empty_like(off_uv)
        grad_d = torch.empty_like(off_d)
        grad_logits = torch.empty_like(logits)
        ext_module.dfa3d_attn3d_backward_ragged(value, dist, shapes, lsi, ref, off_uv, off_d, logits, q_off,
                                                ctx.max_queries, grad_output.contiguous(), grad_value,
                                                grad_dist, grad_uv, grad_d, grad_logits,
                                                dist_map=ctx.dist_map)
        return grad_value, grad_dist, None, None, None, grad_uv, grad_d, grad_logits, None, None, None


def _fp32_variant(cls, name):
    """Same Function with inputs cast to float32 when autocast is active."""
    fwd = torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float32)(cls.forward)
    bwd = torch.amp.custom_bwd(device_type="cuda")(cls.backward)
    return type(name, (Function,), {"forward": staticmethod(fwd), "backward": staticmethod(bwd)})


MultiScaleDepthScoreSampleFunction_fp32 = _fp32_variant(
    MultiScaleDepthScoreSampleFunction, "MultiScaleDepthScoreSampleFunction_fp32")
WeightedMultiScaleDeformableAttnFunction_fp32 = _fp32_variant(
    WeightedMultiScaleDeformableAttnFunction, "WeightedMultiScaleDeformableAttnFunction_fp32")
MultiScale3DDeformableAttnFunction_fp32 = _fp32_variant(
    MultiScale3DDeformableAttnFunction, "MultiScale3DDeformableAttnFunction_fp32")
MultiScaleDeformableAttnFunction_fp32 = _fp32_variant(
    MultiScaleDeformableAttnFunction, "MultiScaleDeformableAttnFunction_fp32")
DeformableAttn3DFromOffsetsFunction_fp32 = _fp32_variant(
    DeformableAttn3DFromOffsetsFunction, "DeformableAttn3DFromOffsetsFunction_fp32")
MultiScale3DDeformableAttnRaggedFunction_fp32 = _fp32_variant(
    MultiScale3DDeformableAttnRaggedFunction, "MultiScale3DDeformableAttnRaggedFunction_fp32")
DeformableAttn3DFromOffsetsRaggedFunction_fp32 = _fp32_variant(
    DeformableAttn3DFromOffsetsRaggedFunction, "DeformableAttn3DFromOffsetsRaggedFunction_fp32")


def _fp16_variant(cls, name, storage):
    """Half-precision variant of `cls`.  `storage` = positions of the tensors that stay half for the kernels
    (value, value_dpt_dist); every other half tensor is widened to float32 first, and when any argument was
    half the outputs are returned as half.  Gradients are computed in float32; autograd casts them to the
    dtype of the inputs they belong to."""

    def forward(ctx, *args):
        args = list(args)
        half = any(torch.is_tensor(a) and a.dtype == torch.float16 for a in args)
        for i, a in enumerate(args):
            if not torch.is_tensor(a) or not a.is_floating_point():
                continue
            if i in storage:
                args[i] = a.half() if half else a       # value and dist share one storage type
            elif a.dtype == torch.float16:
                args[i] = a.float()
        out = cls.forward(ctx, *args)
        if not half:
            return out
        if torch.is_tensor(out):
            return out.half()
        return tuple(o.half() if torch.is_tensor(o) else o for o in out)

    def backward(ctx, *grads):
        return cls.backward(ctx, *[g.float() if torch.is_tensor(g) and g.dtype == torch.float16 else g
                                   for g in grads])

    fwd = torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)(forward)
    bwd = torch.amp.custom_bwd(device_type="cuda")(backward)
    return type(name, (Function,), {"forward": staticmethod(fwd), "backward": staticmethod(bwd)})


MultiScaleDepthScoreSampleFunction_fp16 = _fp16_variant(
    MultiScaleDepthScoreSampleFunction, "MultiScaleDepthScoreSampleFunction_fp16", (0,))
WeightedMultiScaleDeformableAttnFunction_fp16 = _fp16_variant(
    WeightedMultiScaleDeformableAttnFunction, "WeightedMultiScaleDeformableAttnFunction_fp16", (0,))
MultiScale3DDeformableAttnFunction_fp16 = _fp16_variant(
    MultiScale3DDeformableAttnFunction, "MultiScale3DDeformableAttnFunction_fp16", (0, 1))
MultiScaleDeformableAttnFunction_fp16 = _fp16_variant(
    MultiScaleDeformableAttnFunction, "MultiScaleDeformableAttnFunction_fp16", (0,))
