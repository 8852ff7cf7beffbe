"""mmcv-free restatement of the callers of the DFA3D operator in BEVFormer-DFA3D.

  * ``MSDeformableAttention3D_DFA3D``  -- BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/
    spatial_cross_attention.py:409-587 (and its parent's parameters/initialisation, :182-277)
  * ``SpatialCrossAttention_DFA3D``    -- same file :616-751
  * ``SCAEncoderLayer`` / ``SCAEncoderStack`` -- the cross-attention -> norm -> FFN -> norm part of one
    BEVFormer encoder layer (…/modules/encoder.py:249-413 with the 'cross_attn', 'norm', 'ffn',
    'norm' operation order), used for the training-step configuration.

  * ``TemporalSelfAttention`` -- the BEV self-attention over the previous and the current BEV
    (…/modules/temporal_self_attention.py:26-272), the caller of the plain 2-D operator.
  * ``CustomMSDeformableAttention`` -- the detection decoder's cross-attention from object queries to
    the BEV (…/modules/decoder.py:133-345), the other caller of the 2-D operator.
  * ``point_sampling`` -- the projection of the pillar reference points into the cameras that yields
    ``reference_points_cam`` and ``bev_mask`` (…/modules/encoder.py:421-476).

Parameter names, shapes and initialisation follow the reference so that its checkpoints load; the
registry / config plumbing of mmcv is not reproduced.  Differences in how the operator is fed:
the depth distribution is passed as (B, N, D) shared by all heads instead of being repeated per head
(:497 in the reference); the per-camera re-batching keeps exactly the (camera, query) pairs that are
visible, as packed rows moved by kernels (``rebatch.RebatchPlan``), instead of Python loops over tensors
padded to the longest camera, and the operator is called once for all cameras with their row offsets.
The layers' norms are ``layer_ops.AddLayerNorm`` (torch LayerNorm parameters; the residual add happens
inside the norm kernel) and the projections ``layer_ops.Linear`` (bias gradient by a column-sum kernel).
"""
import math

import torch
import torch.nn as nn

from .functions import (MultiScaleDeformableAttnFunction_fp32,
                        DeformableAttn3DFromOffsetsFunction_fp32,
                        DeformableAttn3DFromOffsetsRaggedFunction_fp32,
                        MultiScale3DDeformableAttnFunction_fp32,
                        MultiScale3DDeformableAttnRaggedFunction_fp32)
from .layer_ops import AddLayerNorm, Linear
from .rebatch import (CombineCamerasFunction, GatherQueriesFunction, GatherSharedRowsFunction, RebatchPlan,
                      gather_per_camera)


def bev_reference_points(bev_h, bev_w, pillar_height=8, num_points_in_pillar=4, dim="3d", bs=1,
                         device="cuda", dtype=torch.float32):
    """Reference points of the BEV queries (encoder.py:61-99).  dim="3d": (bs, num_points_in_pillar,
    bev_h*bev_w, 3) = (x, y, z) in [0,1]^3, the pillar anchors that `point_sampling` projects into the
    cameras; dim="2d": (bs, bev_h*bev_w, 1, 2), the cell centres the temporal self-attention looks
    around."""
    if dim == "3d":
        Z, n = pillar_height, num_points_in_pillar
        zs = torch.linspace(0.5, Z - 0.5, n, dtype=dtype, device=device).view(-1, 1, 1).expand(n, bev_h, bev_w) / Z
        xs = torch.linspace(0.5, bev_w - 0.5, bev_w, dtype=dtype, device=device).view(1, 1, bev_w) \
            .expand(n, bev_h, bev_w) / bev_w
        ys = torch.linspace(0.5, bev_h - 0.5, bev_h, dtype=dtype, device=device).view(1, bev_h, 1) \
            .expand(n, bev_h, bev_w) / bev_h
        ref = torch.stack((xs, ys, zs), -1).permute(0, 3, 1, 2).flatten(2).permute(0, 2, 1)
        return ref[None].repeat(bs, 1, 1, 1)
    if dim == "2d":
        ref_y, ref_x = torch.meshgrid(torch.linspace(0.5, bev_h - 0.5, bev_h, dtype=dtype, device=device),
                                      torch.linspace(0.5, bev_w - 0.5, bev_w, dtype=dtype, device=device),
                                      indexing="ij")
        ref = torch.stack((ref_x.reshape(-1)[None] / bev_w, ref_y.reshape(-1)[None] / bev_h), -1)
        return ref.repeat(bs, 1, 1).unsqueeze(2)
    raise ValueError("dim must be '3d' or '2d'")


def point_sampling(reference_points, pc_range, lidar2img, img_shape, d_bound):
    """Project the pillar reference points into every camera (encoder.py:421-476).

    reference_points (bs, Z, Q, 3) in [0,1]^3 of the BEV volume; pc_range = (x0, y0, z0, x1, y1, z1);
    lidar2img (bs, cams, 4, 4); img_shape = (height, width) of the padded images; d_bound = (near, far,
    step) of the depth bins.  Returns reference_points_cam (cams, bs, Q, Z, 3) = (x / width, y / height,
    (depth - near) / (far - near)) and bev_mask (cams, bs, Q, Z): in front of the camera and inside the
    image."""
    ref = reference_points.clone().float()
    ref[..., 0:1] = ref[..., 0:1] * (pc_range[3] - pc_range[0]) + pc_range[0]
    ref[..., 1:2] = ref[..., 1:2] * (pc_range[4] - pc_range[1]) + pc_range[1]
    ref[..., 2:3] = ref[..., 2:3] * (pc_range[5] - pc_range[2]) + pc_range[2]
    ref = torch.cat((ref, torch.ones_like(ref[..., :1])), -1).permute(1, 0, 2, 3)      # (Z, bs, Q, 4)
    Z, bs, Q = ref.shape[:3]
    cams = lidar2img.size(1)
    ref = ref.view(Z, bs, 1, Q, 4, 1)
    mat = lidar2img.float().view(1, bs, cams, 1, 4, 4)
    cam = torch.matmul(mat, ref).squeeze(-1)                                           # (Z, bs, cams, Q, 4)
    eps = 1e-5
    mask = cam[..., 2:3] > eps
    xy = cam[..., 0:2] / torch.maximum(cam[..., 2:3], torch.ones_like(cam[..., 2:3]) * eps)
    x = xy[..., 0] / img_shape[1]
    y = xy[..., 1] / img_shape[0]
    z = (cam[..., 2] - d_bound[0]) / (d_bound[1] - d_bound[0])
    out = torch.stack((x, y, z), -1)
    mask = (mask & (out[..., 1:2] > 0.0) & (out[..., 1:2] < 1.0) & (out[..., 0:1] < 1.0)
            & (out[..., 0:1] > 0.0))
    mask = torch.nan_to_num(mask)
    return out.permute(2, 1, 3, 0, 4).contiguous(), mask.permute(2, 1, 3, 0, 4).squeeze(-1).contiguous()


def assemble_sampling_locations(reference_points, offsets_uv, offsets_depth, spatial_shapes, depth_bins):
    """Sampling locations from reference points and predicted offsets
    (spatial_cross_attention.py:498-538).

    reference_points (bs, Q, Z, 3) in [0,1] (x, y, depth); offsets_uv (bs, Q, H, L, P_all, 2) and
    offsets_depth (bs, Q, H, L, P_all, 1) in pixels / bins; spatial_shapes (L, 2) = (h, w).
    P_all = P * Z: the P_all sampling points of a level are split over the Z anchors of the pillar.
    Returns (bs, Q, H, L, P_all, 3)."""
    bs, Q, Z, three = reference_points.shape
    assert three == 3
    _, _, H, L, P_all, _ = offsets_uv.shape
    assert P_all % Z == 0
    normalizer = torch.stack([spatial_shapes[:, 1], spatial_shapes[:, 0],
                              torch.full_like(spatial_shapes[:, 0], depth_bins)], -1).to(offsets_uv.dtype)
    offsets = torch.cat([offsets_uv, offsets_depth], -1) / normalizer[None, None, None, :, None, :]
    offsets = offsets.view(bs, Q, H, L, P_all // Z, Z, 3)
    loc = reference_points[:, :, None, None, None, :, :] + offsets
    return loc.view(bs, Q, H, L, P_all, 3)


class MSDeformableAttention3D_DFA3D(nn.Module):
    """3-D deformable attention over multi-level camera features and their depth distributions."""

    def __init__(self, embed_dims=256, num_heads=8, num_levels=4, num_points=8, im2col_step=64,
                 batch_first=True, compute_weight_update=True, fuse_input_ops=True):
        super().__init__()
        # fuse_input_ops: let the kernels form the sampling locations and the softmax from the Linear
        # outputs (used whenever weight_update is not needed; numerically the same operations)
        self.fuse_input_ops = fuse_input_ops
        # weight_update (:579) needs the (B,Q,H,L,P,4) depth_score tensor written out; callers that do
        # not use it (SpatialCrossAttention_DFA3D with use_empty=False) can switch it off
        self.compute_weight_update = compute_weight_update
        if embed_dims % num_heads != 0:
            raise ValueError(f"embed_dims must be divisible by num_heads, but got {embed_dims} and "
                             f"{num_heads}")
        self.embed_dims, self.num_heads = embed_dims, num_heads
        self.num_levels, self.num_points = num_levels, num_points
        self.im2col_step, self.batch_first = im2col_step, batch_first
        self.sampling_offsets = Linear(embed_dims, num_heads * num_levels * num_points * 2)
        self.sampling_offsets_depth = Linear(embed_dims, num_heads * num_levels * num_points)
        self.attention_weights = Linear(embed_dims, num_heads * num_levels * num_points)
        self.value_proj = Linear(embed_dims, embed_dims)
        self.init_weights()

    def init_weights(self):
        """spatial_cross_attention.py:256-276 (u,v offsets, attention, value_proj) and :414-426 (depth
        offsets)."""
        H, L, P = self.num_heads, self.num_levels, self.num_points
        nn.init.zeros_(self.sampling_offsets.weight)
        thetas = torch.arange(H, dtype=torch.float32) * (2.0 * math.pi / H)
        grid = torch.stack([thetas.cos(), thetas.sin()], -1)
        grid = (grid / grid.abs().max(-1, keepdim=True)[0]).view(H, 1, 1, 2).repeat(1, L, P, 1)
        scale = torch.arange(1, P + 1, dtype=torch.float32).view(1, 1, P, 1)
        with torch.no_grad():
            self.sampling_offsets.bias.copy_((grid * scale).view(-1))
            nn.init.zeros_(self.sampling_offsets_depth.weight)
            gd = ((thetas.cos() + thetas.sin()) / 2).view(H, 1, 1, 1).repeat(1, L, P, 1)
            self.sampling_offsets_depth.bias.copy_((gd * scale).view(-1))
            nn.init.zeros_(self.attention_weights.weight)
            nn.init.zeros_(self.attention_weights.bias)
            nn.init.xavier_uniform_(self.value_proj.weight)
            nn.init.zeros_(self.value_proj.bias)

    def forward(self, query, value, value_dpt_dist, reference_points, spatial_shapes, level_start_index,
                query_pos=None, key_padding_mask=None, query_offsets=None, max_queries=None,
                dist_map=None):
        """query (bs, Q, E); value (bs, N, E); value_dpt_dist (bs, N, D); reference_points
        (bs, Q, Z, 3); spatial_shapes (L, 2) int64; level_start_index (L) int64.
        Returns (output (bs, Q, E), weight_update (bs, Q, H, 1))  -- :428-583.

        Packed rows (cameras with different numbers of queries): pass ``query_offsets`` (bs+1 int32,
        CUDA; element b of value owns the rows [query_offsets[b], query_offsets[b+1])) and
        ``max_queries``; then query is (R, E), reference_points (R, Z, 3), and the results are
        (R, E) and (R, H, 1).  value / value_dpt_dist are batch-first in this mode.

        ``dist_map=(h, w)``: value_dpt_dist is one h x w map per camera, (bs, h*w, D), that every level
        reads with nearest-neighbour indexing (instead of one resized copy per level)."""
        ragged = query_offsets is not None
        if query_pos is not None:
            query = query + query_pos
        if not self.batch_first and not ragged:
            query, value = query.permute(1, 0, 2), value.permute(1, 0, 2)
        lead = query.shape[:-1]                              # (bs, Q) or (R,)
        bs, N, _ = value.shape
        H, L, P = self.num_heads, self.num_levels, self.num_points
        D = value_dpt_dist.shape[-1]
        value = self.value_proj(value)
        if key_padding_mask is not None:
            value = value.masked_fill(key_padding_mask[..., None], 0.0)
        value = value.view(bs, N, H, -1)
        if reference_points.shape[-1] != 3:
            raise ValueError("Last dim of reference_points must be 3 (x, y, depth), but got "
                             f"{reference_points.shape[-1]} instead.")
        shapes3 = torch.cat([spatial_shapes, torch.full_like(spatial_shapes[:, :1], D)], -1).contiguous()
        off_uv = self.sampling_offsets(query).view(*lead, H, L, P, 2)
        off_d = self.sampling_offsets_depth(query).view(*lead, H, L, P, 1)
        logits = self.attention_weights(query).view(*lead, H, L * P)
        if self.fuse_input_ops and not self.compute_weight_update:
            if ragged:
                output = DeformableAttn3DFromOffsetsRaggedFunction_fp32.apply(
                    value.contiguous(), value_dpt_dist.contiguous(), shapes3, level_start_index,
                    reference_points.contiguous(), off_uv, off_d, logits, query_offsets, max_queries,
                    dist_map)
                return output, None
            output = DeformableAttn3DFromOffsetsFunction_fp32.apply(
                value.contiguous(), value_dpt_dist.contiguous(), shapes3, level_start_index,
                reference_points.contiguous(), off_uv, off_d, logits, dist_map)
            return (output if self.batch_first else output.permute(1, 0, 2)), None
        attn = logits.softmax(-1).view(*lead, H, L, P)
        if ragged:
            loc = assemble_sampling_locations(reference_points[None], off_uv[None], off_d[None],
                                              spatial_shapes, D)[0]
            output, depth_score = MultiScale3DDeformableAttnRaggedFunction_fp32.apply(
                value.contiguous(), value_dpt_dist.contiguous(), shapes3, level_start_index,
                loc.contiguous(), attn.contiguous(), query_offsets, max_queries, self.compute_weight_update,
                dist_map)
        else:
            loc = assemble_sampling_locations(reference_points, off_uv, off_d, spatial_shapes, D)
            output, depth_score = MultiScale3DDeformableAttnFunction_fp32.apply(
                value.contiguous(), value_dpt_dist.contiguous(), shapes3, level_start_index,
                loc.contiguous(), attn.contiguous(), self.im2col_step, self.compute_weight_update, dist_map)
        weight_update = None
        if self.compute_weight_update:
            # mean depth score of a point's four corners, weighted by the attention (:579)
            weight_update = (depth_score.mean(-1) * attn).flatten(-2).sum(-1, keepdim=True)
        if not self.batch_first and not ragged:
            output = output.permute(1, 0, 2)
        return output, weight_update


class SpatialCrossAttention_DFA3D(nn.Module):
    """BEV queries attend to the cameras that see them (spatial_cross_attention.py:616-751)."""

    def __init__(self, embed_dims=256, num_cams=6, dropout=0.1, deformable_attention=None,
                 bev_h=200, bev_w=200, num_head=8, use_empty=False):
        super().__init__()
        self.embed_dims, self.num_cams = embed_dims, num_cams
        self.bev_h, self.bev_w, self.num_head, self.use_empty = bev_h, bev_w, num_head, use_empty
        self.deformable_attention = deformable_attention or MSDeformableAttention3D_DFA3D(embed_dims)
        if not use_empty:
            self.deformable_attention.compute_weight_update = False
        self.output_proj = Linear(embed_dims, embed_dims)
        self.dropout = nn.Dropout(dropout)
        if use_empty:
            self.empty_query = nn.Embedding(bev_h * bev_w * num_head, embed_dims)
        nn.init.xavier_uniform_(self.output_proj.weight)
        nn.init.zeros_(self.output_proj.bias)

    def forward(self, query, key=None, value=None, value_dpt_dist=None, reference_points_cam=None,
                bev_mask=None, spatial_shapes=None, level_start_index=None, residual=None,
                query_pos=None, rebatch_plan=None, dist_map=None, return_residual=False):
        """query (bs, Q, E); value (num_cams, N, bs, E) (`key` is accepted and, as in the reference,
        not used by the attention); value_dpt_dist (num_cams, N, bs, D);
        reference_points_cam (num_cams, bs, Q, Z, 3); bev_mask (num_cams, bs, Q, Z).
        ``rebatch_plan``: a ``RebatchPlan`` of this bev_mask built earlier (bev_mask is geometry: one
        plan serves every layer of a frame); without it the plan is built here, which reads the packed
        row count back from the device once.  ``dist_map=(h, w)``: value_dpt_dist is one h x w map per
        camera, (num_cams, h*w, bs, D), read by all levels with nearest indexing.  Returns (bs, Q, E);
        with ``return_residual`` the two summands (attention branch, residual) separately, for a norm that
        adds them itself."""
        inp_residual = query if residual is None else residual
        if query_pos is not None:
            query = query + query_pos
        bs, Q, E = query.shape
        cams = self.num_cams
        plan = rebatch_plan if rebatch_plan is not None else RebatchPlan(bev_mask)
        if (plan.cams, plan.bs, plan.Q) != (cams, bs, Q):
            raise RuntimeError("rebatch_plan does not belong to this bev_mask / query")
        q_rows = GatherQueriesFunction.apply(query.float(), plan)                 # (bs*T, E)
        ref_rows = gather_per_camera(reference_points_cam.float(), plan)          # (bs*T, Z, 3)
        N = value.shape[1]
        value = value.permute(2, 0, 1, 3).reshape(bs * cams, N, E)                # element j*cams + i
        dist = value_dpt_dist.permute(2, 0, 1, 3).reshape(bs * cams, N, -1)
        out_rows, update_weight = self.deformable_attention(
            query=q_rows, value=value, value_dpt_dist=dist, reference_points=ref_rows,
            spatial_shapes=spatial_shapes, level_start_index=level_start_index,
            query_offsets=plan.op_offsets, max_queries=plan.max_queries, dist_map=dist_map)
        if self.use_empty:
            # :721-722, :739-740 -- rows whose depth-weighted attention found little get the learned
            # per-(BEV cell, head) empty embedding instead
            empty = GatherSharedRowsFunction.apply(
                self.empty_query.weight.view(self.bev_h * self.bev_w, self.num_head * E), plan)
            out_rows = out_rows + ((1 - update_weight) * empty.view(-1, self.num_head, E)).mean(-2)
        slots = CombineCamerasFunction.apply(out_rows, plan)                      # sum over cameras / count
        slots = self.dropout(self.output_proj(slots))
        return (slots, inp_residual) if return_residual else slots + inp_residual


class TemporalSelfAttention(nn.Module):
    """BEV queries attend to the previous and the current BEV with 2-D multi-scale deformable attention
    (temporal_self_attention.py:26-272; parameters and initialisation :103-127).  The operator is the
    plain 2-D one, here on the depth-weighted kernels with all depth scores 1
    (``MultiScaleDeformableAttnFunction_fp32``); the reference takes it from the mmcv extension."""

    def __init__(self, embed_dims=256, num_heads=8, num_levels=4, num_points=4, num_bev_queue=2,
                 im2col_step=64, dropout=0.1, batch_first=True):
        super().__init__()
        if embed_dims % num_heads != 0:
            raise ValueError(f"embed_dims must be divisible by num_heads, but got {embed_dims} and "
                             f"{num_heads}")
        self.embed_dims, self.num_heads = embed_dims, num_heads
        self.num_levels, self.num_points, self.num_bev_queue = num_levels, num_points, num_bev_queue
        self.im2col_step, self.batch_first = im2col_step, batch_first
        self.dropout = nn.Dropout(dropout)
        self.sampling_offsets = Linear(embed_dims * num_bev_queue,
                                          num_bev_queue * num_heads * num_levels * num_points * 2)
        self.attention_weights = Linear(embed_dims * num_bev_queue,
                                           num_bev_queue * num_heads * num_levels * num_points)
        self.value_proj = Linear(embed_dims, embed_dims)
        self.output_proj = Linear(embed_dims, embed_dims)
        self.init_weights()

    def init_weights(self):
        H, LQ, P = self.num_heads, self.num_levels * self.num_bev_queue, self.num_points
        nn.init.zeros_(self.sampling_offsets.weight)
        thetas = torch.arange(H, dtype=torch.float32) * (2.0 * math.pi / H)
        grid = torch.stack([thetas.cos(), thetas.sin()], -1)
        grid = (grid / grid.abs().max(-1, keepdim=True)[0]).view(H, 1, 1, 2).repeat(1, LQ, P, 1)
        grid = grid * torch.arange(1, P + 1, dtype=torch.float32).view(1, 1, P, 1)
        with torch.no_grad():
            self.sampling_offsets.bias.copy_(grid.view(-1))
            nn.init.zeros_(self.attention_weights.weight)
            nn.init.zeros_(self.attention_weights.bias)
            nn.init.xavier_uniform_(self.value_proj.weight)
            nn.init.zeros_(self.value_proj.bias)
            nn.init.xavier_uniform_(self.output_proj.weight)
            nn.init.zeros_(self.output_proj.bias)

    def forward(self, query, key=None, value=None, identity=None, query_pos=None, key_padding_mask=None,
                reference_points=None, spatial_shapes=None, level_start_index=None, return_residual=False):
        """query (bs, Q, E); value (bs*num_bev_queue, Q, E) = [previous BEV, current BEV] per batch
        element, or None (then the current queries stand for both, :180-184); reference_points
        (bs*num_bev_queue, Q, num_levels, 2); spatial_shapes (L, 2); level_start_index (L).
        Returns (bs, Q, E)  -- :130-272; with ``return_residual`` the attention branch and the identity
        separately."""
        if self.num_bev_queue != 2:
            raise ValueError("the BEV queue holds the previous and the current BEV: num_bev_queue == 2")
        if value is None:
            if not self.batch_first:
                raise ValueError("value=None needs batch_first=True")
            bs, len_bev, c = query.shape
            value = torch.stack([query, query], 1).reshape(bs * 2, len_bev, c)
        if identity is None:
            identity = query
        if query_pos is not None:
            query = query + query_pos
        if not self.batch_first:
            query, value = query.permute(1, 0, 2), value.permute(1, 0, 2)
        bs, Q, E = query.shape
        N = value.shape[1]
        H, L, P, NQ = self.num_heads, self.num_levels, self.num_points, self.num_bev_queue
        query = torch.cat([value[:bs], query], -1)                        # :197
        value = self.value_proj(value)
        if key_padding_mask is not None:
            value = value.masked_fill(key_padding_mask[..., None], 0.0)
        value = value.reshape(bs * NQ, N, H, -1)
        offsets = self.sampling_offsets(query).view(bs, Q, H, NQ, L, P, 2)
        attn = self.attention_weights(query).view(bs, Q, H, NQ, L * P).softmax(-1).view(bs, Q, H, NQ, L, P)
        attn = attn.permute(0, 3, 1, 2, 4, 5).reshape(bs * NQ, Q, H, L, P).contiguous()
        offsets = offsets.permute(0, 3, 1, 2, 4, 5, 6).reshape(bs * NQ, Q, H, L, P, 2)
        if reference_points.shape[-1] == 2:
            normalizer = torch.stack([spatial_shapes[..., 1], spatial_shapes[..., 0]], -1).to(offsets.dtype)
            loc = reference_points[:, :, None, :, None, :] + offsets / normalizer[None, None, None, :, None, :]
        elif reference_points.shape[-1] == 4:
            loc = reference_points[:, :, None, :, None, :2] \
                + offsets / P * reference_points[:, :, None, :, None, 2:] * 0.5
        else:
            raise ValueError("Last dim of reference_points must be 2 or 4, but get "
                             f"{reference_points.shape[-1]} instead.")
        out = MultiScaleDeformableAttnFunction_fp32.apply(value.contiguous(), spatial_shapes, level_start_index,
                                                          loc.contiguous(), attn, self.im2col_step)
        # mean over the previous and the current BEV (:257-262); batch element j owns rows j*NQ .. j*NQ+NQ-1
        out = out.view(bs, NQ, Q, E).mean(1)
        out = self.output_proj(out)
        if not self.batch_first:
            out = out.permute(1, 0, 2)
        out = self.dropout(out)
        return (out, identity) if return_residual else out + identity


class SCAEncoderLayer(nn.Module):
    """cross-attention -> LayerNorm -> FFN -> LayerNorm (encoder.py:389-411 operation order without the
    temporal self-attention, which uses a different, 2-D operator)."""

    def __init__(self, embed_dims=256, ffn_dims=512, num_cams=6, num_heads=8, num_levels=4, num_points=8,
                 dropout=0.1):
        super().__init__()
        self.cross_attn = SpatialCrossAttention_DFA3D(
            embed_dims, num_cams, dropout,
            MSDeformableAttention3D_DFA3D(embed_dims, num_heads, num_levels, num_points))
        self.norm1 = AddLayerNorm(embed_dims)
        self.ffn = nn.Sequential(Linear(embed_dims, ffn_dims), nn.ReLU(inplace=True), nn.Dropout(dropout),
                                 Linear(ffn_dims, embed_dims), nn.Dropout(dropout))
        self.norm2 = AddLayerNorm(embed_dims)

    def forward(self, query, **kw):
        query = self.norm1(*self.cross_attn(query, return_residual=True, **kw))     # norm(branch + residual)
        return self.norm2(self.ffn(query), query)


class CustomMSDeformableAttention(nn.Module):
    """Object queries attend to the BEV features with 2-D multi-scale deformable attention
    (decoder.py:133-345; parameters and initialisation :200-227).  batch_first=False by default, like
    the reference: query (Q, bs, E), value (N, bs, E)."""

    def __init__(self, embed_dims=256, num_heads=8, num_levels=4, num_points=4, im2col_step=64, dropout=0.1,
                 batch_first=False):
        super().__init__()
        if embed_dims % num_heads != 0:
            raise ValueError(f"embed_dims must be divisible by num_heads, but got {embed_dims} and "
                             f"{num_heads}")
        self.embed_dims, self.num_heads = embed_dims, num_heads
        self.num_levels, self.num_points = num_levels, num_points
        self.im2col_step, self.batch_first = im2col_step, batch_first
        self.dropout = nn.Dropout(dropout)
        self.sampling_offsets = Linear(embed_dims, num_heads * num_levels * num_points * 2)
        self.attention_weights = Linear(embed_dims, num_heads * num_levels * num_points)
        self.value_proj = Linear(embed_dims, embed_dims)
        self.output_proj = Linear(embed_dims, embed_dims)
        self.init_weights()

    def init_weights(self):
        H, L, P = self.num_heads, self.num_levels, self.num_points
        nn.init.zeros_(self.sampling_offsets.weight)
        thetas = torch.arange(H, dtype=torch.float32) * (2.0 * math.pi / H)
        grid = torch.stack([thetas.cos(), thetas.sin()], -1)
        grid = (grid / grid.abs().max(-1, keepdim=True)[0]).view(H, 1, 1, 2).repeat(1, L, P, 1)
        grid = grid * torch.arange(1, P + 1, dtype=torch.float32).view(1, 1, P, 1)
        with torch.no_grad():
            self.sampling_offsets.bias.copy_(grid.view(-1))
            nn.init.zeros_(self.attention_weights.weight)
            nn.init.zeros_(self.attention_weights.bias)
            nn.init.xavier_uniform_(self.value_proj.weight)
            nn.init.zeros_(self.value_proj.bias)
            nn.init.xavier_uniform_(self.output_proj.weight)
            nn.init.zeros_(self.output_proj.bias)

    def forward(self, query, key=None, value=None, identity=None, query_pos=None, key_padding_mask=None,
                reference_points=None, spatial_shapes=None, level_start_index=None):
        """reference_points (bs, Q, L, 2) normalised positions, or (bs, Q, L, 4) boxes (cx, cy, w, h).
        Returns dropout(output_proj(attention)) + identity, in the layout of `query`  -- :231-345."""
        if value is None:
            value = query
        if identity is None:
            identity = query
        if query_pos is not None:
            query = query + query_pos
        if not self.batch_first:
            query, value = query.permute(1, 0, 2), value.permute(1, 0, 2)
        bs, Q, _ = query.shape
        N = value.shape[1]
        H, L, P = self.num_heads, self.num_levels, self.num_points
        value = self.value_proj(value)
        if key_padding_mask is not None:
            value = value.masked_fill(key_padding_mask[..., None], 0.0)
        value = value.view(bs, N, H, -1)
        offsets = self.sampling_offsets(query).view(bs, Q, H, L, P, 2)
        attn = self.attention_weights(query).view(bs, Q, H, L * P).softmax(-1).view(bs, Q, H, L, P)
        if reference_points.shape[-1] == 2:
            normalizer = torch.stack([spatial_shapes[..., 1], spatial_shapes[..., 0]], -1).to(offsets.dtype)
            loc = reference_points[:, :, None, :, None, :] + offsets / normalizer[None, None, None, :, None, :]
        elif reference_points.shape[-1] == 4:
            loc = reference_points[:, :, None, :, None, :2] \
                + offsets / P * reference_points[:, :, None, :, None, 2:] * 0.5
        else:
            raise ValueError("Last dim of reference_points must be 2 or 4, but get "
                             f"{reference_points.shape[-1]} instead.")
        out = MultiScaleDeformableAttnFunction_fp32.apply(value.contiguous(), spatial_shapes, level_start_index,
                                                          loc.contiguous(), attn.contiguous(), self.im2col_step)
        out = self.output_proj(out)
        if not self.batch_first:
            out = out.permute(1, 0, 2)
        return self.dropout(out) + identity


class BEVFormerEncoderLayer(nn.Module):
    """One full BEVFormer-DFA3D encoder layer: temporal self-attention -> norm -> spatial
    cross-attention -> norm -> FFN -> norm (operation order of bevformer_base_DFA3D.py:123-124 as executed
    by encoder.py:363-411; post-norm, so every block adds its own input as the residual)."""

    def __init__(self, embed_dims=256, ffn_dims=512, num_cams=6, num_heads=8, num_levels=4, num_points=8,
                 bev_h=200, bev_w=200, dropout=0.1):
        super().__init__()
        self.bev_h, self.bev_w = bev_h, bev_w
        self.self_attn = TemporalSelfAttention(embed_dims, num_heads, num_levels=1, num_points=4,
                                               dropout=dropout)
        self.norm0 = AddLayerNorm(embed_dims)
        self.cross_attn = SpatialCrossAttention_DFA3D(
            embed_dims, num_cams, dropout,
            MSDeformableAttention3D_DFA3D(embed_dims, num_heads, num_levels, num_points), bev_h=bev_h,
            bev_w=bev_w, num_head=num_heads)
        self.norm1 = AddLayerNorm(embed_dims)
        self.ffn = nn.Sequential(Linear(embed_dims, ffn_dims), nn.ReLU(inplace=True), nn.Dropout(dropout),
                                 Linear(ffn_dims, embed_dims), nn.Dropout(dropout))
        self.norm2 = AddLayerNorm(embed_dims)

    def forward(self, query, prev_bev=None, bev_pos=None, ref_2d=None, **cross_kw):
        """query (bs, bev_h*bev_w, E); prev_bev: None or (bs*2, Q, E) = [previous, current] BEV per batch
        element (encoder.py:519-528 stacks them); ref_2d (bs*2, Q, 1, 2) (`bev_reference_points(dim="2d")`,
        shifted for the previous BEV by the caller); cross_kw: the spatial cross-attention's inputs."""
        dev = query.device
        if ref_2d is None:
            ref_2d = bev_reference_points(self.bev_h, self.bev_w, dim="2d", bs=query.shape[0] * 2, device=dev,
                                          dtype=query.dtype)
        shapes = torch.tensor([[self.bev_h, self.bev_w]], dtype=torch.int64, device=dev)
        lsi = torch.zeros(1, dtype=torch.int64, device=dev)
        query = self.norm0(*self.self_attn(query, value=prev_bev, query_pos=bev_pos, reference_points=ref_2d,
                                           spatial_shapes=shapes, level_start_index=lsi, return_residual=True))
        query = self.norm1(*self.cross_attn(query, return_residual=True, **cross_kw))
        return self.norm2(self.ffn(query), query)


class SCAEncoderStack(nn.Module):
    def __init__(self, num_layers=6, **layer_kw):
        super().__init__()
        self.layers = nn.ModuleList(SCAEncoderLayer(**layer_kw) for _ in range(num_layers))

    def forward(self, query, **kw):
        if kw.get("rebatch_plan") is None:          # bev_mask is the same for every layer: one plan
            kw = dict(kw, rebatch_plan=RebatchPlan(kw["bev_mask"]))
        for layer in self.layers:
            query = layer(query, **kw)
        return query
