/* dfa3d_b200 -- C ABI of the B200 (sm_100a) DFA3D operator library (libdfa3d_b200.so).
 *
 * The library replaces the device side of the reference's `dfa3D._ext` extension module.  Every entry
 * point takes raw DEVICE pointers, a problem descriptor of plain integers and a CUDA stream; it
 * allocates nothing, keeps no pointer after returning, launches asynchronously on `stream` and returns
 * DFA3D_OK or a negative error code (never aborts, never traps the GPU).  `dfa3d_last_error()` gives
 * the message of the calling thread's last failure.
 *
 * Tensor layouts are the reference's (all contiguous, row-major):
 *   value        (B, N, H, C)           fp32, bf16 or fp16  N = sum over levels of h_l * w_l
 *   dist         (B, N, H, D) or (B, N, D) shared by all heads   fp32, bf16 or fp16, per-pixel depth distribution
 *   loc3 / loc2  (B, Q, H, L, P, 3|2)   fp32   (x, y[, z]) in units of the level's width/height/depth
 *   attn         (B, Q, H, L, P)        fp32
 *   depth_score  (B, Q, H, L, P, 4)     fp32   corner order 0=(y0,x0) 1=(y0,x1) 2=(y1,x1) 3=(y1,x0)
 *   out          (B, Q, H*C)            fp32
 *   spatial_shapes (L, 3|2) int64 = (h, w[, d]) and level_start_index (L) int64, both in DEVICE
 *   memory: the kernels read them there, as the reference's kernels do
 *   (DFA3D/dfa3D/ops/csrc/common/cuda/wms_deform_attn_cuda_kernel.cuh:273-276).
 * Gradients are fp32 whatever the storage type of value/dist.
 */
#ifndef DFA3D_B200_H_
#define DFA3D_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DFA3D_ABI_VERSION 2

#define DFA3D_OK 0
#define DFA3D_ERR_INVALID_ARGUMENT (-1) /* null pointer, non-positive size, bad enum, misaligned pointer */
#define DFA3D_ERR_UNSUPPORTED (-2)      /* shape outside what the kernels cover (see DFA3D_MAX_*) */
#define DFA3D_ERR_CUDA (-3)             /* a CUDA runtime call or the launch failed */

#define DFA3D_DTYPE_F32 0
#define DFA3D_DTYPE_BF16 1
#define DFA3D_DTYPE_F64 2 /* the *_f64 entry points only: every floating-point tensor is double */
#define DFA3D_DTYPE_F16 3 /* IEEE half storage of value and dist together (what the reference's *_fp16
                             Functions pass); arithmetic, the other tensors and all gradients stay fp32 */

#define DFA3D_ACT_SOFTMAX 0 /* dfa3d_dist_from_logits: softmax over the D channels */
#define DFA3D_ACT_SIGMOID 1 /* element-wise sigmoid */

#define DFA3D_MAX_LEVELS 32   /* L */
#define DFA3D_MAX_CHANNELS 1024 /* C; reference kernels for C > 1024 are themselves broken
                                   (wms_deform_attn_cuda_kernel.cuh:968-971 pass un-offset pointers) */

/* Problem descriptor shared by all entry points (plain integers, fixed widths, no padding). */
typedef struct dfa3d_problem {
  int32_t B;  /* batch * cameras */
  int32_t N;  /* pixels over all levels */
  int32_t H;  /* heads */
  int32_t C;  /* channels per head, any value up to DFA3D_MAX_CHANNELS.  Vectorised kernels: fp32 value
                 C in {8,16,32,64,128}; bf16 / fp16 value C in {16,32,64,128,256} forward and
                 {8,16,32,64,128} backward.  Every other width runs a lane-strided kernel with the same
                 results, several times slower. */
  int32_t D;  /* depth bins = channel count of dist */
  int32_t L;  /* levels */
  int32_t Q;  /* queries */
  int32_t P;  /* sampling points per level */
  int32_t value_dtype;       /* DFA3D_DTYPE_* of `value` */
  int32_t dist_dtype;        /* DFA3D_DTYPE_* of `dist`  */
  int64_t dist_head_stride;  /* elements between heads of one pixel in `dist`: D for (B,N,H,D);
                                0 for (B,N,D) shared by all heads (then grad_dist is (B,N,D) too,
                                already summed over heads) */
  int32_t dist_map_h;        /* 0, 0: `dist` has one row per pixel of `value` (N rows per camera).  */
  int32_t dist_map_w;        /* h, w > 0: `dist` is ONE map of h x w pixels per camera (h*w rows) that
                                every level samples with nearest-neighbour indexing -- the depth
                                network predicts at one resolution and the reference resizes that map
                                to every feature level with F.interpolate(mode="nearest")
                                (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/dense_heads/
                                depth_head.py:273-276); pixel (y, x) of a level of size (H_l, W_l) reads
                                map pixel (min(floor(y * (float)h / H_l), h-1), min(floor(x * (float)w /
                                W_l), w-1)), which is that resize.  grad_dist then has the map's layout
                                and holds the sum over all level pixels that read a map pixel. */
} dfa3d_problem;

/* ABI version of the loaded library (== DFA3D_ABI_VERSION of the header it was built from). */
int dfa3d_abi_version(void);

/* Message of the last error raised on the calling thread ("" if none). */
const char *dfa3d_last_error(void);

/* Depth-score sampling, forward.  Replaces ms_depth_score_sample_forward
 * (DFA3D/dfa3D/ops/csrc/pybind.cpp:55-59 -> cuda/ms_depth_score_sample_cuda.cu:49-111 ->
 * common/cuda/ms_depth_score_sample_cuda_kernel.cuh:94-148).
 * Writes every element of depth_score (no pre-zeroing needed).  shapes3 is (L,3). */
int dfa3d_depth_score_forward(const dfa3d_problem *p, const void *dist, const int64_t *shapes3,
                              const int64_t *level_start, const float *loc3, float *depth_score,
                              void *stream);

/* Depth-score sampling, backward.  Replaces ms_depth_score_sample_backward
 * (pybind.cpp:60-66 -> ms_depth_score_sample_cuda.cu:137-202 -> kernel.cuh:242-327).
 * grad_dist is ACCUMULATED into with atomics (caller zeroes it, as the reference's Function does);
 * grad_loc3 (B,Q,H,L,P,3) is overwritten: (0, 0, dL/dz). */
int dfa3d_depth_score_backward(const dfa3d_problem *p, const void *dist, const int64_t *shapes3,
                               const int64_t *level_start, const float *loc3,
                               const float *grad_depth_score, float *grad_dist, float *grad_loc3,
                               void *stream);

/* Depth-weighted multi-scale deformable attention, forward, depth_score given.  Replaces
 * wms_deform_attn_forward (pybind.cpp:43-47 -> cuda/wms_deform_attn_cuda.cu:213-288 ->
 * common/cuda/wms_deform_attn_cuda_kernel.cuh:240-303).  shapes2 is (L,2), loc2 is (...,2).
 * Writes every element of out. */
int dfa3d_wms_attn_forward(const dfa3d_problem *p, const void *value, const int64_t *shapes2,
                           const int64_t *level_start, const float *loc2, const float *attn,
                           const float *depth_score, float *out, void *stream);

/* Depth-weighted attention, backward.  Replaces wms_deform_attn_backward (pybind.cpp:48-54 ->
 * wms_deform_attn_cuda.cu:291-370 -> kernel.cuh:305-419 and its five sibling kernels).
 * grad_value (B,N,H,C) fp32 is ACCUMULATED into (caller zeroes it); grad_loc2, grad_attn and
 * grad_depth_score are overwritten. */
int dfa3d_wms_attn_backward(const dfa3d_problem *p, const void *value, const int64_t *shapes2,
                            const int64_t *level_start, const float *loc2, const float *attn,
                            const float *depth_score, const float *grad_out, float *grad_value,
                            float *grad_loc2, float *grad_attn, float *grad_depth_score,
                            void *stream);

/* One-stage forward: both reference kernels in one launch, depth_score never leaves the SM unless
 * depth_score_out is non-null.  Replaces the forward of MultiScale3DDeformableAttnFunction_fp32
 * (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/
 *  multi_scale_3ddeformable_attn_function.py:279-305).  shapes3 is (L,3), loc3 is (...,3). */
int dfa3d_fused_forward(const dfa3d_problem *p, const void *value, const void *dist,
                        const int64_t *shapes3, const int64_t *level_start, const float *loc3,
                        const float *attn, float *out, float *depth_score_out, void *stream);

/* One-stage backward: replaces the backward of the same Function (:306-352), i.e. both reference
 * backward kernels, the slice copies and four of its six memsets.  grad_value and grad_dist are
 * ACCUMULATED into (caller zeroes them); grad_loc3 (x, y and z parts) and grad_attn are overwritten. */
int dfa3d_fused_backward(const dfa3d_problem *p, const void *value, const void *dist,
                         const int64_t *shapes3, const int64_t *level_start, const float *loc3,
                         const float *attn, const float *grad_out, float *grad_value,
                         float *grad_dist, float *grad_loc3, float *grad_attn, void *stream);

/* Plain 2-D multi-scale deformable attention: the depth-weighted kernels with every depth score 1.
 * BEVFormer_DFA3D calls this operator (through the third-party mmcv extension, not vendored in the
 * reference checkout) from its temporal self-attention and decoder,
 * BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/multi_scale_deformable_attn_function.py:10-12
 * (ms_deform_attn_forward / ms_deform_attn_backward).  Same layouts as dfa3d_wms_attn_*: shapes2 (L,2),
 * loc2 (...,2).  grad_value is ACCUMULATED into; grad_loc2 and grad_attn are overwritten. */
int dfa3d_msda_forward(const dfa3d_problem *p, const void *value, const int64_t *shapes2,
                       const int64_t *level_start, const float *loc2, const float *attn, float *out,
                       void *stream);
int dfa3d_msda_backward(const dfa3d_problem *p, const void *value, const int64_t *shapes2,
                        const int64_t *level_start, const float *loc2, const float *attn,
                        const float *grad_out, float *grad_value, float *grad_loc2, float *grad_attn,
                        void *stream);

/* The attention module's tensor code folded into the operator.  Replaces, around the one-stage
 * Function, the location assembly and the softmax of MSDeformableAttention3D_DFA3D.forward
 * (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/spatial_cross_attention.py:503-538):
 *   loc[b,q,h,l,p] = ref_points[b,q,p % num_anchors] + (offsets_uv / (w_l, h_l), offsets_depth / D)
 *   attn[b,q,h,:]  = softmax over the L*P logits
 * ref_points (B,Q,num_anchors,3), offsets_uv (B,Q,H,L,P,2), offsets_depth (B,Q,H,L,P),
 * logits (B,Q,H,L*P), all fp32; num_anchors must divide P.  Writes every element of out. */
int dfa3d_attn3d_forward(const dfa3d_problem *p, int32_t num_anchors, const void *value,
                         const void *dist, const int64_t *shapes3, const int64_t *level_start,
                         const float *ref_points, const float *offsets_uv, const float *offsets_depth,
                         const float *logits, float *out, void *stream);

/* Backward of dfa3d_attn3d_forward, i.e. of the Function's backward (:306-352) chained with the
 * autograd of the division, the addition and the softmax.  grad_value and grad_dist are ACCUMULATED
 * into (caller zeroes them); grad_offsets_uv, grad_offsets_depth and grad_logits are overwritten.
 * The reference points get no gradient (in BEVFormer they come from fixed geometry). */
int dfa3d_attn3d_backward(const dfa3d_problem *p, int32_t num_anchors, const void *value,
                          const void *dist, const int64_t *shapes3, const int64_t *level_start,
                          const float *ref_points, const float *offsets_uv,
                          const float *offsets_depth, const float *logits, const float *grad_out,
                          float *grad_value, float *grad_dist, float *grad_offsets_uv,
                          float *grad_offsets_depth, float *grad_logits, void *stream);

/* The one-stage and the offsets/logits entry points for cameras with DIFFERENT numbers of queries
 * (BEVFormer: every camera sees its own subset of the BEV queries; the reference pads all of them to the
 * longest list, spatial_cross_attention.py:707-722).  query_offsets (B+1 int32, device) gives camera b
 * the packed rows [query_offsets[b], query_offsets[b+1]) of every per-query tensor, which therefore lose
 * their batch dimension: loc3 (R,H,L,P,3), attn (R,H,L,P), out (R,H*C), ref_points (R,Z,3), ... with
 * R = query_offsets[B].  p->Q is then only an upper bound of the queries of any one camera (it sizes the
 * launch); value / dist and their gradients keep their (B, N, ...) layout.  Everything else is as in
 * the entry point of the same name without the suffix. */
int dfa3d_fused_forward_ragged(const dfa3d_problem *p, const int32_t *query_offsets, const void *value,
                               const void *dist, const int64_t *shapes3, const int64_t *level_start,
                               const float *loc3, const float *attn, float *out,
                               float *depth_score_out, void *stream);
int dfa3d_fused_backward_ragged(const dfa3d_problem *p, const int32_t *query_offsets, const void *value,
                                const void *dist, const int64_t *shapes3, const int64_t *level_start,
                                const float *loc3, const float *attn, const float *grad_out,
                                float *grad_value, float *grad_dist, float *grad_loc3,
                                float *grad_attn, void *stream);
int dfa3d_attn3d_forward_ragged(const dfa3d_problem *p, int32_t num_anchors,
                                const int32_t *query_offsets, const void *value, const void *dist,
                                const int64_t *shapes3, const int64_t *level_start,
                                const float *ref_points, const float *offsets_uv,
                                const float *offsets_depth, const float *logits, float *out,
                                void *stream);
int dfa3d_attn3d_backward_ragged(const dfa3d_problem *p, int32_t num_anchors,
                                 const int32_t *query_offsets, const void *value, const void *dist,
                                 const int64_t *shapes3, const int64_t *level_start,
                                 const float *ref_points, const float *offsets_uv,
                                 const float *offsets_depth, const float *logits, const float *grad_out,
                                 float *grad_value, float *grad_dist, float *grad_offsets_uv,
                                 float *grad_offsets_depth, float *grad_logits, void *stream);

/* Per-camera re-batching of the BEV queries.  Replaces the host loops of
 * SpatialCrossAttention_DFA3D.forward (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/
 * spatial_cross_attention.py:700-722 build the per-camera index lists with nonzero() and copy the
 * queries / reference points into zero-padded (bs, cams, max_len, ...) tensors; :741-748 add the
 * per-camera results back into BEV order and divide by the number of cameras that see each query).
 *
 * dfa3d_rebatch_plan: bev_mask (cams, bs, Q, Z) bytes (0 / non-0), device.  Camera i sees query q when any
 * of the Z entries of batch element 0 is set (:703-705).  Outputs (device, written entirely):
 *   counts (cams)            queries seen per camera
 *   offsets (cams+1)         exclusive prefix sums; T = offsets[cams] rows per batch element
 *   op_offsets (bs*cams+1)   j*T + offsets[i] at index j*cams + i: the query_offsets of the *_ragged
 *                            entry points for B = bs*cams
 *   packed_query, packed_camera (capacity cams*Q each; the first T entries are written)
 *                            BEV query and camera of packed row p, cameras in order, queries ascending
 *   row_of (cams, Q)         packed row of (camera, query) or -1
 *   inv_count (bs, Q)        1 / max(1, cameras that see q in batch element j)          (:745-747)
 * No host synchronisation; the caller learns T by reading offsets[cams] when it needs exact sizes. */
int dfa3d_rebatch_plan(const uint8_t *bev_mask, int32_t cams, int32_t bs, int32_t Q, int32_t Z,
                       int32_t *counts, int32_t *offsets, int32_t *op_offsets, int32_t *packed_query,
                       int32_t *packed_camera, int32_t *row_of, float *inv_count, void *stream);

/* dst[j*T + p, :] = scale[j, q] * src[camera*src_camera_stride + j*src_batch_stride + q, :] with
 * q = packed_query[p], camera = packed_camera[p]; rows of `width` floats; strides in rows (0 = the
 * source is shared by all cameras / batch elements); scale (bs, Q) or null.  rows_bound >= bs*T sizes
 * the launch (bs*cams*Q always suffices).  Replaces :710-722; with scale = inv_count it is also the
 * backward of dfa3d_rebatch_combine. */
int dfa3d_rebatch_gather(const float *src, const int32_t *packed_query, const int32_t *packed_camera,
                         const int32_t *offsets, int32_t cams, int32_t bs, int32_t Q, int32_t width,
                         int64_t src_camera_stride, int64_t src_batch_stride, const float *scale,
                         float *dst, int64_t rows_bound, void *stream);

/* dst[j, q, :] = scale[j, q] * sum over the cameras i that see q of src[j*T + row_of[i, q], :]
 * (zeros where no camera sees q; every element of dst is written; no atomics: each output row is
 * formed by one thread group).  Replaces :741-748; without scale it is the backward of
 * dfa3d_rebatch_gather for a source shared by all cameras. */
int dfa3d_rebatch_combine(const float *src, const int32_t *row_of, const int32_t *offsets, int32_t cams,
                          int32_t bs, int32_t Q, int32_t width, const float *scale, float *dst,
                          void *stream);

/* Producer of `dist`: the depth network's logits (B, D, map_h, map_w) fp32 become the operator's
 * dist (B, N, D), fp32, bf16 or fp16, in one pass: softmax over D (or sigmoid), nearest-neighbour resize to
 * every level (spatial_shapes (L, shape_stride) / level_start (L), int64, device), channel-last layout.
 * Replaces BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/dense_heads/depth_head.py:265-276
 * (feat_dpt.softmax(1) | sigmoid(); F.interpolate(dpt_dist, size=scale, mode="nearest") per level) and
 * the flatten / permute / cat of …/modules/transformer.py:368-391 with the permute of
 * spatial_cross_attention.py:727-728.  With L = 1 and the level equal to the map it writes the single
 * map that dfa3d_problem.dist_map_h/w describe.  D <= 256.  Writes every element of dist. */
int dfa3d_dist_from_logits(const float *logits, int32_t B, int32_t D, int32_t map_h, int32_t map_w,
                           const int64_t *spatial_shapes, int32_t shape_stride,
                           const int64_t *level_start, int32_t L, int32_t N, int32_t activation,
                           int32_t dist_dtype, void *dist, void *stream);

/* Its backward: grad_dist (B, N, D) fp32 -> grad_logits (B, D, map_h, map_w) fp32, i.e. autograd of the
 * interpolate calls (sum over the level pixels that read a map pixel) chained with the softmax /
 * sigmoid backward; the normalised bins are recomputed from the logits.  Writes every element of
 * grad_logits. */
int dfa3d_dist_from_logits_backward(const float *logits, int32_t B, int32_t D, int32_t map_h,
                                    int32_t map_w, const int64_t *spatial_shapes, int32_t shape_stride,
                                    const int64_t *level_start, int32_t L, int32_t N,
                                    int32_t activation, const float *grad_dist, float *grad_logits,
                                    void *stream);

/* Double precision.  The reference instantiates its kernels for float and double
 * (AT_DISPATCH_FLOATING_TYPES, DFA3D/dfa3D/ops/csrc/cuda/wms_deform_attn_cuda.cu:267,344 and
 * cuda/ms_depth_score_sample_cuda.cu:94,184).  The *_f64 entry points are the double instantiations of
 * the entry points of the same name: every floating-point tensor -- value, dist, locations, attention
 * weights, depth scores, outputs, all gradients -- is double, p->value_dtype and p->dist_dtype are
 * DFA3D_DTYPE_F64, dist is (B,N,H,D) or (B,N,D) (no single-map option).  Accumulated gradients are
 * caller-zeroed, the others overwritten, as in single precision.  These kernels are written for
 * gradient checks and reference-grade comparisons, not for speed. */
int dfa3d_depth_score_forward_f64(const dfa3d_problem *p, const double *dist, const int64_t *shapes3,
                                  const int64_t *level_start, const double *loc3, double *depth_score,
                                  void *stream);
int dfa3d_depth_score_backward_f64(const dfa3d_problem *p, const double *dist, const int64_t *shapes3,
                                   const int64_t *level_start, const double *loc3,
                                   const double *grad_depth_score, double *grad_dist, double *grad_loc3,
                                   void *stream);
int dfa3d_wms_attn_forward_f64(const dfa3d_problem *p, const double *value, const int64_t *shapes2,
                               const int64_t *level_start, const double *loc2, const double *attn,
                               const double *depth_score, double *out, void *stream);
int dfa3d_wms_attn_backward_f64(const dfa3d_problem *p, const double *value, const int64_t *shapes2,
                                const int64_t *level_start, const double *loc2, const double *attn,
                                const double *depth_score, const double *grad_out, double *grad_value,
                                double *grad_loc2, double *grad_attn, double *grad_depth_score,
                                void *stream);
int dfa3d_fused_forward_f64(const dfa3d_problem *p, const double *value, const double *dist,
                            const int64_t *shapes3, const int64_t *level_start, const double *loc3,
                            const double *attn, double *out, double *depth_score_out, void *stream);
int dfa3d_fused_backward_f64(const dfa3d_problem *p, const double *value, const double *dist,
                             const int64_t *shapes3, const int64_t *level_start, const double *loc3,
                             const double *attn, const double *grad_out, double *grad_value,
                             double *grad_dist, double *grad_loc3, double *grad_attn, void *stream);

/* ---- row operations of the encoder layer around the operator ------------------------------------
 * The layer applies norm(x + branch(x)) after each block (BEVFormer_DFA3D/projects/mmdet3d_plugin/
 * bevformer/modules/encoder.py:363-411: self_attn, norm, cross_attn, norm, ffn, norm; the reference
 * builds the norms as torch LayerNorm and adds the residual inside each attention / FFN module).
 * fp32, rows of E columns, E a multiple of 4 up to 1024 (multiples of 128 use every lane), all row
 * pointers 16-byte aligned.
 *
 * y = LayerNorm(x + residual) * gamma + beta over the last dimension (biased variance, eps inside the
 * square root, like torch.nn.LayerNorm).  residual and sum_out may be NULL together (plain LayerNorm of
 * x); with a residual, sum_out receives x + residual, the tensor the backward reads.  mean and rstd
 * (rows) receive the row statistics. */
int dfa3d_add_layer_norm_forward(const float *x, const float *residual, const float *gamma,
                                 const float *beta, int64_t rows, int32_t E, float eps, float *sum_out,
                                 float *y, float *mean, float *rstd, void *stream);

/* Its backward.  `in` is what was normalised (x, or sum_out).  grad_in (rows, E) is overwritten (it is
 * the gradient of x and of the residual alike); grad_gamma and grad_beta (E) are accumulated into and
 * must be zeroed by the caller; both 16-byte aligned. */
int dfa3d_layer_norm_backward(const float *grad_y, const float *in, const float *gamma,
                              const float *mean, const float *rstd, int64_t rows, int32_t E,
                              float *grad_in, float *grad_gamma, float *grad_beta, void *stream);

/* dst[c] += sum over rows of src[r, c]: the bias gradient of a Linear layer (torch computes it as
 * grad_output.sum(0)).  cols a multiple of 4; dst accumulated into, zeroed by the caller, 16-byte
 * aligned like src. */
int dfa3d_column_sum(const float *src, int64_t rows, int32_t cols, float *dst, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DFA3D_B200_H_ */
