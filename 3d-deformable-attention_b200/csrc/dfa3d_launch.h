// Internal: host-side launchers implemented by the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

struct dfa3d_problem;
namespace dfa3d {
struct KArgs;
// mode: dfa3d::Mode
cudaError_t launch_forward(const KArgs &a, int value_dtype, int dist_dtype, int mode, cudaStream_t s);
cudaError_t launch_depth_score_forward(const KArgs &a, int dist_dtype, cudaStream_t s);
cudaError_t launch_backward(const KArgs &a, int value_dtype, int dist_dtype, int mode, cudaStream_t s);
cudaError_t launch_depth_score_backward(const KArgs &a, int dist_dtype, cudaStream_t s);
// per-camera re-batching (dfa3d_rebatch.cu)
cudaError_t launch_rebatch_plan(const uint8_t *mask, int cams, int bs, int Q, int Z, int32_t *counts,
                                int32_t *offsets, int32_t *op_offsets, int32_t *packed_query,
                                int32_t *packed_camera, int32_t *row_of, float *inv_count,
                                cudaStream_t s);
cudaError_t launch_rebatch_gather(const float *src, const int32_t *packed_query,
                                  const int32_t *packed_camera, const int32_t *offsets, int cams, int bs,
                                  int Q, int W, long long cam_stride, long long batch_stride,
                                  const float *scale, float *dst, long long rows_bound, cudaStream_t s);
cudaError_t launch_rebatch_combine(const float *src, const int32_t *row_of, const int32_t *offsets,
                                   int cams, int bs, int Q, int W, const float *scale, float *dst,
                                   cudaStream_t s);
// double-precision kernels (dfa3d_fp64.cu); `from_dist`: depth scores are sampled from dist (one-stage)
// instead of being given (two-stage attention; a null ds_in then means all ones)
cudaError_t launch_forward64(const dfa3d_problem *p, const double *value, const double *dist,
                             const int64_t *shapes, int shape_stride, const int64_t *lsi,
                             const double *loc, int loc_stride, const double *attn, const double *ds_in,
                             bool from_dist, double *out, double *ds_out, cudaStream_t s);
cudaError_t launch_backward64(const dfa3d_problem *p, const double *value, const double *dist,
                              const int64_t *shapes, int shape_stride, const int64_t *lsi,
                              const double *loc, int loc_stride, const double *attn, const double *ds_in,
                              bool from_dist, const double *grad_out, double *grad_value,
                              double *grad_dist, double *grad_loc, double *grad_attn, double *grad_ds_out,
                              cudaStream_t s);
cudaError_t launch_depth_forward64(const dfa3d_problem *p, const double *dist, const int64_t *shapes3,
                                   const int64_t *lsi, const double *loc3, double *ds_out,
                                   cudaStream_t s);
cudaError_t launch_depth_backward64(const dfa3d_problem *p, const double *dist, const int64_t *shapes3,
                                    const int64_t *lsi, const double *loc3, const double *grad_ds,
                                    double *grad_dist, double *grad_loc3, cudaStream_t s);
// depth-distribution producer (dfa3d_dist_producer.cu)
int dist_producer_max_bins();
// dist_dtype: DFA3D_DTYPE_F32 (0), _BF16 (1) or _F16 (3)
cudaError_t launch_dist_from_logits(const float *logits, const int64_t *shapes, int shape_stride,
                                    const int64_t *lsi, void *dist, int dist_dtype, int B, int D, int hs,
                                    int ws, int N, int L, bool sigmoid, cudaStream_t s);
cudaError_t launch_dist_from_logits_backward(const float *logits, const int64_t *shapes, int shape_stride,
                                             const int64_t *lsi, const float *grad_dist,
                                             float *grad_logits, int B, int D, int hs, int ws, int N,
                                             int L, bool sigmoid, cudaStream_t s);
// encoder-layer row operations (dfa3d_layer_ops.cu); E = columns of a row, a multiple of 4 up to 1024
int layer_norm_max_columns();
cudaError_t launch_add_layer_norm_forward(const float *x, const float *residual, const float *gamma,
                                          const float *beta, long long rows, int E, float eps,
                                          float *sum_out, float *y, float *mean, float *rstd,
                                          cudaStream_t s);
cudaError_t launch_layer_norm_backward(const float *grad_y, const float *in, const float *gamma,
                                       const float *mean, const float *rstd, long long rows, int E,
                                       float *grad_in, float *grad_gamma, float *grad_beta,
                                       cudaStream_t s);
cudaError_t launch_column_sum(const float *src, long long rows, int cols, float *dst, cudaStream_t s);
}  // namespace dfa3d
