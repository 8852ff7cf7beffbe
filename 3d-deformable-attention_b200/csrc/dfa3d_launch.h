// Internal: host-side launchers implemented by the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dfa3d {
struct KArgs;
// mode: dfa3d::Mode
cudaError_t launch_forward(const KArgs &a, bool value_bf16, bool dist_bf16, int mode, cudaStream_t s);
cudaError_t launch_depth_score_forward(const KArgs &a, bool dist_bf16, cudaStream_t s);
cudaError_t launch_backward(const KArgs &a, bool value_bf16, bool dist_bf16, int mode, cudaStream_t s);
cudaError_t launch_depth_score_backward(const KArgs &a, bool dist_bf16, cudaStream_t s);
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
// depth-distribution producer (dfa3d_dist_producer.cu)
int dist_producer_max_bins();
cudaError_t launch_dist_from_logits(const float *logits, const int64_t *shapes, int shape_stride,
                                    const int64_t *lsi, void *dist, bool dist_bf16, int B, int D, int hs,
                                    int ws, int N, int L, bool sigmoid, cudaStream_t s);
cudaError_t launch_dist_from_logits_backward(const float *logits, const int64_t *shapes, int shape_stride,
                                             const int64_t *lsi, const float *grad_dist,
                                             float *grad_logits, int B, int D, int hs, int ws, int N,
                                             int L, bool sigmoid, cudaStream_t s);
}  // namespace dfa3d
