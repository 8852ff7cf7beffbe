// extern "C" entry points of libdfa3d_b200.so: argument validation, kernel-argument assembly, error
// reporting.  Declarations and the reference interfaces they replace: include/dfa3d_b200.h.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "dfa3d_b200.h"
#include "dfa3d_common.cuh"
#include "dfa3d_launch.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Checks the descriptor; `need_value` / `need_dist` say which tensors the call reads.
int check_problem(const dfa3d_problem *p, bool need_value, bool need_dist) {
  if (!p) return fail(DFA3D_ERR_INVALID_ARGUMENT, "problem descriptor is null");
  if (p->B < 0 || p->Q < 0) return fail(DFA3D_ERR_INVALID_ARGUMENT, "B and Q must be >= 0");
  if (p->N <= 0 || p->H <= 0 || p->L <= 0 || p->P <= 0)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "N, H, L, P must be positive (got %d %d %d %d)", p->N,
                p->H, p->L, p->P);
  if (p->L > DFA3D_MAX_LEVELS)
    return fail(DFA3D_ERR_UNSUPPORTED, "L=%d exceeds DFA3D_MAX_LEVELS=%d", p->L, DFA3D_MAX_LEVELS);
  if ((long long)p->L * p->P > (1 << 20))
    return fail(DFA3D_ERR_UNSUPPORTED, "L*P=%lld is too large", (long long)p->L * p->P);
  if ((long long)p->Q * p->H >= (1LL << 31) - 8)
    return fail(DFA3D_ERR_UNSUPPORTED, "Q*H must stay below 2^31");
  if (need_value) {
    if (p->C <= 0 || p->C > DFA3D_MAX_CHANNELS)
      return fail(DFA3D_ERR_UNSUPPORTED, "C=%d outside [1, %d]", p->C, DFA3D_MAX_CHANNELS);
    if (p->value_dtype != DFA3D_DTYPE_F32 && p->value_dtype != DFA3D_DTYPE_BF16 &&
        p->value_dtype != DFA3D_DTYPE_F16)
      return fail(DFA3D_ERR_INVALID_ARGUMENT, "value_dtype %d is not a DFA3D_DTYPE_*", p->value_dtype);
    if ((long long)p->N * p->H * p->C >= (1LL << 31))
      return fail(DFA3D_ERR_UNSUPPORTED, "N*H*C must stay below 2^31 (one camera's value slice)");
  }
  if (need_dist) {
    if (p->D <= 0) return fail(DFA3D_ERR_INVALID_ARGUMENT, "D must be positive (got %d)", p->D);
    if (p->dist_dtype != DFA3D_DTYPE_F32 && p->dist_dtype != DFA3D_DTYPE_BF16 &&
        p->dist_dtype != DFA3D_DTYPE_F16)
      return fail(DFA3D_ERR_INVALID_ARGUMENT, "dist_dtype %d is not a DFA3D_DTYPE_*", p->dist_dtype);
    if (need_value && (p->value_dtype == DFA3D_DTYPE_F16) != (p->dist_dtype == DFA3D_DTYPE_F16))
      return fail(DFA3D_ERR_UNSUPPORTED, "fp16 storage: value and dist must both be DFA3D_DTYPE_F16 "
                  "(got value_dtype %d, dist_dtype %d)", p->value_dtype, p->dist_dtype);
    if (p->dist_head_stride != 0 && p->dist_head_stride != p->D)
      return fail(DFA3D_ERR_INVALID_ARGUMENT, "dist_head_stride must be 0 (shared) or D (per head), got %lld",
                  (long long)p->dist_head_stride);
    if ((p->dist_map_h > 0) != (p->dist_map_w > 0) || p->dist_map_h < 0 || p->dist_map_w < 0)
      return fail(DFA3D_ERR_INVALID_ARGUMENT, "dist_map_h and dist_map_w must both be 0 or both positive "
                  "(got %d, %d)", p->dist_map_h, p->dist_map_w);
    const long long rows = p->dist_map_h > 0 ? (long long)p->dist_map_h * p->dist_map_w : p->N;
    if (rows * p->H * p->D >= (1LL << 31))
      return fail(DFA3D_ERR_UNSUPPORTED, "rows*H*D of one camera's dist slice must stay below 2^31");
  }
  return DFA3D_OK;
}

#define REQUIRE_PTR(ptr)                                                                 \
  do {                                                                                    \
    if (!(ptr)) return fail(DFA3D_ERR_INVALID_ARGUMENT, "argument `%s` is null", #ptr);   \
  } while (0)
#define REQUIRE_ALIGNED(ptr)                                                                          \
  do {                                                                                                 \
    if (!aligned16(ptr)) return fail(DFA3D_ERR_INVALID_ARGUMENT, "`%s` must be 16-byte aligned", #ptr); \
  } while (0)

dfa3d::KArgs base_args(const dfa3d_problem *p, int shape_stride, int loc_stride) {
  dfa3d::KArgs a;
  memset(&a, 0, sizeof(a));
  a.B = p->B; a.N = p->N; a.H = p->H; a.C = p->C; a.D = p->D; a.L = p->L; a.Q = p->Q; a.P = p->P;
  a.LP = p->L * p->P;
  a.shape_stride = shape_stride;
  a.loc_stride = loc_stride;
  a.items = (long long)p->B * p->Q * p->H;
  a.items_per_cam = p->Q * p->H;
  a.dist_head_stride = (int)p->dist_head_stride;
  a.dist_pix_stride = p->dist_head_stride == 0 ? p->D : p->H * p->D;
  a.dmap_h = p->dist_map_h; a.dmap_w = p->dist_map_w;
  a.Nd = p->dist_map_h > 0 ? p->dist_map_h * p->dist_map_w : p->N;
  return a;
}

int finish(cudaError_t e, const char *what) {
  if (e != cudaSuccess)
    return fail(DFA3D_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return DFA3D_OK;
}

}  // namespace

extern "C" {

int dfa3d_abi_version(void) { return DFA3D_ABI_VERSION; }

const char *dfa3d_last_error(void) { return g_err; }

int dfa3d_depth_score_forward(const dfa3d_problem *p, const void *dist, const int64_t *shapes3,
                              const int64_t *level_start, const float *loc3, float *depth_score,
                              void *stream) {
  if (int rc = check_problem(p, false, true)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start); REQUIRE_PTR(loc3);
  REQUIRE_PTR(depth_score); REQUIRE_ALIGNED(depth_score);
  dfa3d::KArgs a = base_args(p, 3, 3);
  a.dist = dist; a.shapes = shapes3; a.lsi = level_start; a.loc = loc3; a.ds_out = depth_score;
  return finish(dfa3d::launch_depth_score_forward(a, p->dist_dtype,
                                                  (cudaStream_t)stream),
                "dfa3d_depth_score_forward launch");
}

int dfa3d_depth_score_backward(const dfa3d_problem *p, const void *dist, const int64_t *shapes3,
                               const int64_t *level_start, const float *loc3,
                               const float *grad_depth_score, float *grad_dist, float *grad_loc3,
                               void *stream) {
  if (int rc = check_problem(p, false, true)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start); REQUIRE_PTR(loc3);
  REQUIRE_PTR(grad_depth_score); REQUIRE_PTR(grad_dist); REQUIRE_PTR(grad_loc3);
  REQUIRE_ALIGNED(grad_depth_score);
  dfa3d::KArgs a = base_args(p, 3, 3);
  a.dist = dist; a.shapes = shapes3; a.lsi = level_start; a.loc = loc3;
  a.grad_ds_in = grad_depth_score; a.grad_dist = grad_dist; a.grad_loc = grad_loc3;
  return finish(dfa3d::launch_depth_score_backward(a, p->dist_dtype,
                                                   (cudaStream_t)stream),
                "dfa3d_depth_score_backward launch");
}

int dfa3d_wms_attn_forward(const dfa3d_problem *p, const void *value, const int64_t *shapes2,
                           const int64_t *level_start, const float *loc2, const float *attn,
                           const float *depth_score, float *out, void *stream) {
  if (int rc = check_problem(p, true, false)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(shapes2); REQUIRE_PTR(level_start); REQUIRE_PTR(loc2);
  REQUIRE_PTR(attn); REQUIRE_PTR(depth_score); REQUIRE_PTR(out);
  REQUIRE_ALIGNED(value); REQUIRE_ALIGNED(depth_score); REQUIRE_ALIGNED(out);
  dfa3d::KArgs a = base_args(p, 2, 2);
  a.value = value; a.shapes = shapes2; a.lsi = level_start; a.loc = loc2; a.attn = attn;
  a.ds_in = depth_score; a.out = out;
  return finish(dfa3d::launch_forward(a, p->value_dtype, DFA3D_DTYPE_F32,
                                      dfa3d::kGivenDepthScore, (cudaStream_t)stream),
                "dfa3d_wms_attn_forward launch");
}

int dfa3d_wms_attn_backward(const dfa3d_problem *p, const void *value, const int64_t *shapes2,
                            const int64_t *level_start, const float *loc2, const float *attn,
                            const float *depth_score, const float *grad_out, float *grad_value,
                            float *grad_loc2, float *grad_attn, float *grad_depth_score,
                            void *stream) {
  if (int rc = check_problem(p, true, false)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(shapes2); REQUIRE_PTR(level_start); REQUIRE_PTR(loc2);
  REQUIRE_PTR(attn); REQUIRE_PTR(depth_score); REQUIRE_PTR(grad_out); REQUIRE_PTR(grad_value);
  REQUIRE_PTR(grad_loc2); REQUIRE_PTR(grad_attn); REQUIRE_PTR(grad_depth_score);
  REQUIRE_ALIGNED(value); REQUIRE_ALIGNED(depth_score); REQUIRE_ALIGNED(grad_out);
  REQUIRE_ALIGNED(grad_value); REQUIRE_ALIGNED(grad_depth_score);
  dfa3d::KArgs a = base_args(p, 2, 2);
  a.value = value; a.shapes = shapes2; a.lsi = level_start; a.loc = loc2; a.attn = attn;
  a.ds_in = depth_score; a.grad_out = grad_out; a.grad_value = grad_value; a.grad_loc = grad_loc2;
  a.grad_attn = grad_attn; a.grad_ds_out = grad_depth_score;
  return finish(dfa3d::launch_backward(a, p->value_dtype, DFA3D_DTYPE_F32,
                                       dfa3d::kGivenDepthScore, (cudaStream_t)stream),
                "dfa3d_wms_attn_backward launch");
}

static int fused_forward_impl(const dfa3d_problem *p, const int32_t *query_offsets, const void *value,
                              const void *dist, const int64_t *shapes3, const int64_t *level_start,
                              const float *loc3, const float *attn, float *out, float *depth_score_out,
                              void *stream) {
  if (int rc = check_problem(p, true, true)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start);
  REQUIRE_PTR(loc3); REQUIRE_PTR(attn); REQUIRE_PTR(out);
  REQUIRE_ALIGNED(value); REQUIRE_ALIGNED(out); REQUIRE_ALIGNED(depth_score_out);
  dfa3d::KArgs a = base_args(p, 3, 3);
  a.value = value; a.dist = dist; a.shapes = shapes3; a.lsi = level_start; a.loc = loc3;
  a.attn = attn; a.out = out; a.ds_out = depth_score_out; a.q_off = query_offsets;
  return finish(dfa3d::launch_forward(a, p->value_dtype,
                                      p->dist_dtype, dfa3d::kFused,
                                      (cudaStream_t)stream),
                "dfa3d_fused_forward launch");
}

int dfa3d_fused_forward(const dfa3d_problem *p, const void *value, const void *dist,
                        const int64_t *shapes3, const int64_t *level_start, const float *loc3,
                        const float *attn, float *out, float *depth_score_out, void *stream) {
  return fused_forward_impl(p, nullptr, value, dist, shapes3, level_start, loc3, attn, out,
                            depth_score_out, stream);
}

int dfa3d_fused_forward_ragged(const dfa3d_problem *p, const int32_t *query_offsets, const void *value,
                               const void *dist, const int64_t *shapes3, const int64_t *level_start,
                               const float *loc3, const float *attn, float *out,
                               float *depth_score_out, void *stream) {
  REQUIRE_PTR(query_offsets);
  return fused_forward_impl(p, query_offsets, value, dist, shapes3, level_start, loc3, attn, out,
                            depth_score_out, stream);
}

static int fused_backward_impl(const dfa3d_problem *p, const int32_t *query_offsets, const void *value,
                               const void *dist, const int64_t *shapes3, const int64_t *level_start,
                               const float *loc3, const float *attn, const float *grad_out,
                               float *grad_value, float *grad_dist, float *grad_loc3, float *grad_attn,
                               void *stream) {
  if (int rc = check_problem(p, true, true)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start);
  REQUIRE_PTR(loc3); REQUIRE_PTR(attn); REQUIRE_PTR(grad_out); REQUIRE_PTR(grad_value);
  REQUIRE_PTR(grad_dist); REQUIRE_PTR(grad_loc3); REQUIRE_PTR(grad_attn);
  REQUIRE_ALIGNED(value); REQUIRE_ALIGNED(grad_out); REQUIRE_ALIGNED(grad_value);
  dfa3d::KArgs a = base_args(p, 3, 3);
  a.value = value; a.dist = dist; a.shapes = shapes3; a.lsi = level_start; a.loc = loc3;
  a.attn = attn; a.grad_out = grad_out; a.grad_value = grad_value; a.grad_dist = grad_dist;
  a.grad_loc = grad_loc3; a.grad_attn = grad_attn; a.q_off = query_offsets;
  return finish(dfa3d::launch_backward(a, p->value_dtype,
                                       p->dist_dtype, dfa3d::kFused,
                                       (cudaStream_t)stream),
                "dfa3d_fused_backward launch");
}

int dfa3d_fused_backward(const dfa3d_problem *p, const void *value, const void *dist,
                         const int64_t *shapes3, const int64_t *level_start, const float *loc3,
                         const float *attn, const float *grad_out, float *grad_value,
                         float *grad_dist, float *grad_loc3, float *grad_attn, void *stream) {
  return fused_backward_impl(p, nullptr, value, dist, shapes3, level_start, loc3, attn, grad_out,
                             grad_value, grad_dist, grad_loc3, grad_attn, stream);
}

int dfa3d_fused_backward_ragged(const dfa3d_problem *p, const int32_t *query_offsets, const void *value,
                                const void *dist, const int64_t *shapes3, const int64_t *level_start,
                                const float *loc3, const float *attn, const float *grad_out,
                                float *grad_value, float *grad_dist, float *grad_loc3,
                                float *grad_attn, void *stream) {
  REQUIRE_PTR(query_offsets);
  return fused_backward_impl(p, query_offsets, value, dist, shapes3, level_start, loc3, attn, grad_out,
                             grad_value, grad_dist, grad_loc3, grad_attn, stream);
}

int dfa3d_msda_forward(const dfa3d_problem *p, const void *value, const int64_t *shapes2,
                       const int64_t *level_start, const float *loc2, const float *attn, float *out,
                       void *stream) {
  if (int rc = check_problem(p, true, false)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(shapes2); REQUIRE_PTR(level_start); REQUIRE_PTR(loc2);
  REQUIRE_PTR(attn); REQUIRE_PTR(out);
  REQUIRE_ALIGNED(value); REQUIRE_ALIGNED(out);
  dfa3d::KArgs a = base_args(p, 2, 2);
  a.value = value; a.shapes = shapes2; a.lsi = level_start; a.loc = loc2; a.attn = attn; a.out = out;
  return finish(dfa3d::launch_forward(a, p->value_dtype, DFA3D_DTYPE_F32,
                                      dfa3d::kGivenDepthScore, (cudaStream_t)stream),
                "dfa3d_msda_forward launch");
}

int dfa3d_msda_backward(const dfa3d_problem *p, const void *value, const int64_t *shapes2,
                        const int64_t *level_start, const float *loc2, const float *attn,
                        const float *grad_out, float *grad_value, float *grad_loc2, float *grad_attn,
                        void *stream) {
  if (int rc = check_problem(p, true, false)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(shapes2); REQUIRE_PTR(level_start); REQUIRE_PTR(loc2);
  REQUIRE_PTR(attn); REQUIRE_PTR(grad_out); REQUIRE_PTR(grad_value); REQUIRE_PTR(grad_loc2);
  REQUIRE_PTR(grad_attn);
  REQUIRE_ALIGNED(value); REQUIRE_ALIGNED(grad_out); REQUIRE_ALIGNED(grad_value);
  dfa3d::KArgs a = base_args(p, 2, 2);
  a.value = value; a.shapes = shapes2; a.lsi = level_start; a.loc = loc2; a.attn = attn;
  a.grad_out = grad_out; a.grad_value = grad_value; a.grad_loc = grad_loc2; a.grad_attn = grad_attn;
  return finish(dfa3d::launch_backward(a, p->value_dtype, DFA3D_DTYPE_F32,
                                       dfa3d::kGivenDepthScore, (cudaStream_t)stream),
                "dfa3d_msda_backward launch");
}

static int attn3d_forward_impl(const dfa3d_problem *p, int32_t num_anchors,
                               const int32_t *query_offsets, const void *value, const void *dist,
                               const int64_t *shapes3, const int64_t *level_start,
                               const float *ref_points, const float *offsets_uv,
                               const float *offsets_depth, const float *logits, float *out,
                               void *stream) {
  if (int rc = check_problem(p, true, true)) return rc;
  if (num_anchors <= 0 || p->P % num_anchors != 0)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "num_anchors=%d must be positive and divide P=%d",
                num_anchors, p->P);
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start);
  REQUIRE_PTR(ref_points); REQUIRE_PTR(offsets_uv); REQUIRE_PTR(offsets_depth); REQUIRE_PTR(logits);
  REQUIRE_PTR(out);
  REQUIRE_ALIGNED(value); REQUIRE_ALIGNED(out);
  dfa3d::KArgs a = base_args(p, 3, 3);
  a.value = value; a.dist = dist; a.shapes = shapes3; a.lsi = level_start; a.ref = ref_points;
  a.off_uv = offsets_uv; a.off_d = offsets_depth; a.logits = logits; a.Z = num_anchors; a.out = out;
  a.q_off = query_offsets;
  return finish(dfa3d::launch_forward(a, p->value_dtype,
                                      p->dist_dtype, dfa3d::kCallerFused,
                                      (cudaStream_t)stream),
                "dfa3d_attn3d_forward launch");
}

int dfa3d_attn3d_forward(const dfa3d_problem *p, int32_t num_anchors, const void *value,
                         const void *dist, const int64_t *shapes3, const int64_t *level_start,
                         const float *ref_points, const float *offsets_uv, const float *offsets_depth,
                         const float *logits, float *out, void *stream) {
  return attn3d_forward_impl(p, num_anchors, nullptr, value, dist, shapes3, level_start, ref_points,
                             offsets_uv, offsets_depth, logits, out, stream);
}

int dfa3d_attn3d_forward_ragged(const dfa3d_problem *p, int32_t num_anchors,
                                const int32_t *query_offsets, const void *value, const void *dist,
                                const int64_t *shapes3, const int64_t *level_start,
                                const float *ref_points, const float *offsets_uv,
                                const float *offsets_depth, const float *logits, float *out,
                                void *stream) {
  REQUIRE_PTR(query_offsets);
  return attn3d_forward_impl(p, num_anchors, query_offsets, value, dist, shapes3, level_start, ref_points,
                             offsets_uv, offsets_depth, logits, out, stream);
}

static int attn3d_backward_impl(const dfa3d_problem *p, int32_t num_anchors,
                                const int32_t *query_offsets, const void *value, const void *dist,
                                const int64_t *shapes3, const int64_t *level_start,
                                const float *ref_points, const float *offsets_uv,
                                const float *offsets_depth, const float *logits, const float *grad_out,
                                float *grad_value, float *grad_dist, float *grad_offsets_uv,
                                float *grad_offsets_depth, float *grad_logits, void *stream) {
  if (int rc = check_problem(p, true, true)) return rc;
  if (num_anchors <= 0 || p->P % num_anchors != 0)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "num_anchors=%d must be positive and divide P=%d",
                num_anchors, p->P);
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start);
  REQUIRE_PTR(ref_points); REQUIRE_PTR(offsets_uv); REQUIRE_PTR(offsets_depth); REQUIRE_PTR(logits);
  REQUIRE_PTR(grad_out); REQUIRE_PTR(grad_value); REQUIRE_PTR(grad_dist); REQUIRE_PTR(grad_offsets_uv);
  REQUIRE_PTR(grad_offsets_depth); REQUIRE_PTR(grad_logits);
  REQUIRE_ALIGNED(value); REQUIRE_ALIGNED(grad_out); REQUIRE_ALIGNED(grad_value);
  dfa3d::KArgs a = base_args(p, 3, 3);
  a.value = value; a.dist = dist; a.shapes = shapes3; a.lsi = level_start; a.ref = ref_points;
  a.off_uv = offsets_uv; a.off_d = offsets_depth; a.logits = logits; a.Z = num_anchors;
  a.grad_out = grad_out; a.grad_value = grad_value; a.grad_dist = grad_dist;
  a.grad_off_uv = grad_offsets_uv; a.grad_off_d = grad_offsets_depth; a.grad_logits = grad_logits;
  a.q_off = query_offsets;
  return finish(dfa3d::launch_backward(a, p->value_dtype,
                                       p->dist_dtype, dfa3d::kCallerFused,
                                       (cudaStream_t)stream),
                "dfa3d_attn3d_backward launch");
}

int dfa3d_attn3d_backward(const dfa3d_problem *p, int32_t num_anchors, const void *value,
                          const void *dist, const int64_t *shapes3, const int64_t *level_start,
                          const float *ref_points, const float *offsets_uv,
                          const float *offsets_depth, const float *logits, const float *grad_out,
                          float *grad_value, float *grad_dist, float *grad_offsets_uv,
                          float *grad_offsets_depth, float *grad_logits, void *stream) {
  return attn3d_backward_impl(p, num_anchors, nullptr, value, dist, shapes3, level_start, ref_points,
                              offsets_uv, offsets_depth, logits, grad_out, grad_value, grad_dist,
                              grad_offsets_uv, grad_offsets_depth, grad_logits, stream);
}

int dfa3d_attn3d_backward_ragged(const dfa3d_problem *p, int32_t num_anchors,
                                 const int32_t *query_offsets, const void *value, const void *dist,
                                 const int64_t *shapes3, const int64_t *level_start,
                                 const float *ref_points, const float *offsets_uv,
                                 const float *offsets_depth, const float *logits, const float *grad_out,
                                 float *grad_value, float *grad_dist, float *grad_offsets_uv,
                                 float *grad_offsets_depth, float *grad_logits, void *stream) {
  REQUIRE_PTR(query_offsets);
  return attn3d_backward_impl(p, num_anchors, query_offsets, value, dist, shapes3, level_start,
                              ref_points, offsets_uv, offsets_depth, logits, grad_out, grad_value,
                              grad_dist, grad_offsets_uv, grad_offsets_depth, grad_logits, stream);
}

// ---- per-camera re-batching -----------------------------------------------------------------
int dfa3d_rebatch_plan(const uint8_t *bev_mask, int32_t cams, int32_t bs, int32_t Q, int32_t Z,
                       int32_t *counts, int32_t *offsets, int32_t *op_offsets, int32_t *packed_query,
                       int32_t *packed_camera, int32_t *row_of, float *inv_count, void *stream) {
  if (cams <= 0 || bs <= 0 || Q < 0 || Z <= 0)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "cams, bs, Z must be positive and Q >= 0 (got %d %d %d %d)",
                cams, bs, Z, Q);
  if ((long long)cams * Q >= (1LL << 31) || (long long)bs * cams * Q >= (1LL << 31))
    return fail(DFA3D_ERR_UNSUPPORTED, "bs * cams * Q must stay below 2^31");
  REQUIRE_PTR(counts); REQUIRE_PTR(offsets); REQUIRE_PTR(op_offsets);
  if (Q > 0) {      // with no queries the per-query tables are empty and may have no storage
    REQUIRE_PTR(bev_mask); REQUIRE_PTR(packed_query); REQUIRE_PTR(packed_camera); REQUIRE_PTR(row_of);
    REQUIRE_PTR(inv_count);
  }
  return finish(dfa3d::launch_rebatch_plan(bev_mask, cams, bs, Q, Z, counts, offsets, op_offsets,
                                           packed_query, packed_camera, row_of, inv_count,
                                           (cudaStream_t)stream),
                "dfa3d_rebatch_plan launch");
}

int dfa3d_rebatch_gather(const float *src, const int32_t *packed_query, const int32_t *packed_camera,
                         const int32_t *offsets, int32_t cams, int32_t bs, int32_t Q, int32_t width,
                         int64_t src_camera_stride, int64_t src_batch_stride, const float *scale,
                         float *dst, int64_t rows_bound, void *stream) {
  if (cams <= 0 || bs <= 0 || Q < 0 || width <= 0 || rows_bound < 0 || src_camera_stride < 0 ||
      src_batch_stride < 0)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "dfa3d_rebatch_gather: bad size");
  if (rows_bound == 0) return DFA3D_OK;
  REQUIRE_PTR(src); REQUIRE_PTR(packed_query); REQUIRE_PTR(packed_camera); REQUIRE_PTR(offsets);
  REQUIRE_PTR(dst);
  return finish(dfa3d::launch_rebatch_gather(src, packed_query, packed_camera, offsets, cams, bs, Q, width,
                                             src_camera_stride, src_batch_stride, scale, dst, rows_bound,
                                             (cudaStream_t)stream),
                "dfa3d_rebatch_gather launch");
}

int dfa3d_rebatch_combine(const float *src, const int32_t *row_of, const int32_t *offsets, int32_t cams,
                          int32_t bs, int32_t Q, int32_t width, const float *scale, float *dst,
                          void *stream) {
  if (cams <= 0 || bs <= 0 || Q < 0 || width <= 0)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "dfa3d_rebatch_combine: bad size");
  if (Q == 0) return DFA3D_OK;
  REQUIRE_PTR(src); REQUIRE_PTR(row_of); REQUIRE_PTR(offsets); REQUIRE_PTR(dst);
  return finish(dfa3d::launch_rebatch_combine(src, row_of, offsets, cams, bs, Q, width, scale, dst,
                                              (cudaStream_t)stream),
                "dfa3d_rebatch_combine launch");
}

// ---- depth-distribution producer --------------------------------------------------------------
static int check_producer(int32_t B, int32_t D, int32_t map_h, int32_t map_w, int32_t shape_stride,
                          int32_t L, int32_t N, int32_t activation) {
  if (B < 0 || N < 0) return fail(DFA3D_ERR_INVALID_ARGUMENT, "B and N must be >= 0");
  if (D <= 0 || map_h <= 0 || map_w <= 0 || L <= 0)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "D, map_h, map_w, L must be positive (got %d %d %d %d)", D, map_h,
                map_w, L);
  if (D > dfa3d::dist_producer_max_bins())
    return fail(DFA3D_ERR_UNSUPPORTED, "D=%d exceeds the producer's limit of %d bins", D,
                dfa3d::dist_producer_max_bins());
  if (L > DFA3D_MAX_LEVELS) return fail(DFA3D_ERR_UNSUPPORTED, "L=%d exceeds DFA3D_MAX_LEVELS", L);
  if (shape_stride != 2 && shape_stride != 3)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "shape_stride must be 2 or 3 (got %d)", shape_stride);
  if (activation != DFA3D_ACT_SOFTMAX && activation != DFA3D_ACT_SIGMOID)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "activation %d is not a DFA3D_ACT_*", activation);
  if ((long long)N * D >= (1LL << 31) || (long long)D * map_h * map_w >= (1LL << 31))
    return fail(DFA3D_ERR_UNSUPPORTED, "N*D and D*map_h*map_w must stay below 2^31");
  return DFA3D_OK;
}

int dfa3d_dist_from_logits(const float *logits, int32_t B, int32_t D, int32_t map_h, int32_t map_w,
                           const int64_t *spatial_shapes, int32_t shape_stride,
                           const int64_t *level_start, int32_t L, int32_t N, int32_t activation,
                           int32_t dist_dtype, void *dist, void *stream) {
  if (int rc = check_producer(B, D, map_h, map_w, shape_stride, L, N, activation)) return rc;
  if (dist_dtype != DFA3D_DTYPE_F32 && dist_dtype != DFA3D_DTYPE_BF16 && dist_dtype != DFA3D_DTYPE_F16)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "dist_dtype %d is not a DFA3D_DTYPE_*", dist_dtype);
  if (B == 0 || N == 0) return DFA3D_OK;
  REQUIRE_PTR(logits); REQUIRE_PTR(spatial_shapes); REQUIRE_PTR(level_start); REQUIRE_PTR(dist);
  return finish(dfa3d::launch_dist_from_logits(logits, spatial_shapes, shape_stride, level_start, dist,
                                               dist_dtype, B, D, map_h, map_w, N, L,
                                               activation == DFA3D_ACT_SIGMOID, (cudaStream_t)stream),
                "dfa3d_dist_from_logits launch");
}

int dfa3d_dist_from_logits_backward(const float *logits, int32_t B, int32_t D, int32_t map_h,
                                    int32_t map_w, const int64_t *spatial_shapes, int32_t shape_stride,
                                    const int64_t *level_start, int32_t L, int32_t N,
                                    int32_t activation, const float *grad_dist, float *grad_logits,
                                    void *stream) {
  if (int rc = check_producer(B, D, map_h, map_w, shape_stride, L, N, activation)) return rc;
  if (B == 0) return DFA3D_OK;
  REQUIRE_PTR(logits); REQUIRE_PTR(spatial_shapes); REQUIRE_PTR(level_start); REQUIRE_PTR(grad_logits);
  if (N > 0) REQUIRE_PTR(grad_dist);
  return finish(dfa3d::launch_dist_from_logits_backward(logits, spatial_shapes, shape_stride, level_start,
                                                        grad_dist, grad_logits, B, D, map_h, map_w, N, L,
                                                        activation == DFA3D_ACT_SIGMOID,
                                                        (cudaStream_t)stream),
                "dfa3d_dist_from_logits_backward launch");
}

// ---- encoder-layer row operations --------------------------------------------------------------
static int check_rows(int64_t rows, int32_t E) {
  if (rows < 0) return fail(DFA3D_ERR_INVALID_ARGUMENT, "rows must be >= 0 (got %lld)", (long long)rows);
  if (E <= 0) return fail(DFA3D_ERR_INVALID_ARGUMENT, "E must be positive (got %d)", E);
  if (E % 4 != 0 || E > dfa3d::layer_norm_max_columns())
    return fail(DFA3D_ERR_UNSUPPORTED, "E=%d: rows of a multiple of 4 columns up to %d are covered", E,
                dfa3d::layer_norm_max_columns());
  return DFA3D_OK;
}

int dfa3d_add_layer_norm_forward(const float *x, const float *residual, const float *gamma,
                                 const float *beta, int64_t rows, int32_t E, float eps, float *sum_out,
                                 float *y, float *mean, float *rstd, void *stream) {
  if (int rc = check_rows(rows, E)) return rc;
  if (!(eps >= 0.f)) return fail(DFA3D_ERR_INVALID_ARGUMENT, "eps must be >= 0");
  if ((residual == nullptr) != (sum_out == nullptr))
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "residual and sum_out must be given together or not at all");
  if (rows == 0) return DFA3D_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(gamma); REQUIRE_PTR(beta); REQUIRE_PTR(y); REQUIRE_PTR(mean); REQUIRE_PTR(rstd);
  REQUIRE_ALIGNED(x); REQUIRE_ALIGNED(residual); REQUIRE_ALIGNED(gamma); REQUIRE_ALIGNED(beta);
  REQUIRE_ALIGNED(sum_out); REQUIRE_ALIGNED(y);
  return finish(dfa3d::launch_add_layer_norm_forward(x, residual, gamma, beta, rows, E, eps, sum_out, y, mean,
                                                     rstd, (cudaStream_t)stream),
                "dfa3d_add_layer_norm_forward launch");
}

int dfa3d_layer_norm_backward(const float *grad_y, const float *in, const float *gamma,
                              const float *mean, const float *rstd, int64_t rows, int32_t E,
                              float *grad_in, float *grad_gamma, float *grad_beta, void *stream) {
  if (int rc = check_rows(rows, E)) return rc;
  if (rows == 0) return DFA3D_OK;
  REQUIRE_PTR(grad_y); REQUIRE_PTR(in); REQUIRE_PTR(gamma); REQUIRE_PTR(mean); REQUIRE_PTR(rstd);
  REQUIRE_PTR(grad_in); REQUIRE_PTR(grad_gamma); REQUIRE_PTR(grad_beta);
  REQUIRE_ALIGNED(grad_y); REQUIRE_ALIGNED(in); REQUIRE_ALIGNED(gamma); REQUIRE_ALIGNED(grad_in);
  REQUIRE_ALIGNED(grad_gamma); REQUIRE_ALIGNED(grad_beta);
  return finish(dfa3d::launch_layer_norm_backward(grad_y, in, gamma, mean, rstd, rows, E, grad_in, grad_gamma,
                                                  grad_beta, (cudaStream_t)stream),
                "dfa3d_layer_norm_backward launch");
}

int dfa3d_column_sum(const float *src, int64_t rows, int32_t cols, float *dst, void *stream) {
  if (rows < 0 || cols < 0)
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "rows and cols must be >= 0 (got %lld, %d)", (long long)rows, cols);
  if (cols % 4 != 0) return fail(DFA3D_ERR_UNSUPPORTED, "cols=%d must be a multiple of 4", cols);
  if (rows == 0 || cols == 0) return DFA3D_OK;
  REQUIRE_PTR(src); REQUIRE_PTR(dst);
  REQUIRE_ALIGNED(src); REQUIRE_ALIGNED(dst);
  return finish(dfa3d::launch_column_sum(src, rows, cols, dst, (cudaStream_t)stream), "dfa3d_column_sum launch");
}

// ---- double precision -------------------------------------------------------------------------
// Same checks as check_problem(); both dtype fields must say DFA3D_DTYPE_F64 and dist must be laid out
// like value (no single-map option in double).
static int check_problem64(const dfa3d_problem *p, bool need_value, bool need_dist) {
  if (!p) return fail(DFA3D_ERR_INVALID_ARGUMENT, "problem descriptor is null");
  if ((need_value && p->value_dtype != DFA3D_DTYPE_F64) || (need_dist && p->dist_dtype != DFA3D_DTYPE_F64))
    return fail(DFA3D_ERR_INVALID_ARGUMENT, "the *_f64 entry points take DFA3D_DTYPE_F64 tensors only");
  if (p->dist_map_h != 0 || p->dist_map_w != 0)
    return fail(DFA3D_ERR_UNSUPPORTED, "the single-map dist option is not available in double precision");
  dfa3d_problem q = *p;
  q.value_dtype = DFA3D_DTYPE_F32; q.dist_dtype = DFA3D_DTYPE_F32;   // the size checks are type-independent
  return check_problem(&q, need_value, need_dist);
}

int dfa3d_depth_score_forward_f64(const dfa3d_problem *p, const double *dist, const int64_t *shapes3,
                                  const int64_t *level_start, const double *loc3, double *depth_score,
                                  void *stream) {
  if (int rc = check_problem64(p, false, true)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start); REQUIRE_PTR(loc3);
  REQUIRE_PTR(depth_score);
  return finish(dfa3d::launch_depth_forward64(p, dist, shapes3, level_start, loc3, depth_score,
                                              (cudaStream_t)stream),
                "dfa3d_depth_score_forward_f64 launch");
}

int dfa3d_depth_score_backward_f64(const dfa3d_problem *p, const double *dist, const int64_t *shapes3,
                                   const int64_t *level_start, const double *loc3,
                                   const double *grad_depth_score, double *grad_dist, double *grad_loc3,
                                   void *stream) {
  if (int rc = check_problem64(p, false, true)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start); REQUIRE_PTR(loc3);
  REQUIRE_PTR(grad_depth_score); REQUIRE_PTR(grad_dist); REQUIRE_PTR(grad_loc3);
  return finish(dfa3d::launch_depth_backward64(p, dist, shapes3, level_start, loc3, grad_depth_score,
                                               grad_dist, grad_loc3, (cudaStream_t)stream),
                "dfa3d_depth_score_backward_f64 launch");
}

int dfa3d_wms_attn_forward_f64(const dfa3d_problem *p, const double *value, const int64_t *shapes2,
                               const int64_t *level_start, const double *loc2, const double *attn,
                               const double *depth_score, double *out, void *stream) {
  if (int rc = check_problem64(p, true, false)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(shapes2); REQUIRE_PTR(level_start); REQUIRE_PTR(loc2);
  REQUIRE_PTR(attn); REQUIRE_PTR(depth_score); REQUIRE_PTR(out);
  return finish(dfa3d::launch_forward64(p, value, nullptr, shapes2, 2, level_start, loc2, 2, attn,
                                        depth_score, false, out, nullptr, (cudaStream_t)stream),
                "dfa3d_wms_attn_forward_f64 launch");
}

int dfa3d_wms_attn_backward_f64(const dfa3d_problem *p, const double *value, const int64_t *shapes2,
                                const int64_t *level_start, const double *loc2, const double *attn,
                                const double *depth_score, const double *grad_out, double *grad_value,
                                double *grad_loc2, double *grad_attn, double *grad_depth_score,
                                void *stream) {
  if (int rc = check_problem64(p, true, false)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(shapes2); REQUIRE_PTR(level_start); REQUIRE_PTR(loc2);
  REQUIRE_PTR(attn); REQUIRE_PTR(depth_score); REQUIRE_PTR(grad_out); REQUIRE_PTR(grad_value);
  REQUIRE_PTR(grad_loc2); REQUIRE_PTR(grad_attn); REQUIRE_PTR(grad_depth_score);
  return finish(dfa3d::launch_backward64(p, value, nullptr, shapes2, 2, level_start, loc2, 2, attn,
                                         depth_score, false, grad_out, grad_value, nullptr, grad_loc2,
                                         grad_attn, grad_depth_score, (cudaStream_t)stream),
                "dfa3d_wms_attn_backward_f64 launch");
}

int dfa3d_fused_forward_f64(const dfa3d_problem *p, const double *value, const double *dist,
                            const int64_t *shapes3, const int64_t *level_start, const double *loc3,
                            const double *attn, double *out, double *depth_score_out, void *stream) {
  if (int rc = check_problem64(p, true, true)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start);
  REQUIRE_PTR(loc3); REQUIRE_PTR(attn); REQUIRE_PTR(out);
  return finish(dfa3d::launch_forward64(p, value, dist, shapes3, 3, level_start, loc3, 3, attn, nullptr,
                                        true, out, depth_score_out, (cudaStream_t)stream),
                "dfa3d_fused_forward_f64 launch");
}

int dfa3d_fused_backward_f64(const dfa3d_problem *p, const double *value, const double *dist,
                             const int64_t *shapes3, const int64_t *level_start, const double *loc3,
                             const double *attn, const double *grad_out, double *grad_value,
                             double *grad_dist, double *grad_loc3, double *grad_attn, void *stream) {
  if (int rc = check_problem64(p, true, true)) return rc;
  if (p->B == 0 || p->Q == 0) return DFA3D_OK;
  REQUIRE_PTR(value); REQUIRE_PTR(dist); REQUIRE_PTR(shapes3); REQUIRE_PTR(level_start);
  REQUIRE_PTR(loc3); REQUIRE_PTR(attn); REQUIRE_PTR(grad_out); REQUIRE_PTR(grad_value);
  REQUIRE_PTR(grad_dist); REQUIRE_PTR(grad_loc3); REQUIRE_PTR(grad_attn);
  return finish(dfa3d::launch_backward64(p, value, dist, shapes3, 3, level_start, loc3, 3, attn, nullptr,
                                         true, grad_out, grad_value, grad_dist, grad_loc3, grad_attn,
                                         nullptr, (cudaStream_t)stream),
                "dfa3d_fused_backward_f64 launch");
}

}  // extern "C"
