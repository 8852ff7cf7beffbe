// Per-camera re-batching of BEV queries (sm_100a): which queries each camera sees, packed rows for
// exactly those queries (no padding to the longest camera), and the combination of the per-camera
// results back into BEV order.
//
// Replaces the Python loops, the `nonzero()` host synchronisations and the zero-padded
// (bs, cams, max_len, ...) tensors of SpatialCrossAttention_DFA3D.forward
// (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/spatial_cross_attention.py:700-722 and
// :741-748).  Semantics kept from there: camera i's query list is taken from batch element 0 of
// bev_mask (:703-705), in ascending query order; the divisor of the combination is the number of
// cameras that see the query in the SAME batch element, at least 1 (:745-748).
//
// Packed layout: batch element j, camera i, its r-th visible query sits in row
//   j * T + offsets[i] + r,     T = offsets[cams] = visible (camera, query) pairs of one batch element,
// which is also the order of the operator's "cameras" b = j * cams + i, so op_offsets[b] = j*T +
// offsets[i] is the operator's per-camera query offset table.
#include <stdint.h>

#include "dfa3d_b200.h"
#include "dfa3d_launch.h"

namespace dfa3d {
namespace {

constexpr int kPlanThreads = 1024;

__device__ __forceinline__ bool sees(const uint8_t *mask, long long base, int Z) {
  bool any = false;
  for (int z = 0; z < Z; ++z) any |= mask[base + z] != 0;
  return any;
}

// Exclusive prefix count of `flag` over the CTA (kPlanThreads threads); returns the CTA total in `total`.
__device__ __forceinline__ int block_exclusive_count(bool flag, int &total, int *warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned ballot = __ballot_sync(0xffffffffu, flag);
  const int in_warp = __popc(ballot & ((1u << lane) - 1u));
  if (lane == 0) warp_sums[warp] = __popc(ballot);
  __syncthreads();
  int before = 0, all = 0;
  for (int w = 0; w < kPlanThreads / 32; ++w) {
    const int s = warp_sums[w];
    before += w < warp ? s : 0;
    all += s;
  }
  __syncthreads();
  total = all;
  return before + in_warp;
}

// One CTA per camera: number of queries the camera sees (batch element 0).
__global__ void __launch_bounds__(kPlanThreads)
rebatch_count_kernel(const uint8_t *mask, int bs, int Q, int Z, int32_t *counts) {
  __shared__ int warp_sums[kPlanThreads / 32];
  const int cam = blockIdx.x;
  int running = 0;
  for (int q0 = 0; q0 < Q; q0 += kPlanThreads) {
    const int q = q0 + threadIdx.x;
    const bool f = q < Q && sees(mask, ((long long)cam * bs * Q + q) * Z, Z);
    int total;
    block_exclusive_count(f, total, warp_sums);
    running += total;
  }
  if (threadIdx.x == 0) counts[cam] = running;
}

// One warp: offsets[i] = sum of counts[< i]; op_offsets[j*cams + i] = j*T + offsets[i].
__global__ void rebatch_offsets_kernel(const int32_t *counts, int cams, int bs, int32_t *offsets,
                                       int32_t *op_offsets) {
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < cams; ++i) { offsets[i] = run; run += counts[i]; }
    offsets[cams] = run;
  }
  __syncwarp();
  const int T = offsets[cams];
  for (int b = threadIdx.x; b <= cams * bs; b += 32)
    op_offsets[b] = b == cams * bs ? bs * T : (b / cams) * T + offsets[b % cams];
}

// One CTA per camera: fill packed_query / packed_camera and the inverse map row_of.
__global__ void __launch_bounds__(kPlanThreads)
rebatch_fill_kernel(const uint8_t *mask, int bs, int Q, int Z, const int32_t *offsets,
                    int32_t *packed_query, int32_t *packed_camera, int32_t *row_of) {
  __shared__ int warp_sums[kPlanThreads / 32];
  const int cam = blockIdx.x;
  int running = offsets[cam];
  for (int q0 = 0; q0 < Q; q0 += kPlanThreads) {
    const int q = q0 + threadIdx.x;
    const bool f = q < Q && sees(mask, ((long long)cam * bs * Q + q) * Z, Z);
    int total;
    const int pos = running + block_exclusive_count(f, total, warp_sums);
    if (f) { packed_query[pos] = q; packed_camera[pos] = cam; }
    if (q < Q) row_of[(long long)cam * Q + q] = f ? pos : -1;
    running += total;
  }
}

// inv_count[j, q] = 1 / max(1, number of cameras that see q in batch element j).
__global__ void rebatch_inv_count_kernel(const uint8_t *mask, int cams, int bs, int Q, int Z,
                                         float *inv_count) {
  const long long n = (long long)bs * Q;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n;
       t += (long long)gridDim.x * blockDim.x) {
    int c = 0;
    for (int i = 0; i < cams; ++i) c += sees(mask, ((long long)i * bs * Q + t) * Z, Z) ? 1 : 0;
    inv_count[t] = 1.f / (float)(c < 1 ? 1 : c);
  }
}

// dst[j*T + p, :] = scale[j, q] * src[cam*cam_stride + j*batch_stride + q, :],  q = packed_query[p],
// cam = packed_camera[p].  VEC = 4: rows of W floats handled as float4 (W % 4 == 0, aligned bases).
template <int VEC>
__global__ void __launch_bounds__(256)
rebatch_gather_kernel(const float *src, const int32_t *packed_query, const int32_t *packed_camera,
                      const int32_t *offsets, int cams, int bs, int Q, int W, long long cam_stride,
                      long long batch_stride, const float *scale, float *dst) {
  const int T = offsets[cams];
  const int wv = W / VEC;
  const long long n = (long long)bs * T * wv;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n;
       t += (long long)gridDim.x * blockDim.x) {
    const long long row = t / wv;
    const int v = (int)(t - row * wv);
    const int j = (int)(row / T), p = (int)(row - (long long)j * T);
    const int q = packed_query[p], cam = packed_camera[p];
    const float s = scale ? scale[(long long)j * Q + q] : 1.f;
    const float *sp = src + ((long long)cam * cam_stride + (long long)j * batch_stride + q) * W;
    if (VEC == 4) {
      float4 x = __ldg(reinterpret_cast<const float4 *>(sp) + v);
      x.x *= s; x.y *= s; x.z *= s; x.w *= s;
      reinterpret_cast<float4 *>(dst + row * W)[v] = x;
    } else {
      dst[row * W + v] = s * __ldg(sp + v);
    }
  }
}

// dst[j, q, :] = scale[j, q] * sum over cameras i that see q of src[j*T + row_of[i, q], :]
// (every element of dst is written: queries no camera sees get zeros).
template <int VEC>
__global__ void __launch_bounds__(256)
rebatch_combine_kernel(const float *src, const int32_t *row_of, const int32_t *offsets, int cams,
                       int bs, int Q, int W, const float *scale, float *dst) {
  const int T = offsets[cams];
  const int wv = W / VEC;
  const long long n = (long long)bs * Q * wv;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n;
       t += (long long)gridDim.x * blockDim.x) {
    const long long jq = t / wv;
    const int v = (int)(t - jq * wv);
    const int j = (int)(jq / Q), q = (int)(jq - (long long)j * Q);
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    // eight cameras at a time: their row indices first, then the rows, so that the loads of one thread
    // overlap instead of forming an index -> row chain per camera
    for (int cam0 = 0; cam0 < cams; cam0 += 8) {
      int r[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) r[i] = cam0 + i < cams ? __ldg(row_of + (long long)(cam0 + i) * Q + q) : -1;
      if (VEC == 4) {
        float4 x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          x[i] = r[i] >= 0 ? __ldg(reinterpret_cast<const float4 *>(src + ((long long)j * T + r[i]) * W) + v)
                           : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; ++i) { acc[0] += x[i].x; acc[1] += x[i].y; acc[2] += x[i].z; acc[3] += x[i].w; }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (r[i] >= 0) acc[0] += __ldg(src + ((long long)j * T + r[i]) * W + v);
      }
    }
    const float s = scale ? scale[jq] : 1.f;
    if (VEC == 4)
      reinterpret_cast<float4 *>(dst + jq * W)[v] = make_float4(s * acc[0], s * acc[1], s * acc[2], s * acc[3]);
    else
      dst[jq * W + v] = s * acc[0];
  }
}

unsigned grid_for(long long n, int threads) {
  long long g = (n + threads - 1) / threads;
  const long long cap = 148LL * 16;
  return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

bool vec4_ok(const void *a, const void *b, int W) {
  return W % 4 == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15u) == 0;
}

}  // namespace

cudaError_t launch_rebatch_plan(const uint8_t *mask, int cams, int bs, int Q, int Z, int32_t *counts,
                                int32_t *offsets, int32_t *op_offsets, int32_t *packed_query,
                                int32_t *packed_camera, int32_t *row_of, float *inv_count,
                                cudaStream_t s) {
  rebatch_count_kernel<<<cams, kPlanThreads, 0, s>>>(mask, bs, Q, Z, counts);
  rebatch_offsets_kernel<<<1, 32, 0, s>>>(counts, cams, bs, offsets, op_offsets);
  rebatch_fill_kernel<<<cams, kPlanThreads, 0, s>>>(mask, bs, Q, Z, offsets, packed_query, packed_camera,
                                                    row_of);
  rebatch_inv_count_kernel<<<grid_for((long long)bs * Q, 256), 256, 0, s>>>(mask, cams, bs, Q, Z,
                                                                            inv_count);
  return cudaGetLastError();
}

cudaError_t launch_rebatch_gather(const float *src, const int32_t *packed_query,
                                  const int32_t *packed_camera, const int32_t *offsets, int cams, int bs,
                                  int Q, int W, long long cam_stride, long long batch_stride,
                                  const float *scale, float *dst, long long rows_bound, cudaStream_t s) {
  if (rows_bound <= 0) return cudaSuccess;
  if (vec4_ok(src, dst, W))
    rebatch_gather_kernel<4><<<grid_for(rows_bound * (W / 4), 256), 256, 0, s>>>(
        src, packed_query, packed_camera, offsets, cams, bs, Q, W, cam_stride, batch_stride, scale, dst);
  else
    rebatch_gather_kernel<1><<<grid_for(rows_bound * W, 256), 256, 0, s>>>(
        src, packed_query, packed_camera, offsets, cams, bs, Q, W, cam_stride, batch_stride, scale, dst);
  return cudaGetLastError();
}

cudaError_t launch_rebatch_combine(const float *src, const int32_t *row_of, const int32_t *offsets,
                                   int cams, int bs, int Q, int W, const float *scale, float *dst,
                                   cudaStream_t s) {
  if ((long long)bs * Q <= 0) return cudaSuccess;
  if (vec4_ok(src, dst, W))
    rebatch_combine_kernel<4><<<grid_for((long long)bs * Q * (W / 4), 256), 256, 0, s>>>(
        src, row_of, offsets, cams, bs, Q, W, scale, dst);
  else
    rebatch_combine_kernel<1><<<grid_for((long long)bs * Q * W, 256), 256, 0, s>>>(
        src, row_of, offsets, cams, bs, Q, W, scale, dst);
  return cudaGetLastError();
}

}  // namespace dfa3d
