// Row-wise helpers of the encoder layer that surrounds the attention operator (sm_100a):
//
//   * residual add + LayerNorm, forward and backward.  The layer applies `norm(x + branch(x))` after
//     each of its blocks (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/encoder.py:363-411:
//     operation order self_attn, norm, cross_attn, norm, ffn, norm); one kernel reads both summands,
//     writes the sum (the backward needs it) and the normalised rows.
//   * column sums of a (rows, cols) matrix: the bias gradient of a Linear layer.
//
// All three are bound by HBM: every operand is read once and every result written once.  A warp owns a
// row (LayerNorm) or a CTA a band of rows (column sums); per-column results that are summed over rows
// (grad_gamma, grad_beta, the column sums) are accumulated in registers over a CTA's rows, combined in
// shared memory and added to the caller-zeroed output with one `red.global.add.f32` per column and CTA.
#include <stdint.h>

#include "dfa3d_launch.h"

namespace dfa3d {
namespace {

constexpr int kLnWarps = 8;
constexpr int kLnThreads = kLnWarps * 32;
constexpr int kCtasPerSm = 4;
constexpr int kSms = 148;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float4 ld4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
// Streaming variants for data touched once.
__device__ __forceinline__ float4 ld4_stream(const float *p) { return __ldcs(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }

// One 16-byte vector reduction into global memory (sm_90+).
__device__ __forceinline__ void red_add_v4(float *addr, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

// Rows of E columns, E a multiple of 4 with 128 * (K - 1) < E <= 128 * K; lane l holds the float4 groups
// l, l + 32, ... of its row (groups at or beyond E are idle).
template <int K>
__global__ void __launch_bounds__(kLnThreads, K <= 4 ? kCtasPerSm : 2)
add_layer_norm_forward_kernel(const float *__restrict__ x, const float *__restrict__ residual,
                              const float *__restrict__ gamma, const float *__restrict__ beta,
                              long long rows, int E, float eps, float *__restrict__ sum_out,
                              float *__restrict__ y, float *__restrict__ mean_out,
                              float *__restrict__ rstd_out) {
  const float inv_e = 1.f / (float)E;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  const long long stride = (long long)gridDim.x * kLnWarps;
  for (long long row = warp0; row < rows; row += stride) {
    const float *xr = x + row * E;
    float4 v[K];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int c = (lane + 32 * j) * 4;
      v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c >= E) continue;
      v[j] = ld4_stream(xr + c);
      if (residual) {
        const float4 r = ld4_stream(residual + row * E + c);
        v[j].x += r.x; v[j].y += r.y; v[j].z += r.z; v[j].w += r.w;
      }
      s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = warp_sum(s) * inv_e;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if ((lane + 32 * j) * 4 >= E) continue;
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
      q += (a * a + b * b) + (c * c + d * d);
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_e + eps);
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int c = (lane + 32 * j) * 4;
      if (c >= E) continue;
      if (sum_out) st4(sum_out + row * E + c, v[j]);
      const float4 g = ld4(gamma + c), b = ld4(beta + c);
      float4 o;
      o.x = (v[j].x - mean) * rstd * g.x + b.x;
      o.y = (v[j].y - mean) * rstd * g.y + b.y;
      o.z = (v[j].z - mean) * rstd * g.z + b.z;
      o.w = (v[j].w - mean) * rstd * g.w + b.w;
      st4(y + row * E + c, o);
    }
    if (lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
  }
}

// grad_in = rstd * (g*gamma - mean(g*gamma) - xhat * mean(g*gamma*xhat)); grad_gamma += g*xhat;
// grad_beta += g, both summed over rows.
template <int K>
__global__ void __launch_bounds__(kLnThreads, K <= 1 ? kCtasPerSm : (K == 2 ? 3 : (K <= 4 ? 2 : 1)))
layer_norm_backward_kernel(const float *__restrict__ grad_y, const float *__restrict__ in,
                           const float *__restrict__ gamma, const float *__restrict__ mean_in,
                           const float *__restrict__ rstd_in, long long rows, int E,
                           float *__restrict__ grad_in, float *__restrict__ grad_gamma,
                           float *__restrict__ grad_beta) {
  const float inv_e = 1.f / (float)E;
  __shared__ float4 part[kLnWarps][32 * K];      // one warp's per-column partial sums
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * kLnWarps + warp;
  const long long stride = (long long)gridDim.x * kLnWarps;
  float4 dg[K], db[K];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    dg[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    db[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // R rows of a warp are in flight together (narrow rows leave registers for it): their loads are issued
  // before any of them is reduced
  constexpr int R = K <= 2 ? 2 : 1;
  for (long long row0 = warp0; row0 < rows; row0 += stride * R) {
    float4 g[R][K], xh[R][K];
    float mean[R], rstd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long long row = row0 + r * stride;
      const bool live = row < rows;
      mean[r] = live ? __ldg(mean_in + row) : 0.f;
      rstd[r] = live ? __ldg(rstd_in + row) : 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const int c = (lane + 32 * j) * 4;
        g[r][j] = make_float4(0.f, 0.f, 0.f, 0.f);
        xh[r][j] = g[r][j];
        if (live && c < E) {
          g[r][j] = ld4_stream(grad_y + row * E + c);
          xh[r][j] = ld4_stream(in + row * E + c);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long long row = row0 + r * stride;
      if (row >= rows) break;
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const int c = (lane + 32 * j) * 4;
        if (c >= E) continue;
        float4 &G = g[r][j], &X = xh[r][j];
        X = make_float4((X.x - mean[r]) * rstd[r], (X.y - mean[r]) * rstd[r], (X.z - mean[r]) * rstd[r],
                        (X.w - mean[r]) * rstd[r]);
        dg[j].x += G.x * X.x; dg[j].y += G.y * X.y; dg[j].z += G.z * X.z; dg[j].w += G.w * X.w;
        db[j].x += G.x; db[j].y += G.y; db[j].z += G.z; db[j].w += G.w;
        const float4 gam = ld4(gamma + c);
        G.x *= gam.x; G.y *= gam.y; G.z *= gam.z; G.w *= gam.w;
        s1 += (G.x + G.y) + (G.z + G.w);
        s2 += (G.x * X.x + G.y * X.y) + (G.z * X.z + G.w * X.w);
      }
      const float c1 = warp_sum(s1) * inv_e, c2 = warp_sum(s2) * inv_e;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const int c = (lane + 32 * j) * 4;
        if (c >= E) continue;
        const float4 G = g[r][j], X = xh[r][j];
        float4 o;
        o.x = rstd[r] * (G.x - c1 - X.x * c2);
        o.y = rstd[r] * (G.y - c1 - X.y * c2);
        o.z = rstd[r] * (G.z - c1 - X.z * c2);
        o.w = rstd[r] * (G.w - c1 - X.w * c2);
        st4(grad_in + row * E + c, o);
      }
    }
  }
  // combine the CTA's warps, then one reduction per column and CTA; gamma first, beta second
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
    for (int j = 0; j < K; ++j) part[warp][lane + 32 * j] = pass == 0 ? dg[j] : db[j];
    __syncthreads();
    float *dst = pass == 0 ? grad_gamma : grad_beta;
    for (int c4 = threadIdx.x; c4 * 4 < E; c4 += kLnThreads) {
      float4 t = part[0][c4];
#pragma unroll
      for (int w = 1; w < kLnWarps; ++w) {
        const float4 u = part[w][c4];
        t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
      }
      red_add_v4(dst + c4 * 4, t);
    }
    __syncthreads();
  }
}

// Column sums: a CTA is 64 float4 column groups x 8 row lanes; blockIdx.y picks the band of 256 columns,
// blockIdx.x the rows (grid-strided).  dst is accumulated into (caller-zeroed).  Few, long-lived CTAs: every
// CTA ends with one vector reduction per column group into the same few sectors of dst, and those
// serialise in L2.
constexpr int kCsGroups = 64, kCsLanes = 8, kCsThreads = kCsGroups * kCsLanes;

__global__ void __launch_bounds__(kCsThreads)
column_sum_kernel(const float *__restrict__ src, long long rows, int cols, float *__restrict__ dst) {
  __shared__ float4 part[kCsLanes][kCsGroups];
  const int grp = threadIdx.x % kCsGroups, rl = threadIdx.x / kCsGroups;
  const int col = (blockIdx.y * kCsGroups + grp) * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (col < cols) {
    const long long step = (long long)gridDim.x * kCsLanes;
    long long r = (long long)blockIdx.x * kCsLanes + rl;
    // four independent loads in flight per thread
    for (; r + 3 * step < rows; r += 4 * step) {
      const float4 a = ld4_stream(src + r * cols + col), b = ld4_stream(src + (r + step) * cols + col);
      const float4 c = ld4_stream(src + (r + 2 * step) * cols + col);
      const float4 d = ld4_stream(src + (r + 3 * step) * cols + col);
      acc.x += (a.x + b.x) + (c.x + d.x); acc.y += (a.y + b.y) + (c.y + d.y);
      acc.z += (a.z + b.z) + (c.z + d.z); acc.w += (a.w + b.w) + (c.w + d.w);
    }
    for (; r < rows; r += step) {
      const float4 a = ld4_stream(src + r * cols + col);
      acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
    }
  }
  part[rl][grp] = acc;
  __syncthreads();
  if (rl == 0 && col < cols) {
    float4 t = part[0][grp];
#pragma unroll
    for (int i = 1; i < kCsLanes; ++i) {
      t.x += part[i][grp].x; t.y += part[i][grp].y; t.z += part[i][grp].z; t.w += part[i][grp].w;
    }
    red_add_v4(dst + col, t);
  }
}

unsigned row_grid(long long rows) {
  const long long want = (rows + kLnWarps - 1) / kLnWarps;
  const long long cap = (long long)kSms * kCtasPerSm;
  return (unsigned)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace

int layer_norm_max_columns() { return 1024; }

cudaError_t launch_add_layer_norm_forward(const float *x, const float *residual, const float *gamma,
                                          const float *beta, long long rows, int E, float eps,
                                          float *sum_out, float *y, float *mean, float *rstd,
                                          cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  const unsigned grid = row_grid(rows);
#define DFA3D_LN_FWD(K)                                                                              \
  case K:                                                                                            \
    add_layer_norm_forward_kernel<K><<<grid, kLnThreads, 0, s>>>(x, residual, gamma, beta, rows, E,  \
                                                                 eps, sum_out, y, mean, rstd);       \
    break;
  switch ((E + 127) / 128) {
    DFA3D_LN_FWD(1) DFA3D_LN_FWD(2) DFA3D_LN_FWD(3) DFA3D_LN_FWD(4)
    DFA3D_LN_FWD(5) DFA3D_LN_FWD(6) DFA3D_LN_FWD(7) DFA3D_LN_FWD(8)
    default: return cudaErrorInvalidValue;
  }
#undef DFA3D_LN_FWD
  return cudaGetLastError();
}

cudaError_t launch_layer_norm_backward(const float *grad_y, const float *in, const float *gamma,
                                       const float *mean, const float *rstd, long long rows, int E,
                                       float *grad_in, float *grad_gamma, float *grad_beta,
                                       cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  // as many CTAs as are resident at once (the kernel's launch bounds), each with at least 8 rows per warp:
  // every CTA ends with E/4 vector reductions per output
  const int K = (E + 127) / 128;
  const long long want = (rows + kLnWarps * 8 - 1) / (kLnWarps * 8);
  const long long cap = (long long)kSms * (K <= 1 ? kCtasPerSm : (K == 2 ? 3 : (K <= 4 ? 2 : 1)));
  const unsigned grid = (unsigned)(want < cap ? (want > 0 ? want : 1) : cap);
#define DFA3D_LN_BWD(K)                                                                               \
  case K:                                                                                             \
    layer_norm_backward_kernel<K><<<grid, kLnThreads, 0, s>>>(grad_y, in, gamma, mean, rstd, rows, E,  \
                                                              grad_in, grad_gamma, grad_beta);        \
    break;
  switch (K) {
    DFA3D_LN_BWD(1) DFA3D_LN_BWD(2) DFA3D_LN_BWD(3) DFA3D_LN_BWD(4)
    DFA3D_LN_BWD(5) DFA3D_LN_BWD(6) DFA3D_LN_BWD(7) DFA3D_LN_BWD(8)
    default: return cudaErrorInvalidValue;
  }
#undef DFA3D_LN_BWD
  return cudaGetLastError();
}

cudaError_t launch_column_sum(const float *src, long long rows, int cols, float *dst, cudaStream_t s) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  const unsigned bands = (unsigned)((cols / 4 + kCsGroups - 1) / kCsGroups);
  long long gx = (long long)kSms * 2 / bands;                            // two 512-thread CTAs per SM
  const long long most = (rows + kCsLanes * 8 - 1) / (kCsLanes * 8);     // at least 8 rows per thread
  if (gx > most) gx = most;
  if (gx < 1) gx = 1;
  column_sum_kernel<<<dim3((unsigned)gx, bands, 1), kCsThreads, 0, s>>>(src, rows, cols, dst);
  return cudaGetLastError();
}

}  // namespace dfa3d
