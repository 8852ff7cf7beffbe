// Producer of the depth distribution in the operator's layout (sm_100a).
//
// The depth network ends in a (B, D, hs, ws) map of logits.  The reference turns it into what the
// attention reads in four steps, each a pass over HBM: softmax (or sigmoid) over the D channels
// (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/dense_heads/depth_head.py:265-268), one
// F.interpolate(mode="nearest") per feature level (:273-276), flatten + permute + cat of the levels
// (…/modules/transformer.py:368-391) and the permute to (bs*cams, sum hw, D) of the spatial
// cross-attention (spatial_cross_attention.py:727-728).  Here one kernel reads the logits once and
// writes dist (B, N, D) -- fp32, bf16 or fp16 -- for all levels, channel-last; its backward reads the
// gradient of that tensor and the logits once and writes the gradient of the logits.
//
// Nearest resize, as torch computes it: source index = min(floor(dst * scale), size - 1) with
// scale = (float)source size / (float)level size.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "dfa3d_b200.h"
#include "dfa3d_launch.h"

namespace dfa3d {
namespace {

constexpr int kTile = 32;          // destination (forward) / source (backward) pixels per CTA
constexpr int kMaxBins = 256;      // D limit of the shared-memory tile
constexpr int kProdThreads = 256;

struct ProdArgs {
  const float *logits;      // (B, D, hs, ws)
  const int64_t *shapes;    // (L, shape_stride) int64: (h, w, ...) per level
  const int64_t *lsi;       // (L) int64
  void *dist;               // (B, N, D) fp32 | bf16 | fp16
  const float *grad_dist;   // (B, N, D) fp32
  float *grad_logits;       // (B, D, hs, ws)
  int B, D, hs, ws, N, L, shape_stride;
  int sigmoid;              // 0: softmax over D, 1: element-wise sigmoid
};

__device__ __forceinline__ int nearest_src(int dst, float scale, int size) {
  return min((int)floorf((float)dst * scale), size - 1);
}

__device__ __forceinline__ void store_bin(float *p, float v) { *p = v; }
__device__ __forceinline__ void store_bin(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void store_bin(__half *p, float v) { *p = __float2half_rn(v); }

// Forward: a CTA owns kTile consecutive rows n of one camera.  The logits of their source pixels are
// staged transposed in shared memory (loads run along the map's x axis: coalesced where the level has
// the map's width); each warp then normalises whole pixels and writes their D contiguous bins.
template <typename OT>
__global__ void __launch_bounds__(kProdThreads)
dist_from_logits_kernel(const ProdArgs a) {
  __shared__ float tile[kMaxBins][kTile + 1];
  __shared__ int src_off[kTile];
  const int b = blockIdx.y;
  const int n0 = blockIdx.x * kTile;
  if (threadIdx.x < kTile) {
    const int n = n0 + threadIdx.x;
    int off = -1;
    if (n < a.N) {
      int l = 0;
      while (l + 1 < a.L && n >= (int)a.lsi[l + 1]) ++l;
      const int h = (int)a.shapes[l * a.shape_stride], w = (int)a.shapes[l * a.shape_stride + 1];
      const int r = n - (int)a.lsi[l];
      const int y = r / w, x = r - y * w;
      if (y < h)
        off = nearest_src(y, (float)a.hs / (float)h, a.hs) * a.ws + nearest_src(x, (float)a.ws / (float)w, a.ws);
    }
    src_off[threadIdx.x] = off;
  }
  __syncthreads();
  const long long plane = (long long)a.hs * a.ws;
  const float *lg = a.logits + (long long)b * a.D * plane;
  for (int t = threadIdx.x; t < a.D * kTile; t += kProdThreads) {
    const int d = t / kTile, i = t - d * kTile;
    const int off = src_off[i];
    tile[d][i] = off >= 0 ? __ldg(lg + d * plane + off) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  OT *out = reinterpret_cast<OT *>(a.dist) + ((long long)b * a.N + n0) * a.D;
  for (int i = warp; i < kTile; i += kProdThreads / 32) {
    if (src_off[i] < 0) continue;
    if (a.sigmoid) {
      for (int d = lane; d < a.D; d += 32) store_bin(out + (long long)i * a.D + d, 1.f / (1.f + expf(-tile[d][i])));
      continue;
    }
    float mx = -INFINITY;
    for (int d = lane; d < a.D; d += 32) mx = fmaxf(mx, tile[d][i]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float sum = 0.f;
    for (int d = lane; d < a.D; d += 32) sum += expf(tile[d][i] - mx);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    for (int d = lane; d < a.D; d += 32)
      store_bin(out + (long long)i * a.D + d, __fdiv_rn(expf(tile[d][i] - mx), sum));
  }
}

// Backward: a CTA owns kTile consecutive map pixels of one map row.  Per pixel a warp recomputes the
// normalised bins p from the logits, sums the incoming gradient over every level pixel that the resize
// mapped to this map pixel (G), and forms p * (G - <p, G>) (softmax) or p * (1 - p) * G (sigmoid).
// Results go through shared memory so that the stores run along x.
__global__ void __launch_bounds__(kProdThreads)
dist_from_logits_backward_kernel(const ProdArgs a) {
  __shared__ float tile[kMaxBins][kTile + 1];
  const int b = blockIdx.z, sy = blockIdx.y, sx0 = blockIdx.x * kTile;
  const long long plane = (long long)a.hs * a.ws;
  const float *lg = a.logits + (long long)b * a.D * plane + (long long)sy * a.ws;
  for (int t = threadIdx.x; t < a.D * kTile; t += kProdThreads) {
    const int d = t / kTile, i = t - d * kTile;
    tile[d][i] = sx0 + i < a.ws ? __ldg(lg + d * plane + sx0 + i) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = warp; i < kTile; i += kProdThreads / 32) {
    const int sx = sx0 + i;
    if (sx >= a.ws) continue;            // warp-uniform
    // p in registers: D <= kMaxBins -> at most kMaxBins/32 bins per lane
    float p[kMaxBins / 32], G[kMaxBins / 32];
    float mx = -INFINITY;
    for (int d = lane; d < a.D; d += 32) mx = fmaxf(mx, tile[d][i]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxBins / 32; ++j) {
      const int d = lane + 32 * j;
      p[j] = 0.f; G[j] = 0.f;
      if (d < a.D) {
        p[j] = a.sigmoid ? 1.f / (1.f + expf(-tile[d][i])) : expf(tile[d][i] - mx);
        sum += p[j];
      }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    if (!a.sigmoid) {
#pragma unroll
      for (int j = 0; j < kMaxBins / 32; ++j) p[j] = __fdiv_rn(p[j], sum);
    }
    // every level pixel (y, x) whose nearest source is (sy, sx)
    for (int l = 0; l < a.L; ++l) {
      const int h = (int)a.shapes[l * a.shape_stride], w = (int)a.shapes[l * a.shape_stride + 1];
      const float scy = (float)a.hs / (float)h, scx = (float)a.ws / (float)w;
      // candidates start a little below sy / scale; the map is monotone, so walk up until it passes
      int y = max(0, (int)((float)sy / scy) - 2);
      while (y < h && nearest_src(y, scy, a.hs) < sy) ++y;
      for (; y < h && nearest_src(y, scy, a.hs) == sy; ++y) {
        int x = max(0, (int)((float)sx / scx) - 2);
        while (x < w && nearest_src(x, scx, a.ws) < sx) ++x;
        for (; x < w && nearest_src(x, scx, a.ws) == sx; ++x) {
          const float *g = a.grad_dist + ((long long)b * a.N + (int)a.lsi[l] + y * w + x) * a.D;
#pragma unroll
          for (int j = 0; j < kMaxBins / 32; ++j) {
            const int d = lane + 32 * j;
            if (d < a.D) G[j] += __ldg(g + d);
          }
        }
      }
    }
    float pg = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxBins / 32; ++j) pg = fmaf(p[j], G[j], pg);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) pg += __shfl_xor_sync(0xffffffffu, pg, s);
#pragma unroll
    for (int j = 0; j < kMaxBins / 32; ++j) {
      const int d = lane + 32 * j;
      if (d < a.D) tile[d][i] = a.sigmoid ? p[j] * (1.f - p[j]) * G[j] : p[j] * (G[j] - pg);
    }
  }
  __syncthreads();
  float *gl = a.grad_logits + (long long)b * a.D * plane + (long long)sy * a.ws;
  for (int t = threadIdx.x; t < a.D * kTile; t += kProdThreads) {
    const int d = t / kTile, i = t - d * kTile;
    if (sx0 + i < a.ws) gl[d * plane + sx0 + i] = tile[d][i];
  }
}

}  // namespace

int dist_producer_max_bins() { return kMaxBins; }

cudaError_t launch_dist_from_logits(const float *logits, const int64_t *shapes, int shape_stride,
                                    const int64_t *lsi, void *dist, int dist_dtype, int B, int D, int hs,
                                    int ws, int N, int L, bool sigmoid, cudaStream_t s) {
  if (B == 0 || N == 0) return cudaSuccess;
  ProdArgs a{};
  a.logits = logits; a.shapes = shapes; a.lsi = lsi; a.dist = dist;
  a.B = B; a.D = D; a.hs = hs; a.ws = ws; a.N = N; a.L = L; a.shape_stride = shape_stride;
  a.sigmoid = sigmoid ? 1 : 0;
  for (int b0 = 0; b0 < B; b0 += 65535) {
    ProdArgs c = a;
    c.logits = logits + (long long)b0 * D * hs * ws;
    c.dist = static_cast<char *>(dist) + (long long)b0 * N * D * (dist_dtype == 0 ? 4 : 2);
    const dim3 grid((unsigned)((N + kTile - 1) / kTile), (unsigned)min(65535, B - b0), 1);
    if (dist_dtype == 3) dist_from_logits_kernel<__half><<<grid, kProdThreads, 0, s>>>(c);
    else if (dist_dtype == 1) dist_from_logits_kernel<__nv_bfloat16><<<grid, kProdThreads, 0, s>>>(c);
    else dist_from_logits_kernel<float><<<grid, kProdThreads, 0, s>>>(c);
  }
  return cudaGetLastError();
}

cudaError_t launch_dist_from_logits_backward(const float *logits, const int64_t *shapes, int shape_stride,
                                             const int64_t *lsi, const float *grad_dist,
                                             float *grad_logits, int B, int D, int hs, int ws, int N,
                                             int L, bool sigmoid, cudaStream_t s) {
  if (B == 0 || hs == 0 || ws == 0) return cudaSuccess;
  ProdArgs a{};
  a.logits = logits; a.shapes = shapes; a.lsi = lsi; a.grad_dist = grad_dist; a.grad_logits = grad_logits;
  a.B = B; a.D = D; a.hs = hs; a.ws = ws; a.N = N; a.L = L; a.shape_stride = shape_stride;
  a.sigmoid = sigmoid ? 1 : 0;
  for (int b0 = 0; b0 < B; b0 += 65535) {
    ProdArgs c = a;
    c.logits = logits + (long long)b0 * D * hs * ws;
    c.grad_logits = grad_logits + (long long)b0 * D * hs * ws;
    c.grad_dist = grad_dist + (long long)b0 * N * D;
    const dim3 grid((unsigned)((ws + kTile - 1) / kTile), (unsigned)hs, (unsigned)min(65535, B - b0));
    dist_from_logits_backward_kernel<<<grid, kProdThreads, 0, s>>>(c);
  }
  return cudaGetLastError();
}

}  // namespace dfa3d
