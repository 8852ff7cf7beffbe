// Memory-primitive rate probes for the DFA3D kernels (sm_100a) -- measurement code, not part of the
// operator.  Built into libdfa3d_rates.so, driven by dfa3d_b200/rates.py.
//
// A probe launch replays the ADDRESS STREAM of one operator launch -- one warp per (camera, query,
// head) item, 32 sampling points per item (L levels x P points, L*P = 32), per point the four
// bilinear corner rows of `value` / `grad_value` (128-byte rows, 8 heads x 32 fp32 channels per pixel)
// and the (z0, z0+1) pairs of the four corner pixels of `dist` / `grad_dist` -- with pseudo-random
// uniformly distributed corner positions and none of the operator's arithmetic.  The `ops` mask picks
// which memory operations are issued, so that each primitive can be timed alone and together:
//   GATHER_ROWS   16-byte loads, 8 lanes per value row, 4 rows per warp-wide request
//   RED_ROWS      red.global.add.v4.f32, 8 lanes per grad_value row
//   GATHER_PAIRS  one 8-byte load per lane and corner from dist (B, N, D)
//   RED_PAIRS     one red.global.add.v2.f32 per lane and corner into grad_dist (B, N, D)
//   GATHER_CELLS  two 16-byte loads per lane from the corner-interleaved copy of dist
//   RED_CELLS     two red.global.add.v4.f32 per lane into the corner-interleaved gradient
//   BULK_RED_ROWS rows staged in shared memory and added with cp.reduce.async.bulk (the TMA unit)
// `level_mask` restricts the points to some levels (bit l set = level l keeps its P points; points of
// the other levels are dropped), which shows the cost of many updates landing on few rows.
#include <cuda_runtime.h>
#include <stdint.h>

#include "dfa3d_rates.h"

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

struct Levels {
  int h[8], w[8], start[8], cell_start[8];
};

struct PArgs {
  const float *value;   // (B, N, 8, 32)
  float *grad_value;    // (B, N, 8, 32)
  const float *dist;    // (B, N, D)
  float *grad_dist;     // (B, N, D)
  const float *cells;   // (B, NC, D, 4): per 2x2 cell (y0, x0) of a level, per bin, its 4 corners
  float *grad_cells;    // (B, NC, D, 4)
  float *sink;          // one float per warp; written only if a sum turns out NaN (keeps loads alive)
  Levels lv;
  int L, P, N, NC, D, Q;
  int ops, level_mask;
  float dead_fraction;  // fraction of points outside the image (no memory operations at all)
};

__device__ __forceinline__ uint32_t mix(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

__device__ __forceinline__ void red_v4(float *p, float a) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %1, %1, %1};" ::"l"(p), "f"(a) : "memory");
}
__device__ __forceinline__ void red_v2(float *p, float a) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %1};" ::"l"(p), "f"(a) : "memory");
}

__global__ void __launch_bounds__(kThreads, 4) probe_kernel(const PArgs a) {
  __shared__ int rows[kWarps][128];
  __shared__ __align__(128) float stage[kWarps][2][16][32];   // bulk-reduction staging: 2 x 16 rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned idx = blockIdx.x * kWarps + warp;            // (query, head) of camera blockIdx.y
  if (idx >= (unsigned)a.Q * 8u) return;
  const int b = blockIdx.y, h = idx & 7;
  const long long item = (long long)b * a.Q * 8 + idx;

  // the lane's point: level, cell (y0, x0) in [-1, H-1] x [-1, W-1], lower depth bin z0 in [-1, D-1]
  const int l = lane / a.P;
  const uint32_t r0 = mix((uint32_t)(item * 32 + lane) * 2654435761u + 12345u);
  const uint32_t r1 = mix(r0 + 0x9e3779b9u), r2 = mix(r1 + 0x9e3779b9u);
  const int Hh = a.lv.h[l], W = a.lv.w[l];
  const int x0 = (int)(((uint64_t)r0 * (uint32_t)(W + 1)) >> 32) - 1;
  const int y0 = (int)(((uint64_t)r1 * (uint32_t)(Hh + 1)) >> 32) - 1;
  const int z0 = (int)(((uint64_t)(r2 >> 8) * (uint32_t)a.D) >> 24) - 1;   // -1 .. D-2 (both bins in range
  const int z0c = z0 < 0 ? 0 : z0;                                          //  except at the lower edge)
  const bool live = l < a.L && ((a.level_mask >> l) & 1) &&
                    (float)(r2 & 0xff) >= a.dead_fraction * 256.f;
  int pix[4];
  {
    const int base = a.lv.start[l] + y0 * W + x0;
    const bool xl = x0 >= 0, xh = x0 + 1 <= W - 1, yl = y0 >= 0, yh = y0 + 1 <= Hh - 1;
    pix[0] = live && yl && xl ? base : -1;
    pix[1] = live && yl && xh ? base + 1 : -1;
    pix[2] = live && yh && xh ? base + W + 1 : -1;
    pix[3] = live && yh && xl ? base + W : -1;
  }
  float sum = 0.f;

  // ---- depth-distribution operations: one lane = one point ----------------------------------
  if (a.ops & (DFA3D_RATE_GATHER_PAIRS | DFA3D_RATE_RED_PAIRS)) {
    const long long cam = (long long)b * a.N * a.D;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (pix[k] >= 0) {
        const long long o = cam + (long long)pix[k] * a.D + (z0c & ~1);     // 8-byte aligned pair
        if (a.ops & DFA3D_RATE_GATHER_PAIRS) {
          const float2 t = __ldg(reinterpret_cast<const float2 *>(a.dist + o));
          sum += t.x + t.y;
        }
        if (a.ops & DFA3D_RATE_RED_PAIRS) red_v2(a.grad_dist + o, 1.f);
      }
  }
  if ((a.ops & (DFA3D_RATE_GATHER_CELLS | DFA3D_RATE_RED_CELLS)) && live) {
    const int cell = a.lv.cell_start[l] + (y0 + 1) * (W + 1) + (x0 + 1);
    const long long o = ((long long)b * a.NC + cell) * a.D * 4 + z0c * 4;   // 16-byte aligned
    if (a.ops & DFA3D_RATE_GATHER_CELLS) {
      const float4 t0 = __ldg(reinterpret_cast<const float4 *>(a.cells + o));
      const float4 t1 = __ldg(reinterpret_cast<const float4 *>(a.cells + o + 4));
      sum += t0.x + t0.y + t0.z + t0.w + t1.x + t1.y + t1.z + t1.w;
    }
    if (a.ops & DFA3D_RATE_RED_CELLS) {
      red_v4(a.grad_cells + o, 1.f);
      red_v4(a.grad_cells + o + 4, 1.f);
    }
  }

  // ---- row operations: 8 lanes = one 128-byte row, 4 rows per warp-wide request ----------------
  if (a.ops & (DFA3D_RATE_GATHER_ROWS | DFA3D_RATE_RED_ROWS | DFA3D_RATE_BULK_RED_ROWS)) {
#pragma unroll
    for (int k = 0; k < 4; ++k) rows[warp][lane * 4 + k] = pix[k] >= 0 ? pix[k] * 256 : -1;
    __syncwarp();
    const int sub = lane & 7, grp = lane >> 3;
    const long long slice = ((long long)b * a.N * 8 + h) * 32 + sub * 4;
    const float *vbase = a.value + slice;
    float *gbase = a.grad_value + slice;
    if (a.ops & (DFA3D_RATE_GATHER_ROWS | DFA3D_RATE_RED_ROWS)) {
#pragma unroll 1
      for (int r = 0; r < 128; r += 16) {
        int off[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) off[u] = rows[warp][r + u * 4 + grp];
        if (a.ops & DFA3D_RATE_GATHER_ROWS) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (off[u] >= 0) {
              const float4 t = __ldg(reinterpret_cast<const float4 *>(vbase + off[u]));
              sum += t.x + t.y + t.z + t.w;
            }
        }
        if (a.ops & DFA3D_RATE_RED_ROWS) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (off[u] >= 0) red_v4(gbase + off[u], 1.f);
        }
      }
    }
    if (a.ops & DFA3D_RATE_BULK_RED_ROWS) {
      // 16 rows per batch: every lane writes its 16 bytes of 4 x 4 rows, then lanes 0..15 hand one
      // row each to the TMA unit; two staging buffers alternate
      float *gv_head = a.grad_value + ((long long)b * a.N * 8 + h) * 32;
      int buf = 0;
#pragma unroll 1
      for (int r = 0; r < 128; r += 16, buf ^= 1) {
        // the bulk operations that read this buffer two batches ago must have finished reading
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 4; ++u)
          *reinterpret_cast<float4 *>(&stage[warp][buf][u * 4 + grp][sub * 4]) =
              make_float4(1.f, 1.f, 1.f, 1.f);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane < 16) {
          const int off = rows[warp][r + lane];
          if (off >= 0) {
            const uint32_t src = (uint32_t)__cvta_generic_to_shared(&stage[warp][buf][lane][0]);
            asm volatile(
                "cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], 128;" ::"l"(
                    gv_head + off),
                "r"(src)
                : "memory");
          }
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  }
  if (sum != sum) a.sink[blockIdx.x * kWarps + warp] = sum;
}

}  // namespace

extern "C" int dfa3d_rate_probe(const dfa3d_rate_problem *p, const float *value, float *grad_value,
                                const float *dist, float *grad_dist, const float *cells,
                                float *grad_cells, float *sink, void *stream) {
  if (!p || p->L <= 0 || p->L > 8 || p->P <= 0 || p->L * p->P != 32 || p->B <= 0 || p->B > 65535 ||
      p->Q <= 0 || p->D < 2)
    return -1;
  PArgs a;
  a.value = value; a.grad_value = grad_value; a.dist = dist; a.grad_dist = grad_dist;
  a.cells = cells; a.grad_cells = grad_cells; a.sink = sink;
  int n = 0, nc = 0;
  for (int l = 0; l < 8; ++l) {
    const bool on = l < p->L;
    a.lv.h[l] = on ? p->level_h[l] : 1;
    a.lv.w[l] = on ? p->level_w[l] : 1;
    a.lv.start[l] = n;
    a.lv.cell_start[l] = nc;
    if (on) {
      n += p->level_h[l] * p->level_w[l];
      nc += (p->level_h[l] + 1) * (p->level_w[l] + 1);
    }
  }
  a.L = p->L; a.P = p->P; a.N = n; a.NC = nc; a.D = p->D; a.Q = p->Q;
  a.ops = p->ops; a.level_mask = p->level_mask; a.dead_fraction = p->dead_fraction;
  if ((a.ops & (DFA3D_RATE_GATHER_ROWS)) && !value) return -1;
  if ((a.ops & (DFA3D_RATE_RED_ROWS | DFA3D_RATE_BULK_RED_ROWS)) && !grad_value) return -1;
  if ((a.ops & DFA3D_RATE_GATHER_PAIRS) && !dist) return -1;
  if ((a.ops & DFA3D_RATE_RED_PAIRS) && !grad_dist) return -1;
  if ((a.ops & DFA3D_RATE_GATHER_CELLS) && !cells) return -1;
  if ((a.ops & DFA3D_RATE_RED_CELLS) && !grad_cells) return -1;
  if (!sink) return -1;
  const dim3 grid((unsigned)((p->Q * 8 + kWarps - 1) / kWarps), (unsigned)p->B, 1);
  probe_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int dfa3d_rate_sizes(const dfa3d_rate_problem *p, int64_t *pixels, int64_t *cells) {
  if (!p || p->L <= 0 || p->L > 8) return -1;
  int64_t n = 0, nc = 0;
  for (int l = 0; l < p->L; ++l) {
    n += (int64_t)p->level_h[l] * p->level_w[l];
    nc += (int64_t)(p->level_h[l] + 1) * (p->level_w[l] + 1);
  }
  *pixels = n; *cells = nc;
  return 0;
}
