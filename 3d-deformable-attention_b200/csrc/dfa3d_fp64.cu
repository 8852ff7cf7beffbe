// Double-precision DFA3D kernels (sm_100a).
//
// The reference instantiates its kernels for float and double (AT_DISPATCH_FLOATING_TYPES in
// DFA3D/dfa3D/ops/csrc/cuda/wms_deform_attn_cuda.cu:267,344 and ms_depth_score_sample_cuda.cu:94,184).
// The float path of this library is the tuned one (dfa3d_forward.cu / dfa3d_backward.cu); double exists
// for what double is used for -- gradient checks and reference-grade comparisons -- so these kernels
// favour being obviously right over speed: one warp per (camera, query, head) item, the item's sampling
// points taken one after the other with the geometry computed redundantly by all lanes, lanes striding
// over the channels, fp64 atomics for the accumulated gradients.  Every tensor is double (the
// reference requires one scalar type for all of them); level tables stay int64.
//
// Semantics are those of the float kernels (see dfa3d_common.cuh): pixel = fma(loc, size, -0.5), strict
// range tests, corner order 0=(y0,x0) 1=(y0,x1) 2=(y1,x1) 3=(y1,x0), grad_depth_score not gated by the
// depth-range test, depth backward drops points that fail it.
#include <stdint.h>

#include "dfa3d_b200.h"
#include "dfa3d_launch.h"

namespace dfa3d {
namespace {

constexpr int kWarps64 = 4;
constexpr int kMaxLv = DFA3D_MAX_LEVELS;

struct Geo64 {
  double lw, lh, ld;
  int pix[4];      // pixel index inside the camera or -1
  int z0, W, Hh, Dd;
  bool ok2, ok3;
};

__device__ __forceinline__ Geo64 geometry64(double x, double y, double z, bool has_z, int Hh, int W, int Dd,
                                            int start, int N) {
  Geo64 g;
  g.W = W; g.Hh = Hh; g.Dd = Dd;
  const double w_im = fma(x, (double)W, -0.5), h_im = fma(y, (double)Hh, -0.5);
  g.ok2 = h_im > -1.0 && w_im > -1.0 && h_im < (double)Hh && w_im < (double)W;
  double d_im = 0.0;
  g.ok3 = false;
  if (has_z) {
    d_im = fma(z, (double)Dd, -0.5);
    g.ok3 = g.ok2 && d_im > -1.0 && d_im < (double)Dd;
  }
  const double wf = floor(w_im), hf = floor(h_im), df = floor(d_im);
  const int x0 = g.ok2 ? (int)wf : 0, y0 = g.ok2 ? (int)hf : 0;
  g.lw = w_im - wf; g.lh = h_im - hf; g.ld = d_im - df;
  g.z0 = g.ok3 ? (int)df : 0;
  const bool xl = x0 >= 0, xh = x0 + 1 <= W - 1, yl = y0 >= 0, yh = y0 + 1 <= Hh - 1;
  const int base = start + y0 * W + x0;
  const unsigned n = (unsigned)N;
  g.pix[0] = (g.ok2 && yl && xl && (unsigned)base < n) ? base : -1;
  g.pix[1] = (g.ok2 && yl && xh && (unsigned)(base + 1) < n) ? base + 1 : -1;
  g.pix[2] = (g.ok2 && yh && xh && (unsigned)(base + W + 1) < n) ? base + W + 1 : -1;
  g.pix[3] = (g.ok2 && yh && xl && (unsigned)(base + W) < n) ? base + W : -1;
  return g;
}

struct Args64 {
  const double *value, *dist, *loc, *attn, *ds_in, *grad_out, *grad_ds_in;
  const int64_t *shapes, *lsi;
  double *out, *ds_out, *grad_value, *grad_dist, *grad_loc, *grad_attn, *grad_ds_out;
  int B, N, H, C, D, L, Q, P, LP, shape_stride, loc_stride;
  int dist_pix_stride, dist_head_stride;
  bool from_dist;   // depth scores come from dist (one-stage) instead of ds_in (two-stage attention)
};

struct Levels64 {
  int h[kMaxLv], w[kMaxLv], d[kMaxLv], start[kMaxLv];
};

__device__ __forceinline__ void stage64(Levels64 &t, const Args64 &a) {
  for (int l = threadIdx.x; l < a.L; l += blockDim.x) {
    t.h[l] = (int)a.shapes[l * a.shape_stride];
    t.w[l] = (int)a.shapes[l * a.shape_stride + 1];
    t.d[l] = a.shape_stride == 3 ? (int)a.shapes[l * 3 + 2] : a.D;
    t.start[l] = (int)a.lsi[l];
  }
  __syncthreads();
}

// The two bins z0, z0+1 of a corner pixel (0 outside [0, Dlim-1]).
__device__ __forceinline__ void bins64(const double *dist_bh, int stride, int pix, int z0, int Dlim,
                                       double &lo, double &hi) {
  lo = 0.0; hi = 0.0;
  if (pix < 0) return;
  const double *p = dist_bh + ((long long)pix * stride + z0);
  if (z0 >= 0 && z0 < Dlim) lo = p[0];
  if (z0 + 1 >= 0 && z0 + 1 < Dlim) hi = p[1];
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

// Per-corner depth scores of one point (all lanes compute the same values).
__device__ __forceinline__ void depth_scores64(const Args64 &a, const Geo64 &g, int b, int h, long long pt,
                                               double (&ds)[4], double (&dz)[4]) {
  if (a.from_dist) {
    const double *dist_bh = a.dist + ((long long)b * a.N * a.dist_pix_stride + h * a.dist_head_stride);
    const int Dlim = min(g.Dd, a.D);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      double lo, hi;
      bins64(dist_bh, a.dist_pix_stride, g.ok3 ? g.pix[k] : -1, g.z0, Dlim, lo, hi);
      ds[k] = g.ok3 ? lo * (1.0 - g.ld) + hi * g.ld : 0.0;
      dz[k] = hi - lo;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      ds[k] = g.pix[k] >= 0 ? (a.ds_in ? a.ds_in[pt * 4 + k] : 1.0) : 0.0;
      dz[k] = 0.0;
    }
  }
}

__global__ void __launch_bounds__(kWarps64 * 32) forward64_kernel(const Args64 a) {
  __shared__ Levels64 lv;
  stage64(lv, a);
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kWarps64 + (threadIdx.x >> 5);
  if (item >= (long long)a.B * a.Q * a.H) return;
  const int h = (int)(item % a.H);
  const int b = (int)(item / ((long long)a.Q * a.H));
  const double *vbase = a.value + ((long long)b * a.N * a.H + h) * a.C;
  const int row = a.H * a.C;
  for (int c0 = 0; c0 < a.C; c0 += 32) {
    const int ch = c0 + lane;
    double acc = 0.0;
    for (int j = 0; j < a.LP; ++j) {
      const int l = j / a.P;
      const long long pt = item * a.LP + j;
      const double *lp = a.loc + pt * a.loc_stride;
      const Geo64 g = geometry64(lp[0], lp[1], a.from_dist ? lp[2] : 0.0, a.from_dist, lv.h[l], lv.w[l],
                                 lv.d[l], lv.start[l], a.N);
      double ds[4], dz[4];
      depth_scores64(a, g, b, h, pt, ds, dz);
      if (a.ds_out && c0 == 0 && lane < 4) a.ds_out[pt * 4 + lane] = ds[lane];
      if (!g.ok2 || ch >= a.C) continue;
      const double hw = 1.0 - g.lw, hh = 1.0 - g.lh;
      const double bw[4] = {hh * hw, hh * g.lw, g.lh * g.lw, g.lh * hw};
      const double aw = a.attn[pt];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (g.pix[k] >= 0) acc += aw * (bw[k] * ds[k]) * vbase[(long long)g.pix[k] * row + ch];
    }
    if (ch < a.C) a.out[item * a.C + ch] = acc;
  }
}

__global__ void __launch_bounds__(kWarps64 * 32) backward64_kernel(const Args64 a) {
  __shared__ Levels64 lv;
  stage64(lv, a);
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kWarps64 + (threadIdx.x >> 5);
  if (item >= (long long)a.B * a.Q * a.H) return;
  const int h = (int)(item % a.H);
  const int b = (int)(item / ((long long)a.Q * a.H));
  const long long slice = ((long long)b * a.N * a.H + h) * a.C;
  const double *vbase = a.value + slice;
  double *gvbase = a.grad_value + slice;
  const double *go = a.grad_out + item * a.C;
  const int row = a.H * a.C;
  for (int j = 0; j < a.LP; ++j) {
    const int l = j / a.P;
    const long long pt = item * a.LP + j;
    const double *lp = a.loc + pt * a.loc_stride;
    const Geo64 g = geometry64(lp[0], lp[1], a.from_dist ? lp[2] : 0.0, a.from_dist, lv.h[l], lv.w[l],
                               lv.d[l], lv.start[l], a.N);
    double ds[4], dz[4];
    depth_scores64(a, g, b, h, pt, ds, dz);
    const double hw = 1.0 - g.lw, hh = 1.0 - g.lh;
    const double bw[4] = {hh * hw, hh * g.lw, g.lh * g.lw, g.lh * hw};
    const double aw = a.attn[pt];
    double t[4] = {0.0, 0.0, 0.0, 0.0};
    if (g.ok2) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (g.pix[k] < 0) continue;
        const double wgt = aw * (bw[k] * ds[k]);
        double d = 0.0;
        for (int ch = lane; ch < a.C; ch += 32) {
          const long long o = (long long)g.pix[k] * row + ch;
          d = fma(vbase[o], go[ch], d);
          if (wgt != 0.0) atomicAdd(gvbase + o, wgt * go[ch]);
        }
        t[k] = warp_sum(d);
      }
    }
    if (lane != 0) continue;
    double g_attn = 0.0, g_x = 0.0, g_y = 0.0, g_z = 0.0, gds[4] = {0.0, 0.0, 0.0, 0.0};
    if (g.ok2) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        g_attn = fma(bw[k] * ds[k], t[k], g_attn);
        gds[k] = g.pix[k] >= 0 ? aw * (bw[k] * t[k]) : 0.0;
      }
      const double e0 = ds[0] * t[0], e1 = ds[1] * t[1], e2 = ds[2] * t[2], e3 = ds[3] * t[3];
      g_x = (double)g.W * aw * (hh * (e1 - e0) + g.lh * (e2 - e3));
      g_y = (double)g.Hh * aw * (hw * (e3 - e0) + g.lw * (e2 - e1));
      if (a.from_dist && g.ok3) {
        double *gd_bh = a.grad_dist + ((long long)b * a.N * a.dist_pix_stride + h * a.dist_head_stride);
        const int Dlim = min(g.Dd, a.D);
        double acc = 0.0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (g.pix[k] < 0) continue;
          double *p = gd_bh + ((long long)g.pix[k] * a.dist_pix_stride + g.z0);
          if (gds[k] != 0.0) {
            if (g.z0 >= 0 && g.z0 < Dlim) atomicAdd(p, (1.0 - g.ld) * gds[k]);
            if (g.z0 + 1 >= 0 && g.z0 + 1 < Dlim) atomicAdd(p + 1, g.ld * gds[k]);
          }
          acc = fma(gds[k], dz[k], acc);
        }
        g_z = (double)g.Dd * acc;
      }
    }
    a.grad_attn[pt] = g_attn;
    double *gl = a.grad_loc + pt * a.loc_stride;
    gl[0] = g_x; gl[1] = g_y;
    if (a.from_dist) gl[2] = g_z;
    if (a.grad_ds_out) {
#pragma unroll
      for (int k = 0; k < 4; ++k) a.grad_ds_out[pt * 4 + k] = gds[k];
    }
  }
}

// depth scores alone / their backward: one thread per sampling point
__global__ void depth_forward64_kernel(const Args64 a) {
  __shared__ Levels64 lv;
  stage64(lv, a);
  const long long npts = (long long)a.B * a.Q * a.H * a.LP;
  for (long long pt = (long long)blockIdx.x * blockDim.x + threadIdx.x; pt < npts;
       pt += (long long)gridDim.x * blockDim.x) {
    const long long item = pt / a.LP;
    const int l = (int)(pt - item * a.LP) / a.P;
    const int h = (int)(item % a.H), b = (int)(item / ((long long)a.Q * a.H));
    const double *lp = a.loc + pt * 3;
    const Geo64 g = geometry64(lp[0], lp[1], lp[2], true, lv.h[l], lv.w[l], lv.d[l], lv.start[l], a.N);
    double ds[4], dz[4];
    depth_scores64(a, g, b, h, pt, ds, dz);
#pragma unroll
    for (int k = 0; k < 4; ++k) a.ds_out[pt * 4 + k] = ds[k];
  }
}

__global__ void depth_backward64_kernel(const Args64 a) {
  __shared__ Levels64 lv;
  stage64(lv, a);
  const long long npts = (long long)a.B * a.Q * a.H * a.LP;
  for (long long pt = (long long)blockIdx.x * blockDim.x + threadIdx.x; pt < npts;
       pt += (long long)gridDim.x * blockDim.x) {
    const long long item = pt / a.LP;
    const int l = (int)(pt - item * a.LP) / a.P;
    const int h = (int)(item % a.H), b = (int)(item / ((long long)a.Q * a.H));
    const double *lp = a.loc + pt * 3;
    const Geo64 g = geometry64(lp[0], lp[1], lp[2], true, lv.h[l], lv.w[l], lv.d[l], lv.start[l], a.N);
    double g_z = 0.0;
    if (g.ok3) {
      const long long bh = (long long)b * a.N * a.dist_pix_stride + h * a.dist_head_stride;
      const int Dlim = min(g.Dd, a.D);
      double acc = 0.0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (g.pix[k] < 0) continue;
        double lo, hi;
        bins64(a.dist + bh, a.dist_pix_stride, g.pix[k], g.z0, Dlim, lo, hi);
        const double gk = a.grad_ds_in[pt * 4 + k];
        double *p = a.grad_dist + bh + ((long long)g.pix[k] * a.dist_pix_stride + g.z0);
        if (g.z0 >= 0 && g.z0 < Dlim) atomicAdd(p, (1.0 - g.ld) * gk);
        if (g.z0 + 1 >= 0 && g.z0 + 1 < Dlim) atomicAdd(p + 1, g.ld * gk);
        acc = fma(gk, hi - lo, acc);
      }
      g_z = (double)g.Dd * acc;
    }
    double *gl = a.grad_loc + pt * 3;
    gl[0] = 0.0; gl[1] = 0.0; gl[2] = g_z;
  }
}

Args64 args_from(const dfa3d_problem *p, int shape_stride, int loc_stride, bool from_dist) {
  Args64 a{};
  a.B = p->B; a.N = p->N; a.H = p->H; a.C = p->C; a.D = p->D; a.L = p->L; a.Q = p->Q; a.P = p->P;
  a.LP = p->L * p->P;
  a.shape_stride = shape_stride; a.loc_stride = loc_stride; a.from_dist = from_dist;
  a.dist_head_stride = (int)p->dist_head_stride;
  a.dist_pix_stride = p->dist_head_stride == 0 ? p->D : p->H * p->D;
  return a;
}

unsigned item_grid64(const dfa3d_problem *p) {
  const long long items = (long long)p->B * p->Q * p->H;
  return (unsigned)((items + kWarps64 - 1) / kWarps64);
}

unsigned point_grid64(const dfa3d_problem *p) {
  const long long n = (long long)p->B * p->Q * p->H * p->L * p->P;
  const long long g = (n + 255) / 256;
  return (unsigned)(g > 148 * 64 ? 148 * 64 : (g < 1 ? 1 : g));
}

}  // namespace

cudaError_t launch_forward64(const dfa3d_problem *p, const double *value, const double *dist,
                             const int64_t *shapes, int shape_stride, const int64_t *lsi,
                             const double *loc, int loc_stride, const double *attn, const double *ds_in,
                             bool from_dist, double *out, double *ds_out, cudaStream_t s) {
  Args64 a = args_from(p, shape_stride, loc_stride, from_dist);
  a.value = value; a.dist = dist; a.shapes = shapes; a.lsi = lsi; a.loc = loc; a.attn = attn;
  a.ds_in = ds_in; a.out = out; a.ds_out = ds_out;
  forward64_kernel<<<item_grid64(p), kWarps64 * 32, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_backward64(const dfa3d_problem *p, const double *value, const double *dist,
                              const int64_t *shapes, int shape_stride, const int64_t *lsi,
                              const double *loc, int loc_stride, const double *attn, const double *ds_in,
                              bool from_dist, const double *grad_out, double *grad_value,
                              double *grad_dist, double *grad_loc, double *grad_attn, double *grad_ds_out,
                              cudaStream_t s) {
  Args64 a = args_from(p, shape_stride, loc_stride, from_dist);
  a.value = value; a.dist = dist; a.shapes = shapes; a.lsi = lsi; a.loc = loc; a.attn = attn;
  a.ds_in = ds_in; a.grad_out = grad_out; a.grad_value = grad_value; a.grad_dist = grad_dist;
  a.grad_loc = grad_loc; a.grad_attn = grad_attn; a.grad_ds_out = grad_ds_out;
  backward64_kernel<<<item_grid64(p), kWarps64 * 32, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_depth_forward64(const dfa3d_problem *p, const double *dist, const int64_t *shapes3,
                                   const int64_t *lsi, const double *loc3, double *ds_out,
                                   cudaStream_t s) {
  Args64 a = args_from(p, 3, 3, true);
  a.dist = dist; a.shapes = shapes3; a.lsi = lsi; a.loc = loc3; a.ds_out = ds_out;
  depth_forward64_kernel<<<point_grid64(p), 256, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_depth_backward64(const dfa3d_problem *p, const double *dist, const int64_t *shapes3,
                                    const int64_t *lsi, const double *loc3, const double *grad_ds,
                                    double *grad_dist, double *grad_loc3, cudaStream_t s) {
  Args64 a = args_from(p, 3, 3, true);
  a.dist = dist; a.shapes = shapes3; a.lsi = lsi; a.loc = loc3; a.grad_ds_in = grad_ds;
  a.grad_dist = grad_dist; a.grad_loc = grad_loc3;
  depth_backward64_kernel<<<point_grid64(p), 256, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace dfa3d
