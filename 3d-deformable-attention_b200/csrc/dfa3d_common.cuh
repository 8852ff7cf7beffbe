// Shared device helpers of the DFA3D kernels (sm_100a).
//
// Geometry conventions are the reference's
// (DFA3D/dfa3D/ops/csrc/common/cuda/ms_depth_score_sample_cuda_kernel.cuh:128-141 and
//  wms_deform_attn_cuda_kernel.cuh:280-294):
//   pixel coordinate  = fma(loc, size, -0.5)  -- ONE rounding.  The reference writes `loc * size - 0.5`
//                       and nvcc's default contraction turns it into a fused multiply-add; with a
//                       separately rounded product about 1e-5 of the points of a BEVFormer-base
//                       sized problem fall into the neighbouring cell, which changes the
//                       (discontinuous) depth_score slots and location gradients against the
//                       reference op.  With fmaf none were observed to.
//   2-D range test    = h > -1 && w > -1 && h < H && w < W          (strict)
//   3-D range test    = 2-D test && d > -1 && d < D
//   corner k          : 0=(y0,x0) 1=(y0,x1) 2=(y1,x1) 3=(y1,x0);  in-image iff 0 <= y <= H-1, 0 <= x <= W-1
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dfa3d {

constexpr int kMaxLevels = 32;

// What the kernels are given per sampling point.
//   kFused            location (x,y,z) + attention weight; depth scores computed from dist
//   kGivenDepthScore  location (x,y) + attention weight + the four depth scores (two-stage API);
//                     without a depth-score tensor the scores are 1: plain 2-D deformable attention
//   kCallerFused      reference point + raw offsets + raw attention logits: the caller's location
//                     assembly and softmax (BEVFormer_DFA3D/projects/mmdet3d_plugin/bevformer/modules/
//                     spatial_cross_attention.py:498-538) happen in the prologue; depth scores from dist
enum Mode { kFused = 0, kGivenDepthScore = 1, kCallerFused = 2 };
// Storage type codes = DFA3D_DTYPE_F32 / _BF16 / _F16 of the C header.
enum StorageType { kDtypeF32 = 0, kDtypeBF16 = 1, kDtypeF16 = 3 };
__host__ __device__ constexpr bool mode_has_depth(int m) { return m != kGivenDepthScore; }
constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;

// Compile-time tuning knobs (defaults = the measured optimum on B200 at the BEVFormer-base shape).
//   *_ITEMS_PER_WARP  consecutive CTA-sized groups of items a CTA works through before it retires:
//                     fewer, longer-lived CTAs (a CTA that handles one item per warp lives ~2 us)
//   *_MIN_CTAS        __launch_bounds__ residency target, i.e. the register cap
#ifndef DFA3D_FWD_ITEMS_PER_WARP
#define DFA3D_FWD_ITEMS_PER_WARP 8
#endif
#ifndef DFA3D_BWD_ITEMS_PER_WARP
#define DFA3D_BWD_ITEMS_PER_WARP 4
#endif
#ifndef DFA3D_FWD_MIN_CTAS
#define DFA3D_FWD_MIN_CTAS 5
#endif
#ifndef DFA3D_BWD_MIN_CTAS
#define DFA3D_BWD_MIN_CTAS 4
#endif
//   *_HEAD_MAJOR      1: the items of a camera are walked head by head (all queries of head 0, then
//                     head 1, ...) instead of query by query, so that the CTAs resident at one time
//                     gather from, and reduce into, one or two heads' slices.  Measured: backward
//                     -1.8 %, forward +1 % (+4 % when neighbouring queries look at neighbouring pixels,
//                     because the eight heads of a query then share their depth-distribution lines)
#ifndef DFA3D_FWD_HEAD_MAJOR
#define DFA3D_FWD_HEAD_MAJOR 0
#endif
#ifndef DFA3D_BWD_HEAD_MAJOR
#define DFA3D_BWD_HEAD_MAJOR 1
#endif

// Kernel argument block (device pointers + sizes).  Unused pointers are null.
struct KArgs {
  const void *value;       // (B,N,H,C) fp32|bf16|fp16
  const void *dist;        // (B,N,H,D) or (B,N,D) fp32|bf16|fp16
  const int64_t *shapes;   // (L, shape_stride) int64
  const int64_t *lsi;      // (L) int64
  const float *loc;        // (B,Q,H,L,P,loc_stride)
  const float *attn;       // (B,Q,H,L,P)
  const float *ds_in;      // (B,Q,H,L,P,4) given depth score (two-stage attention)
  const float *grad_out;   // (B,Q,H*C)
  // caller-fused mode: locations and attention weights are formed inside the kernel
  const float *ref;        // (B,Q,Z,3) reference points
  const float *off_uv;     // (B,Q,H,L,P,2) raw x/y offsets in pixels
  const float *off_d;      // (B,Q,H,L,P) raw depth offsets in bins
  const float *logits;     // (B,Q,H,L*P) raw attention logits
  float *grad_off_uv;      // (B,Q,H,L,P,2), overwritten
  float *grad_off_d;       // (B,Q,H,L,P), overwritten
  float *grad_logits;      // (B,Q,H,L*P), overwritten
  int Z;                   // reference points (pillar anchors) per query
  // ragged queries: camera b owns the packed query rows [q_off[b], q_off[b+1]) of every per-query
  // tensor; Q is then only the bound the grid is sized for.  Null = every camera has Q queries.
  const int32_t *q_off;
  const float *grad_ds_in; // (B,Q,H,L,P,4) incoming depth-score gradient (two-stage depth backward)
  float *out;              // (B,Q,H*C)
  float *ds_out;           // (B,Q,H,L,P,4) or null
  float *grad_value;       // (B,N,H,C) fp32, accumulated
  float *grad_dist;        // layout of dist, fp32, accumulated
  float *grad_loc;         // (B,Q,H,L,P,loc_stride), overwritten
  float *grad_attn;        // (B,Q,H,L,P), overwritten
  float *grad_ds_out;      // (B,Q,H,L,P,4), overwritten, or null
  int B, N, H, C, D, L, Q, P;
  int LP;                  // L*P
  int items_per_cam;       // Q*H: one warp per (query, head) of a camera
  int b0;                  // camera index of blockIdx.y == 0 (launches cover <= 65535 cameras each)
  int shape_stride;        // 2 or 3
  int loc_stride;          // 2 or 3
  long long items;         // B*Q*H
  int dist_pix_stride;     // elements between pixels of dist: H*D or D
  int dist_head_stride;    // D or 0
  int Nd;                  // rows of dist per camera: N, or dmap_h * dmap_w
  int dmap_h, dmap_w;      // > 0: dist is one dmap_h x dmap_w map per camera, read by every level with
                           // nearest-neighbour indexing (F.interpolate(mode="nearest") semantics)
};

// Level table staged in shared memory once per CTA.
struct LevelTable {
  int h[kMaxLevels], w[kMaxLevels], d[kMaxLevels], start[kMaxLevels];
  float map_sy[kMaxLevels], map_sx[kMaxLevels];   // dist map: (float)map size / level size per axis
};

__device__ __forceinline__ void stage_levels(LevelTable &t, const KArgs &a) {
  for (int l = threadIdx.x; l < a.L; l += blockDim.x) {
    t.h[l] = (int)a.shapes[l * a.shape_stride];
    t.w[l] = (int)a.shapes[l * a.shape_stride + 1];
    t.d[l] = a.shape_stride == 3 ? (int)a.shapes[l * 3 + 2] : a.D;
    t.start[l] = (int)a.lsi[l];
    // the resize's scale, formed in fp32 from the two sizes as torch's nearest interpolation forms it
    t.map_sy[l] = a.dmap_h > 0 ? (float)a.dmap_h / (float)t.h[l] : 1.f;
    t.map_sx[l] = a.dmap_w > 0 ? (float)a.dmap_w / (float)t.w[l] : 1.f;
  }
  __syncthreads();
}

// What a warp knows about its (camera b, query q, head h) item: 64-bit bases computed once, so that
// the per-point and per-row arithmetic stays 32-bit.
struct ItemCtx {
  int b, h;
  long long bq;             // b*Q + q
  long long item;           // (b*Q + q)*H + h
  const float *loc;         // first location of the item
  const float *attn;        // first attention weight of the item
  long long pt0;            // index of the item's first point: item * LP
};

// blockIdx.y (+ b0) selects the camera; the CTA's `group`-th group of kWarpsPerCta items starts at
// (blockIdx.x * groups_per_cta + group) * kWarpsPerCta, warp w takes item w of it: a (query, head)
// pair of that camera.  Returns false for the warps past the end of the camera.
template <bool HEAD_MAJOR = false>
__device__ __forceinline__ bool item_context(const KArgs &a, int warp, unsigned group, ItemCtx &c) {
  const unsigned idx = group * kWarpsPerCta + warp;
  if (idx >= (unsigned)a.items_per_cam) return false;
  c.b = (int)blockIdx.y + a.b0;
  if (HEAD_MAJOR) {
    if (a.q_off) {
      const int q0 = __ldg(a.q_off + c.b);
      const unsigned nq = (unsigned)(__ldg(a.q_off + c.b + 1) - q0);
      if (idx >= nq * (unsigned)a.H) return false;
      c.h = (int)(idx / nq);
      c.bq = (long long)q0 + (idx - (unsigned)c.h * nq);
    } else {
      c.h = (int)(idx / (unsigned)a.Q);
      c.bq = (long long)c.b * a.Q + (idx - (unsigned)c.h * (unsigned)a.Q);
    }
    c.item = c.bq * a.H + c.h;
  } else {
    const unsigned q = idx / (unsigned)a.H;
    c.h = (int)(idx - q * (unsigned)a.H);
    if (a.q_off) {
      const int q0 = __ldg(a.q_off + c.b);
      if ((int)q >= __ldg(a.q_off + c.b + 1) - q0) return false;
      c.bq = (long long)q0 + q;
      c.item = c.bq * a.H + c.h;
    } else {
      c.bq = (long long)c.b * a.Q + q;
      c.item = (long long)c.b * a.items_per_cam + idx;
    }
  }
  c.pt0 = c.item * a.LP;
  c.loc = a.loc + c.pt0 * a.loc_stride;      // (not dereferenced in caller-fused mode)
  c.attn = a.attn + c.pt0;
  return true;
}

// Softmax of an item's L*P attention logits (caller-fused mode): maximum and sum of exp(l - max),
// formed with warp shuffles; lane j later turns its own logit into exp(l_j - max) / sum.
struct SoftmaxStats {
  float mx, sum;
};

__device__ __forceinline__ SoftmaxStats item_softmax_stats(const KArgs &a, const ItemCtx &c, int lane) {
  const float *lg = a.logits + c.pt0;
  float mx = -INFINITY;
  for (int j = lane; j < a.LP; j += 32) mx = fmaxf(mx, __ldg(lg + j));
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
  float sum = 0.f;
  for (int j = lane; j < a.LP; j += 32) sum += expf(__ldg(lg + j) - mx);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
  return SoftmaxStats{mx, sum};
}

// Location and attention weight of point j of the item, from whatever the mode provides.
// Caller-fused: loc = reference point of the point's anchor + offset / (W, H, D), the division and the
// addition rounded separately as the tensor expressions of the caller are
// (spatial_cross_attention.py:527-533); anchor of point p of a level = p % Z (:530-531).
template <int MODE>
__device__ __forceinline__ void read_point(const KArgs &a, const LevelTable &lv, const ItemCtx &c, int j,
                                           int l, const SoftmaxStats &sm, float &x, float &y, float &z,
                                           float &aw) {
  if (MODE == kCallerFused) {
    const int zi = (j - l * a.P) % a.Z;
    const float *r = a.ref + (c.bq * a.Z + zi) * 3;
    const float *o = a.off_uv + (c.pt0 + j) * 2;
    x = __fadd_rn(__ldg(r), __fdiv_rn(__ldg(o), (float)lv.w[l]));
    y = __fadd_rn(__ldg(r + 1), __fdiv_rn(__ldg(o + 1), (float)lv.h[l]));
    z = __fadd_rn(__ldg(r + 2), __fdiv_rn(__ldg(a.off_d + c.pt0 + j), (float)a.D));
    aw = __fdiv_rn(expf(__ldg(a.logits + c.pt0 + j) - sm.mx), sm.sum);
  } else {
    const float *lp = c.loc + j * a.loc_stride;
    x = __ldg(lp);
    y = __ldg(lp + 1);
    z = (MODE == kFused) ? __ldg(lp + 2) : 0.f;
    aw = __ldg(c.attn + j);
  }
}

// Geometry of one sampling point.
struct PointGeo {
  float lw, lh, ld;   // fractional parts; hw = 1-lw etc.
  int pix[4];         // pixel index inside the camera (level start included), -1 if corner k unusable
  int dpix[4];        // row of dist that belongs to corner k (== pix[k] unless dist is a single map)
  int z0;             // lower depth bin (may be -1); upper = z0+1
  int W, Hh, Dd;
  bool ok2, ok3;
};

// `has_z`: the location carries a depth coordinate (3-D range test applies to ok3).
// Corner pixels are additionally bounded by N so that inconsistent shape tables cannot make the
// kernels touch memory outside the tensors (such corners are treated as outside the image).
// Row of the dist map that pixel (y, x) of a level reads: nearest-neighbour resize,
// src = min(floor(dst * scale), size - 1) with scale = (float)map size / (float)level size.
__device__ __forceinline__ int map_row(int y, int x, float sy, float sx, int mh, int mw) {
  const int my = min((int)floorf((float)y * sy), mh - 1);
  const int mx = min((int)floorf((float)x * sx), mw - 1);
  return my * mw + mx;
}

struct DistMap {
  int h, w;           // 0, 0: dist is laid out like value
  float sy, sx;
};
__device__ __forceinline__ DistMap dist_map_of(const KArgs &a, const LevelTable &lv, int l) {
  return DistMap{a.dmap_h, a.dmap_w, lv.map_sy[l], lv.map_sx[l]};
}

__device__ __forceinline__ PointGeo point_geometry(float x, float y, float z, bool has_z, int Hh,
                                                   int W, int Dd, int start, int N,
                                                   const DistMap dm = DistMap{0, 0, 1.f, 1.f}) {
  PointGeo g;
  g.W = W; g.Hh = Hh; g.Dd = Dd;
  const float w_im = fmaf(x, (float)W, -0.5f);
  const float h_im = fmaf(y, (float)Hh, -0.5f);
  g.ok2 = (h_im > -1.f) && (w_im > -1.f) && (h_im < (float)Hh) && (w_im < (float)W);
  float d_im = 0.f;
  g.ok3 = false;
  if (has_z) {
    d_im = fmaf(z, (float)Dd, -0.5f);
    g.ok3 = g.ok2 && (d_im > -1.f) && (d_im < (float)Dd);
  }
  const float wf = floorf(w_im), hf = floorf(h_im), df = floorf(d_im);
  const int x0 = g.ok2 ? (int)wf : 0, y0 = g.ok2 ? (int)hf : 0;
  g.lw = w_im - wf; g.lh = h_im - hf; g.ld = d_im - df;
  g.z0 = g.ok3 ? (int)df : 0;
  const int x1 = x0 + 1, y1 = y0 + 1;
  const bool xl = x0 >= 0, xh = x1 <= W - 1, yl = y0 >= 0, yh = y1 <= Hh - 1;
  const int base = start + y0 * W + x0;
  const int p0 = base, p1 = base + 1, p2 = base + W + 1, p3 = base + W;
  const unsigned n = (unsigned)N;      // unsigned compare: also rejects indices that wrapped negative
  g.pix[0] = (g.ok2 && yl && xl && (unsigned)p0 < n) ? p0 : -1;
  g.pix[1] = (g.ok2 && yl && xh && (unsigned)p1 < n) ? p1 : -1;
  g.pix[2] = (g.ok2 && yh && xh && (unsigned)p2 < n) ? p2 : -1;
  g.pix[3] = (g.ok2 && yh && xl && (unsigned)p3 < n) ? p3 : -1;
#pragma unroll
  for (int k = 0; k < 4; ++k) g.dpix[k] = g.pix[k];
  if (has_z && dm.h > 0) {
    if (g.pix[0] >= 0) g.dpix[0] = map_row(y0, x0, dm.sy, dm.sx, dm.h, dm.w);
    if (g.pix[1] >= 0) g.dpix[1] = map_row(y0, x1, dm.sy, dm.sx, dm.h, dm.w);
    if (g.pix[2] >= 0) g.dpix[2] = map_row(y1, x1, dm.sy, dm.sx, dm.h, dm.w);
    if (g.pix[3] >= 0) g.dpix[3] = map_row(y1, x0, dm.sy, dm.sx, dm.h, dm.w);
  }
  return g;
}

__device__ __forceinline__ void bilinear_weights(const PointGeo &g, float bw[4]) {
  const float hw = 1.f - g.lw, hh = 1.f - g.lh;
  bw[0] = hh * hw; bw[1] = hh * g.lw; bw[2] = g.lh * g.lw; bw[3] = g.lh * hw;
}

__device__ __forceinline__ float load_scalar(const float *p) { return __ldg(p); }
__device__ __forceinline__ float load_scalar(const __nv_bfloat16 *p) {
  return __bfloat162float(__ldg(p));
}
__device__ __forceinline__ float load_scalar(const __half *p) { return __half2float(__ldg(p)); }

// Two packed fp16 values (low half first) widened to fp32.
__device__ __forceinline__ float2 widen_half2(uint32_t bits) {
  return __half22float2(*reinterpret_cast<const __half2 *>(&bits));
}

// One gathered row: where it starts and what it is multiplied by.
struct __align__(8) RowEntry {
  int off;    // element offset of the row inside the (b, h) slice of value; -1 = skip
  float wgt;  // attention * bilinear * depth score
};

// A warp's table of 32 points x 4 corners: entry (p, k) in slot p*4 + k.  (Swizzling the two 16-byte
// halves of a lane's store to avoid its 2-way bank conflict was measured: the extra index arithmetic
// in the readers cost more than the conflicts.)
__device__ __forceinline__ void store_rows(RowEntry *table, int lane, const int (&off)[4],
                                           const float (&wgt)[4]) {
  uint4 *dst = reinterpret_cast<uint4 *>(table) + lane * 2;
  dst[0] = make_uint4((uint32_t)off[0], __float_as_uint(wgt[0]), (uint32_t)off[1], __float_as_uint(wgt[1]));
  dst[1] = make_uint4((uint32_t)off[2], __float_as_uint(wgt[2]), (uint32_t)off[3], __float_as_uint(wgt[3]));
}

// Two adjacent depth bins p[0], p[1] that are both in range: one naturally aligned 8-byte (fp32) or
// 4-byte (bf16) load when the pair happens to be aligned, two scalar loads otherwise (the second then
// hits the sector the first brought into L1).  Measured 3-5 % on the kernels against always-scalar;
// wider windows with element extraction were measured slower.
__device__ __forceinline__ void load_pair(const float *p, float &lo, float &hi) {
  if ((reinterpret_cast<uintptr_t>(p) & 7) == 0) {
    const float2 t = __ldg(reinterpret_cast<const float2 *>(p));
    lo = t.x; hi = t.y;
  } else {
    lo = __ldg(p); hi = __ldg(p + 1);
  }
}
__device__ __forceinline__ void load_pair(const __nv_bfloat16 *p, float &lo, float &hi) {
  if ((reinterpret_cast<uintptr_t>(p) & 3) == 0) {
    const uint32_t t = __ldg(reinterpret_cast<const uint32_t *>(p));
    lo = __uint_as_float(t << 16); hi = __uint_as_float(t & 0xffff0000u);
  } else {
    lo = load_scalar(p); hi = load_scalar(p + 1);
  }
}

__device__ __forceinline__ void load_pair(const __half *p, float &lo, float &hi) {
  if ((reinterpret_cast<uintptr_t>(p) & 3) == 0) {
    const float2 t = widen_half2(__ldg(reinterpret_cast<const uint32_t *>(p)));
    lo = t.x; hi = t.y;
  } else {
    lo = load_scalar(p); hi = load_scalar(p + 1);
  }
}

// The two depth bins z0, z0+1 of one corner pixel (0 where a bin is outside [0, Dlim-1] or the corner
// is unusable).  Dlim = min(depth size of the level, channel count of dist).
template <typename DT>
__device__ __forceinline__ void load_depth_pair(const DT *dist_bh, int pix_stride, int pix, int z0,
                                                int Dlim, bool ok3, float &lo, float &hi) {
  lo = 0.f; hi = 0.f;
  if (ok3 && pix >= 0) {
    const DT *p = dist_bh + ((long long)pix * pix_stride + z0);
    const bool vlo = z0 >= 0 && z0 < Dlim, vhi = z0 + 1 < Dlim;
    if (vlo && vhi) load_pair(p, lo, hi);
    else if (vlo) lo = load_scalar(p);
    else if (vhi) hi = load_scalar(p + 1);
  }
}

// Read-only load of a lane's value-row fragment, widened to fp32.
template <typename VT> struct RowVec;
template <> struct RowVec<float> {
  static constexpr int kElems = 4;
  __device__ static __forceinline__ void load(const float *p, float (&v)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
};
template <> struct RowVec<__nv_bfloat16> {
  // Forward: 8 elements (16 bytes) per lane -- half the requests and row-table reads per point.
  static constexpr int kElems = 8;
  __device__ static __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {           // bf16 -> fp32 is a 16-bit shift
      v[2 * i] = __uint_as_float(u[i] << 16);
      v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
};

template <> struct RowVec<__half> {
  static constexpr int kElems = 8;
  __device__ static __forceinline__ void load(const __half *p, float (&v)[8]) {
    const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = widen_half2(u[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
};

// Backward: 4 channels per lane for every storage type, so that the lane-to-channel mapping, the
// register footprint and the one 16-byte vector reduction per lane are those of fp32 rows (measured:
// with 8 bf16 per lane the backward needs 80+ registers and runs 30 % slower than the fp32 one).
template <typename VT> struct RowVec4 : RowVec<VT> {};
template <> struct RowVec4<__nv_bfloat16> {
  static constexpr int kElems = 4;
  __device__ static __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[4]) {
    const uint2 t = __ldg(reinterpret_cast<const uint2 *>(p));
    v[0] = __uint_as_float(t.x << 16);
    v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16);
    v[3] = __uint_as_float(t.y & 0xffff0000u);
  }
};

template <> struct RowVec4<__half> {
  static constexpr int kElems = 4;
  __device__ static __forceinline__ void load(const __half *p, float (&v)[4]) {
    const uint2 t = __ldg(reinterpret_cast<const uint2 *>(p));
    const float2 a = widen_half2(t.x), b = widen_half2(t.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
};

// Vectorised fire-and-forget fp32 reduction into global memory (one 16-byte L2 atomic, sm_90+).
__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}
__device__ __forceinline__ void red_add(float *addr, float a) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ void red_add_v2(float *addr, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

// grad_dist[pix, z0] += a_lo ; grad_dist[pix, z0+1] += a_hi  (each only if the bin is inside
// [0, Dlim-1]).  The pair is adjacent, so it goes out as one 8-byte vector reduction when it is 8-byte
// aligned, as one 16-byte reduction padded with zeros when it sits in the middle of an aligned 16-byte
// block that lies wholly inside the pixel's row, and as two scalars otherwise: 1.25 L2 reduction
// packets per corner on average where two scalars were 2.
__device__ __forceinline__ void red_depth_pair(float *gd_bh, int pix_stride, int pix, int z0, int Dlim,
                                               int Dchan, float a_lo, float a_hi) {
  const bool vlo = z0 >= 0 && z0 < Dlim, vhi = z0 + 1 >= 0 && z0 + 1 < Dlim;
  float *p = gd_bh + ((long long)pix * pix_stride + z0);
  if (vlo && vhi) {
    const uintptr_t addr = reinterpret_cast<uintptr_t>(p);
    if ((addr & 7) == 0) {
      red_add_v2(p, a_lo, a_hi);
    } else if ((addr & 15) == 4 && z0 >= 1 && z0 + 2 < Dchan) {
      red_add_v4(p - 1, 0.f, a_lo, a_hi, 0.f);
    } else {
      red_add(p, a_lo);
      red_add(p + 1, a_hi);
    }
  } else if (vlo) {
    red_add(p, a_lo);
  } else if (vhi) {
    red_add(p + 1, a_hi);
  }
}

}  // namespace dfa3d
