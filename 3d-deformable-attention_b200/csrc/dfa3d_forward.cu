// DFA3D forward kernels (sm_100a).
//
// One warp owns one (camera b, query q, head h) item.  The L*P sampling points of the item are taken
// 32 at a time:
//   prologue  -- lane j owns point j: it reads its location and attention weight (coalesced), derives
//                the four bilinear corners, and (fused mode) gathers the 8 depth-distribution values
//                that give the four per-corner depth scores; it leaves one {row offset, weight} pair
//                per corner in the warp's slice of shared memory;
//   gather    -- the warp walks the (point, corner) rows; a group of G lanes reads one value row with
//                16-byte loads (4 fp32 or 8 bf16 channels per lane), so one warp-wide request fetches
//                32/G rows, and every lane
//                accumulates weight * row fragment;
//   epilogue  -- the 32/G partial sums are folded with xor-shuffles and G lanes store the output row.
// This replaces the reference's pair of kernels (one thread per (b,q,h) for the depth scores,
// ms_depth_score_sample_cuda_kernel.cuh:94-148; one thread per output channel for the attention,
// wms_deform_attn_cuda_kernel.cuh:240-303) and the depth_score round trip through HBM between them.
//
// The kernels are issue-bound as much as memory-bound (ncu: issue slots 2/3 busy), so index
// arithmetic is kept 32-bit: the grid's y dimension is the camera, 64-bit bases are formed once per
// warp, and when L*P is a multiple of 32 (FULL) the row loop has a compile-time trip count.
#include "dfa3d_common.cuh"
#include "dfa3d_launch.h"

namespace dfa3d {

// ------------------------------------------------------------------------------------------------
// prologue: per-lane point -> 4 row entries (+ depth scores)
// ------------------------------------------------------------------------------------------------
template <typename DT, int MODE>
__device__ __forceinline__ void fwd_point(const KArgs &a, const LevelTable &lv, const ItemCtx &c, int j,
                                          const SoftmaxStats &sm, float (&ds)[4], float (&wgt)[4],
                                          int (&off)[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) { ds[k] = 0.f; wgt[k] = 0.f; off[k] = -1; }
  if (j >= a.LP) return;
  const int l = j / a.P;
  float x, y, z, aw;
  read_point<MODE>(a, lv, c, j, l, sm, x, y, z, aw);
  const PointGeo g = point_geometry(x, y, z, mode_has_depth(MODE), lv.h[l], lv.w[l], lv.d[l], lv.start[l],
                                    a.N, dist_map_of(a, lv, l));
  if (!g.ok2) return;
  float bw[4];
  bilinear_weights(g, bw);
  if (mode_has_depth(MODE)) {
    const DT *dist_bh = reinterpret_cast<const DT *>(a.dist) +
                        ((long long)c.b * a.Nd * a.dist_pix_stride + c.h * a.dist_head_stride);
    float lo[4], hi[4];
    const int Dlim = min(g.Dd, a.D);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      load_depth_pair(dist_bh, a.dist_pix_stride, g.dpix[k], g.z0, Dlim, g.ok3, lo[k], hi[k]);
    const float hd = 1.f - g.ld;
#pragma unroll
    for (int k = 0; k < 4; ++k) ds[k] = g.ok3 ? lo[k] * hd + hi[k] * g.ld : 0.f;
  } else {
    // no depth-score tensor = plain 2-D multi-scale deformable attention: every in-image corner counts 1
    const float4 t = a.ds_in ? __ldg(reinterpret_cast<const float4 *>(a.ds_in) + (c.pt0 + j))
                             : make_float4(1.f, 1.f, 1.f, 1.f);
    ds[0] = g.pix[0] >= 0 ? t.x : 0.f;
    ds[1] = g.pix[1] >= 0 ? t.y : 0.f;
    ds[2] = g.pix[2] >= 0 ? t.z : 0.f;
    ds[3] = g.pix[3] >= 0 ? t.w : 0.f;
  }
  const int row = a.H * a.C;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float w = aw * (bw[k] * ds[k]);
    if (g.pix[k] >= 0 && w != 0.f) {     // rows that would add nothing are not fetched
      off[k] = g.pix[k] * row;
      wgt[k] = w;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// fused / given-depth-score / caller-fused forward; C/V a power of two, V = channels per 16 bytes
// ------------------------------------------------------------------------------------------------
// One item: the L*P points of (camera c.b, query, head c.h), 32 at a time; `table` is the warp's slice
// of the row table in shared memory.
template <typename VT, typename DT, int C, int MODE, bool WRITE_DS, bool FULL>
__device__ __forceinline__ void forward_item(const KArgs &a, const LevelTable &lv, const ItemCtx &c,
                                             RowEntry *table, int lane) {
  constexpr int V = RowVec<VT>::kElems;   // channels per lane
  constexpr int G = C / V;                // lanes per row
  constexpr int R = 32 / G;               // rows per warp-wide request
  constexpr int U = 4;                    // requests in flight per lane
  static_assert(G >= 1 && G <= 32 && (G & (G - 1)) == 0, "C/V must be a power of two <= 32");
  const VT *vbase = reinterpret_cast<const VT *>(a.value) + (((long long)c.b * a.N * a.H + c.h) * C +
                                                             (lane % G) * V);
  const RowEntry *my = table + lane / G;

  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  SoftmaxStats sm{0.f, 1.f};
  if (MODE == kCallerFused) sm = item_softmax_stats(a, c, lane);

  for (int chunk = 0; chunk < a.LP; chunk += 32) {
    float ds[4], wgt[4];
    int off[4];
    fwd_point<DT, MODE>(a, lv, c, chunk + lane, sm, ds, wgt, off);
    store_rows(table, lane, off, wgt);
    if (WRITE_DS && chunk + lane < a.LP)
      reinterpret_cast<float4 *>(a.ds_out)[c.pt0 + chunk + lane] = make_float4(ds[0], ds[1], ds[2], ds[3]);
    __syncwarp();
    // R*U rows per step: U independent row-fragment loads in flight per lane, then U fused multiply-adds.
    auto step = [&](int r0, int nrows) {
      RowEntry e[U];
      float v[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = r0 + u * R;
        e[u] = (FULL || r + lane / G < nrows) ? my[r] : RowEntry{-1, 0.f};
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (e[u].off >= 0) {
          RowVec<VT>::load(vbase + e[u].off, v[u]);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) v[u][i] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fmaf(e[u].wgt, v[u][i], acc[i]);
    };
    if (FULL) {          // 128 rows: compile-time trip count, table offsets become immediates
#pragma unroll
      for (int r0 = 0; r0 < 128; r0 += R * U) step(r0, 128);
    } else {
      const int nrows = min(32, a.LP - chunk) * 4;
#pragma unroll 1
      for (int r0 = 0; r0 < nrows; r0 += R * U) step(r0, nrows);
    }
    __syncwarp();
  }
#pragma unroll
  for (int s = G; s < 32; s <<= 1)
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], s);
  if (lane < G) {
    float *o = a.out + (c.item * C + lane * V);
#pragma unroll
    for (int i = 0; i < V; i += 4)
      *reinterpret_cast<float4 *>(o + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
  }
}

// 5 CTAs (40 warps) per SM: measured best; at 6+ the register cap starts to cost more than the
// extra warps hide.  A CTA walks DFA3D_FWD_ITEMS_PER_WARP consecutive groups of 8 items (the grid's
// ~60 000 CTAs per camera otherwise live ~2 us each and their turnover shows: measured -7 % at 8).
template <typename VT, typename DT, int C, int MODE, bool WRITE_DS, bool FULL>
__global__ void __launch_bounds__(kThreads, DFA3D_FWD_MIN_CTAS)
dfa3d_forward_kernel(const KArgs a) {
  __shared__ LevelTable lv;
  __shared__ __align__(16) RowEntry rows[kWarpsPerCta][128];
  stage_levels(lv, a);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
  for (int it = 0; it < DFA3D_FWD_ITEMS_PER_WARP; ++it) {
    ItemCtx c;
    if (!item_context<DFA3D_FWD_HEAD_MAJOR != 0>(a, warp, blockIdx.x * DFA3D_FWD_ITEMS_PER_WARP + it, c)) return;
    forward_item<VT, DT, C, MODE, WRITE_DS, FULL>(a, lv, c, rows[warp], lane);
  }
}

// ------------------------------------------------------------------------------------------------
// any C: lanes stride over channels, rows walked one by one (correctness path for unusual widths)
// ------------------------------------------------------------------------------------------------
template <typename VT, typename DT, int MODE, bool WRITE_DS>
__global__ void __launch_bounds__(kThreads)
dfa3d_forward_generic_kernel(const KArgs a) {
  __shared__ LevelTable lv;
  __shared__ __align__(16) RowEntry rows[kWarpsPerCta][128];
  stage_levels(lv, a);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  ItemCtx c;
  if (!item_context(a, warp, blockIdx.x, c)) return;
  const int C = a.C;
  const VT *vbase = reinterpret_cast<const VT *>(a.value) + ((long long)c.b * a.N * a.H + c.h) * C;
  RowEntry *my = rows[warp];
  SoftmaxStats sm{0.f, 1.f};
  if (MODE == kCallerFused) sm = item_softmax_stats(a, c, lane);
  for (int c0 = 0; c0 < C; c0 += 32) {          // C <= 1024: at most 32 passes
    const int ch = c0 + lane;
    float acc = 0.f;
    for (int chunk = 0; chunk < a.LP; chunk += 32) {
      float ds[4], wgt[4];
      int off[4];
      fwd_point<DT, MODE>(a, lv, c, chunk + lane, sm, ds, wgt, off);
      store_rows(my, lane, off, wgt);
      if (WRITE_DS && c0 == 0 && chunk + lane < a.LP)
        reinterpret_cast<float4 *>(a.ds_out)[c.pt0 + chunk + lane] =
            make_float4(ds[0], ds[1], ds[2], ds[3]);
      __syncwarp();
      const int nrows = min(32, a.LP - chunk) * 4;
      if (ch < C)
        for (int r = 0; r < nrows; ++r) {
          const RowEntry e = my[r];
          if (e.off >= 0) acc = fmaf(e.wgt, load_scalar(vbase + e.off + ch), acc);
        }
      __syncwarp();
    }
    if (ch < C) a.out[c.item * C + ch] = acc;
  }
}

// ------------------------------------------------------------------------------------------------
// depth scores only (two-stage API): one thread per sampling point
// ------------------------------------------------------------------------------------------------
template <typename DT>
__global__ void __launch_bounds__(kThreads)
dfa3d_depth_score_forward_kernel(const KArgs a) {
  __shared__ LevelTable lv;
  stage_levels(lv, a);
  const long long npts = a.items * a.LP;
  for (long long pt = (long long)blockIdx.x * blockDim.x + threadIdx.x; pt < npts;
       pt += (long long)gridDim.x * blockDim.x) {
    const long long item = pt / a.LP;
    const int j = (int)(pt - item * a.LP);
    const int l = j / a.P;
    const int h = (int)(item % a.H);
    const int b = (int)(item / a.items_per_cam);
    const float *lp = a.loc + pt * 3;
    const PointGeo g = point_geometry(__ldg(lp), __ldg(lp + 1), __ldg(lp + 2), true, lv.h[l], lv.w[l],
                                      lv.d[l], lv.start[l], a.N, dist_map_of(a, lv, l));
    const DT *dist_bh = reinterpret_cast<const DT *>(a.dist) +
                        ((long long)b * a.Nd * a.dist_pix_stride + h * a.dist_head_stride);
    float ds[4];
    const float hd = 1.f - g.ld;
    const int Dlim = min(g.Dd, a.D);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float lo, hi;
      load_depth_pair(dist_bh, a.dist_pix_stride, g.dpix[k], g.z0, Dlim, g.ok3, lo, hi);
      ds[k] = g.ok3 ? lo * hd + hi * g.ld : 0.f;
    }
    reinterpret_cast<float4 *>(a.ds_out)[pt] = make_float4(ds[0], ds[1], ds[2], ds[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// few points per item (L*P = 4, 8 or 16): a warp takes 32 / (L*P) consecutive items at once
// ------------------------------------------------------------------------------------------------
// With one item per warp an item of 4 points (temporal self-attention and the decoder's cross-attention
// use 1 level x 4 points) keeps 4 lanes busy in the prologue and costs a whole chain of dependent
// latencies (locations -> row table -> rows -> sum -> store) for 16 rows.  Here lane j owns point
// j % LP of item j / LP, so the prologue is full and coalesced (the points of consecutive items are
// consecutive in memory); a group of G lanes then sums all rows of one item (or, when the warp holds
// fewer items than groups, a share of them) and writes that item's output itself.
// A warp takes kPackedRounds batches of 32 points before its CTA retires (a batch is several items
// here, so fewer rounds than DFA3D_FWD_ITEMS_PER_WARP keep the grid several waves deep at 40 000 queries).
constexpr int kPackedRounds = 2;

// CTAs per SM the packed forward is compiled for: 6 (48 warps; the kernel waits on chains of dependent
// loads) measured 1-4 % faster than 5 and 4-8 % faster than 4 at 4, 8 and 16 points per item.
#ifndef DFA3D_FWD_PACKED_MIN_CTAS
#define DFA3D_FWD_PACKED_MIN_CTAS 6
#endif
template <typename VT, typename DT, int C, int MODE, bool WRITE_DS, int LP>
__global__ void __launch_bounds__(kThreads, DFA3D_FWD_PACKED_MIN_CTAS)
dfa3d_forward_packed_kernel(const KArgs a) {
  constexpr int V = RowVec<VT>::kElems;
  constexpr int G = C / V;                      // lanes per row
  constexpr int R = 32 / G;                     // groups per warp
  constexpr int K = 32 / LP;                    // items per warp
  constexpr int GPI = R > K ? R / K : 1;        // groups sharing one item
  constexpr int IPG = K > R ? K / R : 1;        // items one group handles in turn
  constexpr int U = 4;
  constexpr int kRows = LP * 4;                 // rows of one item
  static_assert(32 % LP == 0 && 32 % G == 0 && kRows % (GPI * U) == 0, "unsupported packing");
  __shared__ LevelTable lv;
  __shared__ __align__(16) RowEntry rows[kWarpsPerCta][128];
  stage_levels(lv, a);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % G, grp = lane / G;
  const int b = (int)blockIdx.y + a.b0;
  const VT *vbase = reinterpret_cast<const VT *>(a.value) + ((long long)b * a.N * a.H * C + sub * V);
  RowEntry *table = rows[warp];
  // the camera's queries: rows [q0, q0 + nq) of the per-query tensors
  const long long q0 = a.q_off ? (long long)__ldg(a.q_off + b) : (long long)b * a.Q;
  const unsigned nitems = (unsigned)(a.q_off ? __ldg(a.q_off + b + 1) - (int)q0 : a.Q) * (unsigned)a.H;
#pragma unroll 1
  for (int it = 0; it < kPackedRounds; ++it) {
    const unsigned first = ((blockIdx.x * kPackedRounds + it) * kWarpsPerCta + warp) * K;
    if (first >= nitems) return;
    {
      const unsigned idx = first + lane / LP;
      const bool live = idx < nitems;
      ItemCtx c;
      c.b = b;
      const unsigned q = idx / (unsigned)a.H;
      c.h = (int)(idx - q * (unsigned)a.H);
      c.bq = q0 + q;
      c.item = q0 * a.H + idx;
      c.pt0 = c.item * LP;
      c.loc = a.loc + c.pt0 * a.loc_stride;      // (not dereferenced in caller-fused mode)
      c.attn = a.attn + c.pt0;
      const int j = lane % LP;
      SoftmaxStats sm{0.f, 1.f};
      if (MODE == kCallerFused) {                // softmax over the item's LP logits: its own LP lanes
        const float lg = live ? __ldg(a.logits + c.pt0 + j) : -INFINITY;
        float mx = lg;
#pragma unroll
        for (int s = LP / 2; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        float sum = live ? expf(lg - mx) : 0.f;
#pragma unroll
        for (int s = LP / 2; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
        sm = SoftmaxStats{mx, sum};
      }
      float ds[4], wgt[4];
      int off[4];
      fwd_point<DT, MODE>(a, lv, c, live ? j : a.LP, sm, ds, wgt, off);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (off[k] >= 0) off[k] += c.h * C;     // rows of different heads share the table
      store_rows(table, lane, off, wgt);
      if (WRITE_DS && live)
        reinterpret_cast<float4 *>(a.ds_out)[c.pt0 + j] = make_float4(ds[0], ds[1], ds[2], ds[3]);
    }
    __syncwarp();
#pragma unroll
    for (int t = 0; t < IPG; ++t) {
      const int i = grp / GPI + t * (R / GPI);  // item of the warp this group works on
      const RowEntry *my = table + i * kRows + (grp % GPI) * U;
      float acc[V];
#pragma unroll
      for (int x = 0; x < V; ++x) acc[x] = 0.f;
#pragma unroll
      for (int r0 = 0; r0 < kRows; r0 += GPI * U) {
        RowEntry e[U];
        float v[U][V];
#pragma unroll
        for (int u = 0; u < U; ++u) e[u] = my[r0 + u];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (e[u].off >= 0) {
            RowVec<VT>::load(vbase + e[u].off, v[u]);
          } else {
#pragma unroll
            for (int x = 0; x < V; ++x) v[u][x] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int x = 0; x < V; ++x) acc[x] = fmaf(e[u].wgt, v[u][x], acc[x]);
      }
#pragma unroll
      for (int s = G; s < G * GPI; s <<= 1)
#pragma unroll
        for (int x = 0; x < V; ++x) acc[x] += __shfl_xor_sync(0xffffffffu, acc[x], s);
      const unsigned idx = first + i;
      if (grp % GPI == 0 && idx < nitems) {
        float *o = a.out + ((q0 * a.H + idx) * C + sub * V);
#pragma unroll
        for (int x = 0; x < V; x += 4)
          *reinterpret_cast<float4 *>(o + x) = make_float4(acc[x], acc[x + 1], acc[x + 2], acc[x + 3]);
      }
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------------------------------------
// host-side dispatch
// ------------------------------------------------------------------------------------------------
static dim3 item_grid(const KArgs &a, int cams, int items_per_warp) {
  const int per_cta = kWarpsPerCta * items_per_warp;
  return dim3((unsigned)((a.items_per_cam + per_cta - 1) / per_cta), (unsigned)cams, 1);
}

template <typename VT, typename DT, int MODE, bool WRITE_DS, bool FULL>
static void launch_forward_g(const KArgs &a, dim3 grid, cudaStream_t s) {
  constexpr int V = RowVec<VT>::kElems;
  switch ((a.C % V == 0) ? a.C / V : 0) {
    case 2:  dfa3d_forward_kernel<VT, DT, 2 * V, MODE, WRITE_DS, FULL><<<grid, kThreads, 0, s>>>(a); break;
    case 4:  dfa3d_forward_kernel<VT, DT, 4 * V, MODE, WRITE_DS, FULL><<<grid, kThreads, 0, s>>>(a); break;
    case 8:  dfa3d_forward_kernel<VT, DT, 8 * V, MODE, WRITE_DS, FULL><<<grid, kThreads, 0, s>>>(a); break;
    case 16: dfa3d_forward_kernel<VT, DT, 16 * V, MODE, WRITE_DS, FULL><<<grid, kThreads, 0, s>>>(a); break;
    case 32: dfa3d_forward_kernel<VT, DT, 32 * V, MODE, WRITE_DS, FULL><<<grid, kThreads, 0, s>>>(a); break;
    default:
      dfa3d_forward_generic_kernel<VT, DT, MODE, WRITE_DS><<<item_grid(a, (int)grid.y, 1), kThreads, 0, s>>>(a);
      break;
  }
}

// Packed kernels: float storage, 16 / 32 / 64 channels, 4 / 8 / 16 points per item.  Returns false when the
// call is not one of those.
template <int MODE, bool WRITE_DS, int LP>
static bool launch_forward_packed_c(const KArgs &a, dim3 grid, cudaStream_t s) {
  switch (a.C) {
    case 16: dfa3d_forward_packed_kernel<float, float, 16, MODE, WRITE_DS, LP><<<grid, kThreads, 0, s>>>(a); return true;
    case 32: dfa3d_forward_packed_kernel<float, float, 32, MODE, WRITE_DS, LP><<<grid, kThreads, 0, s>>>(a); return true;
    case 64: dfa3d_forward_packed_kernel<float, float, 64, MODE, WRITE_DS, LP><<<grid, kThreads, 0, s>>>(a); return true;
    default: return false;
  }
}

template <int MODE>
static bool launch_forward_packed(const KArgs &a, int cams, cudaStream_t s) {
  if (a.LP != 4 && a.LP != 8 && a.LP != 16) return false;
  const int per_cta = kWarpsPerCta * kPackedRounds * (32 / a.LP);
  const dim3 grid((unsigned)((a.items_per_cam + per_cta - 1) / per_cta), (unsigned)cams, 1);
  constexpr bool kCanWriteDs = MODE != kCallerFused;          // the caller-fused entry points return no depth score
  if (kCanWriteDs && a.ds_out) {
    if (a.LP == 4) return launch_forward_packed_c<MODE, kCanWriteDs, 4>(a, grid, s);
    if (a.LP == 8) return launch_forward_packed_c<MODE, kCanWriteDs, 8>(a, grid, s);
    return launch_forward_packed_c<MODE, kCanWriteDs, 16>(a, grid, s);
  }
  if (a.LP == 4) return launch_forward_packed_c<MODE, false, 4>(a, grid, s);
  if (a.LP == 8) return launch_forward_packed_c<MODE, false, 8>(a, grid, s);
  return launch_forward_packed_c<MODE, false, 16>(a, grid, s);
}

template <typename VT, typename DT> struct IsFloatPair { static constexpr bool value = false; };
template <> struct IsFloatPair<float, float> { static constexpr bool value = true; };

template <typename VT, typename DT, int MODE>
static cudaError_t launch_forward_vd(const KArgs &a0, cudaStream_t s) {
  const bool full = a0.LP % 32 == 0;
  for (int b0 = 0; b0 < a0.B; b0 += 65535) {      // grid.y limit
    KArgs a = a0;
    a.b0 = b0;
    if (IsFloatPair<VT, DT>::value && launch_forward_packed<MODE>(a, min(65535, a0.B - b0), s)) {
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      continue;
    }
    const dim3 grid = item_grid(a, min(65535, a0.B - b0), DFA3D_FWD_ITEMS_PER_WARP);
    if (a.ds_out) {
      if (full) launch_forward_g<VT, DT, MODE, true, true>(a, grid, s);
      else launch_forward_g<VT, DT, MODE, true, false>(a, grid, s);
    } else {
      if (full) launch_forward_g<VT, DT, MODE, false, true>(a, grid, s);
      else launch_forward_g<VT, DT, MODE, false, false>(a, grid, s);
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// Storage types are the DFA3D_DTYPE_* codes of the C header.  fp32 and bf16 combine freely; fp16 value
// goes with fp16 dist (what a half-precision caller passes) -- the C entry points reject the rest.
template <int MODE>
static cudaError_t launch_forward_m(const KArgs &a, int value_dtype, int dist_dtype, cudaStream_t s) {
  if (value_dtype == kDtypeF16) return launch_forward_vd<__half, __half, MODE>(a, s);
  if (value_dtype == kDtypeBF16)
    return dist_dtype == kDtypeBF16 ? launch_forward_vd<__nv_bfloat16, __nv_bfloat16, MODE>(a, s)
                                    : launch_forward_vd<__nv_bfloat16, float, MODE>(a, s);
  return dist_dtype == kDtypeBF16 ? launch_forward_vd<float, __nv_bfloat16, MODE>(a, s)
                                  : launch_forward_vd<float, float, MODE>(a, s);
}

cudaError_t launch_forward(const KArgs &a, int value_dtype, int dist_dtype, int mode, cudaStream_t s) {
  if (a.items == 0) return cudaSuccess;
  if (mode == kGivenDepthScore) {   // dist is not read: its type parameter is irrelevant
    if (value_dtype == kDtypeF16) return launch_forward_vd<__half, float, kGivenDepthScore>(a, s);
    return value_dtype == kDtypeBF16 ? launch_forward_vd<__nv_bfloat16, float, kGivenDepthScore>(a, s)
                                     : launch_forward_vd<float, float, kGivenDepthScore>(a, s);
  }
  if (mode == kCallerFused) return launch_forward_m<kCallerFused>(a, value_dtype, dist_dtype, s);
  return launch_forward_m<kFused>(a, value_dtype, dist_dtype, s);
}

cudaError_t launch_depth_score_forward(const KArgs &a, int dist_dtype, cudaStream_t s) {
  const long long npts = a.items * a.LP;
  if (npts == 0) return cudaSuccess;
  const unsigned grid = (unsigned)min((npts + kThreads - 1) / kThreads, (long long)148 * 64);
  if (dist_dtype == kDtypeF16) dfa3d_depth_score_forward_kernel<__half><<<grid, kThreads, 0, s>>>(a);
  else if (dist_dtype == kDtypeBF16) dfa3d_depth_score_forward_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(a);
  else dfa3d_depth_score_forward_kernel<float><<<grid, kThreads, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace dfa3d
