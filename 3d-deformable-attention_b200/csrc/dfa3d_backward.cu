// DFA3D backward kernels (sm_100a).
//
// Same decomposition as the forward: one warp per (camera, query, head) item, lane j owns sampling
// point j of a 32-point chunk.  Per chunk:
//   prologue -- the lane recomputes its point's geometry and per-corner depth scores from `dist`
//               (fused mode; the (B,Q,H,L,P,4) depth_score tensor is never read back) and publishes
//               {row offset, a * bilinear * depth score} per corner in shared memory;
//   rows     -- a group of G lanes reads one value row (4 channels per lane), takes its dot product with
//               the item's grad_out row (xor-shuffles inside the group) and adds
//               weight * grad_out to grad_value with one 16-byte vector reduction per lane
//               (red.global.add.v4.f32) instead of one scalar atomic per channel;
//   epilogue -- the four dot products t_k of a point return to its owner lane through shared
//               memory; grad_attn, grad_loc (x, y and, fused, z), grad_depth_score and the grad_dist
//               atomics all follow from t_k and the quantities the lane already holds.
// No block-wide barrier and no serial thread-0 reduction remain
// (cf. wms_deform_attn_cuda_kernel.cuh:378-407, ms_depth_score_sample_cuda_kernel.cuh:301-319).
#include "dfa3d_common.cuh"
#include "dfa3d_launch.h"

namespace dfa3d {

// Per-lane state of one sampling point that the epilogue needs.
struct PointState {
  PointGeo g;
  float aw;
  float bw[4], ds[4];
  float dz[4];          // dist[z0+1] - dist[z0] per corner (fused mode): d depth_score / d depth
  bool live;            // j < LP && ok2
};

template <typename DT, int MODE>
__device__ __forceinline__ void bwd_point(const KArgs &a, const LevelTable &lv, const ItemCtx &c, int j,
                                          const SoftmaxStats &sm, PointState &s, float (&wgt)[4],
                                          int (&off)[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    s.ds[k] = 0.f; s.bw[k] = 0.f; s.dz[k] = 0.f; wgt[k] = 0.f; off[k] = -1;
    s.g.pix[k] = -1; s.g.dpix[k] = -1;
  }
  s.live = false; s.aw = 0.f; s.g.ok2 = false; s.g.ok3 = false;
  if (j >= a.LP) return;
  const int l = j / a.P;
  float x, y, z;
  read_point<MODE>(a, lv, c, j, l, sm, x, y, z, s.aw);
  s.g = point_geometry(x, y, z, mode_has_depth(MODE), lv.h[l], lv.w[l], lv.d[l], lv.start[l], a.N,
                       dist_map_of(a, lv, l));
  if (!s.g.ok2) return;
  s.live = true;
  bilinear_weights(s.g, s.bw);
  if (mode_has_depth(MODE)) {
    const DT *dist_bh = reinterpret_cast<const DT *>(a.dist) +
                        ((long long)c.b * a.Nd * a.dist_pix_stride + c.h * a.dist_head_stride);
    const int Dlim = min(s.g.Dd, a.D);
    float lo[4], hi[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      load_depth_pair(dist_bh, a.dist_pix_stride, s.g.dpix[k], s.g.z0, Dlim, s.g.ok3, lo[k], hi[k]);
    const float hd = 1.f - s.g.ld;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      s.ds[k] = s.g.ok3 ? lo[k] * hd + hi[k] * s.g.ld : 0.f;
      s.dz[k] = hi[k] - lo[k];
    }
  } else {
    const float4 t = a.ds_in ? __ldg(reinterpret_cast<const float4 *>(a.ds_in) + (c.pt0 + j))
                             : make_float4(1.f, 1.f, 1.f, 1.f);
    s.ds[0] = s.g.pix[0] >= 0 ? t.x : 0.f;
    s.ds[1] = s.g.pix[1] >= 0 ? t.y : 0.f;
    s.ds[2] = s.g.pix[2] >= 0 ? t.z : 0.f;
    s.ds[3] = s.g.pix[3] >= 0 ? t.w : 0.f;
  }
  const int row = a.H * a.C;
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (s.g.pix[k] >= 0) {
      off[k] = s.g.pix[k] * row;
      wgt[k] = s.aw * (s.bw[k] * s.ds[k]);
    }
}

// Everything that follows from the four dot products t[k] = <value row k, grad_out row>.
// Returns attention weight x its gradient (the point's term of the softmax-backward dot product;
// used in caller-fused mode only).
template <typename DT, int MODE>
__device__ __forceinline__ float bwd_point_epilogue(const KArgs &a, const ItemCtx &c, int j,
                                                    const PointState &s, const float (&t)[4]) {
  if (j >= a.LP) return 0.f;
  const long long pt = c.pt0 + j;
  float g_attn = 0.f, g_x = 0.f, g_y = 0.f, g_z = 0.f;
  float gds[4] = {0.f, 0.f, 0.f, 0.f};
  if (s.live) {
    const float hw = 1.f - s.g.lw, hh = 1.f - s.g.lh;
    float tt[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) tt[k] = s.g.pix[k] >= 0 ? t[k] : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      g_attn = fmaf(s.bw[k] * s.ds[k], tt[k], g_attn);
      gds[k] = s.g.pix[k] >= 0 ? s.aw * (s.bw[k] * tt[k]) : 0.f;
    }
    const float e0 = s.ds[0] * tt[0], e1 = s.ds[1] * tt[1], e2 = s.ds[2] * tt[2], e3 = s.ds[3] * tt[3];
    g_x = (float)s.g.W * s.aw * (hh * (e1 - e0) + s.g.lh * (e2 - e3));
    g_y = (float)s.g.Hh * s.aw * (hw * (e3 - e0) + s.g.lw * (e2 - e1));
    if (mode_has_depth(MODE) && s.g.ok3) {
      float *gd_bh = a.grad_dist + ((long long)c.b * a.Nd * a.dist_pix_stride + c.h * a.dist_head_stride);
      const float hd = 1.f - s.g.ld;
      const int Dlim = min(s.g.Dd, a.D);
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (s.g.pix[k] >= 0) {
          if (gds[k] != 0.f)
            red_depth_pair(gd_bh, a.dist_pix_stride, s.g.dpix[k], s.g.z0, Dlim, a.D, hd * gds[k],
                           s.g.ld * gds[k]);
          acc = fmaf(gds[k], s.dz[k], acc);
        }
      }
      g_z = (float)s.g.Dd * acc;
    }
  }
  if (MODE == kCallerFused) {
    // d loc / d offset = 1 / (W, H, D); the logit gradient needs the whole item's dot product and is
    // finished by finish_logit_grads(): park the attention gradient in its slot for now
    a.grad_logits[pt] = g_attn;
    float *gu = a.grad_off_uv + pt * 2;
    gu[0] = s.live ? __fdiv_rn(g_x, (float)s.g.W) : 0.f;
    gu[1] = s.live ? __fdiv_rn(g_y, (float)s.g.Hh) : 0.f;
    a.grad_off_d[pt] = __fdiv_rn(g_z, (float)a.D);
    return s.aw * g_attn;
  }
  a.grad_attn[pt] = g_attn;
  float *gl = a.grad_loc + pt * a.loc_stride;
  gl[0] = g_x;
  gl[1] = g_y;
  if (MODE == kFused) gl[2] = g_z;
  if (a.grad_ds_out)
    reinterpret_cast<float4 *>(a.grad_ds_out)[pt] = make_float4(gds[0], gds[1], gds[2], gds[3]);
  return 0.f;
}

// Softmax backward of the item's logits: grad_logit_j = a_j * (g_j - sum_k a_k g_k).  `partial` is the
// lane's share of the sum; the g_j were parked in grad_logits by the epilogue (each lane re-reads only
// what it wrote itself).
__device__ __forceinline__ void finish_logit_grads(const KArgs &a, const ItemCtx &c, int lane,
                                                   const SoftmaxStats &sm, float partial) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, s);
  for (int j = lane; j < a.LP; j += 32) {
    const long long pt = c.pt0 + j;
    const float aw = __fdiv_rn(expf(__ldg(a.logits + pt) - sm.mx), sm.sum);
    a.grad_logits[pt] = aw * (a.grad_logits[pt] - partial);
  }
}

// ------------------------------------------------------------------------------------------------
// fused / given-depth-score backward, C/4 a power of two
// ------------------------------------------------------------------------------------------------
// Dot products of U = 4 row fragments with the grad_out fragment, summed over the G lanes of a group.
// For G = 8 the four sums are folded together: after the first exchange a lane keeps two of them, after
// the second one, so the whole reduction takes 4 shuffles instead of 12 and lane `sub` < 4 of every
// group ends up with the total of row u = 2*(sub & 1) + ((sub >> 1) & 1).  Shuffles travel through the
// same pipe as the shared-memory and global accesses this kernel is bound by.
// Returns the lane's total and, in `u_mine`, which of the four rows it belongs to (-1: none).
template <int G>
__device__ __forceinline__ float fold_four_dots(const float (&d)[4], int sub, int &u_mine) {
  if (G == 8) {
    const bool b0 = sub & 1, b1 = sub & 2;
    const float r0 = __shfl_xor_sync(0xffffffffu, b0 ? d[0] : d[2], 1);
    const float r1 = __shfl_xor_sync(0xffffffffu, b0 ? d[1] : d[3], 1);
    const float e0 = (b0 ? d[2] : d[0]) + r0, e1 = (b0 ? d[3] : d[1]) + r1;
    const float r2 = __shfl_xor_sync(0xffffffffu, b1 ? e0 : e1, 2);
    float f = (b1 ? e1 : e0) + r2;
    f += __shfl_xor_sync(0xffffffffu, f, 4);
    u_mine = sub < 4 ? (b0 ? 2 : 0) + (b1 ? 1 : 0) : -1;
    return f;
  }
  // other group widths (G = 4, 16, 32): one butterfly per row, lane u of the group keeps row u
  float mine = 0.f;
  u_mine = -1;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    float t = d[u];
#pragma unroll
    for (int s = 1; s < G; s <<= 1) t += __shfl_xor_sync(0xffffffffu, t, s);
    if (sub == u) { mine = t; u_mine = u; }
  }
  return mine;
}

// One item of the backward: `table` / `dot_slots` are the warp's slices of shared memory.
template <typename VT, typename DT, int C, int MODE, bool FULL>
__device__ __forceinline__ void backward_item(const KArgs &a, const LevelTable &lv, const ItemCtx &c,
                                              RowEntry *table, float *dot_slots, int lane) {
  constexpr int V = RowVec4<VT>::kElems;
  constexpr int G = C / V;
  constexpr int R = 32 / G;
  constexpr int U = 4;
  const int sub = lane % G, grp = lane / G;
  const long long slice = ((long long)c.b * a.N * a.H + c.h) * C + sub * V;
  const VT *vbase = reinterpret_cast<const VT *>(a.value) + slice;
  float *gvbase = a.grad_value + slice;
  const RowEntry *my = table + grp;
  float *myd = dot_slots + grp;

  float go[V];
  {
    const float *gp = a.grad_out + (c.item * C + sub * V);
#pragma unroll
    for (int i = 0; i < V; i += 4) {
      const float4 t = __ldg(reinterpret_cast<const float4 *>(gp + i));
      go[i] = t.x; go[i + 1] = t.y; go[i + 2] = t.z; go[i + 3] = t.w;
    }
  }

  SoftmaxStats sm{0.f, 1.f};
  if (MODE == kCallerFused) sm = item_softmax_stats(a, c, lane);
  float dot = 0.f;

  for (int chunk = 0; chunk < a.LP; chunk += 32) {
    PointState st;
    float wgt[4];
    int off[4];
    bwd_point<DT, MODE>(a, lv, c, chunk + lane, sm, st, wgt, off);
    store_rows(table, lane, off, wgt);
    __syncwarp();
    auto step = [&](int r0, int nrows) {
      RowEntry e[U];
      float v[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = r0 + u * R;
        e[u] = (FULL || r + grp < nrows) ? my[r] : RowEntry{-1, 0.f};
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (e[u].off >= 0) {
          RowVec4<VT>::load(vbase + e[u].off, v[u]);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) v[u][i] = 0.f;
        }
      }
      float d[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        d[u] = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) d[u] = fmaf(v[u][i], go[i], d[u]);
      }
      if (G >= 4) {
        int u_mine;
        const float f = fold_four_dots<G>(d, sub, u_mine);
        const int r = r0 + u_mine * R;
        if (u_mine >= 0 && (FULL || r + grp < nrows)) myd[r] = f;
      } else {
        // groups of 2 lanes (8 channels): a group's first lane stores its four totals one by one
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float t = d[u];
#pragma unroll
          for (int s = 1; s < G; s <<= 1) t += __shfl_xor_sync(0xffffffffu, t, s);
          const int r = r0 + u * R;
          if (sub == 0 && (FULL || r + grp < nrows)) myd[r] = t;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (e[u].off >= 0 && e[u].wgt != 0.f) {
          float *gp = gvbase + e[u].off;
#pragma unroll
          for (int i = 0; i < V; i += 4)
            red_add_v4(gp + i, e[u].wgt * go[i], e[u].wgt * go[i + 1], e[u].wgt * go[i + 2],
                       e[u].wgt * go[i + 3]);
        }
      }
    };
    const int nrows = FULL ? 128 : min(32, a.LP - chunk) * 4;
#pragma unroll 1
    for (int r0 = 0; r0 < nrows; r0 += R * U) step(r0, nrows);
    __syncwarp();
    const float4 tq = reinterpret_cast<const float4 *>(dot_slots)[lane];
    const float t[4] = {tq.x, tq.y, tq.z, tq.w};
    dot += bwd_point_epilogue<DT, MODE>(a, c, chunk + lane, st, t);
    __syncwarp();
  }
  if (MODE == kCallerFused) finish_logit_grads(a, c, lane, sm, dot);
}

// ------------------------------------------------------------------------------------------------
// fused / given-depth-score backward, C/4 a power of two
// ------------------------------------------------------------------------------------------------
// 4 CTAs (32 warps) per SM is the measured optimum (64 registers, a few bytes of spill); a CTA walks
// DFA3D_BWD_ITEMS_PER_WARP consecutive groups of 8 items before it retires.
template <typename VT, typename DT, int C, int MODE, bool FULL>
__global__ void __launch_bounds__(kThreads, DFA3D_BWD_MIN_CTAS)
dfa3d_backward_kernel(const KArgs a) {
  __shared__ LevelTable lv;
  __shared__ __align__(16) RowEntry rows[kWarpsPerCta][128];
  __shared__ __align__(16) float dots[kWarpsPerCta][128];
  stage_levels(lv, a);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
  for (int it = 0; it < DFA3D_BWD_ITEMS_PER_WARP; ++it) {
    ItemCtx c;
    if (!item_context<DFA3D_BWD_HEAD_MAJOR != 0>(a, warp, blockIdx.x * DFA3D_BWD_ITEMS_PER_WARP + it, c)) return;
    backward_item<VT, DT, C, MODE, FULL>(a, lv, c, rows[warp], dots[warp], lane);
  }
}

// ------------------------------------------------------------------------------------------------
// few points per item (L*P = 4, 8 or 16): a warp takes 32 / (L*P) consecutive items at once
// ------------------------------------------------------------------------------------------------
// Lane j owns point j % LP of item j / LP (full, coalesced prologue and epilogue); a group of G lanes
// walks the rows of one item -- or a share of them when the warp holds fewer items than groups -- with
// that item's grad_out fragment.  Same row phase as backward_item otherwise.
constexpr int kPackedRounds = 2;    // batches of 32 points a warp takes before its CTA retires

template <typename VT, typename DT, int C, int MODE, int LP>
__global__ void __launch_bounds__(kThreads, DFA3D_BWD_MIN_CTAS)
dfa3d_backward_packed_kernel(const KArgs a) {
  constexpr int V = RowVec4<VT>::kElems;
  constexpr int G = C / V;
  constexpr int R = 32 / G;
  constexpr int K = 32 / LP;
  constexpr int GPI = R > K ? R / K : 1;
  constexpr int IPG = K > R ? K / R : 1;
  constexpr int U = 4;
  constexpr int kRows = LP * 4;
  static_assert(G >= 4 && 32 % LP == 0 && 32 % G == 0 && kRows % (GPI * U) == 0, "unsupported packing");
  __shared__ LevelTable lv;
  __shared__ __align__(16) RowEntry rows[kWarpsPerCta][128];
  __shared__ __align__(16) float dots[kWarpsPerCta][128];
  stage_levels(lv, a);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % G, grp = lane / G;
  const int b = (int)blockIdx.y + a.b0;
  const long long cam = (long long)b * a.N * a.H * C + sub * V;
  const VT *vbase = reinterpret_cast<const VT *>(a.value) + cam;
  float *gvbase = a.grad_value + cam;
  RowEntry *table = rows[warp];
  float *dot_slots = dots[warp];
  // the camera's queries: rows [q0, q0 + nq) of the per-query tensors
  const long long q0 = a.q_off ? (long long)__ldg(a.q_off + b) : (long long)b * a.Q;
  const unsigned nitems = (unsigned)(a.q_off ? __ldg(a.q_off + b + 1) - (int)q0 : a.Q) * (unsigned)a.H;
#pragma unroll 1
  for (int it = 0; it < kPackedRounds; ++it) {
    const unsigned first = ((blockIdx.x * kPackedRounds + it) * kWarpsPerCta + warp) * K;
    if (first >= nitems) return;
    const unsigned idx = first + lane / LP;
    const bool live = idx < nitems;
    ItemCtx c;
    c.b = b;
    {
      const unsigned q = idx / (unsigned)a.H;
      c.h = (int)(idx - q * (unsigned)a.H);
      c.bq = q0 + q;
    }
    c.item = q0 * a.H + idx;
    c.pt0 = c.item * LP;
    c.loc = a.loc + c.pt0 * a.loc_stride;        // (not dereferenced in caller-fused mode)
    c.attn = a.attn + c.pt0;
    const int j = live ? lane % LP : a.LP;       // a.LP: no such point, the lane stays idle
    SoftmaxStats sm{0.f, 1.f};
    if (MODE == kCallerFused) {                  // softmax over the item's LP logits: its own LP lanes
      const float lg = live ? __ldg(a.logits + c.pt0 + j) : -INFINITY;
      float mx = lg;
#pragma unroll
      for (int s = LP / 2; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
      float sum = live ? expf(lg - mx) : 0.f;
#pragma unroll
      for (int s = LP / 2; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
      sm = SoftmaxStats{mx, sum};
    }
    PointState st;
    {
      float wgt[4];
      int off[4];
      bwd_point<DT, MODE>(a, lv, c, j, sm, st, wgt, off);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (off[k] >= 0) off[k] += c.h * C;
      store_rows(table, lane, off, wgt);
    }
    __syncwarp();
#pragma unroll
    for (int t = 0; t < IPG; ++t) {
      const int i = grp / GPI + t * (R / GPI);
      const unsigned item_i = first + i;
      const int base = i * kRows + (grp % GPI) * U;
      float go[V];
      if (item_i < nitems) {
        const float *gp = a.grad_out + ((q0 * a.H + item_i) * C + sub * V);
#pragma unroll
        for (int x = 0; x < V; x += 4) {
          const float4 q4 = __ldg(reinterpret_cast<const float4 *>(gp + x));
          go[x] = q4.x; go[x + 1] = q4.y; go[x + 2] = q4.z; go[x + 3] = q4.w;
        }
      } else {
#pragma unroll
        for (int x = 0; x < V; ++x) go[x] = 0.f;
      }
#pragma unroll
      for (int r0 = 0; r0 < kRows; r0 += GPI * U) {
        RowEntry e[U];
        float v[U][V];
#pragma unroll
        for (int u = 0; u < U; ++u) e[u] = table[base + r0 + u];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (e[u].off >= 0) {
            RowVec4<VT>::load(vbase + e[u].off, v[u]);
          } else {
#pragma unroll
            for (int x = 0; x < V; ++x) v[u][x] = 0.f;
          }
        }
        float d[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          d[u] = 0.f;
#pragma unroll
          for (int x = 0; x < V; ++x) d[u] = fmaf(v[u][x], go[x], d[u]);
        }
        int u_mine;
        const float f = fold_four_dots<G>(d, sub, u_mine);
        if (u_mine >= 0) dot_slots[base + r0 + u_mine] = f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (e[u].off >= 0 && e[u].wgt != 0.f) {
            float *gp = gvbase + e[u].off;
#pragma unroll
            for (int x = 0; x < V; x += 4)
              red_add_v4(gp + x, e[u].wgt * go[x], e[u].wgt * go[x + 1], e[u].wgt * go[x + 2],
                         e[u].wgt * go[x + 3]);
          }
        }
      }
    }
    __syncwarp();
    const float4 tq = reinterpret_cast<const float4 *>(dot_slots)[lane];
    const float tt[4] = {tq.x, tq.y, tq.z, tq.w};
    float part = bwd_point_epilogue<DT, MODE>(a, c, j, st, tt);
    if (MODE == kCallerFused) {
      // softmax backward, grad_logit_j = a_j * (g_j - sum_k a_k g_k): the sum runs over the item's LP lanes;
      // g_j was parked in grad_logits by the epilogue
#pragma unroll
      for (int s = LP / 2; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
      if (live) a.grad_logits[c.pt0 + j] = st.aw * (a.grad_logits[c.pt0 + j] - part);
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------------------------------------
// any C: lanes stride over channels (correctness path for unusual widths)
// ------------------------------------------------------------------------------------------------
template <typename VT, typename DT, int MODE>
__global__ void __launch_bounds__(kThreads)
dfa3d_backward_generic_kernel(const KArgs a) {
  __shared__ LevelTable lv;
  __shared__ __align__(16) RowEntry rows[kWarpsPerCta][128];
  __shared__ __align__(16) float dots[kWarpsPerCta][128];
  stage_levels(lv, a);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  ItemCtx c;
  if (!item_context(a, warp, blockIdx.x, c)) return;
  const int C = a.C;
  const long long slice = ((long long)c.b * a.N * a.H + c.h) * C;
  const VT *vbase = reinterpret_cast<const VT *>(a.value) + slice;
  float *gvbase = a.grad_value + slice;
  const float *gop = a.grad_out + c.item * C;
  RowEntry *my = rows[warp];
  float *myd = dots[warp];
  SoftmaxStats sm{0.f, 1.f};
  if (MODE == kCallerFused) sm = item_softmax_stats(a, c, lane);
  float dot = 0.f;
  for (int chunk = 0; chunk < a.LP; chunk += 32) {
    PointState st;
    float wgt[4];
    int off[4];
    bwd_point<DT, MODE>(a, lv, c, chunk + lane, sm, st, wgt, off);
    store_rows(my, lane, off, wgt);
    __syncwarp();
    const int nrows = min(32, a.LP - chunk) * 4;
    for (int r = 0; r < nrows; ++r) {
      const RowEntry e = my[r];
      float d = 0.f;
      if (e.off >= 0) {
        for (int ch = lane; ch < C; ch += 32) {
          const float g = __ldg(gop + ch);
          d = fmaf(load_scalar(vbase + e.off + ch), g, d);
          if (e.wgt != 0.f) red_add(gvbase + e.off + ch, e.wgt * g);
        }
      }
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) d += __shfl_xor_sync(0xffffffffu, d, s);
      if (lane == 0) myd[r] = d;
    }
    __syncwarp();
    const float4 tq = reinterpret_cast<const float4 *>(myd)[lane];
    const float t[4] = {tq.x, tq.y, tq.z, tq.w};
    dot += bwd_point_epilogue<DT, MODE>(a, c, chunk + lane, st, t);
    __syncwarp();
  }
  if (MODE == kCallerFused) finish_logit_grads(a, c, lane, sm, dot);
}

// ------------------------------------------------------------------------------------------------
// depth-score backward alone (two-stage API): one thread per sampling point
// ------------------------------------------------------------------------------------------------
template <typename DT>
__global__ void __launch_bounds__(kThreads)
dfa3d_depth_score_backward_kernel(const KArgs a) {
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
    float g_z = 0.f;
    if (g.ok3) {
      const long long bh = (long long)b * a.Nd * a.dist_pix_stride + h * a.dist_head_stride;
      const DT *dist_bh = reinterpret_cast<const DT *>(a.dist) + bh;
      float *gd_bh = a.grad_dist + bh;
      const float4 gq = __ldg(reinterpret_cast<const float4 *>(a.grad_ds_in) + pt);
      const float gds[4] = {gq.x, gq.y, gq.z, gq.w};
      const float hd = 1.f - g.ld;
      const int Dlim = min(g.Dd, a.D);
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (g.pix[k] >= 0) {
          float lo, hi;
          load_depth_pair(dist_bh, a.dist_pix_stride, g.dpix[k], g.z0, Dlim, true, lo, hi);
          red_depth_pair(gd_bh, a.dist_pix_stride, g.dpix[k], g.z0, Dlim, a.D, hd * gds[k], g.ld * gds[k]);
          acc = fmaf(gds[k], hi - lo, acc);
        }
      }
      g_z = (float)g.Dd * acc;
    }
    float *gl = a.grad_loc + pt * 3;
    gl[0] = 0.f; gl[1] = 0.f; gl[2] = g_z;
  }
}

// ------------------------------------------------------------------------------------------------
// host-side dispatch
// ------------------------------------------------------------------------------------------------
template <typename VT, typename DT, int MODE, bool FULL>
static void launch_backward_g(const KArgs &a, dim3 grid, cudaStream_t s) {
  constexpr int V = RowVec4<VT>::kElems;
  switch ((a.C % V == 0) ? a.C / V : 0) {
    case 2:  dfa3d_backward_kernel<VT, DT, 2 * V, MODE, FULL><<<grid, kThreads, 0, s>>>(a); break;
    case 4:  dfa3d_backward_kernel<VT, DT, 4 * V, MODE, FULL><<<grid, kThreads, 0, s>>>(a); break;
    case 8:  dfa3d_backward_kernel<VT, DT, 8 * V, MODE, FULL><<<grid, kThreads, 0, s>>>(a); break;
    case 16: dfa3d_backward_kernel<VT, DT, 16 * V, MODE, FULL><<<grid, kThreads, 0, s>>>(a); break;
    case 32: dfa3d_backward_kernel<VT, DT, 32 * V, MODE, FULL><<<grid, kThreads, 0, s>>>(a); break;
    default: {
      const dim3 g1((unsigned)((a.items_per_cam + kWarpsPerCta - 1) / kWarpsPerCta), grid.y, 1);
      dfa3d_backward_generic_kernel<VT, DT, MODE><<<g1, kThreads, 0, s>>>(a);
      break;
    }
  }
}

// Packed kernels: float storage, 16 / 32 / 64 channels, 4 / 8 / 16 points per item.  Returns false otherwise.
template <int MODE, int LP>
static bool launch_backward_packed_c(const KArgs &a, dim3 grid, cudaStream_t s) {
  switch (a.C) {
    case 16: dfa3d_backward_packed_kernel<float, float, 16, MODE, LP><<<grid, kThreads, 0, s>>>(a); return true;
    case 32: dfa3d_backward_packed_kernel<float, float, 32, MODE, LP><<<grid, kThreads, 0, s>>>(a); return true;
    case 64: dfa3d_backward_packed_kernel<float, float, 64, MODE, LP><<<grid, kThreads, 0, s>>>(a); return true;
    default: return false;
  }
}

template <int MODE>
static bool launch_backward_packed(const KArgs &a, int cams, cudaStream_t s) {
  if (a.LP != 4 && a.LP != 8 && a.LP != 16) return false;
  const int per_cta = kWarpsPerCta * kPackedRounds * (32 / a.LP);
  const dim3 grid((unsigned)((a.items_per_cam + per_cta - 1) / per_cta), (unsigned)cams, 1);
  if (a.LP == 4) return launch_backward_packed_c<MODE, 4>(a, grid, s);
  if (a.LP == 8) return launch_backward_packed_c<MODE, 8>(a, grid, s);
  return launch_backward_packed_c<MODE, 16>(a, grid, s);
}

template <typename VT, typename DT> struct IsFloatPairB { static constexpr bool value = false; };
template <> struct IsFloatPairB<float, float> { static constexpr bool value = true; };

template <typename VT, typename DT, int MODE>
static cudaError_t launch_backward_vd(const KArgs &a0, cudaStream_t s) {
  const bool full = a0.LP % 32 == 0;
  for (int b0 = 0; b0 < a0.B; b0 += 65535) {      // grid.y limit
    KArgs a = a0;
    a.b0 = b0;
    if (IsFloatPairB<VT, DT>::value && launch_backward_packed<MODE>(a, min(65535, a0.B - b0), s)) {
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      continue;
    }
    constexpr int kPerCta = kWarpsPerCta * DFA3D_BWD_ITEMS_PER_WARP;
    const dim3 grid((unsigned)((a.items_per_cam + kPerCta - 1) / kPerCta),
                    (unsigned)min(65535, a0.B - b0), 1);
    if (full) launch_backward_g<VT, DT, MODE, true>(a, grid, s);
    else launch_backward_g<VT, DT, MODE, false>(a, grid, s);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// Storage types are the DFA3D_DTYPE_* codes of the C header.  fp32 and bf16 combine freely; fp16 value
// goes with fp16 dist (what a half-precision caller passes) -- the C entry points reject the rest.
template <int MODE>
static cudaError_t launch_backward_m(const KArgs &a, int value_dtype, int dist_dtype, cudaStream_t s) {
  if (value_dtype == kDtypeF16) return launch_backward_vd<__half, __half, MODE>(a, s);
  if (value_dtype == kDtypeBF16)
    return dist_dtype == kDtypeBF16 ? launch_backward_vd<__nv_bfloat16, __nv_bfloat16, MODE>(a, s)
                                    : launch_backward_vd<__nv_bfloat16, float, MODE>(a, s);
  return dist_dtype == kDtypeBF16 ? launch_backward_vd<float, __nv_bfloat16, MODE>(a, s)
                                  : launch_backward_vd<float, float, MODE>(a, s);
}

cudaError_t launch_backward(const KArgs &a, int value_dtype, int dist_dtype, int mode, cudaStream_t s) {
  if (a.items == 0) return cudaSuccess;
  if (mode == kGivenDepthScore) {
    if (value_dtype == kDtypeF16) return launch_backward_vd<__half, float, kGivenDepthScore>(a, s);
    return value_dtype == kDtypeBF16 ? launch_backward_vd<__nv_bfloat16, float, kGivenDepthScore>(a, s)
                                     : launch_backward_vd<float, float, kGivenDepthScore>(a, s);
  }
  if (mode == kCallerFused) return launch_backward_m<kCallerFused>(a, value_dtype, dist_dtype, s);
  return launch_backward_m<kFused>(a, value_dtype, dist_dtype, s);
}

cudaError_t launch_depth_score_backward(const KArgs &a, int dist_dtype, cudaStream_t s) {
  const long long npts = a.items * a.LP;
  if (npts == 0) return cudaSuccess;
  const unsigned grid = (unsigned)min((npts + kThreads - 1) / kThreads, (long long)148 * 64);
  if (dist_dtype == kDtypeF16) dfa3d_depth_score_backward_kernel<__half><<<grid, kThreads, 0, s>>>(a);
  else if (dist_dtype == kDtypeBF16) dfa3d_depth_score_backward_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(a);
  else dfa3d_depth_score_backward_kernel<float><<<grid, kThreads, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace dfa3d
