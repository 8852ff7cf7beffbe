/* C interface of libdfa3d_rates.so: memory-primitive rate probes (measurement code for the DFA3D
 * kernels' lower bounds; not part of the operator library and not needed to run it). */
#ifndef DFA3D_RATES_H_
#define DFA3D_RATES_H_
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define DFA3D_RATE_GATHER_ROWS 1
#define DFA3D_RATE_RED_ROWS 2
#define DFA3D_RATE_GATHER_PAIRS 4
#define DFA3D_RATE_RED_PAIRS 8
#define DFA3D_RATE_GATHER_CELLS 16
#define DFA3D_RATE_RED_CELLS 32
#define DFA3D_RATE_BULK_RED_ROWS 64

typedef struct dfa3d_rate_problem {
  int32_t B, Q, L, P, D;        /* cameras, queries, levels, points per level (L*P == 32), depth bins */
  int32_t level_h[8], level_w[8];
  int32_t ops;                  /* DFA3D_RATE_* mask */
  int32_t level_mask;           /* bit l: the points of level l are issued */
  float dead_fraction;          /* fraction of points that issue nothing (outside the image) */
} dfa3d_rate_problem;

/* Tensors (device, fp32, 16-byte aligned; only those the mask needs may be non-null):
 * value/grad_value (B, N, 8, 32); dist/grad_dist (B, N, D); cells/grad_cells (B, NC, D, 4);
 * sink: at least ceil(Q*8/8)*8 floats.  N and NC from dfa3d_rate_sizes().  Returns 0, -1 (bad
 * argument) or -3 (launch failed). */
int dfa3d_rate_probe(const dfa3d_rate_problem *p, const float *value, float *grad_value,
                     const float *dist, float *grad_dist, const float *cells, float *grad_cells,
                     float *sink, void *stream);
int dfa3d_rate_sizes(const dfa3d_rate_problem *p, int64_t *pixels, int64_t *cells);

#ifdef __cplusplus
}
#endif
#endif
