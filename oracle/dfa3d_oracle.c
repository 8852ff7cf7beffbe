/* CPU oracle for the DFA3D operator (fp32 and fp64 instantiations of dfa3d_oracle_body.inc).
 *
 * TEST INFRASTRUCTURE ONLY.  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may
 * load the library built from this file; the shipped CUDA library never does.
 *
 * Parity status: the reference's own test (unittest_DFA3D.py:72-73) holds no golden vectors, it only
 * checks "no NaN".  This restatement is pinned instead by (1) outputs of the reference's unmodified
 * CUDA op, generated on a B200 by tests/golden/make_golden.py and committed under tests/golden/, and
 * (2) an independent formulation of the same operator (5-D trilinear grid_sample on value (x) dist,
 * oracle/grid_sample_form.py) in fp64.
 *
 * One deliberate difference from the reference: the reference calls floorf() even when instantiated
 * for double, which rounds the coordinate to float first; the fp64 instantiation here uses floor().
 */
#include <math.h>
#include <stdint.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define REAL float
#define SUF(name) CAT(name, _f32)
#define FMA fmaf
#include "dfa3d_oracle_body.inc"
#undef REAL
#undef SUF
#undef FMA

#define REAL double
#define SUF(name) CAT(name, _f64)
#define FMA fma
#include "dfa3d_oracle_body.inc"
#undef REAL
#undef SUF
#undef FMA

int dfa3d_oracle_abi_version(void) { return 1; }
