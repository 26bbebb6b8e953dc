/* CPU oracle for the mapped-operator path -- TEST INFRASTRUCTURE ONLY.
 *
 * Plain-C restatement of the reference's CPU arithmetic (see
 * sph_oracle_impl.h for the per-function citations).  Used by the parity
 * tests, the smoke check and the benchmark's CPU-baseline leg as the checker;
 * the product library never links, loads or calls it.
 *
 * Parity of this restatement is pinned: tests/test_oracle.py checks it
 * against the known-answer vectors harvested from the reference's own test
 * suite and against outputs of the reference's compiled CPU modules
 * (tests/golden/).
 *
 * Build: make -C oracle   (gcc -O3 -fopenmp -ffp-contract=off)
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define T float
#define TMIN FLT_MIN
#define FN(name) CAT(name, _f32)
#include "sph_oracle_impl.h"
#undef T
#undef TMIN
#undef FN

#define T double
#define TMIN DBL_MIN
#define FN(name) CAT(name, _f64)
#include "sph_oracle_impl.h"
#undef T
#undef TMIN
#undef FN
