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

/* ---- voting resample (integer labels) --------------------------------------
 * core/interpolation.h:249-265 (Vote2D), common/resample.h:109-130,
 * src/cpp/voting_resample_layer.cpp:8-37: every input pixel votes for its
 * label at the output pixel its (integer) map entry names; the output is the
 * label with the most votes, the smallest such label on ties (torch.argmax
 * returns the first maximum), 0 where nobody voted.  Labels outside
 * [0, num_candidates) cast no vote here (the reference would write out of
 * bounds).  Channels are independent here; the reference steps its vote
 * tensor by OH*OW per channel instead of OH*OW*num_candidates
 * (common/resample.h:127-129), so with more than one channel its votes
 * overlap and only the one-channel case is pinned against it. */
void sph_o_voting_resample(const int64_t *x, const int64_t *map, int64_t *out, int64_t B, int64_t C, int64_t IH,
                           int64_t IW, int64_t OH, int64_t OW, int64_t num_candidates) {
  const int64_t n = IH * IW, m = OH * OW;
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++) {
    int64_t *votes = (int64_t *)calloc((size_t)(m * num_candidates), sizeof(int64_t));
    for (int64_t i = 0; i < n; i++) {
      const int64_t xo = map[2 * i], yo = map[2 * i + 1], lab = x[bc * n + i];
      if (xo >= 0 && xo <= OW - 1 && yo >= 0 && yo <= OH - 1 && lab >= 0 && lab < num_candidates)
        votes[(yo * OW + xo) * num_candidates + lab]++;
    }
    for (int64_t o = 0; o < m; o++) {
      int64_t best = 0;
      for (int64_t c = 1; c < num_candidates; c++)
        if (votes[o * num_candidates + c] > votes[o * num_candidates + best]) best = c;
      out[bc * m + o] = best;
    }
    free(votes);
  }
}
