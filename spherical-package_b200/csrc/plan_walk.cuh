// Warp-cooperative walk of a scatter plan: the engine of every adjoint ("scatter") operator.
//
// A plan lists, for every destination pixel q, the entries (source id, weight) that contribute to it, segments laid
// out one after the other in q order.  A warp owns 32 consecutive destination pixels, whose segments are therefore
// one contiguous range of entries.  The walk has two sides:
//   entry side   lane l takes entry t + l of the range: the source ids and weights are read with coalesced loads
//                and the (random) source values of all PL planes are fetched at once - every lane has its loads in
//                flight together, none depends on another;
//   pixel side   the contributions go through a small shared-memory window, and lane l, as the owner of pixel
//                q0 + l, adds the window entries of its own segment in entry order.
// The sum of a pixel is thus taken in map order whatever the scheduling (deterministic), with no zero-fill pass and
// no atomics (the reference's scatter kernels use atomicAdd: ext_modules/include/cuda/resample.cuh:14-47,
// mapped_im2col.cuh:52-91, mapped_max_pool.cuh:57-95).
#pragma once

#include "common.cuh"

namespace sph {

constexpr int kWalkUnroll = 2;                      // entries per lane and window
constexpr int kWalkWindow = 32 * kWalkUnroll;       // entries per window

// Shared memory one warp needs: PL planes (+ 1 row of weights when the sum is normalised) x window entries.
template <typename T, int PL, bool NORM>
__host__ __device__ constexpr int walk_smem_per_warp() { return (PL + (NORM ? 1 : 0)) * kWalkWindow * (int)sizeof(T); }

// Division by a runtime constant as multiply-high + shift (exact for 0 <= x < 2^31 and 1 <= d < 2^31).
struct FastDiv {
  unsigned mul, shift, d;
  __host__ __device__ static FastDiv make(unsigned d) {
    FastDiv f;
    f.d = d;
    unsigned l = 0;
    while ((1ull << l) < d) l++;
    f.shift = l;
    f.mul = (unsigned)((((1ull << l) - d) << 32) / d + 1);
    return f;
  }
  __device__ __forceinline__ unsigned div(unsigned x) const { return (__umulhi(x, mul) + x) >> shift; }
};

// prepare(s) -> per-entry value shared by all planes (source offset, decoded slot ...); contrib(pre, w, j) ->
// contribution of that entry to plane j of this CTA's plane group.  Pixels [q_begin, q_end) are walked by the calling
// CTA's warps; out_plane0 points at plane 0 of the group and planes are n_dst apart; np <= PL planes are written.
template <typename T, int PL, bool NORM, typename FP, typename FC>
__device__ __forceinline__ void plan_walk(const PlanView<T> &plan, bool ok, int n_dst, int q_begin, int q_end, T *cbuf_all,
                                          FP prepare, FC contrib, T *__restrict__ out_plane0, int np) {
  constexpr int ROWS = PL + (NORM ? 1 : 0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  T *cbuf = cbuf_all + (size_t)warp * ROWS * kWalkWindow;
  const bool full = np == PL;
  int q0 = q_begin + warp * 32;
  // segment bounds of the block this warp handles next, fetched one block ahead
  int n0 = 0, n1 = 0;
  if (q0 < q_end && ok) {
    n0 = __ldg(plan.offsets + min(q0 + lane, n_dst));
    n1 = __ldg(plan.offsets + min(q0 + lane + 1, n_dst));
  }
  for (; q0 < q_end; q0 += nwarps * 32) {
    const int q = q0 + lane, e0 = n0, e1 = n1;
    const int qn = q0 + nwarps * 32;
    if (qn < q_end && ok) {
      n0 = __ldg(plan.offsets + min(qn + lane, n_dst));
      n1 = __ldg(plan.offsets + min(qn + lane + 1, n_dst));
    }
    const int a = __shfl_sync(0xffffffffu, e0, 0), b = __shfl_sync(0xffffffffu, e1, 31);
    T acc[PL], wsum = T(0);
#pragma unroll
    for (int j = 0; j < PL; j++) acc[j] = T(0);
    for (int t = a; t < b; t += kWalkWindow) {
      // entry side: lane l takes entries t + l and (if the range is that long) t + 32 + l
      const int nu = (b - t > 32) ? kWalkUnroll : 1;
#pragma unroll
      for (int u = 0; u < kWalkUnroll; u++) {
        if (u < nu) {
          const int e = t + u * 32 + lane;
          bool valid = e < b;
          const int s = valid ? __ldg(plan.src + e) : 0;
          valid = valid && index_ok(s, plan.n_src);
          const T w = valid ? __ldg(plan.w + e) : T(0);
          const auto pre = prepare(s);
#pragma unroll
          for (int j = 0; j < PL; j++) cbuf[j * kWalkWindow + u * 32 + lane] = (valid && (full || j < np)) ? contrib(pre, w, j) : T(0);
          if (NORM) cbuf[PL * kWalkWindow + u * 32 + lane] = w;
        }
      }
      __syncwarp();
      // pixel side: this lane's own segment, in entry order
      const int lo = max(e0, t) - t, hi = min(e1, t + kWalkWindow) - t;
      for (int e = lo; e < hi; e++) {
#pragma unroll
        for (int j = 0; j < PL; j++) acc[j] += cbuf[j * kWalkWindow + e];
        if (NORM) wsum += cbuf[PL * kWalkWindow + e];
      }
      __syncwarp();
    }
    if (q < q_end) {
      T *o = out_plane0 + q;
      if (NORM) {
        const T inv_den = wsum + T(1e-12);
#pragma unroll
        for (int j = 0; j < PL; j++)
          if (full || j < np) o[(size_t)j * n_dst] = acc[j] / inv_den;
      } else {
#pragma unroll
        for (int j = 0; j < PL; j++)
          if (full || j < np) o[(size_t)j * n_dst] = acc[j];
      }
    }
  }
}

}  // namespace sph
