// Shared device/host helpers of libsphmap: exact-rounding arithmetic, the
// sample-map tap decoder and small launch utilities.
#pragma once

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <stdint.h>

#include "sphmap.h"

namespace sph {

constexpr int kPlanesPerThread = 8;  // (b,c) planes one thread walks after decoding a map entry once

// Round-to-nearest arithmetic that the compiler may not contract into FMAs.
// The reference's CPU build evaluates a*b*c and a+b+c+d with separate
// roundings; using these keeps gathers bit-identical to it.
template <typename T> struct RN;
template <> struct RN<float> {
  static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
  static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
  static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
  static __device__ __forceinline__ int round_away(float v) { return (int)roundf(v); }
  static __device__ __forceinline__ int floor_int(float v) { return (int)floorf(v); }
};
template <> struct RN<double> {
  static __device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
  static __device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
  static __device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
  static __device__ __forceinline__ int round_away(double v) { return (int)round(v); }
  static __device__ __forceinline__ int floor_int(double v) { return (int)floor(v); }
};

// ---- checked build (-DSPH_BOUNDS_CHECK) ----------------------------------------------------------------------
// The stand-in for a memory checker on machines where none may run: every data-dependent index a kernel is about to
// use (tap offsets, plan entries, plan positions while a plan is being written) is compared with its range first.
// A violation is recorded in a sticky per-device word, which sph_device_status() reports as bit 2, and the access is
// skipped - nothing traps.  In the normal build index_ok() is the constant true and costs nothing.
#ifdef SPH_BOUNDS_CHECK
static __device__ int g_bad_index;  // one copy per translation unit, collected by sph_device_status()
__device__ __forceinline__ bool index_ok(long long i, long long n) {
  if (i >= 0 && i < n) return true;
  g_bad_index = 1;
  return false;
}
#define SPH_TU_STATUS(name)                                                                       \
  extern "C" int sph_tu_status_##name(int reset) {                                                \
    int v = 0;                                                                                    \
    if (cudaMemcpyFromSymbol(&v, sph::g_bad_index, sizeof(int)) != cudaSuccess) return -1;        \
    if (reset && v) {                                                                             \
      const int zero = 0;                                                                         \
      if (cudaMemcpyToSymbol(sph::g_bad_index, &zero, sizeof(int)) != cudaSuccess) return -1;     \
    }                                                                                             \
    return v;                                                                                     \
  }
#else
__device__ __forceinline__ constexpr bool index_ok(long long, long long) { return true; }
#define SPH_TU_STATUS(name)
#endif

// Up to four taps of one map coordinate: element offset inside a plane
// (negative = outside, contributes zero) and interpolation weight; limit = elements of a plane.
template <typename T> struct Taps {
  int off[4];
  T w[4];
  int limit;
};

// |v| < 1e9, false for NaN.  1e9 is exactly representable in float32, so the float32 comparison decides exactly as the
// float64 one would (and stays off the double-precision pipe).
__device__ __forceinline__ bool coord_in_range(float v) { return fabsf(v) < 1e9f; }
__device__ __forceinline__ bool coord_in_range(double v) { return fabs(v) < 1e9; }

template <int INTERP> struct TapCount { static constexpr int value = (INTERP == SPH_NEAREST) ? 1 : 4; };

// Decode a coordinate exactly as ext_modules/include/core/interpolation.h
// does: nearest = round half away from zero (97-115); bilinear = floor, +1,
// per-corner zero padding, weights (y2-y)(x2-x) ... (17-33,137-162);
// bispherical = x wrapped modulo W, weights from the unwrapped integers
// (191-218).  Coordinates that are NaN or beyond +-1e9 have no valid tap.
template <typename T, int INTERP>
__device__ __forceinline__ void decode(T x, T y, int H, int W, Taps<T> &t) {
  const bool sane = coord_in_range(x) && coord_in_range(y);
  t.limit = H * W;
  if (INTERP == SPH_NEAREST) {
    const int xi = RN<T>::round_away(x), yi = RN<T>::round_away(y);
    const bool ok = sane && xi >= 0 && xi <= W - 1 && yi >= 0 && yi <= H - 1;
    t.off[0] = ok ? yi * W + xi : -1;
    t.w[0] = T(1);
    return;
  }
  if (!sane) {
#pragma unroll
    for (int i = 0; i < 4; i++) { t.off[i] = -1; t.w[i] = T(0); }
    return;
  }
  const int x1 = RN<T>::floor_int(x), y1 = RN<T>::floor_int(y);
  const int x2 = x1 + 1, y2 = y1 + 1;
  const T A = RN<T>::sub((T)y2, y), B = RN<T>::sub((T)x2, x), C = RN<T>::sub(x, (T)x1), D = RN<T>::sub(y, (T)y1);
  t.w[0] = RN<T>::mul(A, B);
  t.w[1] = RN<T>::mul(A, C);
  t.w[2] = RN<T>::mul(D, B);
  t.w[3] = RN<T>::mul(D, C);
  const bool vy1 = y1 >= 0 && y1 <= H - 1, vy2 = y2 >= 0 && y2 <= H - 1;
  int xa = x1, xb = x2;
  bool vx1, vx2;
  if (INTERP == SPH_BISPHERICAL) {
    xa = ((x1 % W) + W) % W;
    xb = ((x2 % W) + W) % W;
    vx1 = vx2 = true;
  } else {
    vx1 = x1 >= 0 && x1 <= W - 1;
    vx2 = x2 >= 0 && x2 <= W - 1;
  }
  t.off[0] = (vx1 && vy1) ? y1 * W + xa : -1;
  t.off[1] = (vx2 && vy1) ? y1 * W + xb : -1;
  t.off[2] = (vx1 && vy2) ? y2 * W + xa : -1;
  t.off[3] = (vx2 && vy2) ? y2 * W + xb : -1;
}

// Interpolated value of one plane at decoded taps: ((w0 v0 + w1 v1) + w2 v2) + w3 v3,
// each product and sum rounded separately (core/interpolation.h:25-32).  Split into the loads and the
// arithmetic so that callers can issue the loads of several taps sets before consuming any.
template <typename T, int INTERP>
__device__ __forceinline__ void gather_load(const T *__restrict__ plane, const Taps<T> &t, T (&v)[TapCount<INTERP>::value]) {
#pragma unroll
  for (int i = 0; i < TapCount<INTERP>::value; i++)
    v[i] = (t.off[i] >= 0 && index_ok(t.off[i], t.limit)) ? __ldg(plane + t.off[i]) : T(0);
}
template <typename T, int INTERP>
__device__ __forceinline__ T gather_combine(const Taps<T> &t, const T (&v)[TapCount<INTERP>::value]) {
  if constexpr (INTERP == SPH_NEAREST) {
    return v[0];
  } else {
    return RN<T>::add(RN<T>::add(RN<T>::add(RN<T>::mul(t.w[0], v[0]), RN<T>::mul(t.w[1], v[1])), RN<T>::mul(t.w[2], v[2])),
                      RN<T>::mul(t.w[3], v[3]));
  }
}
template <typename T, int INTERP>
__device__ __forceinline__ T gather(const T *__restrict__ plane, const Taps<T> &t) {
  T v[TapCount<INTERP>::value];
  gather_load<T, INTERP>(plane, t, v);
  return gather_combine<T, INTERP>(t, v);
}

// Value of one map slot: plain, or the weighted sum over its P points
// (core/resample.h:143-161: acc += w_i * interp_i, in order).
template <typename T, int INTERP, bool WEIGHTED>
__device__ __forceinline__ T gather_slot(const T *__restrict__ plane, const T *__restrict__ m,
                                         const T *__restrict__ iw, int P, int H, int W) {
  Taps<T> t;
  if (!WEIGHTED) {
    decode<T, INTERP>(__ldg(m), __ldg(m + 1), H, W, t);
    return gather<T, INTERP>(plane, t);
  }
  T acc = T(0);
  for (int q = 0; q < P; q++) {
    decode<T, INTERP>(__ldg(m + 2 * q), __ldg(m + 2 * q + 1), H, W, t);
    acc = RN<T>::add(acc, RN<T>::mul(__ldg(iw + q), gather<T, INTERP>(plane, t)));
  }
  return acc;
}

// Device-side view of a scatter plan (CSR keyed by destination pixel * K + slot).
template <typename T> struct PlanView {
  const int *offsets;  // n_keys + 1
  const int *src;      // source position of each entry
  const T *w;          // weight of each entry
  int n_src;           // source positions the plan was built over (entries' src are below it)
};

// First 256 bytes of a plan blob, written on the device by sph_plan_build.
// Consumers locate the arrays through it, so they need not know the P and
// interpolation type the plan was built with.
struct PlanHeader {
  unsigned magic;
  int n_keys, K, dtype, e_max;
  unsigned long long off_offsets, off_src, off_w;
  int max_seg;  // longest segment (entries of one key), written by the sort pass
  int n_src;    // map positions the plan was built over
};
constexpr unsigned kPlanMagic = 0x53504c4eu;  // "SPLN"

// Host-side layout of the opaque plan blob.
struct PlanLayout {
  int64_t n_keys, e_max;
  size_t off_offsets, off_src, off_w, off_cursor, off_sums, total;
  int n_scan_blocks;
};

constexpr int kScanItems = 2048;  // elements one scan block covers

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline bool plan_layout(int64_t n_src, int64_t K, int64_t P, int interp, int64_t dstH, int64_t dstW, int dtype,
                        PlanLayout &L) {
  const int64_t PP = P > 0 ? P : 1, taps = (interp == SPH_NEAREST) ? 1 : 4;
  if (n_src <= 0 || K <= 0 || dstH <= 0 || dstW <= 0) return false;
  L.n_keys = dstH * dstW * K;
  L.e_max = n_src * K * PP * taps;
  const int64_t lim = (int64_t)1 << 31;
  if (L.n_keys + 1 >= lim || n_src * K * PP * 4 >= lim || dstH * dstW >= lim) return false;
  const size_t ts = dtype == SPH_F64 ? 8 : 4;
  L.n_scan_blocks = (int)((L.n_keys + kScanItems - 1) / kScanItems);
  size_t o = 256;  // header
  L.off_offsets = o; o = align_up(o + sizeof(int) * (size_t)(L.n_keys + 1), 256);
  L.off_src = o;     o = align_up(o + sizeof(int) * (size_t)L.e_max, 256);
  L.off_w = o;       o = align_up(o + ts * (size_t)L.e_max, 256);
  L.off_cursor = o;  o = align_up(o + sizeof(int) * (size_t)L.n_keys, 256);
  L.off_sums = o;    o = align_up(o + sizeof(int) * (size_t)(L.n_scan_blocks + 1), 256);
  L.total = o;
  return true;
}

// Resolve the arrays of a plan on the device; `ok` is false when the blob was
// not built for n_keys keys of type T, or (n_src >= 0) not over n_src map positions: the caller then writes zeros
// instead of following entries that were made for tensors of another size.
template <typename T>
__device__ __forceinline__ PlanView<T> plan_view(const void *plan, int n_keys, bool &ok, int n_src = -1) {
  const PlanHeader *h = (const PlanHeader *)plan;
  const char *p = (const char *)plan;
  ok = h->magic == kPlanMagic && h->n_keys == n_keys && h->dtype == (sizeof(T) == 8 ? SPH_F64 : SPH_F32) &&
       (n_src < 0 || h->n_src == n_src);
  return PlanView<T>{(const int *)(p + h->off_offsets), (const int *)(p + h->off_src), (const T *)(p + h->off_w), h->n_src};
}

// NVTX range over one C entry point (header-only NVTX 3: a no-op unless a profiler that injects itself is attached),
// so that a timeline shows which operator the kernels below it belong to.
struct NvtxRange {
  explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange &) = delete;
  NvtxRange &operator=(const NvtxRange &) = delete;
};
#define SPH_RANGE(name) ::sph::NvtxRange sph_nvtx_range_(name)

// Kernel launches issued by this library in this process (tracing aid, see sph_launch_count()).
extern unsigned long long g_launch_count;
inline void note_launches(int n) { __atomic_fetch_add(&g_launch_count, (unsigned long long)n, __ATOMIC_RELAXED); }

// Status of the launches just issued; n = how many kernels the caller enqueued.
inline int launch_status(int n = 1) {
  note_launches(n);
  return cudaGetLastError() == cudaSuccess ? SPH_OK : SPH_ERR_CUDA;
}

inline int cdiv(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// Dispatch a runtime interpolation code to a template parameter.
#define SPH_DISPATCH_INTERP(interp, ...)                                              \
  switch (interp) {                                                                   \
    case SPH_BILINEAR: { constexpr int INTERP = SPH_BILINEAR; __VA_ARGS__; break; }   \
    case SPH_BISPHERICAL: { constexpr int INTERP = SPH_BISPHERICAL; __VA_ARGS__; break; } \
    default: { constexpr int INTERP = SPH_NEAREST; __VA_ARGS__; break; }              \
  }

}  // namespace sph
