// Mapped max pooling (forward: value + argmax index; argmax backward) and mapped average pooling (forward).
#include <float.h>

#include "common.cuh"
#include "plan_walk.cuh"

namespace sph {

// out[p,o] = max over the K map slots of output position o, first strict
// maximum, starting from -FLT_MAX as the reference's CUDA build does
// (ext_modules/include/common/mapped_max_pool.h:27-51).  idx is the offset of
// the winning slot's x coordinate in the flattened map (line 49).  One thread
// per output position walks kPlanesPerThread planes; the whole batch is one
// launch (the reference launches once per image:
// src/cuda/mapped_max_pooling_layer.cu:11-36).
//
// AVG = true turns the same walk into mapped average pooling: the K slot values are added in slot order and the sum
// is divided by K (ext_modules/include/common/mapped_avg_pool.h:12-39, 71-107); idx is not written.
template <typename T, int INTERP, bool WEIGHTED, bool AVG>
__global__ void __launch_bounds__(256)
max_pool_kernel(const T *__restrict__ x, const T *__restrict__ map, const T *__restrict__ iw, T *__restrict__ out,
                int64_t *__restrict__ idx, int n, int planes, int H, int W, int K, int P) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n) return;
  const int p0 = blockIdx.y * kPlanesPerThread;
  const int np = min(kPlanesPerThread, planes - p0);
  const size_t hw = (size_t)H * W;
  const T *xp = x + (size_t)p0 * hw;
  const int PP = WEIGHTED ? P : 1;
  T best[kPlanesPerThread];
  int bk[kPlanesPerThread];
#pragma unroll
  for (int j = 0; j < kPlanesPerThread; j++) { best[j] = AVG ? T(0) : (T)(-FLT_MAX); bk[j] = -1; }
  for (int k = 0; k < K; k++) {
    const size_t e = ((size_t)o * K + k) * PP;
    if (!WEIGHTED) {
      Taps<T> t;
      decode<T, INTERP>(__ldg(map + 2 * e), __ldg(map + 2 * e + 1), H, W, t);
#pragma unroll
      for (int j = 0; j < kPlanesPerThread; j++)
        if (j < np) {
          const T v = gather<T, INTERP>(xp + j * hw, t);
          if (AVG) best[j] = RN<T>::add(best[j], v);
          else if (v > best[j]) { best[j] = v; bk[j] = k; }
        }
    } else {
#pragma unroll
      for (int j = 0; j < kPlanesPerThread; j++)
        if (j < np) {
          const T v = gather_slot<T, INTERP, true>(xp + j * hw, map + 2 * e, iw + e, P, H, W);
          if (AVG) best[j] = RN<T>::add(best[j], v);
          else if (v > best[j]) { best[j] = v; bk[j] = k; }
        }
    }
  }
#pragma unroll
  for (int j = 0; j < kPlanesPerThread; j++)
    if (j < np) {
      if (AVG) {
        out[(size_t)(p0 + j) * n + o] = best[j] / (T)K;
      } else {
        out[(size_t)(p0 + j) * n + o] = best[j];
        idx[(size_t)(p0 + j) * n + o] = bk[j] < 0 ? (int64_t)-1 : ((int64_t)o * K + bk[j]) * PP * 2;
      }
    }
}

// Nearest-neighbour, unweighted pooling with at most kPoolMaxK slots: the K tap offsets of the output position are
// decoded first and kept in registers, then every plane issues its K loads back to back (no load depends on
// another), which is what lets the kernel run at memory speed instead of at K round-trip latencies per plane.
constexpr int kPoolMaxK = 16;

template <typename T, int PPT, int KMAX>
__global__ void __launch_bounds__(256)
max_pool_nearest_kernel(const T *__restrict__ x, const T *__restrict__ map, T *__restrict__ out, int64_t *__restrict__ idx,
                        int n, int planes, int H, int W, int K) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n) return;
  const int p0 = blockIdx.y * PPT;
  const int np = min(PPT, planes - p0);
  const size_t hw = (size_t)H * W;
  int off[KMAX];
#pragma unroll
  for (int k = 0; k < KMAX; k++) {
    off[k] = -1;
    if (k < K) {
      Taps<T> t;
      const size_t e = (size_t)o * K + k;
      decode<T, SPH_NEAREST>(__ldg(map + 2 * e), __ldg(map + 2 * e + 1), H, W, t);
      off[k] = t.off[0];
    }
  }
  T v[PPT][KMAX];
#pragma unroll
  for (int j = 0; j < PPT; j++) {
    const T *plane = x + (size_t)(p0 + (j < np ? j : 0)) * hw;
#pragma unroll
    for (int k = 0; k < KMAX; k++) v[j][k] = (k < K && off[k] >= 0) ? __ldg(plane + off[k]) : T(0);
  }
#pragma unroll
  for (int j = 0; j < PPT; j++) {
    if (j >= np) break;
    T best = (T)(-FLT_MAX);
    int bk = -1;
#pragma unroll
    for (int k = 0; k < KMAX; k++)
      if (k < K && v[j][k] > best) { best = v[j][k]; bk = k; }
    out[(size_t)(p0 + j) * n + o] = best;
    idx[(size_t)(p0 + j) * n + o] = bk < 0 ? (int64_t)-1 : ((int64_t)o * K + bk) * 2;
  }
}

// Argmax backward: the gradient of output (p,o) goes back through the one
// map slot idx names (common/mapped_max_pool.h:60-78, 136-171).  grad_in is
// zeroed first; contributions are added with red.global.add as in the
// reference's CUDA kernel (cuda/mapped_max_pool.cuh:57-95).
template <typename T, int INTERP, bool WEIGHTED>
__global__ void __launch_bounds__(256)
max_unpool_kernel(const T *__restrict__ g, const int64_t *__restrict__ idx, const T *__restrict__ map,
                  const T *__restrict__ iw, T *__restrict__ gin, int n, int planes, int H, int W, int P,
                  int64_t map_elems) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n) return;
  const int p0 = blockIdx.y * kPlanesPerThread;
  const int np = min(kPlanesPerThread, planes - p0);
  const size_t hw = (size_t)H * W;
  const int PP = WEIGHTED ? P : 1;
  for (int j = 0; j < np; j++) {
    const size_t at = (size_t)(p0 + j) * n + o;
    const int64_t s = idx[at];
    if (s < 0 || s + 2 * PP > map_elems) continue;
    const T v = g[at];
    T *plane = gin + (size_t)(p0 + j) * hw;
    Taps<T> t;
    for (int q = 0; q < PP; q++) {
      decode<T, INTERP>(__ldg(map + s + 2 * q), __ldg(map + s + 2 * q + 1), H, W, t);
      const T vq = WEIGHTED ? __ldg(iw + s / 2 + q) * v : v;
#pragma unroll
      for (int i = 0; i < TapCount<INTERP>::value; i++)
        if (t.off[i] >= 0) atomicAdd(plane + t.off[i], INTERP == SPH_NEAREST ? vq : t.w[i] * vq);
    }
  }
}

// Deterministic argmax backward.  `plan_blob` is a scatter plan built over the FLATTENED map slots
// (sph_plan_build with n_src = OH*OW*K positions and K = 1), so the segment of input pixel q lists every
// (output position o, slot k) whose taps touch q, as s = o*K + k, in map order, with the tap weight.  The pixel sums,
// in that fixed order, the entries whose slot is the one the forward pass selected: idx[p,o] == s * 2 * PP.  No
// zero-fill, no atomics, results independent of scheduling (the reference scatters with atomicAdd:
// ext_modules/include/cuda/mapped_max_pool.cuh:57-95).  The plan is walked warp-cooperatively (plan_walk.cuh).
// STAGED: the winning slot of every output of the CTA's PL planes is first decoded into shared memory as one byte
// (255 = none), so the per-entry test reads a byte of shared memory instead of 8 random bytes of idx.
template <typename T, int PL, bool STAGED>
__global__ void __launch_bounds__(1024)
max_unpool_plan_kernel(const T *__restrict__ g, const int64_t *__restrict__ idx, const void *__restrict__ plan_blob,
                       T *__restrict__ gin, int n, int n_dst, int planes, int K, int PP, int chunk, FastDiv divK) {
  extern __shared__ unsigned char unpool_smem[];
  T *cbuf = (T *)unpool_smem;
  uint8_t *ksm = unpool_smem + (size_t)(blockDim.x >> 5) * walk_smem_per_warp<T, PL, false>();  // [PL][n]
  const int p0 = blockIdx.y * PL;
  const int np = min(PL, planes - p0);
  if (STAGED) {
    for (int j = 0; j < PL; j++)
      for (int o = threadIdx.x; o < n; o += blockDim.x) {
        int k = -1;
        if (j < np) {
          const int64_t s = __ldg(idx + (size_t)(p0 + j) * n + o);
          if (s >= 0) {
            const int64_t slot = s / (2 * PP), kk = slot - (int64_t)o * K;
            if (kk >= 0 && kk < K && slot * 2 * PP == s) k = (int)kk;
          }
        }
        ksm[(size_t)j * n + o] = k < 0 ? (uint8_t)255 : (uint8_t)k;
      }
    __syncthreads();
  }
  bool ok;
  const PlanView<T> plan = plan_view<T>(plan_blob, n_dst, ok, n * K);
  const int q_begin = blockIdx.x * chunk, q_end = min(q_begin + chunk, n_dst);
  const T *gp = g + (size_t)p0 * n;
  const int64_t *ip = idx + (size_t)p0 * n;
  struct Slot { int o, k, s; };
  plan_walk<T, PL, false>(plan, ok, n_dst, q_begin, q_end, cbuf,
                          [&](int s) {
                            const int o = (int)divK.div((unsigned)s);
                            return Slot{o, s - o * K, s};
                          },
                          [&](const Slot &e, T w, int j) {
                            const bool hit = STAGED ? ksm[j * n + e.o] == (uint8_t)e.k
                                                    : __ldg(ip + (size_t)j * n + e.o) == (int64_t)e.s * 2 * PP;
                            return hit ? w * __ldg(gp + (size_t)j * n + e.o) : T(0);
                          },
                          gin + (size_t)p0 * n_dst, np);
}

template <typename T>
static int unpool_planned(const void *g, const int64_t *idx, const void *plan, void *gin, int64_t planes, int64_t n_dst,
                          int64_t n, int64_t K, int64_t P, cudaStream_t st) {
  const int PP = (int)(P > 0 ? P : 1);
  constexpr int PL = 4;
  const int groups = cdiv(planes, PL);
  const size_t stage = (size_t)PL * n;
  if (K <= 254 && stage + 32 * (size_t)walk_smem_per_warp<T, PL, false>() <= 200 * 1024) {
    // one CTA of 32 warps per SM (the staged slots fill its shared memory); CTAs = plane groups x pixel chunks
    int chunks = cdiv((int64_t)148 * 2, groups);
    if (chunks > cdiv(n_dst, 1024)) chunks = cdiv(n_dst, 1024);
    const int chunk = cdiv(cdiv(n_dst, chunks), 1024) * 1024;
    const size_t smem = stage + 32 * (size_t)walk_smem_per_warp<T, PL, false>();
    cudaFuncSetAttribute(max_unpool_plan_kernel<T, PL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    max_unpool_plan_kernel<T, PL, true><<<dim3(cdiv(n_dst, chunk), groups), 1024, smem, st>>>(
        (const T *)g, idx, plan, (T *)gin, (int)n, (int)n_dst, (int)planes, (int)K, PP, chunk, FastDiv::make((unsigned)K));
  } else {
    int64_t chunks = ((int64_t)148 * 16 + groups - 1) / groups;
    if (chunks > (n_dst + 255) / 256) chunks = (n_dst + 255) / 256;
    const int chunk = (int)(((n_dst + chunks - 1) / chunks + 255) / 256 * 256);
    const size_t smem = 8 * (size_t)walk_smem_per_warp<T, PL, false>();
    max_unpool_plan_kernel<T, PL, false><<<dim3(cdiv(n_dst, chunk), groups), 256, smem, st>>>(
        (const T *)g, idx, plan, (T *)gin, (int)n, (int)n_dst, (int)planes, (int)K, PP, chunk, FastDiv::make((unsigned)K));
  }
  return launch_status();
}

template <typename T>
static int pool(const void *x, const void *map, const void *iw, void *out, int64_t *idx, int64_t planes, int64_t H,
                int64_t W, int64_t n, int64_t K, int64_t P, int interp, cudaStream_t st, bool avg = false) {
  if (avg) {
    dim3 grid(cdiv(n, 256), cdiv(planes, kPlanesPerThread));
    SPH_DISPATCH_INTERP(interp, {
      if (P > 0)
        max_pool_kernel<T, INTERP, true, true><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, (const T *)iw, (T *)out,
                                                                     nullptr, (int)n, (int)planes, (int)H, (int)W, (int)K, (int)P);
      else
        max_pool_kernel<T, INTERP, false, true><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, nullptr, (T *)out, nullptr,
                                                                      (int)n, (int)planes, (int)H, (int)W, (int)K, 0);
    });
    return launch_status();
  }
  if (interp == SPH_NEAREST && P == 0 && K <= kPoolMaxK) {
    constexpr int PPT = 4;
    dim3 grid(cdiv(n, 256), cdiv(planes, PPT));
#define SPH_POOL_NEAREST(KMAX) \
    max_pool_nearest_kernel<T, PPT, KMAX><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, (T *)out, idx, (int)n, (int)planes, (int)H, (int)W, (int)K)
    if (K <= 4) SPH_POOL_NEAREST(4);
    else if (K <= 9) SPH_POOL_NEAREST(9);
    else SPH_POOL_NEAREST(16);
#undef SPH_POOL_NEAREST
    return launch_status();
  }
  dim3 grid(cdiv(n, 256), cdiv(planes, kPlanesPerThread));
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0)
      max_pool_kernel<T, INTERP, true, false><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, (const T *)iw, (T *)out, idx,
                                                             (int)n, (int)planes, (int)H, (int)W, (int)K, (int)P);
    else
      max_pool_kernel<T, INTERP, false, false><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, nullptr, (T *)out, idx, (int)n,
                                                              (int)planes, (int)H, (int)W, (int)K, 0);
  });
  return launch_status();
}

template <typename T>
static int unpool(const void *g, const int64_t *idx, const void *map, const void *iw, void *gin, int64_t planes,
                  int64_t H, int64_t W, int64_t n, int64_t K, int64_t P, int interp, cudaStream_t st) {
  if (cudaMemsetAsync(gin, 0, sizeof(T) * (size_t)(planes * H * W), st) != cudaSuccess) return SPH_ERR_CUDA;
  dim3 grid(cdiv(n, 256), cdiv(planes, kPlanesPerThread));
  const int64_t map_elems = n * K * (P > 0 ? P : 1) * 2;
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0)
      max_unpool_kernel<T, INTERP, true><<<grid, 256, 0, st>>>((const T *)g, idx, (const T *)map, (const T *)iw, (T *)gin,
                                                               (int)n, (int)planes, (int)H, (int)W, (int)P, map_elems);
    else
      max_unpool_kernel<T, INTERP, false><<<grid, 256, 0, st>>>((const T *)g, idx, (const T *)map, nullptr, (T *)gin, (int)n,
                                                                (int)planes, (int)H, (int)W, 0, map_elems);
  });
  return launch_status();
}

static int check(const void *a, const void *b, const void *c, const void *d, const void *iw, int64_t B, int64_t C,
                 int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp) {
  if (!a || !b || !c || !d || B < 0 || C < 0 || IH <= 0 || IW <= 0 || OH < 0 || OW < 0 || K <= 0 || P < 0 ||
      (P > 0 && !iw) || interp < 0 || interp > 2)
    return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  const int64_t lim = (int64_t)1 << 31;
  if (IH * IW >= lim || OH * OW * K * (P > 0 ? P : 1) * 2 >= lim || B * C / 4 >= 65535)
    return SPH_ERR_TOO_LARGE;
  return SPH_OK;
}

}  // namespace sph

using namespace sph;

SPH_TU_STATUS(pool)

extern "C" int sph_mapped_max_pool(const void *x, const void *map, const void *iw, void *out, int64_t *idx, int64_t B,
                                   int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                                   int dtype, int interp, void *stream) {
  SPH_RANGE("sph_mapped_max_pool");
  const int rc = check(x, map, out, idx, iw, B, C, IH, IW, OH, OW, K, P, dtype, interp);
  if (rc != SPH_OK) return rc;
  if (B * C == 0 || OH * OW == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? pool<float>(x, map, iw, out, idx, B * C, IH, IW, OH * OW, K, P, interp, st)
                          : pool<double>(x, map, iw, out, idx, B * C, IH, IW, OH * OW, K, P, interp, st);
}

extern "C" int sph_mapped_max_unpool(const void *g, const int64_t *idx, const void *map, const void *iw, void *grad_in,
                                     int64_t B, int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                                     int64_t P, int dtype, int interp, void *stream) {
  SPH_RANGE("sph_mapped_max_unpool");
  const int rc = check(g, map, grad_in, idx, iw, B, C, IH, IW, OH, OW, K, P, dtype, interp);
  if (rc != SPH_OK) return rc;
  if (B * C == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (OH * OW == 0)
    return cudaMemsetAsync(grad_in, 0, (dtype == SPH_F64 ? 8 : 4) * (size_t)(B * C * IH * IW), st) == cudaSuccess
               ? SPH_OK : SPH_ERR_CUDA;
  return dtype == SPH_F32 ? unpool<float>(g, idx, map, iw, grad_in, B * C, IH, IW, OH * OW, K, P, interp, st)
                          : unpool<double>(g, idx, map, iw, grad_in, B * C, IH, IW, OH * OW, K, P, interp, st);
}

extern "C" int sph_mapped_max_unpool_planned(const void *g, const int64_t *idx, const void *plan, void *grad_in, int64_t B,
                                             int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                                             int dtype, void *stream) {
  SPH_RANGE("sph_mapped_max_unpool_planned");
  const int rc = check(g, plan, grad_in, idx, nullptr, B, C, IH, IW, OH, OW, K, 0, dtype, 0);
  if (rc != SPH_OK) return rc;
  if (P < 0 || OH * OW * K >= ((int64_t)1 << 31) / (2 * (P > 0 ? P : 1))) return P < 0 ? SPH_ERR_INVALID_ARGUMENT : SPH_ERR_TOO_LARGE;
  if (B * C == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (OH * OW == 0)
    return cudaMemsetAsync(grad_in, 0, (dtype == SPH_F64 ? 8 : 4) * (size_t)(B * C * IH * IW), st) == cudaSuccess
               ? SPH_OK : SPH_ERR_CUDA;
  return dtype == SPH_F32 ? unpool_planned<float>(g, idx, plan, grad_in, B * C, IH * IW, OH * OW, K, P, st)
                          : unpool_planned<double>(g, idx, plan, grad_in, B * C, IH * IW, OH * OW, K, P, st);
}

extern "C" int sph_mapped_avg_pool(const void *x, const void *map, const void *iw, void *out, int64_t B, int64_t C, int64_t IH,
                                   int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                                   void *stream) {
  SPH_RANGE("sph_mapped_avg_pool");
  const int rc = check(x, map, out, out, iw, B, C, IH, IW, OH, OW, K, P, dtype, interp);
  if (rc != SPH_OK) return rc;
  if (B * C == 0 || OH * OW == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? pool<float>(x, map, iw, out, nullptr, B * C, IH, IW, OH * OW, K, P, interp, st, true)
                          : pool<double>(x, map, iw, out, nullptr, B * C, IH, IW, OH * OW, K, P, interp, st, true);
}
