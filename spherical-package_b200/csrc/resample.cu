// resample_from_map (gather) and resample_to_map (adjoint, through a scatter plan).
#include "common.cuh"

namespace sph {

// One thread decodes one map position once and then walks kPlanesPerThread
// (batch, channel) planes with the same taps.  Reference kernel:
// ext_modules/include/cuda/resample.cuh:50-81 (one thread per (c, position), one
// launch per image); arithmetic: common/resample.h:34-52, 85-107.
template <typename T, int INTERP, bool WEIGHTED>
__global__ void __launch_bounds__(256)
resample_from_map_kernel(const T *__restrict__ x, const T *__restrict__ map, const T *__restrict__ iw,
                         T *__restrict__ y, int n, int planes, int H, int W, int P) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int p0 = blockIdx.y * kPlanesPerThread;
  const int np = min(kPlanesPerThread, planes - p0);
  const size_t hw = (size_t)H * W;
  const T *xp = x + (size_t)p0 * hw;
  T *yp = y + (size_t)p0 * n + i;
  Taps<T> t;
  if (!WEIGHTED) {
    decode<T, INTERP>(__ldg(map + 2 * (size_t)i), __ldg(map + 2 * (size_t)i + 1), H, W, t);
#pragma unroll
    for (int j = 0; j < kPlanesPerThread; j++)
      if (j < np) yp[(size_t)j * n] = gather<T, INTERP>(xp + j * hw, t);
  } else {
    T acc[kPlanesPerThread];
#pragma unroll
    for (int j = 0; j < kPlanesPerThread; j++) acc[j] = T(0);
    for (int q = 0; q < P; q++) {
      const size_t e = (size_t)i * P + q;
      decode<T, INTERP>(__ldg(map + 2 * e), __ldg(map + 2 * e + 1), H, W, t);
      const T wq = __ldg(iw + e);
#pragma unroll
      for (int j = 0; j < kPlanesPerThread; j++)
        if (j < np) acc[j] = RN<T>::add(acc[j], RN<T>::mul(wq, gather<T, INTERP>(xp + j * hw, t)));
    }
#pragma unroll
    for (int j = 0; j < kPlanesPerThread; j++)
      if (j < np) yp[(size_t)j * n] = acc[j];
  }
}

// Adjoint as a gather: destination pixel p sums its plan segment in stored
// order.  Replaces the atomicAdd scatter of cuda/resample.cuh:14-47.
template <typename T>
__global__ void __launch_bounds__(256)
resample_to_map_kernel(const T *__restrict__ x, const void *__restrict__ plan_blob, T *__restrict__ out, int n_dst,
                       int n_src, int planes) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_dst) return;
  bool ok;
  const PlanView<T> plan = plan_view<T>(plan_blob, n_dst, ok);
  const int p0 = blockIdx.y * kPlanesPerThread;
  const int np = min(kPlanesPerThread, planes - p0);
  const T *xp = x + (size_t)p0 * n_src;
  T acc[kPlanesPerThread];
#pragma unroll
  for (int j = 0; j < kPlanesPerThread; j++) acc[j] = T(0);
  const int e0 = ok ? __ldg(plan.offsets + p) : 0, e1 = ok ? __ldg(plan.offsets + p + 1) : 0;
  for (int e = e0; e < e1; e++) {
    const int s = __ldg(plan.src + e);
    const T w = __ldg(plan.w + e);
#pragma unroll
    for (int j = 0; j < kPlanesPerThread; j++)
      if (j < np) acc[j] += w * __ldg(xp + (size_t)j * n_src + s);
  }
#pragma unroll
  for (int j = 0; j < kPlanesPerThread; j++)
    if (j < np) out[(size_t)(p0 + j) * n_dst + p] = acc[j];
}

template <typename T>
static int from_map(const void *x, const void *map, const void *iw, void *y, int64_t planes, int64_t H, int64_t W,
                    int64_t n, int64_t P, int interp, cudaStream_t st) {
  dim3 grid(cdiv(n, 256), cdiv(planes, kPlanesPerThread));
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0)
      resample_from_map_kernel<T, INTERP, true><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, (const T *)iw,
                                                                       (T *)y, (int)n, (int)planes, (int)H, (int)W, (int)P);
    else
      resample_from_map_kernel<T, INTERP, false><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, nullptr, (T *)y,
                                                                        (int)n, (int)planes, (int)H, (int)W, 0);
  });
  return launch_status();
}

}  // namespace sph

using namespace sph;

extern "C" int sph_resample_from_map(const void *x, const void *map, const void *iw, void *y, int64_t B, int64_t C,
                                     int64_t H, int64_t W, int64_t MH, int64_t MW, int64_t P, int dtype, int interp,
                                     void *stream) {
  if (!x || !map || !y || B < 0 || C < 0 || H <= 0 || W <= 0 || MH < 0 || MW < 0 || P < 0 || (P > 0 && !iw))
    return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  if (interp < 0 || interp > 2) return SPH_ERR_INVALID_ARGUMENT;
  const int64_t n = MH * MW, planes = B * C, lim = (int64_t)1 << 31;
  if (H * W >= lim || n * (P > 0 ? P : 1) * 2 >= lim || planes / kPlanesPerThread >= 65535) return SPH_ERR_TOO_LARGE;
  if (n == 0 || planes == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? from_map<float>(x, map, iw, y, planes, H, W, n, P, interp, st)
                          : from_map<double>(x, map, iw, y, planes, H, W, n, P, interp, st);
}

extern "C" int sph_resample_to_map(const void *x, const void *plan, void *out, int64_t B, int64_t C, int64_t MH,
                                   int64_t MW, int64_t OH, int64_t OW, int dtype, void *stream) {
  if (!x || !plan || !out || B < 0 || C < 0 || MH <= 0 || MW <= 0 || OH <= 0 || OW <= 0) return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  const int64_t planes = B * C, lim = (int64_t)1 << 31;
  if (OH * OW >= lim || MH * MW >= lim || planes / kPlanesPerThread >= 65535) return SPH_ERR_TOO_LARGE;
  if (planes == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(cdiv(OH * OW, 256), cdiv(planes, kPlanesPerThread));
  if (dtype == SPH_F32)
    resample_to_map_kernel<float><<<grid, 256, 0, st>>>((const float *)x, plan, (float *)out, (int)(OH * OW),
                                                        (int)(MH * MW), (int)planes);
  else
    resample_to_map_kernel<double><<<grid, 256, 0, st>>>((const double *)x, plan, (double *)out, (int)(OH * OW),
                                                         (int)(MH * MW), (int)planes);
  return launch_status();
}
