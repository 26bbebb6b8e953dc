// resample_from_map (gather) and resample_to_map (adjoint, through a scatter plan).
#include <algorithm>

#include "common.cuh"
#include "plan_walk.cuh"

namespace sph {

// One thread decodes one map position once and then walks kPlanesPerThread
// (batch, channel) planes with the same taps.  Reference kernel:
// ext_modules/include/cuda/resample.cuh:50-81 (one thread per (c, position), one
// launch per image); arithmetic: common/resample.h:34-52, 85-107.
//
// With `quad` (UV-map gather, common/resample.h:133-159) every plane holds NT textures of H x W and position i samples
// texture quad[i]; an index outside [0, NT) yields zero.
template <typename T, int INTERP, bool WEIGHTED, int PPT>
__global__ void __launch_bounds__(256)
resample_from_map_kernel(const T *__restrict__ x, const T *__restrict__ map, const T *__restrict__ iw,
                         T *__restrict__ y, int n, int planes, int H, int W, int P, const int64_t *__restrict__ quad,
                         int NT) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int p0 = blockIdx.y * PPT;
  const int np = min(PPT, planes - p0);
  size_t hw = (size_t)H * W;
  const T *xp = x + (size_t)p0 * hw;
  T *yp = y + (size_t)p0 * n + i;
  Taps<T> t;
  bool dead = false;
  if (quad) {
    const int64_t q = __ldg(quad + i);
    dead = q < 0 || q >= NT;
    xp = x + (size_t)p0 * hw * NT + (dead ? 0 : (size_t)q * hw);
    hw *= NT;
  }
  if (!WEIGHTED) {
    decode<T, INTERP>(__ldg(map + 2 * (size_t)i), __ldg(map + 2 * (size_t)i + 1), H, W, t);
    if (dead) {
#pragma unroll
      for (int k = 0; k < 4; k++) t.off[k] = -1;
    }
#pragma unroll
    for (int j = 0; j < PPT; j++)
      if (j < np) yp[(size_t)j * n] = gather<T, INTERP>(xp + j * hw, t);
  } else {
    T acc[PPT];
#pragma unroll
    for (int j = 0; j < PPT; j++) acc[j] = T(0);
    for (int q = 0; q < P; q++) {
      const size_t e = (size_t)i * P + q;
      decode<T, INTERP>(__ldg(map + 2 * e), __ldg(map + 2 * e + 1), H, W, t);
      const T wq = __ldg(iw + e);
#pragma unroll
      for (int j = 0; j < PPT; j++)
        if (j < np) acc[j] = RN<T>::add(acc[j], RN<T>::mul(wq, gather<T, INTERP>(xp + j * hw, t)));
    }
#pragma unroll
    for (int j = 0; j < PPT; j++)
      if (j < np) yp[(size_t)j * n] = acc[j];
  }
}

// How a plan entry's source id s turns into the value it contributes.
//   div == 1   x[s]                       resample_to_map
//   div  > 1   x[s / div] / div           mapped average unpooling: the plan runs over the flattened map slots
//                                         s = o * K + k and every slot carries grad[o] / K
//                                         (common/mapped_avg_pool.h:41-69, 109-143)
template <typename T, bool DIV>
struct SrcValue {
  int div;
  FastDiv fd;
  __device__ __forceinline__ int index(int s) const { return DIV ? (int)fd.div((unsigned)s) : s; }
  __device__ __forceinline__ T value(T v) const { return DIV ? v / (T)div : v; }
};

// Adjoint as a gather through the plan (plan_walk.cuh): a CTA takes a chunk of destination pixels and PL planes.
// NORM: the sum is divided by (sum of the segment's weights + 1e-12), i.e. scatter(x) / (scatter(1) + 1e-12), the
// weight-sum normalisation the reference composes in Python (layers/functional/sphere_ops.py:74-80).
template <typename T, int PL, bool NORM, bool DIV>
__global__ void __launch_bounds__(256)
resample_to_map_kernel(const T *__restrict__ x, const void *__restrict__ plan_blob, T *__restrict__ out, int n_dst,
                       int n_src, int planes, int chunk, SrcValue<T, DIV> sv) {
  extern __shared__ unsigned char walk_smem[];
  bool ok;
  const PlanView<T> plan = plan_view<T>(plan_blob, n_dst, ok, DIV ? n_src * sv.div : n_src);
  const int p0 = blockIdx.y * PL;
  const int np = min(PL, planes - p0);
  const T *xp = x + (size_t)p0 * n_src;
  const int q_begin = blockIdx.x * chunk, q_end = min(q_begin + chunk, n_dst);
  plan_walk<T, PL, NORM>(plan, ok, n_dst, q_begin, q_end, (T *)walk_smem,
                         [&](int s) { return xp + sv.index(s); },
                         [&](const T *src, T w, int j) { return w * sv.value(__ldg(src + (size_t)j * n_src)); },
                         out + (size_t)p0 * n_dst, np);
}

// Planes walked per thread: 8 amortises the tap decode best; small problems use 2 so that enough threads are
// in flight to cover the memory latency.
static int planes_per_thread(int64_t n, int64_t planes) {
  return n * ((planes + 7) / 8) >= (int64_t)148 * 2048 * 2 ? 8 : 2;
}

template <typename T, int PPT>
static void from_map_launch(const void *x, const void *map, const void *iw, void *y, int64_t planes, int64_t H, int64_t W,
                            int64_t n, int64_t P, int interp, cudaStream_t st, const int64_t *quad, int NT) {
  dim3 grid(cdiv(n, 256), cdiv(planes, PPT));
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0)
      resample_from_map_kernel<T, INTERP, true, PPT><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, (const T *)iw, (T *)y,
                                                                           (int)n, (int)planes, (int)H, (int)W, (int)P, nullptr, 1);
    else
      resample_from_map_kernel<T, INTERP, false, PPT><<<grid, 256, 0, st>>>((const T *)x, (const T *)map, nullptr, (T *)y,
                                                                            (int)n, (int)planes, (int)H, (int)W, 0, quad, NT);
  });
}

template <typename T>
static int from_map(const void *x, const void *map, const void *iw, void *y, int64_t planes, int64_t H, int64_t W,
                    int64_t n, int64_t P, int interp, cudaStream_t st, const int64_t *quad = nullptr, int NT = 1) {
  if (planes_per_thread(n, planes) == 8) from_map_launch<T, 8>(x, map, iw, y, planes, H, W, n, P, interp, st, quad, NT);
  else from_map_launch<T, 2>(x, map, iw, y, planes, H, W, n, P, interp, st, quad, NT);
  return launch_status();
}

// n_src: elements per source plane; src_div: see SrcValue.
template <typename T, int PL, bool NORM, bool DIV>
static void to_map_launch(const void *x, const void *plan, void *out, int64_t planes, int64_t n_src, int64_t n_dst, int src_div,
                          cudaStream_t st) {
  const int groups = cdiv(planes, PL);
  // CTAs of 8 warps; enough CTAs for a few waves of the SMs, each warp walking several 32-pixel blocks so that the
  // segment bounds of the next block are in flight while the current one is summed
  int64_t chunks = ((int64_t)148 * 16 + groups - 1) / groups;
  const int64_t max_chunks = (n_dst + 255) / 256;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  const int chunk = (int)(((n_dst + chunks - 1) / chunks + 255) / 256 * 256);
  const size_t smem = 8 * (size_t)walk_smem_per_warp<T, PL, NORM>();
  resample_to_map_kernel<T, PL, NORM, DIV><<<dim3(cdiv(n_dst, chunk), groups), 256, smem, st>>>(
      (const T *)x, plan, (T *)out, (int)n_dst, (int)n_src, (int)planes, chunk, SrcValue<T, DIV>{src_div, FastDiv::make((unsigned)src_div)});
}

template <typename T, bool NORM, bool DIV>
static int to_map_n(const void *x, const void *plan, void *out, int64_t planes, int64_t n_src, int64_t n_dst, int src_div,
                    cudaStream_t st) {
  // planes per CTA: more planes amortise the plan reads and put more stores in flight per warp
  if (sizeof(T) == 4 && planes >= 128) to_map_launch<T, 16, NORM, DIV>(x, plan, out, planes, n_src, n_dst, src_div, st);
  else if (planes >= 8) to_map_launch<T, 8, NORM, DIV>(x, plan, out, planes, n_src, n_dst, src_div, st);
  else to_map_launch<T, 4, NORM, DIV>(x, plan, out, planes, n_src, n_dst, src_div, st);
  return launch_status();
}

template <typename T>
static int to_map(const void *x, const void *plan, void *out, int64_t planes, int64_t n_src, int64_t n_dst, cudaStream_t st,
                  int src_div = 1, bool normalize = false) {
  if (src_div > 1) return to_map_n<T, false, true>(x, plan, out, planes, n_src, n_dst, src_div, st);  // never normalised
  return normalize ? to_map_n<T, true, false>(x, plan, out, planes, n_src, n_dst, 1, st)
                   : to_map_n<T, false, false>(x, plan, out, planes, n_src, n_dst, 1, st);
}

// Voting resample of integer labels through a nearest-neighbour plan: destination pixel o takes the label that most
// of the source pixels mapped onto it carry, the smallest such label on ties, 0 if none does (torch.argmax over a
// vote histogram in the reference: src/cpp/voting_resample_layer.cpp:8-37, core/interpolation.h:249-265).  The
// segment is walked once per entry (segments hold the few source pixels that land on one output pixel), so no
// (pixels x candidates) histogram is materialised.
__global__ void __launch_bounds__(256)
voting_resample_kernel(const int64_t *__restrict__ x, const void *__restrict__ plan_blob, int64_t *__restrict__ out, int n_dst,
                       int n_src, int planes, int64_t num_candidates, int dtype) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x, p = blockIdx.y;
  if (o >= n_dst) return;
  const PlanHeader *h = (const PlanHeader *)plan_blob;
  const bool ok = h->magic == kPlanMagic && h->n_keys == n_dst && h->dtype == dtype && h->n_src == n_src;
  const int *offsets = (const int *)((const char *)plan_blob + h->off_offsets);
  const int *src = (const int *)((const char *)plan_blob + h->off_src);
  const int64_t *xp = x + (size_t)p * n_src;
  const int e0 = ok ? __ldg(offsets + o) : 0, e1 = ok ? __ldg(offsets + o + 1) : 0;
  int64_t best = 0;
  int best_votes = 0;
  for (int i = e0; i < e1; i++) {
    const int64_t li = __ldg(xp + __ldg(src + i));
    if (li < 0 || li >= num_candidates) continue;
    int votes = 0;
    bool first = true;
    for (int j = e0; j < e1; j++)
      if (__ldg(xp + __ldg(src + j)) == li) {
        votes++;
        if (j < i) first = false;
      }
    if (first && (votes > best_votes || (votes == best_votes && li < best))) {
      best = li;
      best_votes = votes;
    }
  }
  out[(size_t)p * n_dst + o] = best;
}

}  // namespace sph

using namespace sph;

SPH_TU_STATUS(resample)

extern "C" int sph_resample_from_map(const void *x, const void *map, const void *iw, void *y, int64_t B, int64_t C,
                                     int64_t H, int64_t W, int64_t MH, int64_t MW, int64_t P, int dtype, int interp,
                                     void *stream) {
  SPH_RANGE("sph_resample_from_map");
  if (!x || !map || !y || B < 0 || C < 0 || H <= 0 || W <= 0 || MH < 0 || MW < 0 || P < 0 || (P > 0 && !iw))
    return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  if (interp < 0 || interp > 2) return SPH_ERR_INVALID_ARGUMENT;
  const int64_t n = MH * MW, planes = B * C, lim = (int64_t)1 << 31;
  if (H * W >= lim || n * (P > 0 ? P : 1) * 2 >= lim || planes / 2 >= 65535) return SPH_ERR_TOO_LARGE;
  if (n == 0 || planes == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? from_map<float>(x, map, iw, y, planes, H, W, n, P, interp, st)
                          : from_map<double>(x, map, iw, y, planes, H, W, n, P, interp, st);
}

extern "C" int sph_resample_to_map(const void *x, const void *plan, void *out, int64_t B, int64_t C, int64_t MH,
                                   int64_t MW, int64_t OH, int64_t OW, int dtype, void *stream) {
  SPH_RANGE("sph_resample_to_map");
  if (!x || !plan || !out || B < 0 || C < 0 || MH <= 0 || MW <= 0 || OH <= 0 || OW <= 0) return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  const int64_t planes = B * C, lim = (int64_t)1 << 31;
  if (OH * OW >= lim || MH * MW >= lim || planes / 2 >= 65535) return SPH_ERR_TOO_LARGE;
  if (planes == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? to_map<float>(x, plan, out, planes, MH * MW, OH * OW, st)
                          : to_map<double>(x, plan, out, planes, MH * MW, OH * OW, st);
}

extern "C" int sph_resample_to_map_normalized(const void *x, const void *plan, void *out, int64_t B, int64_t C, int64_t MH,
                                              int64_t MW, int64_t OH, int64_t OW, int dtype, void *stream) {
  SPH_RANGE("sph_resample_to_map_normalized");
  if (!x || !plan || !out || B < 0 || C < 0 || MH <= 0 || MW <= 0 || OH <= 0 || OW <= 0) return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  const int64_t planes = B * C, lim = (int64_t)1 << 31;
  if (OH * OW >= lim || MH * MW >= lim || planes / 2 >= 65535) return SPH_ERR_TOO_LARGE;
  if (planes == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? to_map<float>(x, plan, out, planes, MH * MW, OH * OW, st, 1, true)
                          : to_map<double>(x, plan, out, planes, MH * MW, OH * OW, st, 1, true);
}

extern "C" int sph_mapped_avg_unpool(const void *g, const void *plan, void *grad_in, int64_t B, int64_t C, int64_t IH,
                                     int64_t IW, int64_t OH, int64_t OW, int64_t K, int dtype, void *stream) {
  SPH_RANGE("sph_mapped_avg_unpool");
  if (!g || !plan || !grad_in || B < 0 || C < 0 || IH <= 0 || IW <= 0 || OH <= 0 || OW <= 0 || K <= 0)
    return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  const int64_t planes = B * C, lim = (int64_t)1 << 31;
  if (OH * OW * K >= lim || IH * IW >= lim || planes / 2 >= 65535) return SPH_ERR_TOO_LARGE;
  if (planes == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? to_map<float>(g, plan, grad_in, planes, OH * OW, IH * IW, st, (int)K)
                          : to_map<double>(g, plan, grad_in, planes, OH * OW, IH * IW, st, (int)K);
}

extern "C" int sph_resample_from_uv_maps(const void *tex, const int64_t *quad_idx, const void *tex_uv, void *out, int64_t B,
                                         int64_t C, int64_t NT, int64_t TH, int64_t TW, int64_t IH, int64_t IW, int dtype,
                                         int interp, void *stream) {
  SPH_RANGE("sph_resample_from_uv_maps");
  if (!tex || !quad_idx || !tex_uv || !out || B < 0 || C < 0 || NT <= 0 || TH <= 0 || TW <= 0 || IH < 0 || IW < 0 ||
      interp < 0 || interp > 2)
    return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  const int64_t n = IH * IW, planes = B * C, lim = (int64_t)1 << 31;
  if (NT * TH * TW >= lim || n * 2 >= lim || planes / 2 >= 65535) return SPH_ERR_TOO_LARGE;
  if (n == 0 || planes == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? from_map<float>(tex, tex_uv, nullptr, out, planes, TH, TW, n, 0, interp, st, quad_idx, (int)NT)
                          : from_map<double>(tex, tex_uv, nullptr, out, planes, TH, TW, n, 0, interp, st, quad_idx, (int)NT);
}

extern "C" int sph_voting_resample_to_map(const int64_t *labels, const void *plan, int plan_dtype, int64_t *out, int64_t B,
                                          int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t num_candidates,
                                          void *stream) {
  SPH_RANGE("sph_voting_resample_to_map");
  if (!labels || !plan || !out || B < 0 || C < 0 || IH <= 0 || IW <= 0 || OH <= 0 || OW <= 0 || num_candidates <= 0)
    return SPH_ERR_INVALID_ARGUMENT;
  if (plan_dtype != SPH_F32 && plan_dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  const int64_t planes = B * C, lim = (int64_t)1 << 31;
  if (OH * OW >= lim || IH * IW >= lim || planes >= 65535) return SPH_ERR_TOO_LARGE;
  if (planes == 0) return SPH_OK;
  voting_resample_kernel<<<dim3(cdiv(OH * OW, 256), (unsigned)planes), 256, 0, (cudaStream_t)stream>>>(
      labels, plan, out, (int)(OH * OW), (int)(IH * IW), (int)planes, num_candidates, plan_dtype);
  return launch_status();
}
