// Scatter plan: the sample map inverted into a CSR table keyed by
// (destination pixel, kernel slot), entries ordered by their position in the
// map so that every adjoint operator sums in one fixed order.
#include "common.cuh"

namespace sph {

// Visit every valid tap of map slot s (= position * K + k): f(key, id, weight).
// With `quad` (UV maps: the destination is NT textures of H x W and position s / K writes into texture quad[s / K],
// ext_modules/include/common/resample.h:161-187) the key is offset by that texture; a texture index outside
// [0, NT) has no taps.
template <typename T, int INTERP, bool WEIGHTED, typename F>
__device__ __forceinline__ void for_each_tap(const T *__restrict__ map, const T *__restrict__ iw, int s, int K, int PP,
                                             int H, int W, const int64_t *__restrict__ quad, int NT, F f) {
  const int k = s % K;
  int base = 0;
  if (quad) {
    const int64_t q = __ldg(quad + s / K);
    if (q < 0 || q >= NT) return;
    base = (int)q * H * W;
  }
  Taps<T> t;
  for (int q = 0; q < PP; q++) {
    const size_t e = (size_t)s * PP + q;
    decode<T, INTERP>(__ldg(map + 2 * e), __ldg(map + 2 * e + 1), H, W, t);
    const T wq = WEIGHTED ? __ldg(iw + e) : T(1);
#pragma unroll
    for (int i = 0; i < TapCount<INTERP>::value; i++)
      if (t.off[i] >= 0) f((base + t.off[i]) * K + k, (int)(e * 4 + i), WEIGHTED ? wq * t.w[i] : t.w[i]);
  }
}

template <typename T, int INTERP, bool WEIGHTED>
__global__ void plan_count_kernel(const T *map, const T *iw, int n_slots, int K, int PP, int H, int W, const int64_t *quad,
                                  int NT, int *cnt) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_slots) return;
  const int n_keys = NT * H * W * K;
  for_each_tap<T, INTERP, WEIGHTED>(map, iw, s, K, PP, H, W, quad, NT, [&](int key, int, T) {
    if (index_ok(key, n_keys)) atomicAdd(cnt + key, 1);
  });
}

template <typename T, int INTERP, bool WEIGHTED>
__global__ void plan_fill_kernel(const T *map, const T *iw, int n_slots, int K, int PP, int H, int W, const int64_t *quad,
                                 int NT, const int *offsets, int *cursor, int *ids, T *w, int e_max) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_slots) return;
  const int n_keys = NT * H * W * K;
  for_each_tap<T, INTERP, WEIGHTED>(map, iw, s, K, PP, H, W, quad, NT, [&](int key, int id, T wt) {
    if (!index_ok(key, n_keys)) return;
    const int pos = offsets[key] + atomicAdd(cursor + key, 1);
    if (!index_ok(pos, e_max)) return;
    ids[pos] = id;
    w[pos] = wt;
  });
}

// One thread per key: order the segment by entry id (the fill order above is not reproducible), then turn ids into
// source positions.  Short segments (the usual case: a handful of samples per pixel) by insertion, longer ones by an
// in-place heap sort, so that a map that sends very many samples to one pixel costs n log n, not n^2.
template <typename T>
__device__ __forceinline__ void sift_down(int *ids, T *w, int root, int n) {
  for (;;) {
    int child = 2 * root + 1;
    if (child >= n) return;
    if (child + 1 < n && ids[child + 1] > ids[child]) child++;
    if (ids[root] >= ids[child]) return;
    const int ti = ids[root];
    ids[root] = ids[child];
    ids[child] = ti;
    const T tw = w[root];
    w[root] = w[child];
    w[child] = tw;
    root = child;
  }
}

template <typename T>
__global__ void plan_sort_kernel(const int *offsets, int *ids, T *w, int n_keys, int id_div, int *max_seg) {
  const int key = blockIdx.x * blockDim.x + threadIdx.x;
  if (key >= n_keys) return;
  const int e0 = offsets[key], e1 = offsets[key + 1], n = e1 - e0;
  if (n > 1) atomicMax(max_seg, n);
  if (n <= 16) {
    for (int i = e0 + 1; i < e1; i++) {
      const int id = ids[i];
      const T wi = w[i];
      int j = i - 1;
      while (j >= e0 && ids[j] > id) {
        ids[j + 1] = ids[j];
        w[j + 1] = w[j];
        j--;
      }
      ids[j + 1] = id;
      w[j + 1] = wi;
    }
  } else {
    int *a = ids + e0;
    T *aw = w + e0;
    for (int r = n / 2 - 1; r >= 0; r--) sift_down(a, aw, r, n);
    for (int end = n - 1; end > 0; end--) {
      const int ti = a[0];
      a[0] = a[end];
      a[end] = ti;
      const T tw = aw[0];
      aw[0] = aw[end];
      aw[end] = tw;
      sift_down(a, aw, 0, end);
    }
  }
  for (int i = e0; i < e1; i++) ids[i] = ids[i] / id_div;
}

// ---- exclusive scan of n ints (three passes, kScanItems per block) -------
constexpr int kScanThreads = 256;
constexpr int kScanPer = kScanItems / kScanThreads;

__device__ __forceinline__ int block_exclusive_scan(int v, int *total) {
  __shared__ int warp_sums[kScanThreads / 32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += u;
  }
  if (lane == 31) warp_sums[wid] = incl;
  __syncthreads();
  if (wid == 0) {
    int s = lane < kScanThreads / 32 ? warp_sums[lane] : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += u;
    }
    if (lane < kScanThreads / 32) warp_sums[lane] = s;
  }
  __syncthreads();
  const int base = wid ? warp_sums[wid - 1] : 0;
  if (total) *total = warp_sums[kScanThreads / 32 - 1];
  __syncthreads();
  return base + incl - v;
}

__global__ void __launch_bounds__(kScanThreads) scan_sums_kernel(const int *in, int n, int *sums) {
  const int base = blockIdx.x * kScanItems + threadIdx.x * kScanPer;
  int s = 0;
#pragma unroll
  for (int i = 0; i < kScanPer; i++)
    if (base + i < n) s += in[base + i];
  int total;
  block_exclusive_scan(s, &total);
  if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanThreads) scan_top_kernel(int *sums, int nb) {
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < nb; b0 += kScanThreads) {
    const int i = b0 + threadIdx.x;
    const int v = i < nb ? sums[i] : 0;
    int total;
    const int ex = block_exclusive_scan(v, &total);
    const int c = carry;
    if (i < nb) sums[i] = c + ex;
    __syncthreads();
    if (threadIdx.x == 0) carry = c + total;
    __syncthreads();
  }
  if (threadIdx.x == 0) sums[nb] = carry;
}

__global__ void __launch_bounds__(kScanThreads) scan_final_kernel(const int *in, int n, const int *sums, int *out) {
  const int base = blockIdx.x * kScanItems + threadIdx.x * kScanPer;
  int v[kScanPer], s = 0;
#pragma unroll
  for (int i = 0; i < kScanPer; i++) {
    v[i] = base + i < n ? in[base + i] : 0;
    s += v[i];
  }
  int run = block_exclusive_scan(s, nullptr) + sums[blockIdx.x];
#pragma unroll
  for (int i = 0; i < kScanPer; i++) {
    if (base + i < n) out[base + i] = run;
    run += v[i];
  }
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) out[n] = sums[gridDim.x];
}

__global__ void plan_header_kernel(PlanHeader *dst, PlanHeader h) { *dst = h; }

template <typename T>
static int build(const void *map, const void *iw, int64_t n_src, int64_t K, int64_t P, int interp, int64_t H,
                 int64_t W, int dtype, void *plan, const PlanLayout &L, cudaStream_t st, const int64_t *quad = nullptr,
                 int NT = 1) {
  char *base = (char *)plan;
  int *offsets = (int *)(base + L.off_offsets), *src = (int *)(base + L.off_src);
  int *cursor = (int *)(base + L.off_cursor), *sums = (int *)(base + L.off_sums);
  T *w = (T *)(base + L.off_w);
  const int n_slots = (int)(n_src * K), PP = (int)(P > 0 ? P : 1), nk = (int)L.n_keys;
  if (cudaMemsetAsync(cursor, 0, sizeof(int) * (size_t)nk, st) != cudaSuccess) return SPH_ERR_CUDA;
  const int gb = cdiv(n_slots, 256);
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0)
      plan_count_kernel<T, INTERP, true><<<gb, 256, 0, st>>>((const T *)map, (const T *)iw, n_slots, (int)K, PP, (int)H, (int)W, quad, NT, cursor);
    else
      plan_count_kernel<T, INTERP, false><<<gb, 256, 0, st>>>((const T *)map, nullptr, n_slots, (int)K, PP, (int)H, (int)W, quad, NT, cursor);
  });
  scan_sums_kernel<<<L.n_scan_blocks, kScanThreads, 0, st>>>(cursor, nk, sums);
  scan_top_kernel<<<1, kScanThreads, 0, st>>>(sums, L.n_scan_blocks);
  scan_final_kernel<<<L.n_scan_blocks, kScanThreads, 0, st>>>(cursor, nk, sums, offsets);
  if (cudaMemsetAsync(cursor, 0, sizeof(int) * (size_t)nk, st) != cudaSuccess) return SPH_ERR_CUDA;
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0)
      plan_fill_kernel<T, INTERP, true><<<gb, 256, 0, st>>>((const T *)map, (const T *)iw, n_slots, (int)K, PP, (int)H, (int)W, quad, NT, offsets, cursor, src, w, (int)L.e_max);
    else
      plan_fill_kernel<T, INTERP, false><<<gb, 256, 0, st>>>((const T *)map, nullptr, n_slots, (int)K, PP, (int)H, (int)W, quad, NT, offsets, cursor, src, w, (int)L.e_max);
  });
  PlanHeader h;
  h.magic = kPlanMagic;
  h.n_keys = nk;
  h.K = (int)K;
  h.dtype = dtype;
  h.e_max = (int)L.e_max;
  h.off_offsets = L.off_offsets;
  h.off_src = L.off_src;
  h.off_w = L.off_w;
  h.max_seg = 1;
  h.n_src = (int)n_src;  // map positions (each with K slots)
  plan_header_kernel<<<1, 1, 0, st>>>((PlanHeader *)plan, h);
  plan_sort_kernel<T><<<cdiv(nk, 256), 256, 0, st>>>(offsets, src, w, nk, (int)(4 * PP * K), &((PlanHeader *)plan)->max_seg);
  return launch_status(7);
}

}  // namespace sph

using namespace sph;

SPH_TU_STATUS(plan)

extern "C" size_t sph_plan_bytes(int64_t n_src, int64_t K, int64_t P, int interp, int64_t dstH, int64_t dstW,
                                 int dtype) {
  PlanLayout L;
  if (P < 0 || !plan_layout(n_src, K, P, interp, dstH, dstW, dtype, L)) return 0;
  return L.total;
}

extern "C" int sph_plan_build(const void *map, const void *iw, int64_t n_src, int64_t K, int64_t P, int interp,
                              int64_t dstH, int64_t dstW, int dtype, void *plan, size_t plan_bytes, void *stream) {
  SPH_RANGE("sph_plan_build");
  if (!map || !plan || P < 0 || (P > 0 && !iw) || interp < 0 || interp > 2) return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  PlanLayout L;
  if (!plan_layout(n_src, K, P, interp, dstH, dstW, dtype, L)) return SPH_ERR_TOO_LARGE;
  if (plan_bytes < L.total) return SPH_ERR_WORKSPACE_TOO_SMALL;
  if (((uintptr_t)plan & 255) != 0) return SPH_ERR_INVALID_ARGUMENT;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? build<float>(map, iw, n_src, K, P, interp, dstH, dstW, dtype, plan, L, st)
                          : build<double>(map, iw, n_src, K, P, interp, dstH, dstW, dtype, plan, L, st);
}

// Plan of the UV-map scatter (resample_to_uv_maps): the destination is NT textures of TH x TW, laid out as one
// (NT*TH) x TW image; interpolation and its zero padding act inside the texture quad_idx names.
extern "C" int sph_plan_build_uv(const void *tex_uv, const int64_t *quad_idx, int64_t n_src, int64_t NT, int64_t TH,
                                 int64_t TW, int interp, int dtype, void *plan, size_t plan_bytes, void *stream) {
  SPH_RANGE("sph_plan_build_uv");
  if (!tex_uv || !quad_idx || !plan || NT <= 0 || interp < 0 || interp > 2) return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  PlanLayout L;
  if (!plan_layout(n_src, 1, 0, interp, NT * TH, TW, dtype, L)) return SPH_ERR_TOO_LARGE;
  if (plan_bytes < L.total) return SPH_ERR_WORKSPACE_TOO_SMALL;
  if (((uintptr_t)plan & 255) != 0) return SPH_ERR_INVALID_ARGUMENT;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == SPH_F32 ? build<float>(tex_uv, nullptr, n_src, 1, 0, interp, TH, TW, dtype, plan, L, st, quad_idx, (int)NT)
                          : build<double>(tex_uv, nullptr, n_src, 1, 0, interp, TH, TW, dtype, plan, L, st, quad_idx, (int)NT);
}

// ---- resample_to_map without any allocation ---------------------------------------------------
// Scratch for callers that cannot allocate: the plan lives in this array, which is part of the library image
// on every device.  In host code the name `g_static_scratch` is only a handle for the runtime, not a device
// address, so the address is looked up once per device and that pointer is what the kernels get.
static __device__ __align__(256) unsigned char g_static_scratch[SPH_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void *g_static_scratch_ptr[kMaxDevices];  // per device, filled by the first call made with that device current
}  // namespace

extern "C" int sph_resample_to_map_static(const void *x, const void *map, const void *iw, void *out, int64_t B, int64_t C,
                                          int64_t MH, int64_t MW, int64_t OH, int64_t OW, int64_t P, int dtype, int interp,
                                          void *stream) {
  if (!x || !map || !out || P < 0 || (P > 0 && !iw) || interp < 0 || interp > 2) return SPH_ERR_INVALID_ARGUMENT;
  if (B < 0 || C < 0 || MH <= 0 || MW <= 0 || OH <= 0 || OW <= 0) return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  // everything sph_resample_to_map would refuse is refused here, before the shared array is touched
  if (OH * OW >= ((int64_t)1 << 31) || MH * MW >= ((int64_t)1 << 31) || B * C / 2 >= 65535) return SPH_ERR_TOO_LARGE;
  PlanLayout L;
  if (!plan_layout(MH * MW, 1, P, interp, OH, OW, dtype, L)) return SPH_ERR_TOO_LARGE;
  if (L.total > (size_t)SPH_STATIC_SCRATCH_BYTES) return SPH_ERR_STATIC_SCRATCH_EXCEEDED;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SPH_ERR_CUDA;
  void *scratch = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!scratch) {
    if (cudaGetSymbolAddress(&scratch, g_static_scratch) != cudaSuccess || !scratch) return SPH_ERR_CUDA;
    __atomic_store_n(&g_static_scratch_ptr[dev], scratch, __ATOMIC_RELEASE);
  }
  const int rc = sph_plan_build(map, iw, MH * MW, 1, P, interp, OH, OW, dtype, scratch, SPH_STATIC_SCRATCH_BYTES, stream);
  if (rc != SPH_OK) return rc;
  return sph_resample_to_map(x, scratch, out, B, C, MH, MW, OH, OW, dtype, stream);
}
