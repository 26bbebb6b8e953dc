// Host side of the drop-in `_spherical_distortion_ext` package: a thin
// PyTorch extension that checks arguments, allocates outputs with torch's
// caching allocator and calls the C ABI of libsphmap.so (include/sphmap.h) on
// the current CUDA stream.  Function names and positional argument order are
// those of the reference's pybind modules (ext_modules/include/layers/*.h);
// the Python files next to this extension re-export them under the reference's
// module names.  There is no CPU path: CPU tensors raise.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>

#include <cstdlib>
#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "sphmap.h"

namespace {

enum class InterpolationType { NEAREST = 0, BILINEAR = 1, BISPHERICAL = 2 };   // include/enums.h:12-16
enum class DistortionType { SIMPLE_RADIAL = 0, BROWN = 1, FISHEYE = 2 };       // include/enums.h:6-10

int g_precision = -1;
bool g_deterministic_unpool = true;  // argmax backward through a plan (fixed summation order) instead of float atomics

int precision() {
  if (g_precision < 0) {
    const char *e = std::getenv("SPHERICAL_MAPPED_PRECISION");
    const std::string s = e ? e : "fp32";
    TORCH_CHECK(s == "fp32" || s == "bf16", "SPHERICAL_MAPPED_PRECISION must be fp32 or bf16, got ", s);
    g_precision = s == "bf16" ? SPH_PRECISION_BF16 : SPH_PRECISION_EXACT;
  }
  return g_precision;
}

void set_precision(const std::string &s) {
  TORCH_CHECK(s == "fp32" || s == "bf16", "precision must be 'fp32' or 'bf16', got ", s);
  g_precision = s == "bf16" ? SPH_PRECISION_BF16 : SPH_PRECISION_EXACT;
}

std::string get_precision() { return precision() == SPH_PRECISION_BF16 ? "bf16" : "fp32"; }

void ok(int status, const char *what) {
  TORCH_CHECK(status == SPH_OK, what, ": ", sph_status_string(status));
}

// SPHERICAL_MAPPED_CHECK_STATUS=1: after every convolution call wait for the device and raise if a bounded wait inside
// a tensor-core kernel gave up (off by default: the check synchronises).
void maybe_check_device(const char *what) {
  static const bool on = [] {
    const char *e = std::getenv("SPHERICAL_MAPPED_CHECK_STATUS");
    return e && *e && std::string(e) != "0";
  }();
  if (!on) return;
  int v = 0;
  ok(sph_device_status(&v, 1), "sph_device_status");
  TORCH_CHECK(v == 0, what, ": a bounded wait inside a tensor-core kernel gave up; the results are invalid");
}

int dtype_of(const torch::Tensor &t) {
  TORCH_CHECK(t.scalar_type() == torch::kFloat || t.scalar_type() == torch::kDouble,
              "mapped operators support float32 and float64 tensors only");
  return t.scalar_type() == torch::kDouble ? SPH_F64 : SPH_F32;
}

// Same preconditions as CHECK_CUDA / CHECK_CONTIGUOUS of include/cuda_helper.h:12-18.
void check(const torch::Tensor &t, const char *name, const torch::Tensor &like) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (this build has no CPU path)");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.device() == like.device(), name, " must be on the same device as the input");
}

void check_float(const torch::Tensor &t, const char *name, const torch::Tensor &like) {
  check(t, name, like);
  TORCH_CHECK(t.scalar_type() == like.scalar_type(), name, " must have the input's dtype");
}

struct MapInfo {
  int64_t H, W, K, P;  // map spatial size, kernel slots (1 if absent), interpolation points (0 if unweighted)
};

// map: (H,W,[K,][P,]2); weights: (H,W,[K,]P)
MapInfo map_info(const torch::Tensor &map, const torch::Tensor *iw, bool has_k, int64_t kernel_size) {
  const int64_t want = 3 + (has_k ? 1 : 0) + (iw ? 1 : 0);
  TORCH_CHECK(map.dim() == want, "sample map must have ", want, " dimensions, got ", map.dim());
  TORCH_CHECK(map.size(-1) == 2, "last dimension of the sample map must be 2");
  MapInfo m{map.size(0), map.size(1), has_k ? map.size(2) : 1, 0};
  if (has_k) TORCH_CHECK(m.K == kernel_size, "kernel size of the sample map (", m.K, ") != kernel_size (", kernel_size, ")");
  if (iw) {
    m.P = map.size(-2);
    TORCH_CHECK(iw->dim() == want - 1 && iw->size(-1) == m.P && iw->size(0) == m.H && iw->size(1) == m.W &&
                    (!has_k || iw->size(2) == m.K),
                "interpolation weights do not match the sample map");
    TORCH_CHECK(m.P > 0, "need at least one interpolation point");
  }
  return m;
}

// ---- scatter-plan cache ---------------------------------------------------
// A plan depends only on the map (and weights); training loops call the same
// layer with the same map every step, so plans are kept, keyed by the
// identity and version of the tensors' storage.
struct PlanKey {
  c10::weak_intrusive_ptr<c10::StorageImpl> map_s, iw_s;
  const void *map_p, *iw_p;
  int64_t map_off, iw_off;
  uint32_t map_v, iw_v;
  int64_t n_src, K, P, dstH, dstW;
  int interp, dtype, device;
  torch::Tensor blob;
  std::shared_ptr<at::cuda::CUDAEvent> built;  // recorded after the build kernels, on the stream that ran them
  cudaStream_t build_stream;
};

// Version counter of a tensor; inference tensors have none (and cannot be modified in place): 0.
uint32_t version_of(const torch::Tensor &t) { return t.is_inference() ? 0u : (uint32_t)t._version(); }
// (The caches are never destroyed: at interpreter shutdown the CUDA runtime may already be gone when static destructors
// run, and releasing an event or a tensor then throws.  The process exit reclaims them.)
std::list<PlanKey> &plan_cache() {
  static auto *cache = new std::list<PlanKey>();
  return *cache;
}
#define g_plans plan_cache()
std::mutex g_plan_mu;
constexpr size_t kMaxPlans = 64;

// uv_textures > 0: `iw` is the int64 texture-index tensor of a UV map and the plan is built by sph_plan_build_uv for
// uv_textures textures of (dstH / uv_textures) x dstW texels.
torch::Tensor get_plan(const torch::Tensor &map, const torch::Tensor *iw, int64_t n_src, int64_t K, int64_t P, int interp,
                       int64_t dstH, int64_t dstW, int64_t uv_textures = 0) {
  const int dtype = dtype_of(map), device = map.get_device();
  if (uv_textures > 0) K = -uv_textures;  // keeps UV plans apart from ordinary ones in the cache
  std::lock_guard<std::mutex> lock(g_plan_mu);
  for (auto it = g_plans.begin(); it != g_plans.end();) {
    if (it->map_s.expired() || (it->iw_p && it->iw_s.expired())) {
      it = g_plans.erase(it);
      continue;
    }
    const bool hit = it->map_p == map.data_ptr() && it->map_off == map.storage_offset() && it->map_v == version_of(map) &&
                     it->map_s.lock().get() == map.storage().unsafeGetStorageImpl() &&
                     (iw ? (it->iw_p == iw->data_ptr() && it->iw_v == version_of(*iw) &&
                            it->iw_s.lock().get() == iw->storage().unsafeGetStorageImpl())
                         : it->iw_p == nullptr) &&
                     it->n_src == n_src && it->K == K && it->P == P && it->dstH == dstH && it->dstW == dstW &&
                     it->interp == interp && it->dtype == dtype && it->device == device;
    if (hit) {
      g_plans.splice(g_plans.begin(), g_plans, it);
      // a caller on another stream than the one that built the plan waits for the build first
      const cudaStream_t cur = at::cuda::getCurrentCUDAStream().stream();
      if (cur != g_plans.front().build_stream) g_plans.front().built->block(at::cuda::getCurrentCUDAStream());
      return g_plans.front().blob;
    }
    ++it;
  }
  const size_t bytes = sph_plan_bytes(n_src, uv_textures > 0 ? 1 : K, P, interp, dstH, dstW, dtype);
  TORCH_CHECK(bytes > 0, "sample map too large for a scatter plan");
  torch::Tensor blob = torch::empty({(int64_t)bytes}, map.options().dtype(torch::kUInt8));
  if (uv_textures > 0)
    ok(sph_plan_build_uv(map.data_ptr(), iw->data_ptr<int64_t>(), n_src, uv_textures, dstH / uv_textures, dstW, interp, dtype,
                         blob.data_ptr(), bytes, at::cuda::getCurrentCUDAStream().stream()),
       "sph_plan_build_uv");
  else
    ok(sph_plan_build(map.data_ptr(), iw ? iw->data_ptr() : nullptr, n_src, K, P, interp, dstH, dstW, dtype, blob.data_ptr(),
                      bytes, at::cuda::getCurrentCUDAStream().stream()),
       "sph_plan_build");
  PlanKey k{c10::weak_intrusive_ptr<c10::StorageImpl>(map.storage().getWeakStorageImpl()),
            iw ? c10::weak_intrusive_ptr<c10::StorageImpl>(iw->storage().getWeakStorageImpl())
               : c10::weak_intrusive_ptr<c10::StorageImpl>(map.storage().getWeakStorageImpl()),
            map.data_ptr(), iw ? iw->data_ptr() : nullptr, map.storage_offset(), iw ? iw->storage_offset() : 0,
            version_of(map), iw ? version_of(*iw) : 0u, n_src, K, P, dstH, dstW, interp, dtype, device, blob,
            std::make_shared<at::cuda::CUDAEvent>(), at::cuda::getCurrentCUDAStream().stream()};
  k.built->record(at::cuda::getCurrentCUDAStream());
  g_plans.push_front(std::move(k));
  if (g_plans.size() > kMaxPlans) g_plans.pop_back();
  return blob;
}

void clear_plan_cache() {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  g_plans.clear();
}

int64_t plan_cache_size() {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  return (int64_t)g_plans.size();
}

// ---- channels-last companions of activations (bf16 precision) -------------------
// The tensor-core kernels gather from a channels-last bf16 copy of their input.  A layer with the fused ReLU writes
// that copy of its output from its own epilogue; it is remembered here under the identity of the output tensor, so
// that the next layer (whose input that tensor is) finds it in forward and in backward and skips its conversion
// pass.  An entry dies with the tensor's storage, on an in-place modification (version counter) or by eviction.
struct CompanionEntry {
  c10::weak_intrusive_ptr<c10::StorageImpl> storage;
  const void *ptr;
  uint32_t version;
  std::vector<int64_t> sizes;
  torch::Tensor companion;
};
std::list<CompanionEntry> &companion_cache() {  // never destroyed, like the plan cache
  static auto *cache = new std::list<CompanionEntry>();
  return *cache;
}
#define g_companions companion_cache()
std::mutex g_companion_mu;
constexpr size_t kMaxCompanions = 8;
bool g_use_companions = true;

const void *find_companion(const torch::Tensor &t) {
  if (!g_use_companions) return nullptr;
  std::lock_guard<std::mutex> lock(g_companion_mu);
  for (auto it = g_companions.begin(); it != g_companions.end();) {
    if (it->storage.expired()) {
      it = g_companions.erase(it);
      continue;
    }
    if (it->ptr == t.data_ptr() && it->version == version_of(t) && it->sizes == t.sizes().vec() &&
        it->storage.lock().get() == t.storage().unsafeGetStorageImpl())
      return it->companion.data_ptr();
    ++it;
  }
  return nullptr;
}

// Fresh companion buffer for a (B, C, H, W) activation: only the zero pixel behind every image (and, if the channel
// count is padded, the padding) has to be cleared; the kernel writes the rest.
torch::Tensor new_companion(const torch::Tensor &like, int64_t B, int64_t C, int64_t H, int64_t W) {
  const size_t bytes = sph_conv_companion_bytes(B, C, H, W);
  TORCH_CHECK(bytes > 0, "activation too large for a channels-last companion");
  const int64_t cp = sph_conv_companion_channels(C);
  if (cp != C) return torch::zeros({(int64_t)bytes}, like.options().dtype(torch::kUInt8));
  torch::Tensor c = torch::empty({(int64_t)bytes}, like.options().dtype(torch::kUInt8));
  const size_t px = (size_t)cp * 2, img = (size_t)(H * W + 1) * px;
  TORCH_CHECK(cudaMemset2DAsync((char *)c.data_ptr() + (size_t)(H * W) * px, img, 0, px, (size_t)B,
                                at::cuda::getCurrentCUDAStream().stream()) == cudaSuccess,
              "clearing the companion's zero pixels failed");
  return c;
}

void register_companion(const torch::Tensor &t, torch::Tensor companion) {
  std::lock_guard<std::mutex> lock(g_companion_mu);
  g_companions.push_front(CompanionEntry{c10::weak_intrusive_ptr<c10::StorageImpl>(t.storage().getWeakStorageImpl()), t.data_ptr(),
                                         version_of(t), t.sizes().vec(), std::move(companion)});
  while (g_companions.size() > kMaxCompanions) g_companions.pop_back();
}

void clear_companions() {
  std::lock_guard<std::mutex> lock(g_companion_mu);
  g_companions.clear();
}

torch::Tensor workspace(size_t bytes, const torch::Tensor &like) {
  return torch::empty({(int64_t)(bytes ? bytes : 1)}, like.options().dtype(torch::kUInt8));
}

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// ---- resample (include/layers/resample_layer.h:40-82, weighted_resample_layer.h:49-105) ----
torch::Tensor resample_from_map_impl(torch::Tensor x, torch::Tensor map, const torch::Tensor *iw, InterpolationType it) {
  TORCH_CHECK(x.dim() == 4, "input must have 4 dimensions");
  check(x, "input", x);
  check_float(map, "sample_map", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw, false, 1);
  c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor y = torch::empty({x.size(0), x.size(1), m.H, m.W}, x.options());
  ok(sph_resample_from_map(x.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr, y.data_ptr(), x.size(0), x.size(1),
                           x.size(2), x.size(3), m.H, m.W, m.P, dtype_of(x), (int)it, stream()),
     "sph_resample_from_map");
  return y;
}

torch::Tensor resample_to_map_impl(torch::Tensor x, torch::Tensor map, const torch::Tensor *iw, int64_t oh, int64_t ow,
                                   InterpolationType it) {
  TORCH_CHECK(x.dim() == 4, "input must have 4 dimensions");
  check(x, "input", x);
  check_float(map, "sample_map", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw, false, 1);
  TORCH_CHECK(x.size(2) == m.H && x.size(3) == m.W, "input spatial size must match the sample map");
  TORCH_CHECK(oh > 0 && ow > 0, "output size must be positive");
  c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor plan = get_plan(map, iw, m.H * m.W, 1, m.P, (int)it, oh, ow);
  torch::Tensor out = torch::empty({x.size(0), x.size(1), oh, ow}, x.options());
  ok(sph_resample_to_map(x.data_ptr(), plan.data_ptr(), out.data_ptr(), x.size(0), x.size(1), m.H, m.W, oh, ow, dtype_of(x),
                         stream()),
     "sph_resample_to_map");
  return out;
}

torch::Tensor resample_to_map(torch::Tensor x, torch::Tensor map, int64_t oh, int64_t ow, InterpolationType it) {
  return resample_to_map_impl(x, map, nullptr, oh, ow, it);
}
torch::Tensor resample_from_map(torch::Tensor x, torch::Tensor map, InterpolationType it) {
  return resample_from_map_impl(x, map, nullptr, it);
}
torch::Tensor weighted_resample_to_map(torch::Tensor x, torch::Tensor map, torch::Tensor iw, int64_t oh, int64_t ow,
                                       InterpolationType it) {
  return resample_to_map_impl(x, map, &iw, oh, ow, it);
}
torch::Tensor weighted_resample_from_map(torch::Tensor x, torch::Tensor map, torch::Tensor iw, InterpolationType it) {
  return resample_from_map_impl(x, map, &iw, it);
}

// scatter(x) / (scatter(1) + 1e-12) in one pass (the normalisation of layers/functional/sphere_ops.py:74-80)
torch::Tensor resample_to_map_normalized(torch::Tensor x, torch::Tensor map, c10::optional<torch::Tensor> iw, int64_t oh,
                                         int64_t ow, InterpolationType it) {
  TORCH_CHECK(x.dim() == 4, "input must have 4 dimensions");
  check(x, "input", x);
  check_float(map, "sample_map", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw ? &*iw : nullptr, false, 1);
  TORCH_CHECK(x.size(2) == m.H && x.size(3) == m.W, "input spatial size must match the sample map");
  TORCH_CHECK(oh > 0 && ow > 0, "output size must be positive");
  c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor plan = get_plan(map, iw ? &*iw : nullptr, m.H * m.W, 1, m.P, (int)it, oh, ow);
  torch::Tensor out = torch::empty({x.size(0), x.size(1), oh, ow}, x.options());
  ok(sph_resample_to_map_normalized(x.data_ptr(), plan.data_ptr(), out.data_ptr(), x.size(0), x.size(1), m.H, m.W, oh, ow,
                                    dtype_of(x), stream()),
     "sph_resample_to_map_normalized");
  return out;
}

// ---- UV-map resampling (include/layers/uv_resample_layer.h:48-100) ----------
void check_uv(const torch::Tensor &quad, const torch::Tensor &uv, const torch::Tensor &like) {
  check(quad, "quad_idx", like);
  check_float(uv, "tex_uv", like);
  TORCH_CHECK(quad.scalar_type() == torch::kLong && quad.dim() == 2, "quad_idx must be an int64 (H, W) tensor");
  TORCH_CHECK(uv.dim() == 3 && uv.size(0) == quad.size(0) && uv.size(1) == quad.size(1) && uv.size(2) == 2,
              "tex_uv must be (H, W, 2) like quad_idx");
}

torch::Tensor resample_from_uv_maps(torch::Tensor tex, torch::Tensor quad, torch::Tensor uv, InterpolationType it) {
  TORCH_CHECK(tex.dim() == 5, "input must be (B, C, textures, TH, TW)");
  check(tex, "input", tex);
  check_uv(quad, uv, tex);
  c10::cuda::CUDAGuard guard(tex.device());
  torch::Tensor out = torch::empty({tex.size(0), tex.size(1), quad.size(0), quad.size(1)}, tex.options());
  ok(sph_resample_from_uv_maps(tex.data_ptr(), quad.data_ptr<int64_t>(), uv.data_ptr(), out.data_ptr(), tex.size(0), tex.size(1),
                               tex.size(2), tex.size(3), tex.size(4), quad.size(0), quad.size(1), dtype_of(tex), (int)it,
                               stream()),
     "sph_resample_from_uv_maps");
  return out;
}

torch::Tensor resample_to_uv_maps(torch::Tensor x, torch::Tensor quad, torch::Tensor uv, int64_t nt, int64_t th, int64_t tw,
                                  InterpolationType it) {
  TORCH_CHECK(x.dim() == 4, "input must have 4 dimensions");
  x = x.contiguous();
  check(x, "input", x);
  check_uv(quad, uv, x);
  TORCH_CHECK(x.size(2) == quad.size(0) && x.size(3) == quad.size(1), "input spatial size must match quad_idx");
  TORCH_CHECK(nt > 0 && th > 0 && tw > 0, "texture sizes must be positive");
  c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor plan = get_plan(uv, &quad, quad.size(0) * quad.size(1), 1, 0, (int)it, nt * th, tw, nt);
  torch::Tensor out = torch::empty({x.size(0), x.size(1), nt, th, tw}, x.options());
  ok(sph_resample_to_map(x.data_ptr(), plan.data_ptr(), out.data_ptr(), x.size(0), x.size(1), x.size(2), x.size(3), nt * th, tw,
                         dtype_of(x), stream()),
     "sph_resample_to_map (uv)");
  return out;
}

// ---- voting resample (include/layers/voting_resample_layer.h:32-58) ---------
torch::Tensor voting_resample_to_map(torch::Tensor x, torch::Tensor map, int64_t oh, int64_t ow, int64_t num_candidates) {
  TORCH_CHECK(x.dim() == 4 && x.scalar_type() == torch::kLong, "input must be an int64 (B, C, H, W) tensor");
  TORCH_CHECK(map.dim() == 3 && map.size(2) == 2 && map.scalar_type() == torch::kLong, "sample_map must be an int64 (H, W, 2) tensor");
  check(x, "input", x);
  check(map, "sample_map", x);
  TORCH_CHECK(x.size(2) == map.size(0) && x.size(3) == map.size(1), "input spatial size must match the sample map");
  TORCH_CHECK(oh > 0 && ow > 0 && num_candidates > 0, "output size and number of candidates must be positive");
  c10::cuda::CUDAGuard guard(x.device());
  // integer coordinates are exact in float64; the nearest-neighbour plan then inverts the map
  torch::Tensor mapf = map.to(torch::kDouble);
  const int64_t n_src = map.size(0) * map.size(1);
  const size_t bytes = sph_plan_bytes(n_src, 1, 0, SPH_NEAREST, oh, ow, SPH_F64);
  TORCH_CHECK(bytes > 0, "sample map too large for a scatter plan");
  torch::Tensor plan = torch::empty({(int64_t)bytes}, x.options().dtype(torch::kUInt8));
  ok(sph_plan_build(mapf.data_ptr(), nullptr, n_src, 1, 0, SPH_NEAREST, oh, ow, SPH_F64, plan.data_ptr(), bytes, stream()),
     "sph_plan_build");
  torch::Tensor out = torch::empty({x.size(0), x.size(1), oh, ow}, x.options());
  ok(sph_voting_resample_to_map(x.data_ptr<int64_t>(), plan.data_ptr(), SPH_F64, out.data_ptr<int64_t>(), x.size(0), x.size(1),
                                x.size(2), x.size(3), oh, ow, num_candidates, stream()),
     "sph_voting_resample_to_map");
  return out;
}

// ---- equirectangular kernel maps built on the device (layers/util/mapping_functions.py:44-163) ----
torch::Tensor build_kernel_map(int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t stride, int64_t dilation,
                               const std::string &kind, torch::Tensor like) {
  TORCH_CHECK(like.is_cuda(), "`like` must be a CUDA tensor (it gives the device and dtype of the map)");
  const int k = kind == "grid" ? SPH_MAP_GRID : kind == "inverse_gnomonic" ? SPH_MAP_INVERSE_GNOMONIC
              : kind == "inverse_equirectangular" ? SPH_MAP_INVERSE_EQUIRECT : -1;
  TORCH_CHECK(k >= 0, "kind must be 'grid', 'inverse_gnomonic' or 'inverse_equirectangular', got ", kind);
  TORCH_CHECK(H > 0 && W > 0 && kh > 0 && kw > 0 && stride > 0 && dilation > 0, "sizes must be positive");
  c10::cuda::CUDAGuard guard(like.device());
  torch::Tensor map = torch::empty({(H + stride - 1) / stride, (W + stride - 1) / stride, kh * kw, 2}, like.options());
  ok(sph_build_kernel_map(map.data_ptr(), H, W, kh, kw, stride, dilation, k, dtype_of(like), stream()), "sph_build_kernel_map");
  return map;
}

// ---- standard convolution (include/layers/convolution_layer.h:52-131, transposed_convolution_layer.h) ----
// Not part of the mapped-operator path: the reference's own im2col + GEMM convolution computes what ATen's
// convolution computes, so these delegate to ATen (cuDNN) with the reference's argument order.
torch::Tensor conv_forward(torch::Tensor x, torch::Tensor w, torch::Tensor b, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                           int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
  TORCH_CHECK(w.dim() == 4 && w.size(2) == kh && w.size(3) == kw, "weight must be (Cout, Cin, kernel_h, kernel_w)");
  return at::conv2d(x, w, b, {sh, sw}, {ph, pw}, {dh, dw}, 1);
}
std::vector<torch::Tensor> conv_backward(torch::Tensor go, torch::Tensor x, torch::Tensor w, torch::Tensor b, int64_t kh,
                                         int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
  auto r = at::convolution_backward(go.contiguous(), x, w, c10::nullopt, {sh, sw}, {ph, pw}, {dh, dw}, false, {0, 0}, 1,
                                    {true, true, false});
  return {std::get<0>(r), std::get<1>(r), go.sum({0, 2, 3})};
}
torch::Tensor transposed_conv_forward(torch::Tensor x, torch::Tensor w, torch::Tensor b, int64_t kh, int64_t kw, int64_t sh,
                                      int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
  TORCH_CHECK(w.dim() == 4 && w.size(2) == kh && w.size(3) == kw, "weight must be (Cin, Cout, kernel_h, kernel_w)");
  return at::conv_transpose2d(x, w, b, {sh, sw}, {ph, pw}, {0, 0}, 1, {dh, dw});
}
std::vector<torch::Tensor> transposed_conv_backward(torch::Tensor go, torch::Tensor x, torch::Tensor w, torch::Tensor b,
                                                    int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                                                    int64_t dh, int64_t dw) {
  auto r = at::convolution_backward(go.contiguous(), x, w, c10::nullopt, {sh, sw}, {ph, pw}, {dh, dw}, true, {0, 0}, 1,
                                    {true, true, false});
  return {std::get<0>(r), std::get<1>(r), go.sum({0, 2, 3})};
}

// ---- max pooling (include/layers/mapped_max_pooling_layer.h:42-97) ---------
std::vector<torch::Tensor> max_pool_impl(torch::Tensor x, torch::Tensor map, const torch::Tensor *iw, int64_t K,
                                         InterpolationType it) {
  TORCH_CHECK(x.dim() == 4, "input must have 4 dimensions");
  check(x, "input", x);
  check_float(map, "sample_map", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw, true, K);
  c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor out = torch::empty({x.size(0), x.size(1), m.H, m.W}, x.options());
  torch::Tensor idx = torch::empty({x.size(0), x.size(1), m.H, m.W}, x.options().dtype(torch::kLong));
  ok(sph_mapped_max_pool(x.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr, out.data_ptr(),
                         idx.data_ptr<int64_t>(), x.size(0), x.size(1), x.size(2), x.size(3), m.H, m.W, m.K, m.P,
                         dtype_of(x), (int)it, stream()),
     "sph_mapped_max_pool");
  return {out, idx};
}

torch::Tensor max_unpool_impl(torch::Tensor g, torch::Tensor idx, torch::Tensor map, const torch::Tensor *iw, int64_t ih,
                              int64_t iwidth, int64_t K, InterpolationType it) {
  TORCH_CHECK(g.dim() == 4, "grad_output must have 4 dimensions");
  g = g.contiguous();
  check(g, "grad_output", g);
  check(idx, "idx_mask", g);
  TORCH_CHECK(idx.scalar_type() == torch::kLong && idx.sizes() == g.sizes(), "idx_mask must be int64 with grad_output's shape");
  check_float(map, "sample_map", g);
  if (iw) check_float(*iw, "interp_weights", g);
  const MapInfo m = map_info(map, iw, true, K);
  TORCH_CHECK(g.size(2) == m.H && g.size(3) == m.W, "grad_output spatial size must match the sample map");
  TORCH_CHECK(ih > 0 && iwidth > 0, "input size must be positive");
  c10::cuda::CUDAGuard guard(g.device());
  torch::Tensor gin = torch::empty({g.size(0), g.size(1), ih, iwidth}, g.options());
  if (g_deterministic_unpool) {
    // plan over the flattened map slots: every input pixel sums the winners that touch it in a fixed order
    torch::Tensor plan = get_plan(map, iw, m.H * m.W * m.K, 1, m.P, (int)it, ih, iwidth);
    ok(sph_mapped_max_unpool_planned(g.data_ptr(), idx.data_ptr<int64_t>(), plan.data_ptr(), gin.data_ptr(), g.size(0),
                                     g.size(1), ih, iwidth, m.H, m.W, m.K, m.P, dtype_of(g), stream()),
       "sph_mapped_max_unpool_planned");
    return gin;
  }
  ok(sph_mapped_max_unpool(g.data_ptr(), idx.data_ptr<int64_t>(), map.data_ptr(), iw ? iw->data_ptr() : nullptr,
                           gin.data_ptr(), g.size(0), g.size(1), ih, iwidth, m.H, m.W, m.K, m.P, dtype_of(g), (int)it,
                           stream()),
     "sph_mapped_max_unpool");
  return gin;
}

// ---- average pooling (include/layers/mapped_avg_pooling_layer.h:40-86, weighted twin) ----
torch::Tensor avg_pool_impl(torch::Tensor x, torch::Tensor map, const torch::Tensor *iw, int64_t K, InterpolationType it) {
  TORCH_CHECK(x.dim() == 4, "input must have 4 dimensions");
  check(x, "input", x);
  check_float(map, "sample_map", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw, true, K);
  c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor out = torch::empty({x.size(0), x.size(1), m.H, m.W}, x.options());
  ok(sph_mapped_avg_pool(x.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr, out.data_ptr(), x.size(0), x.size(1),
                         x.size(2), x.size(3), m.H, m.W, m.K, m.P, dtype_of(x), (int)it, stream()),
     "sph_mapped_avg_pool");
  return out;
}

torch::Tensor avg_unpool_impl(torch::Tensor g, torch::Tensor map, const torch::Tensor *iw, int64_t ih, int64_t iwidth, int64_t K,
                              InterpolationType it) {
  TORCH_CHECK(g.dim() == 4, "grad_output must have 4 dimensions");
  g = g.contiguous();
  check(g, "grad_output", g);
  check_float(map, "sample_map", g);
  if (iw) check_float(*iw, "interp_weights", g);
  const MapInfo m = map_info(map, iw, true, K);
  TORCH_CHECK(g.size(2) == m.H && g.size(3) == m.W, "grad_output spatial size must match the sample map");
  TORCH_CHECK(ih > 0 && iwidth > 0, "input size must be positive");
  c10::cuda::CUDAGuard guard(g.device());
  torch::Tensor plan = get_plan(map, iw, m.H * m.W * m.K, 1, m.P, (int)it, ih, iwidth);
  torch::Tensor gin = torch::empty({g.size(0), g.size(1), ih, iwidth}, g.options());
  ok(sph_mapped_avg_unpool(g.data_ptr(), plan.data_ptr(), gin.data_ptr(), g.size(0), g.size(1), ih, iwidth, m.H, m.W, m.K,
                           dtype_of(g), stream()),
     "sph_mapped_avg_unpool");
  return gin;
}

torch::Tensor mapped_avg_pool(torch::Tensor x, torch::Tensor map, int64_t K, InterpolationType it) {
  return avg_pool_impl(x, map, nullptr, K, it);
}
torch::Tensor mapped_avg_unpool(torch::Tensor g, torch::Tensor map, int64_t ih, int64_t iw, int64_t K, InterpolationType it) {
  return avg_unpool_impl(g, map, nullptr, ih, iw, K, it);
}
torch::Tensor weighted_mapped_avg_pool(torch::Tensor x, torch::Tensor map, torch::Tensor w, int64_t K, InterpolationType it) {
  return avg_pool_impl(x, map, &w, K, it);
}
torch::Tensor weighted_mapped_avg_unpool(torch::Tensor g, torch::Tensor map, torch::Tensor w, int64_t ih, int64_t iw, int64_t K,
                                         InterpolationType it) {
  return avg_unpool_impl(g, map, &w, ih, iw, K, it);
}

std::vector<torch::Tensor> mapped_max_pool(torch::Tensor x, torch::Tensor map, int64_t K, InterpolationType it) {
  return max_pool_impl(x, map, nullptr, K, it);
}
torch::Tensor mapped_max_unpool(torch::Tensor g, torch::Tensor idx, torch::Tensor map, int64_t ih, int64_t iw, int64_t K,
                                InterpolationType it) {
  return max_unpool_impl(g, idx, map, nullptr, ih, iw, K, it);
}
std::vector<torch::Tensor> weighted_mapped_max_pool(torch::Tensor x, torch::Tensor map, torch::Tensor w, int64_t K,
                                                    InterpolationType it) {
  return max_pool_impl(x, map, &w, K, it);
}
torch::Tensor weighted_mapped_max_unpool(torch::Tensor g, torch::Tensor idx, torch::Tensor map, torch::Tensor w, int64_t ih,
                                         int64_t iw, int64_t K, InterpolationType it) {
  return max_unpool_impl(g, idx, map, &w, ih, iw, K, it);
}

// ---- mapped convolution (include/layers/mapped_convolution_layer.h:62-134) --
struct ConvArgs {
  int64_t B, Cin, Cout, IH, IW, OH, OW, K, P;
  int dtype, interp, prec;
};

// relu: the fused variant (sph_mapped_conv_relu_*, an extension without a reference counterpart); shapes the
// library does not fuse fall back to the plain operator plus a separate activation.
torch::Tensor conv_forward_impl(torch::Tensor x, torch::Tensor map, const torch::Tensor *iw, torch::Tensor weight,
                                torch::Tensor bias, int64_t K, InterpolationType it, bool relu = false) {
  TORCH_CHECK(x.dim() == 4 && weight.dim() == 3 && bias.dim() == 1, "input (B,C,H,W), weight (Cout,Cin,K), bias (Cout)");
  check(x, "input", x);
  check_float(map, "sample_map", x);
  check_float(weight, "weight", x);
  check_float(bias, "bias", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw, true, K);
  TORCH_CHECK(weight.size(1) == x.size(1) && weight.size(2) == K && bias.size(0) == weight.size(0),
              "weight / bias shapes do not match the input");
  c10::cuda::CUDAGuard guard(x.device());
  const ConvArgs a{x.size(0), x.size(1), weight.size(0), x.size(2), x.size(3), m.H, m.W, K, m.P, dtype_of(x), (int)it,
                   dtype_of(x) == SPH_F32 ? precision() : SPH_PRECISION_EXACT};
  torch::Tensor out = torch::empty({a.B, a.Cout, a.OH, a.OW}, x.options());
  const size_t wb = sph_conv_workspace_bytes(SPH_CONV_FORWARD, a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype,
                                             a.interp, a.prec);
  torch::Tensor ws = workspace(wb, x);
  if (a.prec == SPH_PRECISION_BF16 && g_use_companions) {
    // channels-last companions: gather from the input's copy if a previous layer left one; with the fused ReLU also
    // write the copy of the output for the next layer
    const void *x_cl = find_companion(x);
    if (x_cl == nullptr && a.Cin * a.K > 63 && x.numel() > 0) {
      // no previous layer left a copy of this input (the reference's own composition: convolution, then a separate
      // activation): convert it once here, for this call and for the weight gradient in backward
      torch::Tensor cl = torch::empty({(int64_t)sph_conv_companion_bytes(a.B, a.Cin, a.IH, a.IW)}, x.options().dtype(torch::kUInt8));
      ok(sph_conv_companion_fill(x.data_ptr(), cl.data_ptr(), a.B, a.Cin, a.IH, a.IW, stream()), "sph_conv_companion_fill");
      register_companion(x, cl);
      x_cl = cl.data_ptr();
    }
    torch::Tensor out_cl;
    if (relu && a.Cout % 8 == 0) out_cl = new_companion(x, a.B, a.Cout, a.OH, a.OW);
    if (x_cl != nullptr || out_cl.defined()) {
      int rc = sph_mapped_conv_forward_cl(x.data_ptr(), x_cl, map.data_ptr(), iw ? iw->data_ptr() : nullptr, weight.data_ptr(),
                                          bias.data_ptr(), out.data_ptr(), out_cl.defined() ? out_cl.data_ptr() : nullptr, a.B,
                                          a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype, a.interp, a.prec, relu ? 1 : 0,
                                          ws.data_ptr(), wb, stream());
      if (rc == SPH_ERR_UNSUPPORTED && out_cl.defined()) {   // this shape cannot write the copy (or cannot fuse): without it
        out_cl = torch::Tensor();
        rc = x_cl == nullptr ? SPH_ERR_UNSUPPORTED
                             : sph_mapped_conv_forward_cl(x.data_ptr(), x_cl, map.data_ptr(), iw ? iw->data_ptr() : nullptr,
                                                          weight.data_ptr(), bias.data_ptr(), out.data_ptr(), nullptr, a.B, a.Cin,
                                                          a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype, a.interp, a.prec,
                                                          relu ? 1 : 0, ws.data_ptr(), wb, stream());
      }
      if (rc != SPH_ERR_UNSUPPORTED) {
        ok(rc, "sph_mapped_conv_forward_cl");
        if (out_cl.defined()) register_companion(out, out_cl);
        maybe_check_device("mapped convolution");
        return out;
      }
    }
  }
  if (relu) {
    const int rc = sph_mapped_conv_relu_forward(x.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr, weight.data_ptr(),
                                                bias.data_ptr(), out.data_ptr(), a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K,
                                                a.P, a.dtype, a.interp, a.prec, ws.data_ptr(), wb, stream());
    if (rc != SPH_ERR_UNSUPPORTED) {
      ok(rc, "sph_mapped_conv_relu_forward");
      maybe_check_device("mapped convolution");
      return out;
    }
  }
  ok(sph_mapped_conv_forward(x.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr, weight.data_ptr(), bias.data_ptr(),
                             out.data_ptr(), a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype, a.interp, a.prec,
                             ws.data_ptr(), wb, stream()),
     "sph_mapped_conv_forward");
  if (relu) out.clamp_min_(0);
  maybe_check_device("mapped convolution");
  return out;
}

std::vector<torch::Tensor> conv_backward_impl(torch::Tensor go, torch::Tensor map, const torch::Tensor *iw, torch::Tensor x,
                                              torch::Tensor weight, torch::Tensor bias, int64_t K, InterpolationType it,
                                              const torch::Tensor *act_out = nullptr) {
  TORCH_CHECK(x.dim() == 4 && go.dim() == 4 && weight.dim() == 3, "input/grad_output (B,C,H,W), weight (Cout,Cin,K)");
  go = go.contiguous();  // the reference never checks grad_output; make it dense here
  check(x, "input", x);
  check_float(go, "grad_output", x);
  check_float(map, "sample_map", x);
  check_float(weight, "weight", x);
  check_float(bias, "bias", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw, true, K);
  TORCH_CHECK(weight.size(1) == x.size(1) && weight.size(2) == K, "weight shape does not match the input");
  TORCH_CHECK(go.size(0) == x.size(0) && go.size(1) == weight.size(0) && go.size(2) == m.H && go.size(3) == m.W,
              "grad_output shape does not match the sample map / weight");
  c10::cuda::CUDAGuard guard(x.device());
  const ConvArgs a{x.size(0), x.size(1), weight.size(0), x.size(2), x.size(3), m.H, m.W, K, m.P, dtype_of(x), (int)it,
                   dtype_of(x) == SPH_F32 ? precision() : SPH_PRECISION_EXACT};
  torch::Tensor gx = torch::empty_like(x), gw = torch::empty_like(weight), gb = torch::empty({a.Cout}, x.options());
  torch::Tensor plan = get_plan(map, iw, a.OH * a.OW, a.K, a.P, a.interp, a.IH, a.IW);
  if (act_out)
    TORCH_CHECK(act_out->is_contiguous() && act_out->sizes() == go.sizes() && act_out->dtype() == go.dtype() &&
                    act_out->device() == go.device(),
                "activation output must be a contiguous tensor like grad_output");
  if (a.prec == SPH_PRECISION_BF16) {
    // all three gradients in one call: grad_output is converted (and masked) once for both of its consumers, and the
    // input's channels-last copy is used if a previous layer left one
    const size_t wbc = sph_conv_workspace_bytes(SPH_CONV_BACKWARD, a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype,
                                                a.interp, a.prec);
    if (wbc > 0) {
      torch::Tensor wsc = workspace(wbc, x);
      const int rc = sph_mapped_conv_backward_cl(go.data_ptr(), act_out ? act_out->data_ptr() : nullptr, x.data_ptr(),
                                                 find_companion(x), plan.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr,
                                                 weight.data_ptr(), gx.data_ptr(), gw.data_ptr(), gb.data_ptr(), a.B, a.Cin, a.Cout,
                                                 a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype, a.interp, a.prec, wsc.data_ptr(), wbc,
                                                 stream());
      if (rc != SPH_ERR_UNSUPPORTED) {
        ok(rc, "sph_mapped_conv_backward_cl");
        maybe_check_device("mapped convolution");
        return {gx, gw, gb};
      }
    }
  }
  size_t wb = sph_conv_workspace_bytes(SPH_CONV_BACKWARD_INPUT, a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P,
                                       a.dtype, a.interp, a.prec);
  torch::Tensor ws = workspace(wb, x);
  size_t wb2 = sph_conv_workspace_bytes(SPH_CONV_BACKWARD_WEIGHT, a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype,
                                        a.interp, a.prec);
  torch::Tensor ws2 = workspace(wb2, x);
  if (act_out) {  // gradient of the fused ReLU: the kernels read grad_output * (act_out > 0)
    const int rc = sph_mapped_conv_relu_backward_input(go.data_ptr(), act_out->data_ptr(), plan.data_ptr(), weight.data_ptr(),
                                                       gx.data_ptr(), a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.dtype,
                                                       a.prec, ws.data_ptr(), wb, stream());
    // The two fused operators are eligible independently (the weight-gradient kernel's tap table is smaller than the
    // gather-GEMM's), so each one that declines falls back on its own to a masked copy and the plain operator.
    bool have_gx = false;
    if (rc != SPH_ERR_UNSUPPORTED) {
      ok(rc, "sph_mapped_conv_relu_backward_input");
      have_gx = true;
      const int rc2 = sph_mapped_conv_relu_backward_weight(go.data_ptr(), act_out->data_ptr(), x.data_ptr(), map.data_ptr(),
                                                           iw ? iw->data_ptr() : nullptr, gw.data_ptr(), gb.data_ptr(), a.B,
                                                           a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype, a.interp,
                                                           a.prec, ws2.data_ptr(), wb2, stream());
      if (rc2 != SPH_ERR_UNSUPPORTED) {
        ok(rc2, "sph_mapped_conv_relu_backward_weight");
        maybe_check_device("mapped convolution");
        return {gx, gw, gb};
      }
    }
    go = at::threshold_backward(go, *act_out, 0);
    if (have_gx) {
      ok(sph_mapped_conv_backward_weight(go.data_ptr(), x.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr,
                                         gw.data_ptr(), gb.data_ptr(), a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P,
                                         a.dtype, a.interp, a.prec, ws2.data_ptr(), wb2, stream()),
         "sph_mapped_conv_backward_weight");
      maybe_check_device("mapped convolution");
      return {gx, gw, gb};
    }
  }
  ok(sph_mapped_conv_backward_input(go.data_ptr(), plan.data_ptr(), weight.data_ptr(), gx.data_ptr(), a.B, a.Cin, a.Cout,
                                    a.IH, a.IW, a.OH, a.OW, a.K, a.dtype, a.prec, ws.data_ptr(), wb, stream()),
     "sph_mapped_conv_backward_input");
  wb = wb2;
  ok(sph_mapped_conv_backward_weight(go.data_ptr(), x.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr,
                                     gw.data_ptr(), gb.data_ptr(), a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P,
                                     a.dtype, a.interp, a.prec, ws2.data_ptr(), wb, stream()),
     "sph_mapped_conv_backward_weight");
  maybe_check_device("mapped convolution");
  return {gx, gw, gb};
}

torch::Tensor mapped_conv_forward(torch::Tensor x, torch::Tensor map, torch::Tensor w, torch::Tensor b, int64_t K,
                                  InterpolationType it) {
  return conv_forward_impl(x, map, nullptr, w, b, K, it);
}
std::vector<torch::Tensor> mapped_conv_backward(torch::Tensor go, torch::Tensor map, torch::Tensor x, torch::Tensor w,
                                                torch::Tensor b, int64_t K, InterpolationType it) {
  return conv_backward_impl(go, map, nullptr, x, w, b, K, it);
}
// fused ReLU variants (extension; interp_weights optional)
torch::Tensor mapped_conv_relu_forward(torch::Tensor x, torch::Tensor map, c10::optional<torch::Tensor> iw, torch::Tensor w,
                                       torch::Tensor b, int64_t K, InterpolationType it) {
  return conv_forward_impl(x, map, iw ? &*iw : nullptr, w, b, K, it, true);
}
std::vector<torch::Tensor> mapped_conv_relu_backward(torch::Tensor go, torch::Tensor act_out, torch::Tensor map,
                                                     c10::optional<torch::Tensor> iw, torch::Tensor x, torch::Tensor w,
                                                     torch::Tensor b, int64_t K, InterpolationType it) {
  return conv_backward_impl(go, map, iw ? &*iw : nullptr, x, w, b, K, it, &act_out);
}
torch::Tensor weighted_mapped_conv_forward(torch::Tensor x, torch::Tensor map, torch::Tensor iw, torch::Tensor w,
                                           torch::Tensor b, int64_t K, InterpolationType it) {
  return conv_forward_impl(x, map, &iw, w, b, K, it);
}
std::vector<torch::Tensor> weighted_mapped_conv_backward(torch::Tensor go, torch::Tensor map, torch::Tensor iw,
                                                         torch::Tensor x, torch::Tensor w, torch::Tensor b, int64_t K,
                                                         InterpolationType it) {
  return conv_backward_impl(go, map, &iw, x, w, b, K, it);
}

// ---- transposed (include/layers/mapped_transposed_convolution_layer.h:62-149) --
torch::Tensor tconv_forward_impl(torch::Tensor x, torch::Tensor map, const torch::Tensor *iw, torch::Tensor weight,
                                 torch::Tensor bias, int64_t oh, int64_t ow, int64_t K, InterpolationType it) {
  TORCH_CHECK(x.dim() == 4 && weight.dim() == 3 && bias.dim() == 1, "input (B,C,H,W), weight (Cin,Cout,K), bias (Cout)");
  check(x, "input", x);
  check_float(map, "sample_map", x);
  check_float(weight, "weight", x);
  check_float(bias, "bias", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw, true, K);
  TORCH_CHECK(x.size(2) == m.H && x.size(3) == m.W, "input spatial size must match the sample map");
  TORCH_CHECK(weight.size(0) == x.size(1) && weight.size(2) == K && bias.size(0) == weight.size(1),
              "weight / bias shapes do not match the input");
  TORCH_CHECK(oh > 0 && ow > 0, "output size must be positive");
  c10::cuda::CUDAGuard guard(x.device());
  const ConvArgs a{x.size(0), x.size(1), weight.size(1), x.size(2), x.size(3), oh, ow, K, m.P, dtype_of(x), (int)it,
                   dtype_of(x) == SPH_F32 ? precision() : SPH_PRECISION_EXACT};
  torch::Tensor plan = get_plan(map, iw, a.IH * a.IW, a.K, a.P, a.interp, a.OH, a.OW);
  torch::Tensor out = torch::empty({a.B, a.Cout, a.OH, a.OW}, x.options());
  const size_t wb = sph_conv_workspace_bytes(SPH_TCONV_FORWARD, a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype,
                                             a.interp, a.prec);
  torch::Tensor ws = workspace(wb, x);
  ok(sph_mapped_tconv_forward(x.data_ptr(), plan.data_ptr(), weight.data_ptr(), bias.data_ptr(), out.data_ptr(), a.B, a.Cin,
                              a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.dtype, a.prec, ws.data_ptr(), wb, stream()),
     "sph_mapped_tconv_forward");
  maybe_check_device("mapped convolution");
  return out;
}

std::vector<torch::Tensor> tconv_backward_impl(torch::Tensor go, torch::Tensor map, const torch::Tensor *iw, torch::Tensor x,
                                               torch::Tensor weight, torch::Tensor bias, int64_t K, InterpolationType it) {
  TORCH_CHECK(x.dim() == 4 && go.dim() == 4 && weight.dim() == 3, "input/grad_output (B,C,H,W), weight (Cin,Cout,K)");
  go = go.contiguous();
  check(x, "input", x);
  check_float(go, "grad_output", x);
  check_float(map, "sample_map", x);
  check_float(weight, "weight", x);
  check_float(bias, "bias", x);
  if (iw) check_float(*iw, "interp_weights", x);
  const MapInfo m = map_info(map, iw, true, K);
  TORCH_CHECK(x.size(2) == m.H && x.size(3) == m.W, "input spatial size must match the sample map");
  TORCH_CHECK(weight.size(0) == x.size(1) && weight.size(2) == K, "weight shape does not match the input");
  TORCH_CHECK(go.size(0) == x.size(0) && go.size(1) == weight.size(1), "grad_output shape does not match the weight");
  c10::cuda::CUDAGuard guard(x.device());
  const ConvArgs a{x.size(0), x.size(1), weight.size(1), x.size(2), x.size(3), go.size(2), go.size(3), K, m.P, dtype_of(x),
                   (int)it, dtype_of(x) == SPH_F32 ? precision() : SPH_PRECISION_EXACT};
  torch::Tensor gx = torch::empty_like(x), gw = torch::empty_like(weight), gb = torch::empty({a.Cout}, x.options());
  size_t wb = sph_conv_workspace_bytes(SPH_TCONV_BACKWARD_INPUT, a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P,
                                       a.dtype, a.interp, a.prec);
  torch::Tensor ws = workspace(wb, x);
  ok(sph_mapped_tconv_backward_input(go.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr, weight.data_ptr(),
                                     gx.data_ptr(), a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype, a.interp,
                                     a.prec, ws.data_ptr(), wb, stream()),
     "sph_mapped_tconv_backward_input");
  wb = sph_conv_workspace_bytes(SPH_TCONV_BACKWARD_WEIGHT, a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P, a.dtype,
                                a.interp, a.prec);
  torch::Tensor ws2 = workspace(wb, x);
  ok(sph_mapped_tconv_backward_weight(go.data_ptr(), x.data_ptr(), map.data_ptr(), iw ? iw->data_ptr() : nullptr,
                                      gw.data_ptr(), gb.data_ptr(), a.B, a.Cin, a.Cout, a.IH, a.IW, a.OH, a.OW, a.K, a.P,
                                      a.dtype, a.interp, a.prec, ws2.data_ptr(), wb, stream()),
     "sph_mapped_tconv_backward_weight");
  maybe_check_device("mapped convolution");
  return {gx, gw, gb};
}

torch::Tensor mapped_transposed_conv_forward(torch::Tensor x, torch::Tensor map, torch::Tensor w, torch::Tensor b, int64_t oh,
                                             int64_t ow, int64_t K, InterpolationType it) {
  return tconv_forward_impl(x, map, nullptr, w, b, oh, ow, K, it);
}
std::vector<torch::Tensor> mapped_transposed_conv_backward(torch::Tensor go, torch::Tensor map, torch::Tensor x,
                                                           torch::Tensor w, torch::Tensor b, int64_t K, InterpolationType it) {
  return tconv_backward_impl(go, map, nullptr, x, w, b, K, it);
}
torch::Tensor weighted_mapped_transposed_conv_forward(torch::Tensor x, torch::Tensor map, torch::Tensor iw, torch::Tensor w,
                                                      torch::Tensor b, int64_t oh, int64_t ow, int64_t K,
                                                      InterpolationType it) {
  return tconv_forward_impl(x, map, &iw, w, b, oh, ow, K, it);
}
std::vector<torch::Tensor> weighted_mapped_transposed_conv_backward(torch::Tensor go, torch::Tensor map, torch::Tensor iw,
                                                                    torch::Tensor x, torch::Tensor w, torch::Tensor b,
                                                                    int64_t K, InterpolationType it) {
  return tconv_backward_impl(go, map, &iw, x, w, b, K, it);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  // include/layers/enum_export.h:8-29
  py::enum_<InterpolationType>(m, "InterpolationType", py::arithmetic(), "How a fractional map coordinate is sampled")
      .value("NEAREST", InterpolationType::NEAREST)
      .value("BILINEAR", InterpolationType::BILINEAR)
      .value("BISPHERICAL", InterpolationType::BISPHERICAL);
  py::enum_<DistortionType>(m, "DistortionType", py::arithmetic(), "Lens distortion model")
      .value("SIMPLE_RADIAL", DistortionType::SIMPLE_RADIAL)
      .value("BROWN", DistortionType::BROWN)
      .value("FISHEYE", DistortionType::FISHEYE);

  m.def("resample_to_map", &resample_to_map);
  m.def("resample_from_map", &resample_from_map);
  m.def("weighted_resample_to_map", &weighted_resample_to_map);
  m.def("weighted_resample_from_map", &weighted_resample_from_map);
  m.def("mapped_max_pool", &mapped_max_pool);
  m.def("mapped_max_unpool", &mapped_max_unpool);
  m.def("weighted_mapped_max_pool", &weighted_mapped_max_pool);
  m.def("weighted_mapped_max_unpool", &weighted_mapped_max_unpool);
  m.def("mapped_avg_pool", &mapped_avg_pool);
  m.def("mapped_avg_unpool", &mapped_avg_unpool);
  m.def("weighted_mapped_avg_pool", &weighted_mapped_avg_pool);
  m.def("weighted_mapped_avg_unpool", &weighted_mapped_avg_unpool);
  m.def("resample_from_uv_maps", &resample_from_uv_maps);
  m.def("resample_to_uv_maps", &resample_to_uv_maps);
  m.def("voting_resample_to_map", &voting_resample_to_map);
  m.def("resample_to_map_normalized", &resample_to_map_normalized, py::arg("input"), py::arg("sample_map"),
        py::arg("interp_weights"), py::arg("output_height"), py::arg("output_width"), py::arg("interpolation"),
        "scatter(input) / (scatter(1) + 1e-12) through the sample map, in one pass");
  m.def("build_kernel_map", &build_kernel_map, py::arg("H"), py::arg("W"), py::arg("kernel_h"), py::arg("kernel_w"),
        py::arg("stride"), py::arg("dilation"), py::arg("kind"), py::arg("like"),
        "equirectangular kernel sample map (ceil(H/stride), ceil(W/stride), kh*kw, 2) built on the device");
  m.def("conv_forward", &conv_forward);
  m.def("conv_backward", &conv_backward);
  m.def("transposed_conv_forward", &transposed_conv_forward);
  m.def("transposed_conv_backward", &transposed_conv_backward);
  m.def("set_companions", [](bool on) { g_use_companions = on; if (!on) clear_companions(); },
        "true (default): with bf16 precision, layers with a fused activation leave a channels-last bf16 copy of their output "
        "for the next layer, which then skips its conversion pass; false: every call converts its own input");
  m.def("clear_companions", &clear_companions);
  m.def("set_deterministic_unpool", [](bool on) { g_deterministic_unpool = on; },
        "true (default): argmax backward sums through a scatter plan in a fixed order; false: float atomics as the reference");
  m.def("mapped_conv_forward", &mapped_conv_forward);
  m.def("mapped_conv_backward", &mapped_conv_backward);
  m.def("mapped_conv_relu_forward", &mapped_conv_relu_forward);
  m.def("mapped_conv_relu_backward", &mapped_conv_relu_backward);
  m.def("weighted_mapped_conv_forward", &weighted_mapped_conv_forward);
  m.def("weighted_mapped_conv_backward", &weighted_mapped_conv_backward);
  m.def("mapped_transposed_conv_forward", &mapped_transposed_conv_forward);
  m.def("mapped_transposed_conv_backward", &mapped_transposed_conv_backward);
  m.def("weighted_mapped_transposed_conv_forward", &weighted_mapped_transposed_conv_forward);
  m.def("weighted_mapped_transposed_conv_backward", &weighted_mapped_transposed_conv_backward);

  m.def("set_precision", &set_precision, "'fp32' (exact SIMT path) or 'bf16' (tcgen05 tensor cores) for float32 convolutions");
  m.def("get_precision", &get_precision);
  m.def("clear_plan_cache", &clear_plan_cache);
  m.def("plan_cache_size", &plan_cache_size);
  m.def("abi_version", []() { return sph_version(); });
  m.def(
      "device_status",
      [](bool reset) {
        int v = -1;
        ok(sph_device_status(&v, reset ? 1 : 0), "sph_device_status");
        return v;
      },
      py::arg("reset") = true,
      "1 if a bounded wait inside a tensor-core kernel gave up on the current device since the last reset (results of "
      "that launch are invalid), else 0; waits for the device's queued work");
}
