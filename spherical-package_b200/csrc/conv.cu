// C entry points of the mapped (transposed) convolution family: argument
// checks and dispatch to the exact SIMT kernels or the bf16 tensor-core path.
#include "common.cuh"
#include "conv_internal.h"

using namespace sph;

namespace {

struct Dims {
  int64_t B, Cin, Cout, IH, IW, OH, OW, K, P;
};

int check_dims(const Dims &d, int dtype, int interp, int precision) {
  if (d.B < 0 || d.Cin <= 0 || d.Cout <= 0 || d.IH <= 0 || d.IW <= 0 || d.OH <= 0 || d.OW <= 0 || d.K <= 0 || d.P < 0)
    return SPH_ERR_INVALID_ARGUMENT;
  if (interp < 0 || interp > 2) return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  if (precision != SPH_PRECISION_EXACT && precision != SPH_PRECISION_BF16) return SPH_ERR_INVALID_ARGUMENT;
  if (precision == SPH_PRECISION_BF16 && dtype != SPH_F32) return SPH_ERR_UNSUPPORTED;
  const int64_t lim = (int64_t)1 << 31, PP = d.P > 0 ? d.P : 1;
  if (d.IH * d.IW >= lim || d.OH * d.OW >= lim || d.B >= 65535) return SPH_ERR_TOO_LARGE;
  if (d.IH * d.IW * d.K * PP * 4 >= lim || d.OH * d.OW * d.K * PP * 4 >= lim) return SPH_ERR_TOO_LARGE;
  if (d.Cin * d.K >= lim || d.Cout * d.K >= lim || d.Cin * d.Cout * d.K >= lim) return SPH_ERR_TOO_LARGE;
  return SPH_OK;
}

}  // namespace

extern "C" const char *sph_status_string(int status) {
  switch (status) {
    case SPH_OK: return "ok";
    case SPH_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, negative size or unknown enum value)";
    case SPH_ERR_UNSUPPORTED: return "unsupported dtype / precision combination";
    case SPH_ERR_WORKSPACE_TOO_SMALL: return "workspace or plan buffer too small";
    case SPH_ERR_CUDA: return "CUDA runtime reported an error at launch";
    case SPH_ERR_TOO_LARGE: return "tensor too large for 32-bit plane indexing";
    case SPH_ERR_STATIC_SCRATCH_EXCEEDED: return "problem needs more scratch than the library's built-in static array holds";
    default: return "unknown status";
  }
}

extern "C" int sph_version(void) { return 100; }

namespace sph {
unsigned long long g_launch_count = 0;
}  // namespace sph
extern "C" unsigned long long sph_launch_count(void) { return __atomic_load_n(&sph::g_launch_count, __ATOMIC_RELAXED); }

namespace {
// Scratch of the kernels an operator falls back on when a thin layer's tensor-core form does not apply.
size_t base_workspace(int op, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                      int64_t P, int dtype, int interp, int precision) {
  const size_t ts = dtype == SPH_F64 ? 8 : 4;
  // thin contractions (few channels on the gathered / produced side) have their own kernels in both precisions
  switch (op) {
    case SPH_CONV_FORWARD: if (small_ok(Cin, K, Cout, ts)) return 0; break;
    case SPH_CONV_BACKWARD_INPUT: if (small_ok(Cin, K, Cout, ts)) return small_premul_workspace(B, Cin, K, OH * OW, ts); break;
    case SPH_CONV_BACKWARD_WEIGHT: if (small_ok(Cin, K, Cout, ts)) return small_dw_workspace(B, OH * OW, Cout, Cin, K, Cout, ts); break;
    case SPH_TCONV_FORWARD: if (small_ok(Cout, K, Cin, ts)) return small_premul_workspace(B, Cout, K, IH * IW, ts); break;
    case SPH_TCONV_BACKWARD_INPUT: if (small_ok(Cout, K, Cin, ts)) return 0; break;
    case SPH_TCONV_BACKWARD_WEIGHT: if (small_ok(Cout, K, Cin, ts)) return small_dw_workspace(B, IH * IW, Cin, Cout, K, Cout, ts); break;
    case SPH_CONV_BACKWARD: if (small_ok(Cin, K, Cout, ts)) return 0; break;  // thin layers: the separate entry points
    default: break;
  }
  if (op == SPH_CONV_BACKWARD)
    return precision == SPH_PRECISION_BF16 ? tc_conv_backward_workspace(B, Cin, Cout, IH, IW, OH, OW, K, P, interp) : 0;
  if (precision == SPH_PRECISION_BF16) return tc_workspace_bytes(op, B, Cin, Cout, IH, IW, OH, OW, K, P, interp);
  switch (op) {
    case SPH_CONV_FORWARD: return simt_gemm_workspace(Cout, Cin, K, ts);
    case SPH_CONV_BACKWARD_INPUT: return simt_adjoint_workspace(B, Cin, Cout, K, OH * OW, IH * IW, ts);
    case SPH_TCONV_FORWARD: return simt_adjoint_workspace(B, Cout, Cin, K, IH * IW, OH * OW, ts);
    case SPH_TCONV_BACKWARD_INPUT: return simt_gemm_workspace(Cin, Cout, K, ts);
    case SPH_CONV_BACKWARD_WEIGHT: return simt_dw_workspace(B, OH * OW, Cout, Cin, K, Cout, ts);
    case SPH_TCONV_BACKWARD_WEIGHT: return simt_dw_workspace(B, IH * IW, Cin, Cout, K, Cout, ts);
    default: return 0;
  }
}
}  // namespace

extern "C" size_t sph_conv_workspace_bytes(int op, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                                           int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                                           int precision) {
  const Dims d{B, Cin, Cout, IH, IW, OH, OW, K, P};
  if (check_dims(d, dtype, interp, precision) != SPH_OK) return 0;
  const size_t base = base_workspace(op, B, Cin, Cout, IH, IW, OH, OW, K, P, dtype, interp, precision);
  if (precision != SPH_PRECISION_BF16 || dtype != SPH_F32) return base;
  // bf16 precision: a convolution whose gathered side has at most 63 columns runs its own tensor-core kernels; they may
  // still decline at call time (an unaligned pointer), so the scratch covers the fallback as well
  size_t thin = 0;
  switch (op) {
    case SPH_CONV_FORWARD: if (tc_thin_forward_ok(Cin, K, Cout, OW)) thin = tc_thin_forward_workspace(Cout); break;
    case SPH_CONV_BACKWARD_INPUT:
    case SPH_CONV_BACKWARD: if (tc_thin_backward_ok(Cin, K, Cout, OH * OW)) thin = tc_thin_backward_workspace(B, Cin, K, OH * OW, true); break;
    case SPH_CONV_BACKWARD_WEIGHT: if (tc_thin_backward_ok(Cin, K, Cout, OH * OW)) thin = tc_thin_backward_workspace(B, Cin, K, OH * OW, false); break;
    default: break;
  }
  return thin > base ? thin : base;
}

#define SPH_BY_DTYPE(fn, ...) (dtype == SPH_F32 ? fn<float>(__VA_ARGS__) : fn<double>(__VA_ARGS__))

namespace {

int conv_forward(const void *x, const void *map, const void *iw, const void *weight, const void *bias, void *out, int64_t B,
                 int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype,
                 int interp, int precision, void *ws, size_t ws_bytes, void *stream, const Fusion &fz) {
  const Dims d{B, Cin, Cout, IH, IW, OH, OW, K, P};
  const int rc = check_dims(d, dtype, interp, precision);
  if (rc != SPH_OK) return rc;
  if (!x || !map || !weight || !bias || !out || (P > 0 && !iw)) return SPH_ERR_INVALID_ARGUMENT;
  if (B == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // bf16 precision, at most 63 gathered columns: one 64-column operand block per tile on the tensor cores, if the output
  // can leave through a tensor map; else (and in the exact precision) thin layers run the register-tiled kernels
  if (precision == SPH_PRECISION_BF16 && tc_thin_forward_ok(Cin, K, Cout, OW)) {
    const int rt = tc_thin_conv_forward(x, map, iw, weight, bias, out, B, Cin, Cout, IH, IW, OH, OW, K, P, interp, ws, ws_bytes, st, fz);
    if (rt != SPH_ERR_UNSUPPORTED) return rt;
  }
  if (small_ok(Cin, K, Cout, dtype == SPH_F64 ? 8 : 4))
    return SPH_BY_DTYPE(small_fwd, x, map, iw, Cin, IH, IW, K, P, OH * OW, interp, weight, Cin * K, K, 1, bias, out, Cout, B, st,
                        fz.relu_out, fz.out_cl);
  if (precision == SPH_PRECISION_BF16)
    return tc_conv_forward(x, map, iw, weight, bias, out, B, Cin, Cout, IH, IW, OH, OW, K, P, interp, ws, ws_bytes, st, fz);
  if (fz.active() || fz.out_cl != nullptr) return SPH_ERR_UNSUPPORTED;
  return SPH_BY_DTYPE(simt_gemm, false, x, map, iw, nullptr, Cin, IH, IW, K, P, OH * OW, interp, weight, Cin * K, K, 1,
                      bias, out, Cout, B, st, ws, ws_bytes);
}

int conv_backward_input(const void *gout, const void *plan, const void *weight, void *gx, int64_t B, int64_t Cin, int64_t Cout,
                        int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int dtype, int precision, void *ws,
                        size_t ws_bytes, void *stream, const Fusion &fz) {
  const Dims d{B, Cin, Cout, IH, IW, OH, OW, K, 0};
  const int rc = check_dims(d, dtype, 0, precision);
  if (rc != SPH_OK) return rc;
  if (!gout || !plan || !weight || !gx) return SPH_ERR_INVALID_ARGUMENT;
  if (B == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // The thin kernels are issue-bound, not memory-bound: reading the mask inside them was measured slower (layer-1 dInput
  // of the encoder 2.1 -> 4.4 ms, dW 2.6 -> 2.9 ms) than one separate masking pass (0.9 ms), so they decline the mask.
  if (precision == SPH_PRECISION_BF16 && tc_thin_backward_ok(Cin, K, Cout, OH * OW)) {
    const int rt = tc_thin_conv_backward(gout, fz.mask, nullptr, plan, nullptr, nullptr, weight, gx, nullptr, nullptr, B, Cin, Cout, IH, IW,
                                         OH, OW, K, 0, 0, ws, ws_bytes, st);
    if (rt != SPH_ERR_UNSUPPORTED) return rt;
  }
  if (small_ok(Cin, K, Cout, dtype == SPH_F64 ? 8 : 4) && fz.mask) return SPH_ERR_UNSUPPORTED;
  if (small_ok(Cin, K, Cout, dtype == SPH_F64 ? 8 : 4))
    return SPH_BY_DTYPE(small_adjoint, gout, plan, Cout, OH * OW, K, IH * IW, weight, K, Cin * K, 1, nullptr, gx, Cin, B, ws,
                        ws_bytes, st);
  if (precision == SPH_PRECISION_BF16)
    return tc_conv_backward_input(gout, plan, weight, gx, B, Cin, Cout, IH, IW, OH, OW, K, ws, ws_bytes, st, fz);
  if (fz.active()) return SPH_ERR_UNSUPPORTED;
  return SPH_BY_DTYPE(simt_gemm, true, gout, nullptr, nullptr, plan, Cout, OH, OW, K, 0, IH * IW, 0, weight, K, Cin * K, 1,
                      nullptr, gx, Cin, B, st, ws, ws_bytes);
}

int conv_backward_weight(const void *gout, const void *x, const void *map, const void *iw, void *gw, void *gb, int64_t B,
                         int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                         int dtype, int interp, int precision, void *ws, size_t ws_bytes, void *stream, const Fusion &fz) {
  const Dims d{B, Cin, Cout, IH, IW, OH, OW, K, P};
  const int rc = check_dims(d, dtype, interp, precision);
  if (rc != SPH_OK) return rc;
  if (!gout || !x || !map || !gw || !gb || (P > 0 && !iw)) return SPH_ERR_INVALID_ARGUMENT;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t ts = dtype == SPH_F64 ? 8 : 4;
  if (B == 0) {
    if (cudaMemsetAsync(gw, 0, ts * (size_t)(Cout * Cin * K), st) != cudaSuccess) return SPH_ERR_CUDA;
    return cudaMemsetAsync(gb, 0, ts * (size_t)Cout, st) == cudaSuccess ? SPH_OK : SPH_ERR_CUDA;
  }
  if (precision == SPH_PRECISION_BF16 && tc_thin_backward_ok(Cin, K, Cout, OH * OW)) {
    const int rt = tc_thin_conv_backward(gout, fz.mask, x, nullptr, map, iw, nullptr, nullptr, gw, gb, B, Cin, Cout, IH, IW, OH, OW, K, P,
                                         interp, ws, ws_bytes, st);
    if (rt != SPH_ERR_UNSUPPORTED) return rt;
  }
  if (small_ok(Cin, K, Cout, ts) && fz.mask) return SPH_ERR_UNSUPPORTED;  // see conv_backward_input
  if (small_ok(Cin, K, Cout, ts))
    return SPH_BY_DTYPE(small_dw, gout, x, map, iw, Cin, IH, IW, K, P, OH * OW, interp, Cout, B, gw, Cin * K, K, 1, gout, Cout,
                        OH * OW, gb, ws, ws_bytes, st);
  if (precision == SPH_PRECISION_BF16)
    return tc_conv_backward_weight(gout, x, map, iw, gw, gb, B, Cin, Cout, IH, IW, OH, OW, K, P, interp, ws, ws_bytes, st, fz);
  if (fz.active()) return SPH_ERR_UNSUPPORTED;
  return SPH_BY_DTYPE(simt_dw, gout, x, map, iw, Cin, IH, IW, K, P, OH * OW, interp, Cout, B, gw, Cin * K, K, 1, gout, Cout,
                      OH * OW, gb, ws, ws_bytes, st);
}

}  // namespace

extern "C" int sph_mapped_conv_forward(const void *x, const void *map, const void *iw, const void *weight,
                                       const void *bias, void *out, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                                       int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                                       int precision, void *ws, size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_conv_forward");
  return conv_forward(x, map, iw, weight, bias, out, B, Cin, Cout, IH, IW, OH, OW, K, P, dtype, interp, precision, ws, ws_bytes,
                      stream, Fusion{});
}

extern "C" int sph_mapped_conv_backward_input(const void *gout, const void *plan, const void *weight, void *gx,
                                              int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH,
                                              int64_t OW, int64_t K, int dtype, int precision, void *ws,
                                              size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_conv_backward_input");
  return conv_backward_input(gout, plan, weight, gx, B, Cin, Cout, IH, IW, OH, OW, K, dtype, precision, ws, ws_bytes, stream,
                             Fusion{});
}

extern "C" int sph_mapped_conv_backward_weight(const void *gout, const void *x, const void *map, const void *iw,
                                               void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                                               int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype,
                                               int interp, int precision, void *ws, size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_conv_backward_weight");
  return conv_backward_weight(gout, x, map, iw, gw, gb, B, Cin, Cout, IH, IW, OH, OW, K, P, dtype, interp, precision, ws,
                              ws_bytes, stream, Fusion{});
}

// ---- convolution with a fused ReLU (no counterpart in the reference; see sphmap.h) -------------------------
extern "C" int sph_mapped_conv_relu_forward(const void *x, const void *map, const void *iw, const void *weight,
                                            const void *bias, void *out, int64_t B, int64_t Cin, int64_t Cout,
                                            int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                                            int dtype, int interp, int precision, void *ws, size_t ws_bytes,
                                            void *stream) {
  SPH_RANGE("sph_mapped_conv_relu_forward");
  return conv_forward(x, map, iw, weight, bias, out, B, Cin, Cout, IH, IW, OH, OW, K, P, dtype, interp, precision, ws, ws_bytes,
                      stream, Fusion{true, nullptr});
}

extern "C" int sph_mapped_conv_relu_backward_input(const void *gout, const void *act_out, const void *plan,
                                                   const void *weight, void *gx, int64_t B, int64_t Cin, int64_t Cout,
                                                   int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int dtype,
                                                   int precision, void *ws, size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_conv_relu_backward_input");
  if (!act_out) return SPH_ERR_INVALID_ARGUMENT;
  return conv_backward_input(gout, plan, weight, gx, B, Cin, Cout, IH, IW, OH, OW, K, dtype, precision, ws, ws_bytes, stream,
                             Fusion{false, act_out});
}

extern "C" int sph_mapped_conv_relu_backward_weight(const void *gout, const void *act_out, const void *x,
                                                    const void *map, const void *iw, void *gw, void *gb, int64_t B,
                                                    int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH,
                                                    int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                                                    int precision, void *ws, size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_conv_relu_backward_weight");
  if (!act_out) return SPH_ERR_INVALID_ARGUMENT;
  return conv_backward_weight(gout, x, map, iw, gw, gb, B, Cin, Cout, IH, IW, OH, OW, K, P, dtype, interp, precision, ws,
                              ws_bytes, stream, Fusion{false, act_out});
}

// ---- channels-last companions and the combined backward (no counterpart in the reference; see sphmap.h) ------
extern "C" size_t sph_conv_companion_bytes(int64_t B, int64_t C, int64_t H, int64_t W) {
  if (B < 0 || C <= 0 || H <= 0 || W <= 0 || H * W >= ((int64_t)1 << 31)) return 0;
  return align_up((size_t)(B * (H * W + 1)) * (size_t)padded_channels(C) * 2, 256);
}

extern "C" int64_t sph_conv_companion_channels(int64_t C) { return C > 0 ? padded_channels(C) : 0; }

extern "C" int sph_conv_companion_fill(const void *x, void *x_cl, int64_t B, int64_t C, int64_t H, int64_t W, void *stream) {
  SPH_RANGE("sph_conv_companion_fill");
  if (!x || !x_cl || ((uintptr_t)x_cl & 15) != 0) return SPH_ERR_INVALID_ARGUMENT;
  if (sph_conv_companion_bytes(B, C, H, W) == 0) return SPH_ERR_INVALID_ARGUMENT;
  if (B == 0) return SPH_OK;
  return tc_fill_companion(x, x_cl, B, C, H * W, (cudaStream_t)stream);
}

extern "C" int sph_mapped_conv_forward_cl(const void *x, const void *x_cl, const void *map, const void *iw, const void *weight,
                                          const void *bias, void *out, void *out_cl, int64_t B, int64_t Cin, int64_t Cout,
                                          int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype,
                                          int interp, int precision, int relu, void *ws, size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_conv_forward_cl");
  Fusion fz;
  fz.relu_out = relu != 0;
  fz.src_cl = x_cl;
  fz.out_cl = out_cl;
  if (x_cl != nullptr && (precision != SPH_PRECISION_BF16 || small_ok(Cin, K, Cout, dtype == SPH_F64 ? 8 : 4) ||
                          tc_thin_forward_ok(Cin, K, Cout, OW)))
    fz.src_cl = nullptr;  // the kernels that run this shape gather from the float32 tensor
  return conv_forward(x, map, iw, weight, bias, out, B, Cin, Cout, IH, IW, OH, OW, K, P, dtype, interp, precision, ws, ws_bytes,
                      stream, fz);
}

extern "C" int sph_mapped_conv_backward_cl(const void *gout, const void *act_out, const void *x, const void *x_cl,
                                           const void *plan, const void *map, const void *iw, const void *weight, void *gx,
                                           void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                                           int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp, int precision,
                                           void *ws, size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_conv_backward_cl");
  const Dims d{B, Cin, Cout, IH, IW, OH, OW, K, P};
  const int rc = check_dims(d, dtype, interp, precision);
  if (rc != SPH_OK) return rc;
  if (!gout || !x || !plan || !map || !weight || !gx || !gw || !gb || (P > 0 && !iw)) return SPH_ERR_INVALID_ARGUMENT;
  if (precision != SPH_PRECISION_BF16 || B == 0) return SPH_ERR_UNSUPPORTED;
  if (tc_thin_backward_ok(Cin, K, Cout, OH * OW)) {
    const int rt = tc_thin_conv_backward(gout, act_out, x, plan, map, iw, weight, gx, gw, gb, B, Cin, Cout, IH, IW, OH, OW, K, P, interp, ws,
                                         ws_bytes, (cudaStream_t)stream);
    if (rt != SPH_ERR_UNSUPPORTED) return rt;
  }
  if (small_ok(Cin, K, Cout, dtype == SPH_F64 ? 8 : 4)) return SPH_ERR_UNSUPPORTED;
  Fusion fz;
  fz.mask = act_out;
  fz.src_cl = x_cl;
  return tc_conv_backward(gout, x, plan, map, iw, weight, gx, gw, gb, B, Cin, Cout, IH, IW, OH, OW, K, P, interp, ws, ws_bytes,
                          (cudaStream_t)stream, fz);
}

extern "C" int sph_mapped_tconv_forward(const void *x, const void *plan, const void *weight, const void *bias,
                                        void *out, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                                        int64_t OH, int64_t OW, int64_t K, int dtype, int precision, void *ws,
                                        size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_tconv_forward");
  const Dims d{B, Cin, Cout, IH, IW, OH, OW, K, 0};
  const int rc = check_dims(d, dtype, 0, precision);
  if (rc != SPH_OK) return rc;
  if (!x || !plan || !weight || !bias || !out) return SPH_ERR_INVALID_ARGUMENT;
  if (B == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (small_ok(Cout, K, Cin, dtype == SPH_F64 ? 8 : 4))
    return SPH_BY_DTYPE(small_adjoint, x, plan, Cin, IH * IW, K, OH * OW, weight, K, Cout * K, 1, bias, out, Cout, B, ws, ws_bytes,
                        st);
  if (precision == SPH_PRECISION_BF16)
    return tc_tconv_forward(x, plan, weight, bias, out, B, Cin, Cout, IH, IW, OH, OW, K, ws, ws_bytes, st);
  return SPH_BY_DTYPE(simt_gemm, true, x, nullptr, nullptr, plan, Cin, IH, IW, K, 0, OH * OW, 0, weight, K, Cout * K, 1,
                      bias, out, Cout, B, st, ws, ws_bytes);
}

extern "C" int sph_mapped_tconv_backward_input(const void *gout, const void *map, const void *iw, const void *weight,
                                               void *gx, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                                               int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                                               int precision, void *ws, size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_tconv_backward_input");
  const Dims d{B, Cin, Cout, IH, IW, OH, OW, K, P};
  const int rc = check_dims(d, dtype, interp, precision);
  if (rc != SPH_OK) return rc;
  if (!gout || !map || !weight || !gx || (P > 0 && !iw)) return SPH_ERR_INVALID_ARGUMENT;
  if (B == 0) return SPH_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (small_ok(Cout, K, Cin, dtype == SPH_F64 ? 8 : 4))
    return SPH_BY_DTYPE(small_fwd, gout, map, iw, Cout, OH, OW, K, P, IH * IW, interp, weight, Cout * K, K, 1, nullptr, gx, Cin, B,
                        st);
  if (precision == SPH_PRECISION_BF16)
    return tc_tconv_backward_input(gout, map, iw, weight, gx, B, Cin, Cout, IH, IW, OH, OW, K, P, interp, ws, ws_bytes, st);
  return SPH_BY_DTYPE(simt_gemm, false, gout, map, iw, nullptr, Cout, OH, OW, K, P, IH * IW, interp, weight, Cout * K, K, 1,
                      nullptr, gx, Cin, B, st, ws, ws_bytes);
}

extern "C" int sph_mapped_tconv_backward_weight(const void *gout, const void *x, const void *map, const void *iw,
                                                void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                                                int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype,
                                                int interp, int precision, void *ws, size_t ws_bytes, void *stream) {
  SPH_RANGE("sph_mapped_tconv_backward_weight");
  const Dims d{B, Cin, Cout, IH, IW, OH, OW, K, P};
  const int rc = check_dims(d, dtype, interp, precision);
  if (rc != SPH_OK) return rc;
  if (!gout || !x || !map || !gw || !gb || (P > 0 && !iw)) return SPH_ERR_INVALID_ARGUMENT;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t ts = dtype == SPH_F64 ? 8 : 4;
  if (B == 0) {
    if (cudaMemsetAsync(gw, 0, ts * (size_t)(Cout * Cin * K), st) != cudaSuccess) return SPH_ERR_CUDA;
    return cudaMemsetAsync(gb, 0, ts * (size_t)Cout, st) == cudaSuccess ? SPH_OK : SPH_ERR_CUDA;
  }
  if (small_ok(Cout, K, Cin, ts))
    return SPH_BY_DTYPE(small_dw, x, gout, map, iw, Cout, OH, OW, K, P, IH * IW, interp, Cin, B, gw, Cout * K, K, 1, gout, Cout,
                        OH * OW, gb, ws, ws_bytes, st);
  if (precision == SPH_PRECISION_BF16)
    return tc_tconv_backward_weight(gout, x, map, iw, gw, gb, B, Cin, Cout, IH, IW, OH, OW, K, P, interp, ws, ws_bytes, st);
  return SPH_BY_DTYPE(simt_dw, x, gout, map, iw, Cout, OH, OW, K, P, IH * IW, interp, Cin, B, gw, Cout * K, K, 1, gout, Cout,
                      OH * OW, gb, ws, ws_bytes, st);
}
