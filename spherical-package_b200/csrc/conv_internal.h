// Internal (non-exported) interfaces between conv.cu, conv_simt.cu and conv_tc.cu.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sph {

// Activation fused into the convolution kernels, passed down by the *_relu entry points: relu_out clamps the
// forward outputs at zero in the epilogue; mask (the saved activation output, same shape as grad_output) makes
// every kernel that reads grad_output see grad_output * (mask > 0).  Code paths that cannot honour it return
// SPH_ERR_UNSUPPORTED before launching anything.
//
// Channels-last copies: the tensor-core kernels gather from a bf16 copy of the source laid out (B, H*W + 1, Cp)
// (Cp = channels padded as padded_channels() says; pixel H*W of every image and the padding channels are zero).  A
// caller that keeps such copies next to its float32 activations passes them here and the conversion pre-passes
// disappear: src_cl is the copy of the gathered tensor, out_cl (forward only) is where the epilogue also writes the
// output in that layout (real channels and pixels only: the buffer is zero-filled once by its owner).
// gt_ready (weight gradient): the gradient tile images and bias partial sums already sit in the workspace.
struct Fusion {
  bool relu_out = false;
  const void *mask = nullptr;
  const void *src_cl = nullptr;
  void *out_cl = nullptr;
  bool gt_ready = false;
  bool active() const { return relu_out || mask != nullptr; }
};

// ---- exact SIMT kernels (conv_simt.cu) -----------------------------------
template <typename T>
int simt_gemm(bool use_plan, const void *src, const void *map, const void *iw, const void *plan, int64_t CH, int64_t SH,
              int64_t SW, int64_t K, int64_t P, int64_t npix, int interp, const void *wgt, int64_t sm, int64_t sc,
              int64_t sk, const void *bias, void *out, int64_t M, int64_t B, cudaStream_t st, void *ws = nullptr,
              size_t ws_bytes = 0);
// scratch simt_gemm can use (optional: a transposed copy of the weights for coalesced reads)
size_t simt_gemm_workspace(int64_t M, int64_t CH, int64_t K, size_t ts);
// the same for plan-mode (adjoint) calls: n_src source and n_dst destination pixels (may select the multiply-first form)
size_t simt_adjoint_workspace(int64_t B, int64_t M, int64_t CH, int64_t K, int64_t n_src, int64_t n_dst, size_t ts);
template <typename T>
int simt_dw(const void *A, const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K,
            int64_t P, int64_t npix, int interp, int64_t M, int64_t B, void *gw, int64_t sm, int64_t sc, int64_t sk,
            const void *gbias_src, int64_t Cbias, int64_t nbias, void *gb, void *ws, size_t ws_bytes, cudaStream_t st);
size_t simt_dw_workspace(int64_t B, int64_t npix, int64_t M, int64_t CH, int64_t K, int64_t Cbias, size_t ts);
size_t simt_bias_workspace(int64_t C, size_t ts);
template <typename T>
int simt_bias_grad(const void *g, int64_t B, int64_t C, int64_t n, void *gb, void *ws, cudaStream_t st);

template <typename T>
int simt_dw_reduce(const void *partial, int splits, int64_t M, int64_t CHK, int64_t K, int64_t sm, int64_t sc, int64_t sk,
                   void *gw, cudaStream_t st);

// ---- thin-contraction kernels (conv_small.cu): side_channels * K <= 32 ----
bool small_ok(int64_t side_channels, int64_t K, int64_t wide_channels, size_t ts);
size_t small_premul_workspace(int64_t B, int64_t M, int64_t K, int64_t n_src, size_t ts);
size_t small_dw_workspace(int64_t B, int64_t npix, int64_t M, int64_t CH, int64_t K, int64_t Cbias, size_t ts);
template <typename T>
int small_fwd(const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K, int64_t P,
              int64_t npix, int interp, const void *wgt, int64_t sm, int64_t sc, int64_t sk, const void *bias, void *out,
              int64_t M, int64_t B, cudaStream_t st, bool relu_out = false, void *out_cl = nullptr);
template <typename T>
int small_adjoint(const void *src, const void *plan, int64_t CH, int64_t n_src, int64_t K, int64_t n_dst, const void *wgt,
                  int64_t sm, int64_t sc, int64_t sk, const void *bias, void *out, int64_t M, int64_t B, void *ws,
                  size_t ws_bytes, cudaStream_t st);
template <typename T>
int small_dw(const void *A, const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K,
             int64_t P, int64_t npix, int interp, int64_t M, int64_t B, void *gw, int64_t sm, int64_t sc, int64_t sk,
             const void *gbias_src, int64_t Cbias, int64_t nbias, void *gb, void *ws, size_t ws_bytes, cudaStream_t st);

// ---- bf16 tcgen05 path (conv_tc.cu); float32 tensors only ----------------
size_t tc_workspace_bytes(int op, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                          int64_t K, int64_t P, int interp);
int tc_conv_forward(const void *x, const void *map, const void *iw, const void *weight, const void *bias, void *out,
                    int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                    int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz = Fusion{});
int tc_conv_backward_input(const void *gout, const void *plan, const void *weight, void *gx, int64_t B, int64_t Cin,
                           int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, void *ws,
                           size_t ws_bytes, cudaStream_t st, const Fusion &fz = Fusion{});
int tc_conv_backward_weight(const void *gout, const void *x, const void *map, const void *iw, void *gw, void *gb,
                            int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                            int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz = Fusion{});
// dInput + dW + dBias of one convolution with grad_output converted once (it feeds both): see conv_tc.cu.
int tc_conv_backward(const void *gout, const void *x, const void *plan, const void *map, const void *iw, const void *weight,
                     void *gx, void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH,
                     int64_t OW, int64_t K, int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz);
size_t tc_conv_backward_workspace(int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                                  int64_t K, int64_t P, int interp);
int padded_channels(int64_t CH);
int tc_fill_companion(const void *x, void *x_cl, int64_t B, int64_t C, int64_t HW, cudaStream_t st);
// Thin gathered side (channels x K <= 63) on the tensor cores, bf16 precision: see conv_tc_thin.cuh.
bool tc_thin_backward_ok(int64_t CH, int64_t K, int64_t N, int64_t npix);
size_t tc_thin_backward_workspace(int64_t B, int64_t CH, int64_t K, int64_t npix, bool with_dx);  // with_dx: gx is wanted
// (a null gx, or null gw and gb, leaves that gradient out)
int tc_thin_conv_backward(const void *gout, const void *act, const void *x, const void *plan, const void *map, const void *iw,
                          const void *weight, void *gx, void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                          int64_t OH, int64_t OW, int64_t K, int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st);
bool tc_thin_forward_ok(int64_t CH, int64_t K, int64_t Nout, int64_t GW);
size_t tc_thin_forward_workspace(int64_t Nout);
int tc_thin_conv_forward(const void *x, const void *map, const void *iw, const void *weight, const void *bias, void *out, int64_t B,
                         int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int interp,
                         void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz);
int tc_tconv_forward(const void *x, const void *plan, const void *weight, const void *bias, void *out, int64_t B,
                     int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, void *ws,
                     size_t ws_bytes, cudaStream_t st);
int tc_tconv_backward_input(const void *gout, const void *map, const void *iw, const void *weight, void *gx, int64_t B,
                            int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                            int interp, void *ws, size_t ws_bytes, cudaStream_t st);
int tc_tconv_backward_weight(const void *gout, const void *x, const void *map, const void *iw, void *gw, void *gb,
                             int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                             int64_t K, int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st);

}  // namespace sph
