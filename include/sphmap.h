/* sphmap.h -- C ABI of the B200 (sm_100a) mapped-operator library, libsphmap.so.
 *
 * These entry points are what the host side of the Spherical-Package extension
 * modules (package `_spherical_distortion_ext`) binds for the mapped-operator
 * path: mapped convolution / transposed convolution forward and backward,
 * mapped max pooling with its argmax backward, and resample_from_map /
 * resample_to_map.  Every pointer is a DEVICE pointer unless said otherwise;
 * tensors are dense, row major ("contiguous NCHW"), float32 or float64.
 * Nothing here allocates, synchronises or throws: every function enqueues its
 * kernels on `stream` (a cudaStream_t passed as void*) and returns a status
 * (0 = SPH_OK).  Scratch memory is supplied by the caller; the sizes come
 * from the *_bytes queries.
 *
 * Conventions shared by all entry points
 *   map     sample map, (OH,OW,K,2) or, with interpolation weights,
 *           (OH,OW,K,P,2); last axis is (x, y) in pixel units of the sampled
 *           image; same dtype as the data.
 *   iw      interpolation weights (OH,OW,K,P), or NULL with P = 0.
 *   interp  0 nearest, 1 bilinear (zero outside), 2 bispherical (x wraps).
 *   dtype   0 float32, 1 float64.
 *   precision  0: arithmetic in the tensor's own type (SIMT path, the one
 *           compared bit-for-bit / to 1e-5 with the reference CPU code);
 *           1: bf16 operands with fp32 accumulation on the tcgen05 tensor
 *           cores (float32 tensors only).
 *
 * Reference interfaces are cited as file:line inside the reference project.
 */
#ifndef SPHMAP_H_
#define SPHMAP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum sph_status {
  SPH_OK = 0,
  SPH_ERR_INVALID_ARGUMENT = 1,
  SPH_ERR_UNSUPPORTED = 2,
  SPH_ERR_WORKSPACE_TOO_SMALL = 3,
  SPH_ERR_CUDA = 4,
  SPH_ERR_TOO_LARGE = 5,
  SPH_ERR_STATIC_SCRATCH_EXCEEDED = 6
};
enum sph_dtype { SPH_F32 = 0, SPH_F64 = 1 };
enum sph_interp { SPH_NEAREST = 0, SPH_BILINEAR = 1, SPH_BISPHERICAL = 2 };
enum sph_precision { SPH_PRECISION_EXACT = 0, SPH_PRECISION_BF16 = 1 };

/* Human-readable text for a status code (host pointer, static storage). */
const char *sph_status_string(int status);
/* Library version, major*10000 + minor*100 + patch. */
int sph_version(void);
/* Number of kernels this library has launched in this process so far (a
 * tracing aid for benchmarks; no counterpart in the reference). */
unsigned long long sph_launch_count(void);

/* ------------------------------------------------------------------------
 * Device status.  Every wait inside the tensor-core kernels (mbarrier waits
 * between the gathering, MMA-issuing and draining warps) is bounded: after
 * 4 s of wall time the waiting warp gives up, all roles of that CTA leave
 * their loops, tensor memory is freed, the kernel returns normally, and the
 * give-up is recorded (a) as 1 in the first 32-bit word of the workspace the
 * call was given and (b) in a sticky word on the device.  Outputs of such a
 * launch are invalid.  The launch itself still returned SPH_OK (nothing
 * synchronises), so a host that wants to know asks here:
 *   sph_device_status  copies the sticky word of the CURRENT device to
 *       *status (host pointer; 0 = no wait ever gave up) and clears it if
 *       reset != 0.  Blocks until the device's queued work is done.
 *   sph_debug_bounded_wait  self check of that mechanism: one small kernel
 *       allocates tensor memory and waits, with the given limit
 *       (nanoseconds, at most 1e9), on a barrier nothing arrives at; it must
 *       write 1 to *status (DEVICE pointer), set the sticky word, free its
 *       tensor memory and return.
 * Checked build.  Compiled with -DSPH_BOUNDS_CHECK (build.py --checked ->
 * libsphmap_checked.so, same ABI) every data-dependent index a kernel is
 * about to use - tap offsets, plan entries, positions while a plan is
 * written - is range-checked first; a violation skips the access and sets
 * bit 1 (value 2) of the status word.  It is the stand-in for a memory
 * checker where none may run; sph_build_is_checked() tells which build is
 * loaded.  In every build a plan that was made for tensors of another size
 * is recognised by its header and the operator writes zeros instead of
 * following it.
 * The reference has no counterpart: its CUDA_CHECK ends the process
 * (ext_modules/include/cuda_helper.h:5-10).
 * ---------------------------------------------------------------------- */
int sph_device_status(int *status, int reset);
int sph_build_is_checked(void);
int sph_debug_bounded_wait(unsigned long long limit_ns, int *status, void *stream);

/* ------------------------------------------------------------------------
 * resample_from_map ("Unresample"): y[b,c,i] = interp(x[b,c], map[i]).
 * Replaces spherical::ResampleFromMap, ext_modules/include/layers/
 * resample_layer.h:62-82 (weighted twin: weighted_resample_layer.h:77-105).
 * x (B,C,H,W); map (MH,MW[,P],2); iw (MH,MW,P) or NULL; y (B,C,MH,MW).
 * ---------------------------------------------------------------------- */
int sph_resample_from_map(const void *x, const void *map, const void *iw, void *y, int64_t B, int64_t C,
                          int64_t H, int64_t W, int64_t MH, int64_t MW, int64_t P, int dtype, int interp,
                          void *stream);

/* ------------------------------------------------------------------------
 * Scatter plan.  Every adjoint ("scatter") operator of the reference adds
 * through float atomics.  This library instead inverts the sample map once
 * into a CSR table keyed by (destination pixel, kernel slot) and every
 * scatter becomes a gather that sums its segment in a fixed order, so the
 * results are deterministic.  A plan depends only on the map, the weights,
 * the interpolation type and the destination size; build it once per map.
 *
 *   n_src   number of map positions (MH*MW, or OH*OW for convolution maps)
 *   K       kernel slots per position (1 for resample maps)
 *   dstH/W  size of the image the map points into
 * The plan blob is opaque; sph_plan_bytes() gives its size (a host function,
 * no device work).  No counterpart in the reference (its scatter kernels are
 * ext_modules/include/cuda/resample.cuh:14-47, mapped_im2col.cuh:52-91).
 * ---------------------------------------------------------------------- */
size_t sph_plan_bytes(int64_t n_src, int64_t K, int64_t P, int interp, int64_t dstH, int64_t dstW, int dtype);
int sph_plan_build(const void *map, const void *iw, int64_t n_src, int64_t K, int64_t P, int interp,
                   int64_t dstH, int64_t dstW, int dtype, void *plan, size_t plan_bytes, void *stream);

/* ------------------------------------------------------------------------
 * resample_to_map ("Resample"): out[b,c] = sum_i scatter(x[b,c,i], map[i]).
 * Replaces spherical::ResampleToMap, resample_layer.h:40-60 (weighted twin:
 * weighted_resample_layer.h:49-75).  `plan` was built from the (MH,MW[,P],2)
 * map with K = 1 and dst = (OH,OW).  x (B,C,MH,MW); out (B,C,OH,OW), fully
 * written (no pre-zeroing needed).
 * ---------------------------------------------------------------------- */
int sph_resample_to_map(const void *x, const void *plan, void *out, int64_t B, int64_t C, int64_t MH,
                        int64_t MW, int64_t OH, int64_t OW, int dtype, void *stream);

/* resample_to_map followed by the weight-sum normalisation,
 *   out = scatter(x) / (scatter(1) + 1e-12),
 * in one pass: every destination pixel divides its sum by the sum of its own
 * segment's weights.  The reference composes this in Python
 * (layers/functional/sphere_ops.py:74-80, 110-116). */
int sph_resample_to_map_normalized(const void *x, const void *plan, void *out, int64_t B, int64_t C, int64_t MH,
                                   int64_t MW, int64_t OH, int64_t OW, int dtype, void *stream);

/* ------------------------------------------------------------------------
 * UV-map resampling between an image and NT square textures (tangent
 * images).  quad_idx (IH,IW) int64 names the texture of every image pixel,
 * tex_uv (IH,IW,2) its (x, y) position inside that texture in texel units;
 * tex is (B,C,NT,TH,TW).  Interpolation and its zero padding act inside the
 * named texture; a texture index outside [0,NT) contributes nothing.
 *   from_uv_maps   out[b,c,i] = interp(tex[b,c,quad[i]], uv[i])      (gather)
 *   to_uv_maps     the adjoint: sph_plan_build_uv once per (quad, uv), then
 *                  sph_resample_to_map(x, plan, tex, B, C, IH, IW,
 *                  OH = NT*TH, OW = TW, ...)
 * Replaces spherical::ResampleFromUVMaps / ResampleToUVMaps,
 * ext_modules/include/layers/uv_resample_layer.h:48-100.
 * sph_plan_bytes(n_src = IH*IW, 1, 0, interp, NT*TH, TW, dtype) sizes the plan.
 * ---------------------------------------------------------------------- */
int sph_resample_from_uv_maps(const void *tex, const int64_t *quad_idx, const void *tex_uv, void *out, int64_t B,
                              int64_t C, int64_t NT, int64_t TH, int64_t TW, int64_t IH, int64_t IW, int dtype,
                              int interp, void *stream);
int sph_plan_build_uv(const void *tex_uv, const int64_t *quad_idx, int64_t n_src, int64_t NT, int64_t TH, int64_t TW,
                      int interp, int dtype, void *plan, size_t plan_bytes, void *stream);

/* ------------------------------------------------------------------------
 * Voting resample of integer labels: out[b,c,o] = the label carried by most
 * of the input pixels whose map entry is output pixel o (the smallest such
 * label on ties, 0 where nothing lands).  `plan` is a nearest-neighbour plan
 * (sph_plan_build with interp = 0, K = 1, P = 0) of the map given as
 * floating-point (x, y) coordinates of type plan_dtype; labels and out are
 * int64.  Labels outside [0, num_candidates) cast no vote.  Replaces
 * spherical::VotingResampleToMap,
 * ext_modules/include/layers/voting_resample_layer.h:32-58, without its
 * (C, OH, OW, num_candidates) vote tensor.
 * ---------------------------------------------------------------------- */
int sph_voting_resample_to_map(const int64_t *labels, const void *plan, int plan_dtype, int64_t *out, int64_t B,
                               int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t num_candidates,
                               void *stream);

/* ------------------------------------------------------------------------
 * Equirectangular kernel maps built on the device.  For every pixel
 * (y, x) = (oy*stride, ox*stride) of an H x W equirectangular image, the
 * kh x kw kernel grid around it in fractional pixel coordinates (x, y) of the
 * same image: map is (ceil(H/stride), ceil(W/stride), kh*kw, 2) of `dtype`.
 *   SPH_MAP_GRID                 offsets on the lat/lon grid (no wrap)
 *   SPH_MAP_INVERSE_GNOMONIC     tangent-plane grid projected back onto the
 *                                sphere; longitude wrapped to [-pi, pi)
 *   SPH_MAP_INVERSE_EQUIRECT     longitude step divided by cos(latitude)
 * Replaces grid_projection_map, inverse_gnomonic_projection_map and
 * inverse_equirectangular_projection_map of the reference's
 * layers/util/mapping_functions.py:44-163 (host tensor code there).
 * ---------------------------------------------------------------------- */
enum sph_map_kind { SPH_MAP_GRID = 0, SPH_MAP_INVERSE_GNOMONIC = 1, SPH_MAP_INVERSE_EQUIRECT = 2 };
int sph_build_kernel_map(void *map, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t stride, int64_t dilation,
                         int kind, int dtype, void *stream);

/* ------------------------------------------------------------------------
 * resample_to_map for callers that cannot allocate device memory.
 * Has no counterpart in the reference.  It is for hosts that must not call
 * cudaMalloc (or any allocating routine) around this library: code running
 * inside a fixed memory budget handed out at start-up, real-time loops where
 * an allocation could stall or fail, or plug-in sandboxes that only receive
 * pre-allocated buffers.  sph_resample_to_map needs a scatter plan in caller
 * scratch; this variant builds the plan from `map` (and `iw`) into a scratch
 * array that is part of the library image itself (a file-scope __device__
 * array of SPH_STATIC_SCRATCH_BYTES, resident on every GPU that loads the
 * library until the process exits) and then runs the same scatter kernel.
 * The caller still passes the input and the output; nothing is allocated or
 * freed by this call, by the CUDA runtime on its behalf, or by torch.
 *
 *  - Limit: the plan for (MH*MW positions, P points, interp, OHxOW) must fit
 *    SPH_STATIC_SCRATCH_BYTES (sph_plan_bytes tells); larger problems return
 *    SPH_ERR_STATIC_SCRATCH_EXCEEDED and launch nothing.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) before launching; make
 *    that first call outside any stream capture.
 *  - Every call on a device shares the one array and overwrites the plan the
 *    previous call left there (the parts that must start at zero are cleared
 *    by the call itself).  Two calls whose GPU work can overlap - different
 *    streams, or host threads on the same device - race on it; serialise
 *    them.
 * Arguments as sph_resample_from_map / sph_resample_to_map: x (B,C,MH,MW),
 * map (MH,MW[,P],2), iw (MH,MW,P) or NULL with P = 0, out (B,C,OH,OW).
 * ---------------------------------------------------------------------- */
#define SPH_STATIC_SCRATCH_BYTES (8u << 20)
int sph_resample_to_map_static(const void *x, const void *map, const void *iw, void *out, int64_t B, int64_t C,
                               int64_t MH, int64_t MW, int64_t OH, int64_t OW, int64_t P, int dtype, int interp,
                               void *stream);

/* ------------------------------------------------------------------------
 * Mapped max pooling.  out[b,c,o] = max_k interp(x[b,c], map[o,k]); idx is
 * the int64 offset of the winning entry's x coordinate in the flattened map
 * (first strict maximum; running maximum starts at -FLT_MAX as in the
 * reference's CUDA build).  Replaces spherical::MappedMaxPoolForward /
 * MappedMaxPoolBackward, ext_modules/include/layers/
 * mapped_max_pooling_layer.h:42-97 (weighted: weighted_mapped_max_pooling_
 * layer.h).  x (B,C,IH,IW); out, idx, g (B,C,OH,OW); grad_in (B,C,IH,IW),
 * fully written by the unpool call.
 * ---------------------------------------------------------------------- */
int sph_mapped_max_pool(const void *x, const void *map, const void *iw, void *out, int64_t *idx, int64_t B,
                        int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                        int dtype, int interp, void *stream);
int sph_mapped_max_unpool(const void *g, const int64_t *idx, const void *map, const void *iw, void *grad_in,
                          int64_t B, int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                          int64_t P, int dtype, int interp, void *stream);

/* Deterministic argmax backward: the same operator with no float atomics and
 * no zero-fill pass.  `plan` is a scatter plan over the FLATTENED map slots,
 * i.e. built by sph_plan_build(map, iw, n_src = OH*OW*K, K = 1, P, interp,
 * dst = (IH,IW)); every input pixel then sums, in map order, the gradients
 * of the outputs whose winning slot (idx) has a tap on it.  Results do not
 * depend on scheduling (run-to-run bit identical).  No counterpart in the
 * reference, whose CUDA kernel scatters with atomicAdd
 * (ext_modules/include/cuda/mapped_max_pool.cuh:57-95). */
int sph_mapped_max_unpool_planned(const void *g, const int64_t *idx, const void *plan, void *grad_in, int64_t B,
                                  int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                                  int dtype, void *stream);

/* ------------------------------------------------------------------------
 * Mapped average pooling.  out[b,c,o] = (sum_k interp(x[b,c], map[o,k])) / K,
 * slots added in order.  The backward sends g[b,c,o] / K back through every
 * slot; `plan` is the flattened-slot plan described above (n_src = OH*OW*K,
 * K = 1, dst = (IH,IW)); grad_in is fully written.  Replaces
 * spherical::MappedAvgPoolforward / MappedAvgPoolbackward,
 * ext_modules/include/layers/mapped_avg_pooling_layer.h:40-86 (weighted:
 * weighted_mapped_avg_pooling_layer.h:48-106).
 * ---------------------------------------------------------------------- */
int sph_mapped_avg_pool(const void *x, const void *map, const void *iw, void *out, int64_t B, int64_t C, int64_t IH,
                        int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp, void *stream);
int sph_mapped_avg_unpool(const void *g, const void *plan, void *grad_in, int64_t B, int64_t C, int64_t IH, int64_t IW,
                          int64_t OH, int64_t OW, int64_t K, int dtype, void *stream);

/* ------------------------------------------------------------------------
 * Mapped convolution.  weight (Cout,Cin,K), bias (Cout), x (B,Cin,IH,IW),
 * out / gout (B,Cout,OH,OW), map (OH,OW,K[,P],2).
 *   forward          out = W * im2col(x) + bias     (no column buffer)
 *   backward_input   gx  = col2im(W^T * gout), through a plan built from the
 *                    map with n_src = OH*OW, K, dst = (IH,IW)
 *   backward_weight  gw  = sum_b gout[b] * im2col(x[b])^T, gb = sum gout
 * Replaces spherical::MappedConvForward / MappedConvBackward,
 * ext_modules/include/layers/mapped_convolution_layer.h:62-134 (weighted:
 * weighted_mapped_convolution_layer.h:69-162).
 * ws/ws_bytes: scratch of at least sph_conv_workspace_bytes(op, ...) bytes, 256-byte aligned
 * (SPH_ERR_INVALID_ARGUMENT otherwise on the bf16 path).  On the bf16 path the first 32-bit
 * word of ws is the call's status word (0, or 1 after a bounded wait gave up: see
 * sph_device_status).
 * ---------------------------------------------------------------------- */
enum sph_conv_op {
  SPH_CONV_FORWARD = 0,
  SPH_CONV_BACKWARD_INPUT = 1,
  SPH_CONV_BACKWARD_WEIGHT = 2,
  SPH_TCONV_FORWARD = 3,
  SPH_TCONV_BACKWARD_INPUT = 4,
  SPH_TCONV_BACKWARD_WEIGHT = 5,
  SPH_CONV_BACKWARD = 6 /* sph_mapped_conv_backward_cl: input, weight and bias gradients in one call */
};
size_t sph_conv_workspace_bytes(int op, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                                int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                                int precision);
int sph_mapped_conv_forward(const void *x, const void *map, const void *iw, const void *weight,
                            const void *bias, void *out, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                            int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                            int precision, void *ws, size_t ws_bytes, void *stream);
int sph_mapped_conv_backward_input(const void *gout, const void *plan, const void *weight, void *gx,
                                   int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH,
                                   int64_t OW, int64_t K, int dtype, int precision, void *ws, size_t ws_bytes,
                                   void *stream);
int sph_mapped_conv_backward_weight(const void *gout, const void *x, const void *map, const void *iw,
                                    void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                                    int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype,
                                    int interp, int precision, void *ws, size_t ws_bytes, void *stream);

/* ------------------------------------------------------------------------
 * Mapped convolution with a fused ReLU: y = max(0, conv(x) + bias).  No counterpart
 * in the reference, which applies the activation as a separate operator (two more
 * passes over the output in forward, three in backward); arguments are those of the
 * three functions above.
 *   relu_forward          writes y; the clamp happens in the kernels' epilogue
 *   relu_backward_input   gout is the gradient w.r.t. y and act_out is y itself
 *   relu_backward_weight  (same shape as gout): the kernels read gout * (act_out > 0)
 *                         wherever they read gout, so no masked copy is made
 * Supported where the convolution runs on the thin-contraction kernels
 * (Cin * K <= 32, either precision) or on the bf16 tensor-core kernels; any other
 * shape returns SPH_ERR_UNSUPPORTED before launching anything, and the caller
 * applies the activation itself.  Workspace sizes are those of the unfused ops.
 * ---------------------------------------------------------------------- */
int sph_mapped_conv_relu_forward(const void *x, const void *map, const void *iw, const void *weight,
                                 const void *bias, void *out, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                                 int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                                 int precision, void *ws, size_t ws_bytes, void *stream);
int sph_mapped_conv_relu_backward_input(const void *gout, const void *act_out, const void *plan,
                                        const void *weight, void *gx, int64_t B, int64_t Cin, int64_t Cout,
                                        int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int dtype,
                                        int precision, void *ws, size_t ws_bytes, void *stream);
int sph_mapped_conv_relu_backward_weight(const void *gout, const void *act_out, const void *x, const void *map,
                                         const void *iw, void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout,
                                         int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                                         int dtype, int interp, int precision, void *ws, size_t ws_bytes,
                                         void *stream);

/* ------------------------------------------------------------------------
 * Channels-last companions and the combined backward (bf16 tensor-core path;
 * no counterpart in the reference).  The tensor-core kernels gather from a
 * bf16 copy of the gathered tensor laid out (B, H*W + 1, Cp): channels last,
 * Cp = C padded to a multiple of 8 that divides 64 or to a multiple of 64,
 * one extra all-zero pixel behind every image.  The plain entry points make
 * that copy in their workspace on every call.  A caller that runs a stack of
 * layers can keep the copies ("companions") next to its float32 activations:
 *   sph_conv_companion_bytes  size of the companion of a (B,C,H,W) tensor.
 *       The owner zero-fills it once (cudaMemsetAsync); the kernels only ever
 *       write real channels of real pixels.
 *   sph_mapped_conv_forward_cl  the forward operator (with the fused ReLU if
 *       relu != 0).  x_cl: companion of x, or NULL (then converted as usual).
 *       out_cl: if not NULL the kernel epilogue also writes the output as a
 *       companion, for the next layer.  Returns SPH_ERR_UNSUPPORTED, before
 *       launching anything, when out_cl cannot be honoured (float64, Cout not
 *       a multiple of 8, shapes that run on the generic SIMT kernels): call
 *       again with out_cl = NULL.
 *   sph_mapped_conv_backward_cl  input, weight and bias gradients in one
 *       call, as the reference's mapped_conv_backward computes them
 *       (ext_modules/include/layers/mapped_convolution_layer.h:89-134):
 *       grad_output is read once and converted for both consumers; act_out
 *       (or NULL) is the fused ReLU's output whose sign masks it; x_cl (or
 *       NULL) the companion of x.  Workspace: op SPH_CONV_BACKWARD.  Returns
 *       SPH_ERR_UNSUPPORTED before launching anything for shapes that do not
 *       run on tensor-core kernels (exact precision; thin layers whose
 *       tensor-core form does not apply): use the separate entry points
 *       there.
 *   sph_conv_companion_fill  writes the companion of an existing float32
 *       tensor (a host that calls the same layer's forward and backward can
 *       convert the input once and pass the copy to both).
 * Results are bit-identical to the separate entry points.
 * ---------------------------------------------------------------------- */
size_t sph_conv_companion_bytes(int64_t B, int64_t C, int64_t H, int64_t W);
int64_t sph_conv_companion_channels(int64_t C); /* Cp, the companion's channel pitch */
int sph_conv_companion_fill(const void *x, void *x_cl, int64_t B, int64_t C, int64_t H, int64_t W, void *stream);
int sph_mapped_conv_forward_cl(const void *x, const void *x_cl, const void *map, const void *iw, const void *weight,
                               const void *bias, void *out, void *out_cl, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                               int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                               int precision, int relu, void *ws, size_t ws_bytes, void *stream);
int sph_mapped_conv_backward_cl(const void *gout, const void *act_out, const void *x, const void *x_cl, const void *plan,
                                const void *map, const void *iw, const void *weight, void *gx, void *gw, void *gb,
                                int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                                int64_t K, int64_t P, int dtype, int interp, int precision, void *ws, size_t ws_bytes,
                                void *stream);

/* Tracing aid for sph_mapped_conv_backward_cl: the NEXT such call made by the
 * calling thread records the given CUDA events (cudaEvent_t passed as
 * void*, up to 4) on its stream at its phase boundaries - [0] entry, [1]
 * grad_output converted, [2] input gradient done, [3] weight and bias
 * gradients done - so that a benchmark can time the kernels inside the one
 * call.  The list is used once.  No counterpart in the reference. */
int sph_trace_phases(void **events, int n_events);

/* ------------------------------------------------------------------------
 * Mapped transposed convolution.  weight (Cin,Cout,K), bias (Cout),
 * x (B,Cin,IH,IW), out / gout (B,Cout,OH,OW); the map has the INPUT's size,
 * (IH,IW,K[,P],2), and points into the (OH,OW) output grid.
 *   forward          out = col2im(W^T * x) + bias, through a plan built from
 *                    the map with n_src = IH*IW, K, dst = (OH,OW)
 *   backward_input   gx  = W * im2col(gout)
 *   backward_weight  gw  = sum_b x[b] * im2col(gout[b])^T, gb = sum gout
 * Replaces spherical::MappedTransposedConvForward / ...Backward,
 * ext_modules/include/layers/mapped_transposed_convolution_layer.h:62-149
 * (weighted: weighted_mapped_transposed_convolution_layer.h).
 * ---------------------------------------------------------------------- */
int sph_mapped_tconv_forward(const void *x, const void *plan, const void *weight, const void *bias, void *out,
                             int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH,
                             int64_t OW, int64_t K, int dtype, int precision, void *ws, size_t ws_bytes,
                             void *stream);
int sph_mapped_tconv_backward_input(const void *gout, const void *map, const void *iw, const void *weight,
                                    void *gx, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                                    int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype, int interp,
                                    int precision, void *ws, size_t ws_bytes, void *stream);
int sph_mapped_tconv_backward_weight(const void *gout, const void *x, const void *map, const void *iw,
                                     void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH,
                                     int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int dtype,
                                     int interp, int precision, void *ws, size_t ws_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SPHMAP_H_ */
