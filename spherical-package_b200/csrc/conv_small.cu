// Mapped convolution kernels for layers whose gathered side is tiny (channels * kernel slots <= 32, e.g. the
// 3-channel first layer of an encoder).  There the contraction is too thin for tensor-core tiles and the
// work is dominated by the gather and by streaming the wide tensor once, so these are SIMT kernels in the
// tensor's own precision (float32 / float64):
//
//   small_fwd_kernel   Out[b,m,pix] = bias[m] + sum_j Wgt[m,j] * Col[b,j,pix]       j = ch*K + k <= 32
//                      (conv forward with few input channels; transposed conv dInput with few output channels)
//   small_premul_kernel + small_plan_gather_kernel
//                      the adjoint in the reference's own order (GEMM first, then col2im:
//                      src/cpp/mapped_convolution_layer.cpp:69-86): T[b,(m,k),o] = sum_ch Wgt[m,ch,k] * Src[b,ch,o],
//                      then Out[b,m,p] = sum_k sum_{e in plan(p,k)} w_e * T[b,(m,k),o_e]   (+ bias), m*K <= 32
//   small_dw_kernel    dW[m,j] = sum_{b,pix} A[b,m,pix] * Col[b,j,pix], split over pixel ranges
#include "common.cuh"
#include "conv_internal.h"

namespace sph {

constexpr int kSmallJ = 32;  // at most this many (channel, slot) columns

template <typename T, int INTERP, bool WEIGHTED>
__device__ __forceinline__ void small_columns(T (&col)[kSmallJ], const T *__restrict__ src, const T *__restrict__ map,
                                              const T *__restrict__ iw, int CH, int K, int P, int SH, int SW, int pix) {
  const int PP = WEIGHTED ? P : 1;
  const size_t shw = (size_t)SH * SW;
#pragma unroll
  for (int j = 0; j < kSmallJ; j++) col[j] = T(0);
  for (int k = 0; k < K; k++) {
    const size_t e = ((size_t)pix * K + k) * PP;
    if (!WEIGHTED) {
      Taps<T> t;
      decode<T, INTERP>(__ldg(map + 2 * e), __ldg(map + 2 * e + 1), SH, SW, t);
      for (int c = 0; c < CH; c++) {
        const T v = gather<T, INTERP>(src + c * shw, t);
#pragma unroll
        for (int j = 0; j < kSmallJ; j++)
          if (j == c * K + k) col[j] = v;
      }
    } else {
      for (int c = 0; c < CH; c++) {
        const T v = gather_slot<T, INTERP, true>(src + c * shw, map + 2 * e, iw + e, P, SH, SW);
#pragma unroll
        for (int j = 0; j < kSmallJ; j++)
          if (j == c * K + k) col[j] = v;
      }
    }
  }
}

// Wgt is staged in shared memory as [M][kSmallJ] (zero padded); thread = one pixel.
template <typename T, int INTERP, bool WEIGHTED>
__global__ void __launch_bounds__(256)
small_fwd_kernel(const T *__restrict__ src, const T *__restrict__ map, const T *__restrict__ iw, const T *__restrict__ wgt,
                 int64_t sm, int64_t sc, int64_t sk, const T *__restrict__ bias, T *__restrict__ out, int CH, int K, int P,
                 int SH, int SW, int npix, int M) {
  extern __shared__ unsigned char small_smem[];
  T *ws = (T *)small_smem;
  for (int i = threadIdx.x; i < M * kSmallJ; i += blockDim.x) {
    const int m = i / kSmallJ, j = i % kSmallJ;
    ws[i] = j < CH * K ? __ldg(wgt + m * sm + (j / K) * sc + (j % K) * sk) : T(0);
  }
  __syncthreads();
  const int pix = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (pix >= npix) return;
  T col[kSmallJ];
  small_columns<T, INTERP, WEIGHTED>(col, src + (size_t)b * CH * SH * SW, map, iw, CH, K, P, SH, SW, pix);
  T *o = out + (size_t)b * M * npix + pix;
  for (int m = 0; m < M; m++) {
    const T *wr = ws + m * kSmallJ;
    T acc = bias ? __ldg(bias + m) : T(0);
#pragma unroll
    for (int j = 0; j < kSmallJ; j++) acc += wr[j] * col[j];
    o[(size_t)m * npix] = acc;
  }
}

// T[b, o, m*K + k] = sum_ch Wgt[m,ch,k] * Src[b,ch,o]; thread = one source position o.
template <typename T>
__global__ void __launch_bounds__(256)
small_premul_kernel(const T *__restrict__ src, const T *__restrict__ wgt, int64_t sm, int64_t sc, int64_t sk,
                    T *__restrict__ tbuf, int CH, int K, int M, int n_src) {
  extern __shared__ unsigned char small_smem[];
  T *ws = (T *)small_smem;  // [CH][kSmallJ]
  for (int i = threadIdx.x; i < CH * kSmallJ; i += blockDim.x) {
    const int ch = i / kSmallJ, j = i % kSmallJ;
    ws[i] = j < M * K ? __ldg(wgt + (j / K) * sm + ch * sc + (j % K) * sk) : T(0);
  }
  __syncthreads();
  const int o = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (o >= n_src) return;
  T acc[kSmallJ];
#pragma unroll
  for (int j = 0; j < kSmallJ; j++) acc[j] = T(0);
  const T *s = src + (size_t)b * CH * n_src + o;
  for (int ch = 0; ch < CH; ch++) {
    const T v = __ldg(s + (size_t)ch * n_src);
    const T *wr = ws + ch * kSmallJ;
#pragma unroll
    for (int j = 0; j < kSmallJ; j++) acc[j] += wr[j] * v;
  }
  T *t = tbuf + ((size_t)b * n_src + o) * kSmallJ;  // one padded row of kSmallJ values per source position
#pragma unroll
  for (int j = 0; j < kSmallJ; j++) t[j] = acc[j];
}

// Out[b,m,p] = bias[m] + sum_k sum_{e in plan(p*K+k)} w_e * T[b, src_e, m*K+k]; thread = one destination pixel of
// kGatherImages consecutive images, so the plan entries are read once per group of images.
constexpr int kGatherImages = 4, kGatherM = 4;  // images per thread; output channels per register block

template <typename T>
__global__ void __launch_bounds__(256)
small_plan_gather_kernel(const T *__restrict__ tbuf, const void *__restrict__ plan_blob, const T *__restrict__ bias,
                         T *__restrict__ out, int K, int M, int n_src, int n_dst, int B) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x, b0 = blockIdx.y * kGatherImages;
  if (p >= n_dst) return;
  bool ok;
  const PlanView<T> pv = plan_view<T>(plan_blob, n_dst * K, ok);
  const int nb = min(kGatherImages, B - b0);
  const size_t img_stride = (size_t)n_src * kSmallJ;
  const T *tb = tbuf + (size_t)b0 * img_stride;
  for (int m0 = 0; m0 < M; m0 += kGatherM) {   // one pass for M <= 4 (e.g. RGB inputs)
    T acc[kGatherImages][kGatherM];
#pragma unroll
    for (int i = 0; i < kGatherImages; i++)
#pragma unroll
      for (int m = 0; m < kGatherM; m++) acc[i][m] = T(0);
    if (ok) {
      int e1 = __ldg(pv.offsets + p * K);
      for (int k = 0; k < K; k++) {
        const int e0 = e1;
        e1 = __ldg(pv.offsets + p * K + k + 1);
        for (int e = e0; e < e1; e++) {
          const T *row = tb + (size_t)__ldg(pv.src + e) * kSmallJ + k;
          const T w = __ldg(pv.w + e);
#pragma unroll
          for (int i = 0; i < kGatherImages; i++)
            if (i < nb) {
#pragma unroll
              for (int m = 0; m < kGatherM; m++)
                if (m0 + m < M) acc[i][m] += w * __ldg(row + i * img_stride + (m0 + m) * K);
            }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kGatherImages; i++)
      if (i < nb) {
#pragma unroll
        for (int m = 0; m < kGatherM; m++)
          if (m0 + m < M) out[((size_t)(b0 + i) * M + m0 + m) * n_dst + p] = acc[i][m] + (bias ? __ldg(bias + m0 + m) : T(0));
      }
  }
}

// dW partial sums: block = (64 rows of A) x (all <= 32 columns) over the pixel chunks of its split.
constexpr int kSdwChunk = 256;
template <typename T> struct SdwPix { static constexpr int value = sizeof(T) == 8 ? 32 : 64; };  // pixels staged per step

template <typename T, int INTERP, bool WEIGHTED>
__global__ void __launch_bounds__(256)
small_dw_kernel(const T *__restrict__ A, const T *__restrict__ src, const T *__restrict__ map, const T *__restrict__ iw,
                int CH, int K, int P, int SH, int SW, int npix, int M, int B, T *__restrict__ partial) {
  constexpr int kSdwPix = SdwPix<T>::value;
  __shared__ T As[kSdwPix][64 + 1];
  __shared__ T Cs[kSdwPix][kSmallJ + 1];
  // four quarters of 64 threads: each quarter takes every fourth staged pixel and holds an 8 x 4 register tile
  // per thread (rows tm + 8 i, columns tj + 8 j); the quarters' sums are kept as separate partials
  const int tid = threadIdx.x, qtr = tid >> 6, tm = (tid & 63) >> 3, tj = tid & 7;
  const int m0 = blockIdx.y * 64, splits = gridDim.x, J = CH * K;
  const int chunks = (npix + kSdwChunk - 1) / kSdwChunk;
  T acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = T(0);
  for (int unit = blockIdx.x; unit < B * chunks; unit += splits) {
    const int b = unit / chunks, pbase = (unit % chunks) * kSdwChunk, pend = min(npix, pbase + kSdwChunk);
    for (int p0 = pbase; p0 < pend; p0 += kSdwPix) {
      {
        // thread = (pixel, slot group): slots k = group, group + G, ... of its pixel, all channels
        constexpr int G = 256 / kSdwPix;
        const int pl = tid % kSdwPix, grp = tid / kSdwPix, pix = p0 + pl;
        const T *img = src + (size_t)b * CH * SH * SW;
        const int PP = WEIGHTED ? P : 1;
        for (int k = grp; k < K; k += G) {
          const size_t e = ((size_t)pix * K + k) * PP;
          for (int c = 0; c < CH; c++)
            Cs[pl][c * K + k] = pix < pend ? gather_slot<T, INTERP, WEIGHTED>(img + (size_t)c * SH * SW, map + 2 * e, iw + e, P, SH, SW)
                                           : T(0);
        }
        for (int j = J + grp; j < kSmallJ; j += G) Cs[pl][j] = T(0);
      }
      for (int e = tid; e < 64 * kSdwPix; e += 256) {
        const int pl = e % kSdwPix, ml = e / kSdwPix, pix = p0 + pl, m = m0 + ml;
        As[pl][ml] = (pix < pend && m < M) ? __ldg(A + ((size_t)b * M + m) * npix + pix) : T(0);
      }
      __syncthreads();
#pragma unroll 2
      for (int pl = qtr; pl < kSdwPix; pl += 4) {
        T c[4], a[8];
#pragma unroll
        for (int j = 0; j < 4; j++) c[j] = Cs[pl][tj + 8 * j];
#pragma unroll
        for (int i = 0; i < 8; i++) a[i] = As[pl][tm + 8 * i];
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] += a[i] * c[j];
      }
      __syncthreads();
    }
  }
  const size_t prow = (size_t)blockIdx.x * 4 + qtr;  // partial index: (split, quarter)
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int m = m0 + tm + 8 * i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++)
      if (tj + 8 * j < J) partial[(prow * M + m) * J + tj + 8 * j] = acc[i][j];
  }
}

// ---- host side ------------------------------------------------------------------------------------------
bool small_ok(int64_t side_channels, int64_t K, int64_t wide_channels, size_t ts) {
  return side_channels * K <= kSmallJ && wide_channels * kSmallJ * (int64_t)ts <= 48 * 1024;
}

static int small_dw_splits(int64_t B, int64_t npix, int64_t M) {
  const int64_t units = B * ((npix + kSdwChunk - 1) / kSdwChunk), mblocks = (M + 63) / 64;
  int64_t s = (4 * 148 + mblocks - 1) / mblocks;
  if (s > units) s = units;
  if (s < 1) s = 1;
  return (int)s;
}

size_t small_premul_workspace(int64_t B, int64_t M, int64_t K, int64_t n_src, size_t ts) {
  (void)M; (void)K;
  return align_up(ts * (size_t)(B * n_src) * kSmallJ, 256);
}

size_t small_dw_workspace(int64_t B, int64_t npix, int64_t M, int64_t CH, int64_t K, int64_t Cbias, size_t ts) {
  return align_up(ts * (size_t)(4 * small_dw_splits(B, npix, M) * M * CH * K), 256) + simt_bias_workspace(Cbias, ts);
}

template <typename T>
int small_fwd(const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K, int64_t P,
              int64_t npix, int interp, const void *wgt, int64_t sm, int64_t sc, int64_t sk, const void *bias, void *out,
              int64_t M, int64_t B, cudaStream_t st) {
  dim3 grid(cdiv(npix, 256), (unsigned)B);
  const size_t smem = sizeof(T) * (size_t)M * kSmallJ;
#define SPH_SMALL_FWD(W)                                                                                              \
  small_fwd_kernel<T, INTERP, W><<<grid, 256, smem, st>>>((const T *)src, (const T *)map, (const T *)iw, (const T *)wgt, sm, \
                                                          sc, sk, (const T *)bias, (T *)out, (int)CH, (int)K, (int)P,   \
                                                          (int)SH, (int)SW, (int)npix, (int)M)
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0) SPH_SMALL_FWD(true);
    else SPH_SMALL_FWD(false);
  });
#undef SPH_SMALL_FWD
  return launch_status();
}

template <typename T>
int small_adjoint(const void *src, const void *plan, int64_t CH, int64_t n_src, int64_t K, int64_t n_dst, const void *wgt,
                  int64_t sm, int64_t sc, int64_t sk, const void *bias, void *out, int64_t M, int64_t B, void *ws,
                  size_t ws_bytes, cudaStream_t st) {
  if (!ws || ws_bytes < small_premul_workspace(B, M, K, n_src, sizeof(T))) return SPH_ERR_WORKSPACE_TOO_SMALL;
  small_premul_kernel<T><<<dim3(cdiv(n_src, 256), (unsigned)B), 256, sizeof(T) * (size_t)CH * kSmallJ, st>>>(
      (const T *)src, (const T *)wgt, sm, sc, sk, (T *)ws, (int)CH, (int)K, (int)M, (int)n_src);
  small_plan_gather_kernel<T><<<dim3(cdiv(n_dst, 256), cdiv(B, kGatherImages)), 256, 0, st>>>(
      (const T *)ws, plan, (const T *)bias, (T *)out, (int)K, (int)M, (int)n_src, (int)n_dst, (int)B);
  return launch_status(2);
}

template <typename T>
int small_dw(const void *A, const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K,
             int64_t P, int64_t npix, int interp, int64_t M, int64_t B, void *gw, int64_t sm, int64_t sc, int64_t sk,
             const void *gbias_src, int64_t Cbias, int64_t nbias, void *gb, void *ws, size_t ws_bytes, cudaStream_t st) {
  if (!ws || ws_bytes < small_dw_workspace(B, npix, M, CH, K, Cbias, sizeof(T))) return SPH_ERR_WORKSPACE_TOO_SMALL;
  const int splits = small_dw_splits(B, npix, M);
  T *partial = (T *)ws;
  void *bias_ws = (char *)ws + align_up(sizeof(T) * (size_t)(4 * splits * M * CH * K), 256);
  dim3 grid(splits, cdiv(M, 64));
#define SPH_SMALL_DW(W)                                                                                               \
  small_dw_kernel<T, INTERP, W><<<grid, 256, 0, st>>>((const T *)A, (const T *)src, (const T *)map, (const T *)iw, (int)CH, \
                                                      (int)K, (int)P, (int)SH, (int)SW, (int)npix, (int)M, (int)B, partial)
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0) SPH_SMALL_DW(true);
    else SPH_SMALL_DW(false);
  });
#undef SPH_SMALL_DW
  const int rc = simt_dw_reduce<T>(partial, 4 * splits, M, CH * K, K, sm, sc, sk, gw, st);
  if (rc != SPH_OK) return rc;
  note_launches(1);
  return simt_bias_grad<T>(gbias_src, B, Cbias, nbias, gb, bias_ws, st);
}

#define SPH_INSTANTIATE_SMALL(T)                                                                                          \
  template int small_fwd<T>(const void *, const void *, const void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, \
                            int, const void *, int64_t, int64_t, int64_t, const void *, void *, int64_t, int64_t,          \
                            cudaStream_t);                                                                                 \
  template int small_adjoint<T>(const void *, const void *, int64_t, int64_t, int64_t, int64_t, const void *, int64_t,     \
                                int64_t, int64_t, const void *, void *, int64_t, int64_t, void *, size_t, cudaStream_t);   \
  template int small_dw<T>(const void *, const void *, const void *, const void *, int64_t, int64_t, int64_t, int64_t,     \
                           int64_t, int64_t, int, int64_t, int64_t, void *, int64_t, int64_t, int64_t, const void *,       \
                           int64_t, int64_t, void *, void *, size_t, cudaStream_t);
SPH_INSTANTIATE_SMALL(float)
SPH_INSTANTIATE_SMALL(double)

}  // namespace sph
