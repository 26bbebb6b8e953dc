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
#include <cuda_bf16.h>

#include "common.cuh"
#include "conv_internal.h"

namespace sph {

constexpr int kSmallJ = 32;  // at most this many (channel, slot) columns
template <typename T> struct alignas(16) SdwVec { T v[16 / sizeof(T)]; };  // 16 bytes of T

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
                 int SH, int SW, int npix, int M, int relu) {
  extern __shared__ __align__(16) unsigned char small_smem[];
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
    o[(size_t)m * npix] = (relu && !(acc > T(0))) ? T(0) : acc;
  }
}

// float32 forward as a tiled product: a block gathers the columns of 256 pixels into shared memory
// (Col[j][pixel], thread = pixel), then multiplies them with the weights as a [256 pixels] x [64 outputs] tile:
// warp w owns outputs 8w..8w+7, lane l pixels 4l..4l+3 and 128+4l..128+4l+3, 64 accumulators per thread held as packed pairs of
// neighbouring pixels (two-wide FMAs).  Per column every thread reads 8 column values and 8 weights for 64
// multiply-adds, so shared-memory traffic stays far below the FMA rate; outputs beyond 64 take further passes
// over the same gathered columns.
__device__ __forceinline__ void ffma2(unsigned long long &d, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ unsigned pack_bf16x2(float lo, float hi) {
  unsigned r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

constexpr int kTilePix = 256, kTileOut = 64;

template <int INTERP, bool WEIGHTED>
__global__ void __launch_bounds__(256, 2)
small_fwd_tile_kernel(const float *__restrict__ src, const float *__restrict__ map, const float *__restrict__ iw,
                      const float *__restrict__ wgt, int64_t sm, int64_t sc, int64_t sk, const float *__restrict__ bias,
                      float *__restrict__ out, int CH, int K, int P, int SH, int SW, int npix, int M, int relu,
                      __nv_bfloat16 *__restrict__ out_cl, int cl_pitch) {
  __shared__ __align__(16) float Cs[kSmallJ][kTilePix];
  __shared__ __align__(16) float Ws[kSmallJ][kTileOut];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, b = blockIdx.y, J = CH * K;
  const int p0 = blockIdx.x * kTilePix;
  const size_t shw = (size_t)SH * SW;
  // ---- gather: thread = pixel ----
  {
    const int pix = p0 + tid;
    const float *img = src + (size_t)b * CH * shw;
    if (pix < npix) {
      const int PP = WEIGHTED ? P : 1;
      const size_t e0 = (size_t)pix * K * PP;
      if (!WEIGHTED) {
        // three slots and up to four channels at a time: all their loads are issued before any is used, so a
        // pixel costs a few memory round trips instead of one per gathered value
        constexpr int NTAP = TapCount<INTERP>::value;
        for (int k0 = 0; k0 < K; k0 += 3) {
          float mx[3], my[3];
#pragma unroll
          for (int u = 0; u < 3; u++)
            if (k0 + u < K) { mx[u] = __ldg(map + 2 * (e0 + k0 + u)); my[u] = __ldg(map + 2 * (e0 + k0 + u) + 1); }
          Taps<float> t[3];
#pragma unroll
          for (int u = 0; u < 3; u++)
            if (k0 + u < K) decode<float, INTERP>(mx[u], my[u], SH, SW, t[u]);
          for (int c0 = 0; c0 < CH; c0 += 4) {
            float raw[3][4][NTAP];
#pragma unroll
            for (int u = 0; u < 3; u++)
#pragma unroll
              for (int v = 0; v < 4; v++)
                if (k0 + u < K && c0 + v < CH) gather_load<float, INTERP>(img + (c0 + v) * shw, t[u], raw[u][v]);
#pragma unroll
            for (int u = 0; u < 3; u++)
#pragma unroll
              for (int v = 0; v < 4; v++)
                if (k0 + u < K && c0 + v < CH) Cs[(c0 + v) * K + k0 + u][tid] = gather_combine<float, INTERP>(t[u], raw[u][v]);
          }
        }
      } else {
        for (int k = 0; k < K; k++) {
          const size_t e = e0 + (size_t)k * PP;
          for (int c = 0; c < CH; c++)
            Cs[c * K + k][tid] = gather_slot<float, INTERP, true>(img + c * shw, map + 2 * e, iw + e, P, SH, SW);
        }
      }
    } else {
      for (int j = 0; j < J; j++) Cs[j][tid] = 0.0f;
    }
  }
  const bool vec_ok = (npix & 3) == 0;  // 16-byte stores need every output row 16-byte aligned
  for (int m0 = 0; m0 < M; m0 += kTileOut) {
    __syncthreads();  // columns complete (first pass) / previous pass done with Ws
    for (int i = tid; i < J * kTileOut; i += 256) {
      const int j = i / kTileOut, m = m0 + i % kTileOut;
      Ws[j][i % kTileOut] = m < M ? __ldg(wgt + m * sm + (j / K) * sc + (j % K) * sk) : 0.0f;
    }
    __syncthreads();
    const int mw = m0 + warp * 8;  // this warp's first output
    if (mw >= M) continue;
    unsigned long long acc[8][4];  // [output][pixel pair]
#pragma unroll
    for (int m = 0; m < 8; m++) {
      const float bv = (bias && mw + m < M) ? __ldg(bias + mw + m) : 0.0f;
#pragma unroll
      for (int q = 0; q < 4; q++) acc[m][q] = pack2(bv, bv);
    }
#pragma unroll 3
    for (int j = 0; j < J; j++) {
      const ulonglong2 c0 = *(const ulonglong2 *)&Cs[j][lane * 4], c1 = *(const ulonglong2 *)&Cs[j][128 + lane * 4];
      const float4 w0 = *(const float4 *)&Ws[j][warp * 8], w1 = *(const float4 *)&Ws[j][warp * 8 + 4];
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int m = 0; m < 8; m++) {
        const unsigned long long ww = pack2(wv[m], wv[m]);
        ffma2(acc[m][0], c0.x, ww);
        ffma2(acc[m][1], c0.y, ww);
        ffma2(acc[m][2], c1.x, ww);
        ffma2(acc[m][3], c1.y, ww);
      }
    }
#pragma unroll
    for (int m = 0; m < 8; m++) {
      if (mw + m >= M) break;
      float v[8];
#pragma unroll
      for (int q = 0; q < 4; q++) unpack2(acc[m][q], v[2 * q], v[2 * q + 1]);
      if (relu) {
#pragma unroll
        for (int q = 0; q < 8; q++) v[q] = v[q] > 0.0f ? v[q] : 0.0f;
      }
#pragma unroll
      for (int h = 0; h < 2; h++) {  // the two groups of four pixels
        const int px = p0 + h * 128 + lane * 4;
        float *o = out + ((size_t)b * M + mw + m) * npix + px;
        if (vec_ok && px + 4 <= npix) {
          *(float4 *)o = make_float4(v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]);
        } else {
#pragma unroll
          for (int q = 0; q < 4; q++)
            if (px + q < npix) o[q] = v[4 * h + q];
        }
      }
    }
    // channels-last bf16 copy of the same outputs: this warp's 8 channels of each of the thread's 8 pixels, 16 bytes
    // per pixel (channels beyond M carry zero weights and bias, so they come out as the zeros the layout wants)
    if (out_cl != nullptr && mw + 8 <= cl_pitch) {
#pragma unroll
      for (int t = 0; t < 8; t++) {
        const int px = p0 + (t >> 2) * 128 + lane * 4 + (t & 3);
        if (px >= npix) continue;
        float c[8];
#pragma unroll
        for (int m = 0; m < 8; m++) {
          float lo, hi;
          unpack2(acc[m][t >> 1], lo, hi);
          c[m] = (t & 1) ? hi : lo;
          if (relu) c[m] = c[m] > 0.0f ? c[m] : 0.0f;
        }
        uint4 o;
        o.x = pack_bf16x2(c[0], c[1]);
        o.y = pack_bf16x2(c[2], c[3]);
        o.z = pack_bf16x2(c[4], c[5]);
        o.w = pack_bf16x2(c[6], c[7]);
        *(uint4 *)(out_cl + ((size_t)b * (npix + 1) + px) * cl_pitch + mw) = o;
      }
    }
  }
}

// Row layout of the adjoint's intermediate T: one row of Rp values per source position, element (k, m) at
// k * Mq + m, where Mq pads the M output channels to 1, 2 or a multiple of 4 so that the plan gather fetches all
// channels of one (position, slot) with one vector load.
__host__ __device__ inline int small_mq(int M) { return M <= 2 ? M : (M + 3) / 4 * 4; }
__host__ __device__ inline int small_row(int M, int K) { return (K * small_mq(M) + 3) / 4 * 4; }
constexpr int kSmallRowMax = 48;  // M * K <= 32 keeps rows within this

// T[b, o, k*Mq + m] = sum_ch Wgt[m,ch,k] * Src[b,ch,o]; thread = two source positions o (256 apart), so that one
// read of a weight vector feeds two pixels.  R4 = row length / 4.
template <typename T, int R4>
__global__ void __launch_bounds__(256)
small_premul_kernel(const T *__restrict__ src, const T *__restrict__ wgt, int64_t sm, int64_t sc, int64_t sk,
                    T *__restrict__ tbuf, int CH, int K, int M, int n_src) {
  constexpr int Rp = 4 * R4, kU = 8;  // kU source channels are loaded ahead of their multiply-adds
  extern __shared__ __align__(16) unsigned char small_smem[];
  T *ws = (T *)small_smem;                   // [CH][Rp] weights
  T *stage = ws + (size_t)CH * Rp;           // [8 warps][32 rows][Rp] output rows on their way to memory
  const int Mq = small_mq(M);
  for (int i = threadIdx.x; i < CH * Rp; i += blockDim.x) {
    const int ch = i / Rp, r = i % Rp, k = r / Mq, m = r % Mq;
    ws[i] = (k < K && m < M) ? __ldg(wgt + m * sm + ch * sc + k * sk) : T(0);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int o0 = blockIdx.x * 512 + threadIdx.x, o1 = o0 + 256, b = blockIdx.y;
  const bool has0 = o0 < n_src, has1 = o1 < n_src;
  T acc0[Rp], acc1[Rp];
#pragma unroll
  for (int r = 0; r < Rp; r++) acc0[r] = acc1[r] = T(0);
  const T *s = src + (size_t)b * CH * n_src;
  for (int c0 = 0; c0 < CH; c0 += kU) {
    T v0[kU], v1[kU];
#pragma unroll
    for (int u = 0; u < kU; u++) {
      const bool in = c0 + u < CH;
      v0[u] = (in && has0) ? __ldg(s + (size_t)(c0 + u) * n_src + o0) : T(0);
      v1[u] = (in && has1) ? __ldg(s + (size_t)(c0 + u) * n_src + o1) : T(0);
    }
#pragma unroll
    for (int u = 0; u < kU; u++) {
      if (c0 + u < CH) {
        const T *wr = ws + (c0 + u) * Rp;
#pragma unroll
        for (int r = 0; r < Rp; r++) {
          acc0[r] += wr[r] * v0[u];
          acc1[r] += wr[r] * v1[u];
        }
      }
    }
  }
  // The 32 rows of a warp are contiguous in T: pass them through shared memory so that the stores are
  // coalesced 16-byte vectors instead of one row per lane.
  using V = SdwVec<T>;
  constexpr int VW = 16 / sizeof(T), kRowVecs = Rp / VW;
  T *wst = stage + (size_t)warp * 32 * Rp;
#pragma unroll
  for (int half = 0; half < 2; half++) {
    const int obase = blockIdx.x * 512 + half * 256 + warp * 32;  // first row of this warp's span
    if (obase >= n_src) break;
    const int rows = min(32, n_src - obase);
#pragma unroll
    for (int r = 0; r < Rp; r++) wst[lane * Rp + r] = half ? acc1[r] : acc0[r];
    __syncwarp();
    V *dst = (V *)(tbuf + ((size_t)b * n_src + obase) * Rp);
    for (int i = lane; i < rows * kRowVecs; i += 32) dst[i] = ((const V *)wst)[i];
    __syncwarp();
  }
}

// Out[b,m,p] = bias[m] + sum_k sum_{e in plan(p*K+k)} w_e * T[b, src_e, k*Mq + m]; thread = one destination pixel of
// kGatherImages consecutive images, so the plan entries are read once per group of images; VM = channels
// fetched per load (1, 2 or 4).
constexpr int kGatherImages = 4;
template <typename T, int VM> struct alignas(sizeof(T) * VM > 16 ? 16 : sizeof(T) * VM) SmallVec { T v[VM]; };

template <typename T, int VM>
__global__ void __launch_bounds__(256)
small_plan_gather_kernel(const T *__restrict__ tbuf, const void *__restrict__ plan_blob, const T *__restrict__ bias,
                         T *__restrict__ out, int K, int M, int n_src, int n_dst, int B) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x, b0 = blockIdx.y * kGatherImages;
  if (p >= n_dst) return;
  bool ok;
  const PlanView<T> pv = plan_view<T>(plan_blob, n_dst * K, ok);
  const int nb = min(kGatherImages, B - b0);
  const int Mq = small_mq(M), Rp = small_row(M, K);
  const size_t img_stride = (size_t)n_src * Rp;
  const T *tb = tbuf + (size_t)b0 * img_stride;
  for (int m0 = 0; m0 < Mq; m0 += VM) {   // one pass for M <= 4 (e.g. RGB inputs)
    T acc[kGatherImages][VM];
#pragma unroll
    for (int i = 0; i < kGatherImages; i++)
#pragma unroll
      for (int m = 0; m < VM; m++) acc[i][m] = T(0);
    if (ok) {
      int e1 = __ldg(pv.offsets + p * K);
      for (int k = 0; k < K; k++) {
        const int e0 = e1;
        e1 = __ldg(pv.offsets + p * K + k + 1);
        for (int e = e0; e < e1; e++) {
          const int sp = __ldg(pv.src + e);
          if (!index_ok(sp, pv.n_src)) continue;
          const T *row = tb + (size_t)sp * Rp + k * Mq + m0;
          const T w = __ldg(pv.w + e);
          SmallVec<T, VM> v[kGatherImages];
#pragma unroll
          for (int i = 0; i < kGatherImages; i++)
            if (i < nb) v[i] = *(const SmallVec<T, VM> *)(row + i * img_stride);
#pragma unroll
          for (int i = 0; i < kGatherImages; i++)
            if (i < nb) {
#pragma unroll
              for (int m = 0; m < VM; m++) acc[i][m] += w * v[i].v[m];
            }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kGatherImages; i++)
      if (i < nb) {
#pragma unroll
        for (int m = 0; m < VM; m++)
          if (m0 + m < M) out[((size_t)(b0 + i) * M + m0 + m) * n_dst + p] = acc[i][m] + (bias ? __ldg(bias + m0 + m) : T(0));
      }
  }
}

// dW partial sums: block = (64 rows of A) x (all <= 32 columns) over its share of the (pixel step, image group)
// units.  Both operands are staged pixel-contiguous ([row][pixel], the layout A already has in memory), and
// every thread reads 16-byte pixel vectors of its 8 rows and 4 columns, so one shared-memory load feeds four
// (two for float64) multiply-adds of each accumulator it touches.  The taps of a pixel step are decoded once
// into shared memory and reused for all images of the unit's group (the map is the same for every image).
constexpr int kSdwImages = 8;  // images per unit
constexpr int kSdwThreads = 128, kSdwParts = kSdwThreads / 64;  // small blocks: four per SM, out of phase with one another
template <typename T> struct SdwPix { static constexpr int value = sizeof(T) == 8 ? 32 : 64; };  // pixels staged per step
template <typename T> struct alignas(16) SdwTaps { Taps<T> t; };  // 16-byte aligned so that it moves as vectors

template <typename T, int INTERP, bool WEIGHTED>
__global__ void __launch_bounds__(kSdwThreads)
small_dw_kernel(const T *__restrict__ A, const T *__restrict__ src, const T *__restrict__ map, const T *__restrict__ iw,
                int CH, int K, int P, int SH, int SW, int npix, int M, int B, T *__restrict__ partial,
                T *__restrict__ bias_partial) {
  constexpr int kSdwPix = SdwPix<T>::value, VW = 16 / sizeof(T), kPitch = kSdwPix + VW;
  // rows 17 words apart (mod 32 banks: 4 apart), so the 16-byte reads of consecutive rows do not collide
  __shared__ __align__(16) T As[64][kPitch];
  __shared__ __align__(16) T Cs[kSmallJ][kPitch];
  extern __shared__ __align__(16) unsigned char small_smem[];
  SdwTaps<T> *tcache = (SdwTaps<T> *)small_smem;  // [K][kSdwPix] decoded taps of the current pixel step (unweighted maps)
  // kSdwParts groups of 64 threads: each group takes every kSdwParts-th pixel vector and holds an 8 x 4 register
  // tile per thread (rows tm + 8 i, columns tj + 8 j); the groups' sums are kept as separate partials
  const int tid = threadIdx.x, qtr = tid >> 6, tm = (tid & 63) >> 3, tj = tid & 7;
  const int m0 = blockIdx.y * 64, splits = gridDim.x, J = CH * K;
  const int steps = (npix + kSdwPix - 1) / kSdwPix, groups = (B + kSdwImages - 1) / kSdwImages;
  const size_t shw = (size_t)SH * SW;
  // With bias_partial set (and J < kSmallJ) the first padding column of Col is all ones, so that column of the
  // product is the row sum of A: the bias gradient when A is grad_output.  Pixels past the end have A = 0.
  const bool ones = bias_partial != nullptr;
  for (int e = tid; e < (kSmallJ - J) * kPitch; e += kSdwThreads) Cs[J + e / kPitch][e % kPitch] = (ones && e < kPitch) ? T(1) : T(0);
  T acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = T(0);
  for (int unit = blockIdx.x; unit < steps * groups; unit += splits) {
    const int p0 = (unit / groups) * kSdwPix, b0 = (unit % groups) * kSdwImages, b1 = min(B, b0 + kSdwImages);
    const int pend = min(npix, p0 + kSdwPix);
    if (!WEIGHTED) {
      for (int idx = tid; idx < K * kSdwPix; idx += kSdwThreads) {
        const int k = idx / kSdwPix, pix = p0 + idx % kSdwPix;
        Taps<T> t;
        if (pix < pend) {
          const size_t e = (size_t)pix * K + k;
          decode<T, INTERP>(__ldg(map + 2 * e), __ldg(map + 2 * e + 1), SH, SW, t);
        } else {
#pragma unroll
          for (int q = 0; q < 4; q++) { t.off[q] = -1; t.w[q] = T(0); }
        }
        tcache[idx].t = t;
      }
      __syncthreads();
    }
    for (int b = b0; b < b1; b++) {
      const T *img = src + (size_t)b * CH * shw;
      for (int e = tid; e < 64 * kSdwPix; e += kSdwThreads) {
        const int pl = e % kSdwPix, ml = e / kSdwPix, pix = p0 + pl, m = m0 + ml;
        As[ml][pl] = (pix < pend && m < M) ? __ldg(A + ((size_t)b * M + m) * npix + pix) : T(0);
      }
      if (!WEIGHTED) {
        // gathered columns, three (slot, pixel) items per thread at a time so that their loads overlap
        for (int base = tid; base < K * kSdwPix; base += 3 * kSdwThreads) {
          Taps<T> t[3];
          int row[3], pl[3];
          bool ok[3];
#pragma unroll
          for (int r = 0; r < 3; r++) {
            const int idx = base + r * kSdwThreads;
            ok[r] = idx < K * kSdwPix;
            row[r] = ok[r] ? idx / kSdwPix : 0;
            pl[r] = idx % kSdwPix;
            t[r] = tcache[ok[r] ? idx : 0].t;
          }
          for (int c = 0; c < CH; c++) {
            T v[3];
#pragma unroll
            for (int r = 0; r < 3; r++) v[r] = gather<T, INTERP>(img + (size_t)c * shw, t[r]);
#pragma unroll
            for (int r = 0; r < 3; r++)
              if (ok[r]) Cs[c * K + row[r]][pl[r]] = v[r];
          }
        }
      } else {
        for (int idx = tid; idx < K * kSdwPix; idx += kSdwThreads) {
          const int k = idx / kSdwPix, pl = idx % kSdwPix, pix = p0 + pl;
          const size_t e = ((size_t)pix * K + k) * P;
          for (int c = 0; c < CH; c++)
            Cs[c * K + k][pl] = pix < pend ? gather_slot<T, INTERP, true>(img + (size_t)c * shw, map + 2 * e, iw + e, P, SH, SW) : T(0);
        }
      }
      __syncthreads();
#pragma unroll 1
      for (int pv = qtr; pv < kSdwPix / VW; pv += kSdwParts) {
        SdwVec<T> a[8], c[4];
#pragma unroll
        for (int i = 0; i < 8; i++) a[i] = *(const SdwVec<T> *)&As[tm + 8 * i][pv * VW];
#pragma unroll
        for (int j = 0; j < 4; j++) c[j] = *(const SdwVec<T> *)&Cs[tj + 8 * j][pv * VW];
#pragma unroll
        for (int x = 0; x < VW; x++)
#pragma unroll
          for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] += a[i].v[x] * c[j].v[x];
      }
      __syncthreads();
    }
  }
  const size_t prow = (size_t)blockIdx.x * kSdwParts + qtr;  // partial index: (split, thread group)
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int m = m0 + tm + 8 * i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      if (tj + 8 * j < J) partial[(prow * M + m) * J + tj + 8 * j] = acc[i][j];
      else if (ones && tj + 8 * j == J) bias_partial[prow * M + m] = acc[i][j];
    }
  }
}

// ---- host side ------------------------------------------------------------------------------------------
bool small_ok(int64_t side_channels, int64_t K, int64_t wide_channels, size_t ts) {
  return side_channels * K <= kSmallJ && wide_channels * kSmallRowMax * (int64_t)ts <= 48 * 1024;
}

static int small_dw_splits(int64_t B, int64_t npix, int64_t M, size_t ts) {
  const int64_t pix = ts == 8 ? 32 : 64;
  const int64_t units = ((B + kSdwImages - 1) / kSdwImages) * ((npix + pix - 1) / pix), mblocks = (M + 63) / 64;
  int64_t s = (8 * 148 + mblocks - 1) / mblocks;
  if (s > units) s = units;
  if (s < 1) s = 1;
  return (int)s;
}

size_t small_premul_workspace(int64_t B, int64_t M, int64_t K, int64_t n_src, size_t ts) {
  return align_up(ts * (size_t)(B * n_src) * small_row((int)M, (int)K), 256);
}

size_t small_dw_workspace(int64_t B, int64_t npix, int64_t M, int64_t CH, int64_t K, int64_t Cbias, size_t ts) {
  const size_t parts = kSdwParts * (size_t)small_dw_splits(B, npix, M, ts);
  return align_up(ts * parts * M * CH * K, 256) + align_up(ts * parts * M, 256) + simt_bias_workspace(Cbias, ts);
}

template <typename T>
int small_fwd(const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K, int64_t P,
              int64_t npix, int interp, const void *wgt, int64_t sm, int64_t sc, int64_t sk, const void *bias, void *out,
              int64_t M, int64_t B, cudaStream_t st, bool relu_out, void *out_cl) {
  if (out_cl != nullptr && (sizeof(T) != 4 || M % 8 != 0)) return SPH_ERR_UNSUPPORTED;
  if constexpr (sizeof(T) == 4) {  // float32: tiled product
    const int cl_pitch = out_cl ? padded_channels(M) : 0;
    const dim3 tgrid(cdiv(npix, kTilePix), (unsigned)B);
#define SPH_FWD_TILE(W)                                                                                                \
  small_fwd_tile_kernel<INTERP, W><<<tgrid, 256, 0, st>>>((const float *)src, (const float *)map, (const float *)iw,     \
                                                          (const float *)wgt, sm, sc, sk, (const float *)bias,          \
                                                          (float *)out, (int)CH, (int)K, (int)P, (int)SH, (int)SW,       \
                                                          (int)npix, (int)M, relu_out ? 1 : 0, (__nv_bfloat16 *)out_cl, cl_pitch)
    SPH_DISPATCH_INTERP(interp, {
      if (P > 0) SPH_FWD_TILE(true);
      else SPH_FWD_TILE(false);
    });
#undef SPH_FWD_TILE
    return launch_status();
  }
  dim3 grid(cdiv(npix, 256), (unsigned)B);
  const size_t smem = sizeof(T) * (size_t)M * kSmallJ;
#define SPH_SMALL_FWD(W)                                                                                              \
  small_fwd_kernel<T, INTERP, W><<<grid, 256, smem, st>>>((const T *)src, (const T *)map, (const T *)iw, (const T *)wgt, sm, \
                                                          sc, sk, (const T *)bias, (T *)out, (int)CH, (int)K, (int)P,   \
                                                          (int)SH, (int)SW, (int)npix, (int)M, relu_out ? 1 : 0)
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0) SPH_SMALL_FWD(true);
    else SPH_SMALL_FWD(false);
  });
#undef SPH_SMALL_FWD
  return launch_status();
}

template <typename T, int R4>
static void launch_premul(const void *src, const void *wgt, int64_t sm, int64_t sc, int64_t sk, void *ws, int64_t CH, int64_t K,
                          int64_t M, int64_t n_src, int64_t B, cudaStream_t st) {
  const size_t smem = sizeof(T) * (size_t)(CH + 256) * 4 * R4;  // weights + one staged row per thread
  cudaFuncSetAttribute(small_premul_kernel<T, R4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  small_premul_kernel<T, R4><<<dim3(cdiv(n_src, 512), (unsigned)B), 256, smem, st>>>(
      (const T *)src, (const T *)wgt, sm, sc, sk, (T *)ws, (int)CH, (int)K, (int)M, (int)n_src);
}

template <typename T>
int small_adjoint(const void *src, const void *plan, int64_t CH, int64_t n_src, int64_t K, int64_t n_dst, const void *wgt,
                  int64_t sm, int64_t sc, int64_t sk, const void *bias, void *out, int64_t M, int64_t B, void *ws,
                  size_t ws_bytes, cudaStream_t st) {
  if (!ws || ws_bytes < small_premul_workspace(B, M, K, n_src, sizeof(T))) return SPH_ERR_WORKSPACE_TOO_SMALL;
  const int r4 = small_row((int)M, (int)K) / 4;
  switch (r4) {
#define SPH_PREMUL_CASE(N) case N: launch_premul<T, N>(src, wgt, sm, sc, sk, ws, CH, K, M, n_src, B, st); break;
    SPH_PREMUL_CASE(1) SPH_PREMUL_CASE(2) SPH_PREMUL_CASE(3) SPH_PREMUL_CASE(4) SPH_PREMUL_CASE(5) SPH_PREMUL_CASE(6)
    SPH_PREMUL_CASE(7) SPH_PREMUL_CASE(8) SPH_PREMUL_CASE(9) SPH_PREMUL_CASE(10) SPH_PREMUL_CASE(11) SPH_PREMUL_CASE(12)
#undef SPH_PREMUL_CASE
    default: return SPH_ERR_INVALID_ARGUMENT;
  }
  const dim3 grid(cdiv(n_dst, 256), cdiv(B, kGatherImages));
  const int mq = small_mq((int)M);
#define SPH_GATHER(VM)                                                                                                   \
  small_plan_gather_kernel<T, VM><<<grid, 256, 0, st>>>((const T *)ws, plan, (const T *)bias, (T *)out, (int)K, (int)M,     \
                                                        (int)n_src, (int)n_dst, (int)B)
  if (mq == 1) SPH_GATHER(1);
  else if (mq == 2) SPH_GATHER(2);
  else SPH_GATHER(4);
#undef SPH_GATHER
  return launch_status(2);
}

template <typename T>
int small_dw(const void *A, const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K,
             int64_t P, int64_t npix, int interp, int64_t M, int64_t B, void *gw, int64_t sm, int64_t sc, int64_t sk,
             const void *gbias_src, int64_t Cbias, int64_t nbias, void *gb, void *ws, size_t ws_bytes, cudaStream_t st) {
  if (!ws || ws_bytes < small_dw_workspace(B, npix, M, CH, K, Cbias, sizeof(T))) return SPH_ERR_WORKSPACE_TOO_SMALL;
  const int splits = small_dw_splits(B, npix, M, sizeof(T));
  T *partial = (T *)ws;
  T *bias_partial = (T *)((char *)ws + align_up(sizeof(T) * (size_t)(kSdwParts * splits * M * CH * K), 256));
  void *bias_ws = (char *)bias_partial + align_up(sizeof(T) * (size_t)(kSdwParts * splits * M), 256);
  // conv dW: the tensor whose rows are staged is also the one whose channel sums give the bias gradient
  const bool fuse_bias = gbias_src == A && Cbias == M && nbias == npix && CH * K < kSmallJ;
  dim3 grid(splits, cdiv(M, 64));
  // tap cache of one pixel step (unweighted maps only)
  const size_t tap_smem = P > 0 ? 0 : (size_t)K * SdwPix<T>::value * sizeof(SdwTaps<T>);
#define SPH_SMALL_DW(W)                                                                                                  \
  do {                                                                                                                   \
    cudaFuncSetAttribute(small_dw_kernel<T, INTERP, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tap_smem);      \
    small_dw_kernel<T, INTERP, W><<<grid, kSdwThreads, tap_smem, st>>>((const T *)A, (const T *)src, (const T *)map,              \
                                                               (const T *)iw, (int)CH, (int)K, (int)P, (int)SH, (int)SW,  \
                                                               (int)npix, (int)M, (int)B, partial,                       \
                                                               fuse_bias ? bias_partial : nullptr);                      \
  } while (0)
  SPH_DISPATCH_INTERP(interp, {
    if (P > 0) SPH_SMALL_DW(true);
    else SPH_SMALL_DW(false);
  });
#undef SPH_SMALL_DW
  const int rc = simt_dw_reduce<T>(partial, kSdwParts * splits, M, CH * K, K, sm, sc, sk, gw, st);
  if (rc != SPH_OK) return rc;
  note_launches(1);
  if (fuse_bias) return simt_dw_reduce<T>(bias_partial, kSdwParts * splits, M, 1, 1, 1, 0, 0, gb, st);
  return simt_bias_grad<T>(gbias_src, B, Cbias, nbias, gb, bias_ws, st);
}

#define SPH_INSTANTIATE_SMALL(T)                                                                                          \
  template int small_fwd<T>(const void *, const void *, const void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, \
                            int, const void *, int64_t, int64_t, int64_t, const void *, void *, int64_t, int64_t,          \
                            cudaStream_t, bool, void *);                                                                           \
  template int small_adjoint<T>(const void *, const void *, int64_t, int64_t, int64_t, int64_t, const void *, int64_t,     \
                                int64_t, int64_t, const void *, void *, int64_t, int64_t, void *, size_t, cudaStream_t);   \
  template int small_dw<T>(const void *, const void *, const void *, const void *, int64_t, int64_t, int64_t, int64_t,     \
                           int64_t, int64_t, int, int64_t, int64_t, void *, int64_t, int64_t, int64_t, const void *,       \
                           int64_t, int64_t, void *, void *, size_t, cudaStream_t);
SPH_INSTANTIATE_SMALL(float)
SPH_INSTANTIATE_SMALL(double)

}  // namespace sph

SPH_TU_STATUS(conv_small)
