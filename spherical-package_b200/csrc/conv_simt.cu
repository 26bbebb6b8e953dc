// Exact-arithmetic (float32 / float64, SIMT) mapped convolution family.
//
// Every operator of the family is one of two fused kernels, neither of which
// materialises the column buffer the reference builds per image
// (src/cpp/mapped_convolution_layer.cpp:24-45):
//
//   conv_gemm_kernel   Out[b,m,pix] = sum_{ch,k} Wgt[m,ch,k] * Col[b,ch,k,pix] (+ bias[m])
//   conv_dw_kernel     dW[m,ch,k]   = sum_{b,pix} A[b,m,pix] * Col[b,ch,k,pix]
//
// where Col is produced on the fly, either straight from the sample map
// (mapped_im2col, common/mapped_im2col.h:11-41, 80-116) or, for the adjoint
// direction (mapped_col2im, :44-77, 119-158), from a scatter plan:
//
//   forward            Col = im2col(x),      Wgt = W  (Cout,Cin,K)      m = co, ch = c
//   backward_input     Col = plan(gout),     Wgt = W  read transposed   m = c,  ch = co
//   tconv forward      Col = plan(x),        Wgt = Wt (Cin,Cout,K) tr.  m = co, ch = ci
//   tconv backward_in  Col = im2col(gout),   Wgt = Wt                   m = ci, ch = co
//   (t)conv backward_weight: A = gout (conv) or x (tconv), Col = im2col(x) or im2col(gout)
#include "common.cuh"
#include "conv_internal.h"

namespace sph {

constexpr int COL_PLAN = 3;   // column source: scatter plan (modes 0..2 are the interpolation types)
constexpr int COL_IDENT = 4;  // the pixel itself (K = 1): a dense product over the source grid

template <typename T> struct ColSrc {
  const T *src;      // (B, CH, SH*SW) tensor the columns are gathered from
  const T *map;      // direct modes
  const T *iw;
  const void *plan;  // plan mode
  int CH, SH, SW, K, P, npix;
};

template <typename T, int MODE, bool WEIGHTED>
__device__ __forceinline__ T col_value(const ColSrc<T> &s, const PlanView<T> &pv, const T *__restrict__ plane, int k,
                                       int pix) {
  if (MODE == COL_IDENT) return __ldg(plane + pix);
  if (MODE == COL_PLAN) {
    const int key = pix * s.K + k;
    const int e0 = __ldg(pv.offsets + key), e1 = __ldg(pv.offsets + key + 1);
    T acc = T(0);
    for (int e = e0; e < e1; e++) {
      const int sp = __ldg(pv.src + e);
      if (index_ok(sp, pv.n_src)) acc += __ldg(pv.w + e) * __ldg(plane + sp);
    }
    return acc;
  } else {
    const int PP = WEIGHTED ? s.P : 1;
    const size_t e = ((size_t)pix * s.K + k) * PP;
    return gather_slot<T, MODE >= COL_PLAN ? 0 : MODE, WEIGHTED>(plane, s.map + 2 * e, s.iw + e, s.P, s.SH, s.SW);
  }
}

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T, int MODE, bool WEIGHTED>
__global__ void __launch_bounds__(256)
conv_gemm_kernel(ColSrc<T> cs, const T *__restrict__ wgt, int64_t sm, int64_t sc, int64_t sk,
                 const T *__restrict__ bias, T *__restrict__ out, int M) {
  __shared__ T Ws[TK][TM + 1];
  __shared__ T Cs[TK][TN];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int b = blockIdx.z, m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int CHK = cs.CH * cs.K;
  const size_t shw = (size_t)cs.SH * cs.SW;
  PlanView<T> pv{};
  bool ok = true;
  if (MODE == COL_PLAN) pv = plan_view<T>(cs.plan, cs.npix * cs.K, ok);
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = T(0);

  for (int kk0 = 0; kk0 < CHK; kk0 += TK) {
    for (int e = tid; e < TK * TM; e += 256) {
      const int kl = e % TK, ml = e / TK, kk = kk0 + kl, m = m0 + ml;
      Ws[kl][ml] = (kk < CHK && m < M) ? __ldg(wgt + m * sm + (kk / cs.K) * sc + (kk % cs.K) * sk) : T(0);
    }
    for (int e = tid; e < TK * TN; e += 256) {
      const int nl = e % TN, kl = e / TN, kk = kk0 + kl, pix = n0 + nl;
      T v = T(0);
      if (ok && kk < CHK && pix < cs.npix)
        v = col_value<T, MODE, WEIGHTED>(cs, pv, cs.src + ((size_t)b * cs.CH + kk / cs.K) * shw, kk % cs.K, pix);
      Cs[kl][nl] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kl = 0; kl < TK; kl++) {
      T a[4], c[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = Ws[kl][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) c[j] = Cs[kl][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += a[i] * c[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
    const T bv = bias ? __ldg(bias + m) : T(0);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int pix = n0 + tx + 16 * j;
      if (pix < cs.npix) out[((size_t)b * M + m) * cs.npix + pix] = acc[i][j] + bv;
    }
  }
}

// The same operator for float32 with at least ~100 output rows: 128 x 128 output tile, 8 x 8 accumulators per thread
// read through 16-byte shared-memory loads, the next step's operands fetched into registers while the current step is
// multiplied, and the columns ordered slot-major (kk = k * CH + ch) so that a thread decodes a map entry once for all
// the channels it gathers with it.
constexpr int GM = 128, GN = 128, GK = 16;
__device__ __forceinline__ void gffma2(unsigned long long &d, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long gpack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void gunpack2(unsigned long long v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// RM = output rows per thread: 8 (128-row tile) or 4 (64-row tile, for operators with about 64 output rows).
template <int MODE, bool WEIGHTED, int RM>
__global__ void __launch_bounds__(256, 2)
conv_gemm128_kernel(ColSrc<float> cs, const float *__restrict__ wgt, int64_t sm, int64_t sc, int64_t sk,
                    const float *__restrict__ bias, float *__restrict__ out, int M, const float *__restrict__ wt) {
  constexpr int GMt = 16 * RM, kWPass = 256 / GMt, kWN = GK / kWPass;  // tile rows; weight rows per pass; passes
  __shared__ __align__(16) float Ws[GK][GMt];
  __shared__ __align__(16) float Cs[GK][GN];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int b = blockIdx.z, m0 = blockIdx.y * GMt, n0 = blockIdx.x * GN;
  const int CHK = cs.CH * cs.K;
  const size_t shw = (size_t)cs.SH * cs.SW;
  PlanView<float> pv{};
  bool ok = true;
  if (MODE == COL_PLAN) pv = plan_view<float>(cs.plan, cs.npix * cs.K, ok);
  const float *img = cs.src + (size_t)b * cs.CH * shw;
  // operand fetch: weights (row wl, kl = wr + kWPass * i), columns (pixel tid & 127, kl = 8 * (tid >> 7) + j)
  const int nl = tid & 127, half = tid >> 7, pix = n0 + nl;
  const int wl = tid % GMt, wr = tid / GMt;
  const bool pix_ok = ok && pix < cs.npix;
  float wreg[kWN], creg[8];
  auto fetch = [&](int kk0) {
#pragma unroll
    for (int i = 0; i < kWN; i++) {
      const int kk = kk0 + wr + kWPass * i, m = m0 + wl;
      float v = 0.0f;
      if (kk < CHK && m < M) {
        if (wt != nullptr) {  // transposed copy [kk][m]: neighbouring threads read neighbouring words
          v = __ldg(wt + (size_t)kk * M + m);
        } else {
          const int k = kk / cs.CH, ch = kk - k * cs.CH;
          v = __ldg(wgt + m * sm + ch * sc + k * sk);
        }
      }
      wreg[i] = v;
    }
    if constexpr (MODE == COL_IDENT) {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int ch = kk0 + half * 8 + j;
        creg[j] = (pix_ok && ch < CHK) ? __ldg(img + (size_t)ch * shw + pix) : 0.0f;
      }
      return;
    }
    if constexpr (MODE == COL_PLAN) {
      // the eight columns are consecutive channels; when they share their slot, the slot's plan entries are read once
      const int kk_first = kk0 + half * 8, k = kk_first / cs.CH, ch0 = kk_first - k * cs.CH;
      if (pix_ok && kk_first + 8 <= CHK && ch0 + 8 <= cs.CH) {
#pragma unroll
        for (int j = 0; j < 8; j++) creg[j] = 0.0f;
        const int key = pix * cs.K + k;
        const int e0 = __ldg(pv.offsets + key), e1 = __ldg(pv.offsets + key + 1);
        const float *plane0 = img + (size_t)ch0 * shw;
        // the first four entries' sources and weights are read together, then their 32 values (a dependent load per
        // entry, one after the other, would leave the chain of latencies exposed); longer segments continue one by one
        int sp4[4];
        float w4[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const bool in = e0 + i < e1;
          sp4[i] = in ? __ldg(pv.src + e0 + i) : -1;
          w4[i] = in ? __ldg(pv.w + e0 + i) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
          if (sp4[i] >= 0 && index_ok(sp4[i], pv.n_src)) {
#pragma unroll
            for (int j = 0; j < 8; j++) creg[j] += w4[i] * __ldg(plane0 + (size_t)j * shw + sp4[i]);
          }
        }
        for (int e = e0 + 4; e < e1; e++) {
          const int sp = __ldg(pv.src + e);
          if (!index_ok(sp, pv.n_src)) continue;
          const float w = __ldg(pv.w + e);
#pragma unroll
          for (int j = 0; j < 8; j++) creg[j] += w * __ldg(plane0 + (size_t)j * shw + sp);
        }
        return;
      }
    }
    if constexpr (MODE != COL_PLAN && !WEIGHTED) {
      // likewise through the map: one division and one decoded map entry for the eight channels
      const int kk_first = kk0 + half * 8, k = kk_first / cs.CH, ch0 = kk_first - k * cs.CH;
      if (pix_ok && kk_first + 8 <= CHK && ch0 + 8 <= cs.CH) {
        Taps<float> t8;
        const float *mp = cs.map + 2 * ((size_t)pix * cs.K + k);
        decode<float, MODE >= COL_PLAN ? 0 : MODE>(__ldg(mp), __ldg(mp + 1), cs.SH, cs.SW, t8);
        const float *plane0 = img + (size_t)ch0 * shw;
#pragma unroll
        for (int j = 0; j < 8; j++) creg[j] = gather<float, MODE >= COL_PLAN ? 0 : MODE>(plane0 + (size_t)j * shw, t8);
        return;
      }
    }
    if constexpr (MODE != COL_PLAN && WEIGHTED) {
      // weighted maps: the slot's P points are decoded once for the eight channels; per channel the sum runs over the
      // points in order, acc += w_q * interp_q with separate roundings (as gather_slot)
      const int kk_first = kk0 + half * 8, k = kk_first / cs.CH, ch0 = kk_first - k * cs.CH;
      if (pix_ok && kk_first + 8 <= CHK && ch0 + 8 <= cs.CH) {
        const size_t e = ((size_t)pix * cs.K + k) * cs.P;
        const float *plane0 = img + (size_t)ch0 * shw;
#pragma unroll
        for (int j = 0; j < 8; j++) creg[j] = 0.0f;
        for (int q = 0; q < cs.P; q++) {
          Taps<float> tq;
          decode<float, MODE >= COL_PLAN ? 0 : MODE>(__ldg(cs.map + 2 * (e + q)), __ldg(cs.map + 2 * (e + q) + 1), cs.SH, cs.SW, tq);
          const float wq = __ldg(cs.iw + e + q);
#pragma unroll
          for (int j = 0; j < 8; j++)
            creg[j] = __fadd_rn(creg[j], __fmul_rn(wq, gather<float, MODE >= COL_PLAN ? 0 : MODE>(plane0 + (size_t)j * shw, tq)));
        }
        return;
      }
    }
    int cur_k = -1;
    Taps<float> t;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int kk = kk0 + half * 8 + j;
      float v = 0.0f;
      if (pix_ok && kk < CHK) {
        const int k = kk / cs.CH, ch = kk - k * cs.CH;
        const float *plane = img + (size_t)ch * shw;
        if constexpr (MODE != COL_PLAN && !WEIGHTED) {
          if (k != cur_k) {
            const float *mp = cs.map + 2 * ((size_t)pix * cs.K + k);
            decode<float, MODE >= COL_PLAN ? 0 : MODE>(__ldg(mp), __ldg(mp + 1), cs.SH, cs.SW, t);
            cur_k = k;
          }
          v = gather<float, MODE >= COL_PLAN ? 0 : MODE>(plane, t);
        } else {
          v = col_value<float, MODE, WEIGHTED>(cs, pv, plane, k, pix);
        }
      }
      creg[j] = v;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int i = 0; i < kWN; i++) Ws[wr + kWPass * i][wl] = wreg[i];
#pragma unroll
    for (int j = 0; j < 8; j++) Cs[half * 8 + j][nl] = creg[j];
  };
  unsigned long long acc2[RM][4];  // RM rows x 4 pixel pairs, multiplied with packed float32 pair FMAs
#pragma unroll
  for (int i = 0; i < RM; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc2[i][j] = 0ull;

  fetch(0);
  stash();
  __syncthreads();
  for (int kk0 = 0; kk0 < CHK; kk0 += GK) {
    const bool more = kk0 + GK < CHK;
    if (more) fetch(kk0 + GK);  // in flight while this step is multiplied
#pragma unroll
    for (int kl = 0; kl < GK; kl++) {
      float a[RM];
#pragma unroll
      for (int i = 0; i < RM; i += 4) {
        const float4 av = *(const float4 *)&Ws[kl][ty * RM + i];
        a[i] = av.x; a[i + 1] = av.y; a[i + 2] = av.z; a[i + 3] = av.w;
      }
      const float4 c0 = *(const float4 *)&Cs[kl][tx * 4], c1 = *(const float4 *)&Cs[kl][64 + tx * 4];
      const unsigned long long c2[4] = {gpack2(c0.x, c0.y), gpack2(c0.z, c0.w), gpack2(c1.x, c1.y), gpack2(c1.z, c1.w)};
#pragma unroll
      for (int i = 0; i < RM; i++) {
        const unsigned long long aa = gpack2(a[i], a[i]);
#pragma unroll
        for (int j = 0; j < 4; j++) gffma2(acc2[i][j], aa, c2[j]);
      }
    }
    __syncthreads();
    if (more) {
      stash();
      __syncthreads();
    }
  }
  float acc[RM][8];
#pragma unroll
  for (int i = 0; i < RM; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) gunpack2(acc2[i][j], acc[i][2 * j], acc[i][2 * j + 1]);
  const bool vec = (cs.npix & 3) == 0 && (((uintptr_t)out) & 15) == 0;
#pragma unroll
  for (int i = 0; i < RM; i++) {
    const int m = m0 + ty * RM + i;
    if (m >= M) continue;
    const float bv = bias ? __ldg(bias + m) : 0.0f;
    float *row = out + ((size_t)b * M + m) * cs.npix;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int p0 = n0 + h * 64 + tx * 4;
      if (vec && p0 + 4 <= cs.npix) {
        *(float4 *)(row + p0) = make_float4(acc[i][4 * h] + bv, acc[i][4 * h + 1] + bv, acc[i][4 * h + 2] + bv, acc[i][4 * h + 3] + bv);
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
          if (p0 + j < cs.npix) row[p0 + j] = acc[i][4 * h + j] + bv;
      }
    }
  }
}

constexpr int kDwChunk = 256;  // pixels per split-K work unit

template <typename T, int MODE, bool WEIGHTED>
__global__ void __launch_bounds__(256)
conv_dw_kernel(ColSrc<T> cs, const T *__restrict__ A, int M, int B, T *__restrict__ partial) {
  __shared__ T As[16][TM + 1];
  __shared__ T Cs[16][TN + 1];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int kk0 = blockIdx.x * TN, m0 = blockIdx.y * TM, splits = gridDim.z;
  const int CHK = cs.CH * cs.K;
  const size_t shw = (size_t)cs.SH * cs.SW;
  const int chunks = (cs.npix + kDwChunk - 1) / kDwChunk;
  PlanView<T> pv{};
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = T(0);

  for (int unit = blockIdx.z; unit < B * chunks; unit += splits) {
    const int b = unit / chunks, pbase = (unit % chunks) * kDwChunk, pend = min(cs.npix, pbase + kDwChunk);
    for (int p0 = pbase; p0 < pend; p0 += 16) {
      for (int e = tid; e < 16 * TM; e += 256) {
        const int pl = e & 15, ml = e >> 4, pix = p0 + pl, m = m0 + ml;
        As[pl][ml] = (pix < pend && m < M) ? __ldg(A + ((size_t)b * M + m) * cs.npix + pix) : T(0);
      }
      for (int e = tid; e < 16 * TN; e += 256) {
        const int pl = e & 15, kl = e >> 4, pix = p0 + pl, kk = kk0 + kl;
        T v = T(0);
        if (pix < pend && kk < CHK)
          v = col_value<T, MODE, WEIGHTED>(cs, pv, cs.src + ((size_t)b * cs.CH + kk / cs.K) * shw, kk % cs.K, pix);
        Cs[pl][kl] = v;
      }
      __syncthreads();
#pragma unroll
      for (int pl = 0; pl < 16; pl++) {
        T a[4], c[4];
#pragma unroll
        for (int i = 0; i < 4; i++) a[i] = As[pl][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; j++) c[j] = Cs[pl][tx + 16 * j];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] += a[i] * c[j];
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int kk = kk0 + tx + 16 * j;
      if (kk < CHK) partial[((size_t)blockIdx.z * M + m) * CHK + kk] = acc[i][j];
    }
  }
}

// Weight gradient for float32 with at least 64 gathered channels: 128 rows x 128 columns per block, 8 x 8 accumulators
// per thread (packed pair multiply-adds), columns slot-major (kk = k * CH + ch).  A block's 128 columns lie in at most
// three slots, so the taps of a 16-pixel step are decoded once per (slot, pixel) into shared memory and every thread
// gathers its column's eight pixels with them; the next step's operands are fetched while the current one is
// multiplied.  partial[split][m][kk] in the same slot-major order (dw_reduce_kernel is told).
// WN: weighted nearest map with at most four points per slot - its value sum_q w_q x[tap_q], added in order, is the
// four-tap combine with the points in the taps' places.
constexpr int kDwSlots = 3;
template <int MODE, bool WN = false>
__global__ void __launch_bounds__(256, 2)
conv_dw128_kernel(ColSrc<float> cs, const float *__restrict__ A, int M, int B, float *__restrict__ partial) {
  __shared__ __align__(16) float As[GK][GM];
  __shared__ __align__(16) float Cs[GK][GN + 4];  // (padded: a thread stores eight columns of one pixel row)
  __shared__ int t_off[2][kDwSlots][GK][4];
  __shared__ float t_w[2][kDwSlots][GK][4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int kk0 = blockIdx.x * GN, m0 = blockIdx.y * GM, splits = gridDim.z;
  const int CHK = cs.CH * cs.K;
  const size_t shw = (size_t)cs.SH * cs.SW;
  const int chunks = (cs.npix + kDwChunk - 1) / kDwChunk;
  const int k_first = kk0 / cs.CH;                       // first slot of the block's columns
  // operand rows: gradient row cl, pixels half * 8 ..; columns: pixel gp of the step, the eight columns 8 * gc .. (a warp
  // reads 16 neighbouring pixels of two channels per load instruction, not 32 channels of one pixel)
  const int cl = tid & 127, half = tid >> 7;
  const int gp = tid & 15, gc = tid >> 4, kk_first = kk0 + gc * 8;
  const int ks0 = kk_first / cs.CH, ch_first = kk_first - ks0 * cs.CH;
  const bool cols_uniform = kk_first + 8 <= CHK && ch_first + 8 <= cs.CH;  // all eight exist and share their slot
  const bool a_ok = m0 + cl < M;
  const bool vec = (cs.npix & 3) == 0 && (((uintptr_t)A) & 15) == 0;
  unsigned long long acc2[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc2[i][j] = 0ull;
  float areg[8], creg[8];
  constexpr int TAPS = WN ? 4 : TapCount<MODE>::value;

  // Taps of the 16 pixels [p0, p0 + 16) for the block's slots (threads 0 .. 16 * kDwSlots - 1), in two parts: the map
  // coordinates (and point weights) are loaded a step early, so that between the two barriers of a step only the
  // arithmetic and the table stores remain.
  constexpr int NPT = WN ? 4 : 1;  // points per slot held in registers
  float cx[NPT], cy[NPT], cw[NPT];
  bool c_have = false;
  auto coords_load = [&](int p0, int pend) {
    c_have = false;
    if (tid < GK * kDwSlots) {
      const int pl = tid % GK, sl = tid / GK, pix = p0 + pl, k = k_first + sl;
      if (pix < pend && k < cs.K) {
        c_have = true;
        if constexpr (WN) {
          const size_t e = ((size_t)pix * cs.K + k) * cs.P;
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const bool in = q < cs.P;
            cx[q] = in ? __ldg(cs.map + 2 * (e + q)) : 0.0f;
            cy[q] = in ? __ldg(cs.map + 2 * (e + q) + 1) : 0.0f;
            cw[q] = in ? __ldg(cs.iw + e + q) : 0.0f;
          }
        } else {
          const float *mp = cs.map + 2 * ((size_t)pix * cs.K + k);
          cx[0] = __ldg(mp);
          cy[0] = __ldg(mp + 1);
          cw[0] = 1.0f;
        }
      }
    }
  };
  auto decode_store = [&](int buf) {
    if (tid < GK * kDwSlots) {
      const int pl = tid % GK, sl = tid / GK;
      Taps<float> t;
#pragma unroll
      for (int i = 0; i < 4; i++) { t.off[i] = -1; t.w[i] = 0.0f; }
      if (c_have) {
        if constexpr (WN) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            if (q < cs.P) {
              Taps<float> tq;
              decode<float, SPH_NEAREST>(cx[q], cy[q], cs.SH, cs.SW, tq);
              t.off[q] = tq.off[0];
              t.w[q] = cw[q];
            }
          }
        } else {
          decode<float, MODE>(cx[0], cy[0], cs.SH, cs.SW, t);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; i++) {
        t_off[buf][sl][pl][i] = (i < TAPS && t.off[i] >= 0 && index_ok(t.off[i], (long long)shw)) ? t.off[i] : -1;
        t_w[buf][sl][pl][i] = t.w[i];
      }
    }
  };
  // operands of the step whose taps are in table `buf`: A rows (row cl, pixels half * 8 ..) and this column's values
  auto fetch = [&](int buf, int b, int p0, int pend) {
    const float *arow = A + ((size_t)b * M + m0 + cl) * cs.npix + p0 + half * 8;
    if (a_ok && vec && p0 + half * 8 + 8 <= pend) {
      const float4 u = __ldg((const float4 *)arow), v = __ldg((const float4 *)arow + 1);
      areg[0] = u.x; areg[1] = u.y; areg[2] = u.z; areg[3] = u.w; areg[4] = v.x; areg[5] = v.y; areg[6] = v.z; areg[7] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) areg[j] = (a_ok && p0 + half * 8 + j < pend) ? __ldg(arow + j) : 0.0f;
    }
    auto value = [&](const float *plane, const int4 &o, const float4 &w) {
      const float v0 = o.x >= 0 ? __ldg(plane + o.x) : 0.0f;
      if constexpr (TAPS == 1) {
        return v0;
      } else {
        const float v1 = o.y >= 0 ? __ldg(plane + o.y) : 0.0f, v2 = o.z >= 0 ? __ldg(plane + o.z) : 0.0f;
        const float v3 = o.w >= 0 ? __ldg(plane + o.w) : 0.0f;
        // ((w0 v0 + w1 v1) + w2 v2) + w3 v3 with separate roundings, as the forward operator
        return __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(w.x, v0), __fmul_rn(w.y, v1)), __fmul_rn(w.z, v2)), __fmul_rn(w.w, v3));
      }
    };
    const float *img = cs.src + (size_t)b * cs.CH * shw;
    if (cols_uniform) {
      const int4 o = *(const int4 *)t_off[buf][ks0 - k_first][gp];
      const float4 w = *(const float4 *)t_w[buf][ks0 - k_first][gp];
#pragma unroll
      for (int j = 0; j < 8; j++) creg[j] = value(img + (size_t)(ch_first + j) * shw, o, w);
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int kk = kk_first + j;
        float v = 0.0f;
        if (kk < CHK) {
          const int k = kk / cs.CH, ch = kk - k * cs.CH;
          v = value(img + (size_t)ch * shw, *(const int4 *)t_off[buf][k - k_first][gp], *(const float4 *)t_w[buf][k - k_first][gp]);
        }
        creg[j] = v;
      }
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int j = 0; j < 8; j++) As[half * 8 + j][cl] = areg[j];
    *(float4 *)&Cs[gp][gc * 8] = make_float4(creg[0], creg[1], creg[2], creg[3]);
    *(float4 *)&Cs[gp][gc * 8 + 4] = make_float4(creg[4], creg[5], creg[6], creg[7]);
  };

  for (int unit = blockIdx.z; unit < B * chunks; unit += splits) {
    const int b = unit / chunks, pbase = (unit % chunks) * kDwChunk, pend = min(cs.npix, pbase + kDwChunk);
    int buf = 0;
    coords_load(pbase, pend);
    decode_store(0);
    __syncthreads();
    fetch(0, b, pbase, pend);
    if (pbase + GK < pend) coords_load(pbase + GK, pend);
    for (int p0 = pbase; p0 < pend; p0 += GK) {
      const bool more = p0 + GK < pend;
      __syncthreads();  // the previous step's tiles have been read
      stash();
      if (more) decode_store(buf ^ 1);  // (coordinates of step p0 + GK: loaded during the previous step)
      __syncthreads();
      if (more) {
        fetch(buf ^ 1, b, p0 + GK, pend);  // in flight while this step is multiplied
        if (p0 + 2 * GK < pend) coords_load(p0 + 2 * GK, pend);
      }
#pragma unroll
      for (int kl = 0; kl < GK; kl++) {
        const float4 a0 = *(const float4 *)&As[kl][ty * 8], a1 = *(const float4 *)&As[kl][ty * 8 + 4];
        const float4 c0 = *(const float4 *)&Cs[kl][tx * 4], c1 = *(const float4 *)&Cs[kl][64 + tx * 4];
        const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const unsigned long long c2[4] = {gpack2(c0.x, c0.y), gpack2(c0.z, c0.w), gpack2(c1.x, c1.y), gpack2(c1.z, c1.w)};
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const unsigned long long aa = gpack2(a[i], a[i]);
#pragma unroll
          for (int j = 0; j < 4; j++) gffma2(acc2[i][j], aa, c2[j]);
        }
      }
      buf ^= 1;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int m = m0 + ty * 8 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float lo, hi;
      gunpack2(acc2[i][j], lo, hi);
      const int c = kk0 + (j >> 1) * 64 + tx * 4 + (j & 1) * 2;
      float *dst = partial + ((size_t)blockIdx.z * M + m) * CHK + c;
      if (c < CHK) dst[0] = lo;
      if (c + 1 < CHK) dst[1] = hi;
    }
  }
}

// gw[m,ch,k] = sum over splits, in a fixed order (deterministic): 32 outputs per block, sixteen threads per
// output each summing every sixteenth split, then the sixteen sums in order.
constexpr int kReduceLanes = 16;
template <typename T>
__global__ void __launch_bounds__(32 * kReduceLanes) dw_reduce_kernel(const T *__restrict__ partial, int splits, int M, int CHK,
                                                                      int K, int64_t sm, int64_t sc, int64_t sk,
                                                                      T *__restrict__ gw, int slot_major = 0) {
  __shared__ T red[kReduceLanes][32];
  const int i = blockIdx.x * 32 + threadIdx.x, zl = threadIdx.y;
  const size_t n = (size_t)M * CHK;
  T s0 = T(0), s1 = T(0), s2 = T(0), s3 = T(0);
  if (i < M * CHK) {
    int z = zl;
    for (; z + 3 * kReduceLanes < splits; z += 4 * kReduceLanes) {
      s0 += partial[(size_t)z * n + i];
      s1 += partial[(size_t)(z + kReduceLanes) * n + i];
      s2 += partial[(size_t)(z + 2 * kReduceLanes) * n + i];
      s3 += partial[(size_t)(z + 3 * kReduceLanes) * n + i];
    }
    for (; z < splits; z += kReduceLanes) s0 += partial[(size_t)z * n + i];
  }
  red[zl][threadIdx.x] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (zl == 0 && i < M * CHK) {
    T s = red[0][threadIdx.x];
#pragma unroll
    for (int j = 1; j < kReduceLanes; j++) s += red[j][threadIdx.x];
    const int m = i / CHK, kk = i % CHK, CH = CHK / K;
    const int ch = slot_major ? kk % CH : kk / K, k = slot_major ? kk / CH : kk % K;
    gw[m * sm + ch * sc + k * sk] = s;
  }
}

// Bias gradient: sum of g over batch and pixels per channel, two fixed-order stages.
constexpr int kBiasSplits = 32;

template <typename T>
__global__ void __launch_bounds__(256) bias_partial_kernel(const T *__restrict__ g, int B, int C, int n, T *__restrict__ part) {
  __shared__ T red[256];
  const int c = blockIdx.x, s = blockIdx.y;
  const int64_t total = (int64_t)B * n, per = (total + kBiasSplits - 1) / kBiasSplits;
  const int64_t i0 = s * per, i1 = min(total, i0 + per);
  T acc = T(0);
  for (int64_t i = i0 + threadIdx.x; i < i1; i += 256) {
    const int64_t b = i / n, p = i % n;
    acc += __ldg(g + ((size_t)b * C + c) * n + p);
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int d = 128; d > 0; d >>= 1) {
    if (threadIdx.x < d) red[threadIdx.x] += red[threadIdx.x + d];
    __syncthreads();
  }
  if (threadIdx.x == 0) part[c * kBiasSplits + s] = red[0];
}

template <typename T>
__global__ void bias_final_kernel(const T *__restrict__ part, int C, T *__restrict__ gb) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  T s = T(0);
  for (int i = 0; i < kBiasSplits; i++) s += part[c * kBiasSplits + i];
  gb[c] = s;
}

template <typename T>
int simt_dw_reduce(const void *partial, int splits, int64_t M, int64_t CHK, int64_t K, int64_t sm, int64_t sc, int64_t sk,
                   void *gw, cudaStream_t st) {
  dw_reduce_kernel<T><<<cdiv(M * CHK, 32), dim3(32, kReduceLanes), 0, st>>>((const T *)partial, splits, (int)M, (int)CHK, (int)K, sm, sc, sk, (T *)gw);
  return launch_status();
}
template int simt_dw_reduce<float>(const void *, int, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, void *, cudaStream_t);
template int simt_dw_reduce<double>(const void *, int, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, void *, cudaStream_t);

size_t simt_bias_workspace(int64_t C, size_t ts) { return align_up(ts * (size_t)(C * kBiasSplits), 256); }

// gb[c] = sum over batch and pixels of g[b,c,:] (two fixed-order stages); ws holds C * kBiasSplits partials.
template <typename T>
int simt_bias_grad(const void *g, int64_t B, int64_t C, int64_t n, void *gb, void *ws, cudaStream_t st) {
  bias_partial_kernel<T><<<dim3((unsigned)C, kBiasSplits), 256, 0, st>>>((const T *)g, (int)B, (int)C, (int)n, (T *)ws);
  bias_final_kernel<T><<<cdiv(C, 128), 128, 0, st>>>((const T *)ws, (int)C, (T *)gb);
  return launch_status(2);
}
template int simt_bias_grad<float>(const void *, int64_t, int64_t, int64_t, void *, void *, cudaStream_t);
template int simt_bias_grad<double>(const void *, int64_t, int64_t, int64_t, void *, void *, cudaStream_t);

// big: the shape the 128 x 128 float32 kernel takes (fewer, larger tiles: more splits to fill the device)
static bool dw_big(int64_t M, int64_t CH, size_t ts) { return ts == 4 && M >= 48 && CH >= 64; }
static int dw_splits(int64_t B, int64_t npix, int64_t M, int64_t CHK, bool big) {
  const int64_t units = B * ((npix + kDwChunk - 1) / kDwChunk);
  const int64_t tn = big ? GN : TN, tm = big ? GM : TM;
  const int64_t tiles = ((CHK + tn - 1) / tn) * ((M + tm - 1) / tm);
  int64_t s = big ? (4 * 148) / tiles : (4 * 148 + tiles - 1) / tiles;  // (large tile: two blocks per SM, two full waves)
  if (s > 64) s = 64;
  if (s > units) s = units;
  if (s < 1) s = 1;
  return (int)s;
}

size_t simt_dw_workspace(int64_t B, int64_t npix, int64_t M, int64_t CH, int64_t K, int64_t Cbias, size_t ts) {
  const int64_t CHK = CH * K;
  return align_up(ts * (size_t)(dw_splits(B, npix, M, CHK, dw_big(M, CH, ts)) * M * CHK), 256) +
         align_up(ts * (size_t)(Cbias * kBiasSplits), 256);
}

// wt[kk][m] = w[m*sm + ch*sc + k*sk] with kk = k * CH + ch (the slot-major column order of conv_gemm128_kernel)
__global__ void weight_transpose_kernel(const float *__restrict__ w, float *__restrict__ wt, int M, int CH, int K, int64_t sm,
                                        int64_t sc, int64_t sk) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * CH * K) return;
  const int m = i % M, kk = i / M, k = kk / CH, ch = kk - k * CH;
  wt[i] = w[m * sm + ch * sc + k * sk];
}

size_t simt_gemm_workspace(int64_t M, int64_t CH, int64_t K, size_t ts);

// ---- multiply-first adjoint (float32) --------------------------------------------------------------------------
// When the destination grid of an adjoint is several times larger than its source grid (a down-sampling map), the
// gather form repeats the channel contraction for every destination pixel, most of whose (pixel, slot) keys are
// empty.  Contract first on the source grid - T[b][k*M + m][p] = sum_ch W[m, ch, k] src[b, ch, p], a dense product
// with the large-tile kernel - then gather planes of T through the plan (the reference's own order: GEMM, then
// mapped_col2im, src/cpp/mapped_convolution_layer.cpp:69-86).
// wt[ch][k*M + m] = w[m*sm + ch*sc + k*sk]: the transposed weight copy the dense product reads
__global__ void premul_weight_transpose_kernel(const float *__restrict__ w, float *__restrict__ wt, int M, int CH, int K, int64_t sm,
                                               int64_t sc, int64_t sk) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * CH * K) return;
  const int mm = i % (K * M), ch = i / (K * M), k = mm / M, m = mm - k * M;
  wt[i] = w[m * sm + ch * sc + k * sk];
}

// out[b][m][q] (+bias) = sum over the plan entries (p, k, w) of destination pixel q, in plan order, of w * T[b][k*M + m][p].
// Thread = destination pixel x 8 output rows: neighbouring pixels read neighbouring words of the same planes.
__global__ void __launch_bounds__(128) plan_gather_planes_kernel(const float *__restrict__ T, const void *__restrict__ plan_blob,
                                                                 const float *__restrict__ bias, float *__restrict__ out, int K, int M,
                                                                 int n_src, int n_dst) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x, m0 = blockIdx.y * 8, b = blockIdx.z;
  if (q >= n_dst) return;
  bool ok;
  const PlanView<float> pv = plan_view<float>(plan_blob, n_dst * K, ok);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; j++) acc[j] = 0.0f;
  if (ok) {
    int e1 = __ldg(pv.offsets + (size_t)q * K);
    for (int k = 0; k < K; k++) {
      const int e0 = e1;
      e1 = __ldg(pv.offsets + (size_t)q * K + k + 1);
      const float *tk = T + ((size_t)b * K * M + (size_t)k * M + m0) * n_src;
      for (int e = e0; e < e1; e++) {
        const int sp = __ldg(pv.src + e);
        if (!index_ok(sp, pv.n_src)) continue;
        const float w = __ldg(pv.w + e);
#pragma unroll
        for (int j = 0; j < 8; j++)
          if (m0 + j < M) acc[j] = fmaf(w, __ldg(tk + (size_t)j * n_src + sp), acc[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; j++)
    if (m0 + j < M) out[((size_t)b * M + m0 + j) * n_dst + q] = acc[j] + (bias ? __ldg(bias + m0 + j) : 0.0f);
}

static bool premul_applies(int64_t M, int64_t CH, int64_t K, int64_t n_src, int64_t n_dst, int64_t B) {
  return n_dst >= 3 * n_src && K * M >= 48 && CH >= 16 && (size_t)(B * K * M * n_src) * 4 <= ((size_t)8 << 30);
}

size_t simt_adjoint_workspace(int64_t B, int64_t M, int64_t CH, int64_t K, int64_t n_src, int64_t n_dst, size_t ts) {
  if (ts == 4 && premul_applies(M, CH, K, n_src, n_dst, B))
    return align_up((size_t)(M * CH * K) * 4, 256) + align_up((size_t)(B * K * M * n_src) * 4, 256);
  return simt_gemm_workspace(M, CH, K, ts);
}

size_t simt_gemm_workspace(int64_t M, int64_t CH, int64_t K, size_t ts) {
  return (ts == 4 && M >= 48) ? align_up((size_t)(M * CH * K) * 4, 256) : 0;
}

template <typename T, int MODE, bool WEIGHTED>
static void launch_gemm(const ColSrc<T> &cs, const T *wgt, int64_t sm, int64_t sc, int64_t sk, const T *bias, T *out, int M,
                        int B, cudaStream_t st, void *ws, size_t ws_bytes) {
  if constexpr (sizeof(T) == 4) {
    if (M >= 48) {  // (a half-empty tile still beats several passes of the small one over the same gathered columns)
      const float *wt = nullptr;
      if (ws != nullptr && ws_bytes >= simt_gemm_workspace(M, cs.CH, cs.K, 4) && (((uintptr_t)ws) & 3) == 0) {
        weight_transpose_kernel<<<cdiv((int64_t)M * cs.CH * cs.K, 256), 256, 0, st>>>(wgt, (float *)ws, M, cs.CH, cs.K, sm, sc, sk);
        note_launches(1);
        wt = (const float *)ws;
      }
      if (M % 128 > 0 && M % 128 <= 64) {  // (the last row block would be at most half full: 64-row tiles)
        dim3 grid64(cdiv(cs.npix, GN), cdiv(M, 64), B);
        conv_gemm128_kernel<MODE, WEIGHTED, 4><<<grid64, 256, 0, st>>>(cs, wgt, sm, sc, sk, bias, out, M, wt);
      } else {
        dim3 grid128(cdiv(cs.npix, GN), cdiv(M, GM), B);
        conv_gemm128_kernel<MODE, WEIGHTED, 8><<<grid128, 256, 0, st>>>(cs, wgt, sm, sc, sk, bias, out, M, wt);
      }
      return;
    }
  }
  dim3 grid(cdiv(cs.npix, TN), cdiv(M, TM), B);
  conv_gemm_kernel<T, MODE, WEIGHTED><<<grid, 256, 0, st>>>(cs, wgt, sm, sc, sk, bias, out, M);
}

// Out[b,m,pix] (+bias) with columns gathered through the map (mode = interp) or through a plan.
template <typename T>
int simt_gemm(bool use_plan, const void *src, const void *map, const void *iw, const void *plan, int64_t CH, int64_t SH,
              int64_t SW, int64_t K, int64_t P, int64_t npix, int interp, const void *wgt, int64_t sm, int64_t sc,
              int64_t sk, const void *bias, void *out, int64_t M, int64_t B, cudaStream_t st, void *ws, size_t ws_bytes) {
  ColSrc<T> cs{(const T *)src, (const T *)map, (const T *)iw, plan, (int)CH, (int)SH, (int)SW, (int)K, (int)P, (int)npix};
  if constexpr (sizeof(T) == 4) {
    const int64_t n_src = SH * SW;
    if (use_plan && premul_applies(M, CH, K, n_src, npix, B) && ws != nullptr && (((uintptr_t)ws) & 15) == 0 &&
        ws_bytes >= simt_adjoint_workspace(B, M, CH, K, n_src, npix, 4)) {
      float *wt = (float *)ws, *Tb = (float *)((char *)ws + align_up((size_t)(M * CH * K) * 4, 256));
      premul_weight_transpose_kernel<<<cdiv(M * CH * K, 256), 256, 0, st>>>((const float *)wgt, wt, (int)M, (int)CH, (int)K, sm, sc, sk);
      ColSrc<float> ci{(const float *)src, nullptr, nullptr, nullptr, (int)CH, (int)SH, (int)SW, 1, 0, (int)n_src};
      const int MM = (int)(K * M);
      if (MM % 128 > 0 && MM % 128 <= 64) {
        conv_gemm128_kernel<COL_IDENT, false, 4><<<dim3(cdiv(n_src, GN), cdiv(MM, 64), (unsigned)B), 256, 0, st>>>(ci, nullptr, 0, 0, 0, nullptr, Tb, MM, wt);
      } else {
        conv_gemm128_kernel<COL_IDENT, false, 8><<<dim3(cdiv(n_src, GN), cdiv(MM, GM), (unsigned)B), 256, 0, st>>>(ci, nullptr, 0, 0, 0, nullptr, Tb, MM, wt);
      }
      plan_gather_planes_kernel<<<dim3(cdiv(npix, 128), cdiv(M, 8), (unsigned)B), 128, 0, st>>>(Tb, plan, (const float *)bias, (float *)out,
                                                                                              (int)K, (int)M, (int)n_src, (int)npix);
      return launch_status(3);
    }
  }
  if (use_plan) {
    launch_gemm<T, COL_PLAN, false>(cs, (const T *)wgt, sm, sc, sk, (const T *)bias, (T *)out, (int)M, (int)B, st, ws, ws_bytes);
  } else {
    SPH_DISPATCH_INTERP(interp, {
      if (P > 0) launch_gemm<T, INTERP, true>(cs, (const T *)wgt, sm, sc, sk, (const T *)bias, (T *)out, (int)M, (int)B, st, ws, ws_bytes);
      else launch_gemm<T, INTERP, false>(cs, (const T *)wgt, sm, sc, sk, (const T *)bias, (T *)out, (int)M, (int)B, st, ws, ws_bytes);
    });
  }
  return launch_status();
}

// gw[m,ch,k] = sum_{b,pix} A[b,m,pix] * im2col(src)[b,ch,k,pix];  gb[c] = sum gbias_src[b,c,:]
template <typename T>
int simt_dw(const void *A, const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K,
            int64_t P, int64_t npix, int interp, int64_t M, int64_t B, void *gw, int64_t sm, int64_t sc, int64_t sk,
            const void *gbias_src, int64_t Cbias, int64_t nbias, void *gb, void *ws, size_t ws_bytes, cudaStream_t st) {
  const int64_t CHK = CH * K;
  const int splits = dw_splits(B, npix, M, CHK, dw_big(M, CH, sizeof(T)));
  if (ws_bytes < simt_dw_workspace(B, npix, M, CH, K, Cbias, sizeof(T)) || !ws) return SPH_ERR_WORKSPACE_TOO_SMALL;
  T *partial = (T *)ws;
  T *bpart = (T *)((char *)ws + align_up(sizeof(T) * (size_t)(splits * M * CHK), 256));
  ColSrc<T> cs{(const T *)src, (const T *)map, (const T *)iw, nullptr, (int)CH, (int)SH, (int)SW, (int)K, (int)P, (int)npix};
  int slot_major = 0;
  if constexpr (sizeof(T) == 4) {
    // the large tile: unweighted maps, enough rows to fill it, and so many channels that a block's columns lie in at
    // most kDwSlots slots
    const bool weighted_nearest = P > 0 && P <= 4 && interp == SPH_NEAREST;
    if ((P == 0 || weighted_nearest) && dw_big(M, CH, sizeof(T))) {
      slot_major = 1;
      dim3 grid128(cdiv(CHK, GN), cdiv(M, GM), splits);
      if (weighted_nearest)
        conv_dw128_kernel<SPH_NEAREST, true><<<grid128, 256, 0, st>>>(cs, (const float *)A, (int)M, (int)B, (float *)partial);
      else
        SPH_DISPATCH_INTERP(interp, (conv_dw128_kernel<INTERP><<<grid128, 256, 0, st>>>(cs, (const float *)A, (int)M, (int)B, (float *)partial)));
    }
  }
  if (!slot_major) {
    dim3 grid(cdiv(CHK, TN), cdiv(M, TM), splits);
    SPH_DISPATCH_INTERP(interp, {
      if (P > 0) conv_dw_kernel<T, INTERP, true><<<grid, 256, 0, st>>>(cs, (const T *)A, (int)M, (int)B, partial);
      else conv_dw_kernel<T, INTERP, false><<<grid, 256, 0, st>>>(cs, (const T *)A, (int)M, (int)B, partial);
    });
  }
  dw_reduce_kernel<T><<<cdiv(M * CHK, 32), dim3(32, kReduceLanes), 0, st>>>(partial, splits, (int)M, (int)CHK, (int)K, sm, sc, sk, (T *)gw,
                                                                           slot_major);
  bias_partial_kernel<T><<<dim3((unsigned)Cbias, kBiasSplits), 256, 0, st>>>((const T *)gbias_src, (int)B, (int)Cbias, (int)nbias, bpart);
  bias_final_kernel<T><<<cdiv(Cbias, 128), 128, 0, st>>>(bpart, (int)Cbias, (T *)gb);
  return launch_status(4);
}

template int simt_gemm<float>(bool, const void *, const void *, const void *, const void *, int64_t, int64_t, int64_t, int64_t,
                              int64_t, int64_t, int, const void *, int64_t, int64_t, int64_t, const void *, void *, int64_t,
                              int64_t, cudaStream_t, void *, size_t);
template int simt_gemm<double>(bool, const void *, const void *, const void *, const void *, int64_t, int64_t, int64_t, int64_t,
                               int64_t, int64_t, int, const void *, int64_t, int64_t, int64_t, const void *, void *, int64_t,
                               int64_t, cudaStream_t, void *, size_t);
template int simt_dw<float>(const void *, const void *, const void *, const void *, int64_t, int64_t, int64_t, int64_t, int64_t,
                            int64_t, int, int64_t, int64_t, void *, int64_t, int64_t, int64_t, const void *, int64_t, int64_t,
                            void *, void *, size_t, cudaStream_t);
template int simt_dw<double>(const void *, const void *, const void *, const void *, int64_t, int64_t, int64_t, int64_t, int64_t,
                             int64_t, int, int64_t, int64_t, void *, int64_t, int64_t, int64_t, const void *, int64_t, int64_t,
                             void *, void *, size_t, cudaStream_t);

}  // namespace sph

SPH_TU_STATUS(conv_simt)
