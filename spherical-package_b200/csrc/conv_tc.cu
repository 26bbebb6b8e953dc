// bf16 tensor-core path of the mapped convolution family (float32 tensors,
// bf16 operands, fp32 accumulation in tensor memory).
//
// Two persistent, warp-specialised kernels cover the six operators:
//
//   tc_gemm_kernel   Out[b, n, pix] = sum_j Col[b, pix, j] * Wt[n, j]  (+ bias[n])
//                    conv forward, conv dInput (through a scatter plan), transposed conv forward (plan) and
//                    transposed conv dInput.  128 pixels (an 8x16 block of the output grid) per tile.
//   tc_dw_kernel     dW[n, j] = sum_{b, pix} G[b, n, pix] * Col[b, pix, j]
//                    weight gradients; split over pixel ranges, partial sums reduced in a fixed order.
//
// j runs over (slot, channel) pairs of the sample map.  Col is never written
// to HBM: eight producer warps gather it (through the sample map's taps, or
// through a scatter plan for the adjoint direction) from a channels-last bf16
// copy of the source image straight into the 128-byte-swizzled shared-memory
// layout tcgen05.mma reads; the other operand (weights, or the gradient tile
// image) arrives by bulk async copies from a pre-swizzled bf16 image; one
// thread issues the MMAs into TMEM; four epilogue warps drain TMEM.  The
// reference does the same work per image as im2col kernel + cuBLAS SGEMM + bias
// kernel with a (Cin*K, OH*OW) column buffer in HBM
// (src/cuda/mapped_convolution_layer.cu:16-193).
#include <cuda.h>
#include <string.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "conv_internal.h"
#include "tc_common.cuh"

namespace sph {

// Channels of the channels-last bf16 copies: padded to a multiple of 8 that divides 64, or to a multiple of 64.
int padded_channels(int64_t CH) {
  int cp = (int)align_up((size_t)CH, 8);
  if (cp > 64) return (int)align_up((size_t)CH, 64);
  while (64 % cp) cp += 8;  // a 16-byte vector never straddles two slots and whole slots tile a chunk
  return cp;
}

namespace {

using namespace tc;

constexpr int kChunk = 64;  // GEMM columns per 128-byte swizzle row
constexpr int kTW = 16;     // pixel tiles are kTW wide; 8 rows (forward-type) or 4 rows (weight gradient)
constexpr int kEpilogueWarps = 4, kProducerWarps = 16;
constexpr int kProducerThreads = 32 * kProducerWarps;
constexpr int kThreads = 32 * (kEpilogueWarps + 1 + kProducerWarps);
constexpr int kFirstProducerThread = 32 * (kEpilogueWarps + 1);
constexpr int kSmemLimit = 227 * 1024;
constexpr int kTmemCols = 512;

enum { MODE_DIRECT = 0, MODE_PLAN = 1 };

// Sticky per-device record of a bounded wait that gave up in any kernel of this file (the kernels also write 1 into
// the first word of the call's workspace); read and cleared by sph_device_status().
__device__ int g_wait_status;

// Developer aid (-DSPH_TC_TIMING): cycles one thread of every role of tc_gemm_kernel spends in each phase, summed
// over all CTAs; read with sph_debug_tc_timing().
#ifdef SPH_TC_TIMING
__device__ unsigned long long g_tc_timing[16];
#define TC_TIC(var) const long long var = clock64()
#define TC_TOC(var, slot) atomicAdd(&g_tc_timing[slot], (unsigned long long)(clock64() - var))
#define TC_COUNT(slot) atomicAdd(&g_tc_timing[slot], 1ull)
#else
#define TC_TIC(var)
#define TC_TOC(var, slot)
#define TC_COUNT(slot)
#endif

// ---- column <-> (slot, channel) mapping -------------------------------------------------------
// Channels are padded to Cp (a multiple of 8 that divides 64, or a multiple of 64).  With Cp >= 64 a chunk
// is 64 channels of one slot and chunks are ordered channel-block major, slot minor, so that consecutive
// chunks re-read the same input neighbourhood; with Cp < 64 a chunk holds 64 / Cp whole slots.
__host__ __device__ inline int num_chunks(int Cp, int K) { return Cp >= 64 ? (Cp / 64) * K : (K * Cp + 63) / 64; }
__host__ __device__ inline void chunk_vec(int Cp, int K, int chunk, int v, int &slot, int &c0) {
  if (Cp >= 64) {
    const int cc = chunk / K;
    slot = chunk - cc * K;
    c0 = cc * 64 + v * 8;
  } else {
    const int q = chunk * 64 + v * 8;
    slot = q / Cp;  // >= K for padding columns
    c0 = q - slot * Cp;
  }
}

struct Gather {
  const __nv_bfloat16 *xh;  // (B, SH*SW + 1, Cp) channels-last bf16 source; the extra last pixel of every image is zero
  const float *map, *iw;    // direct mode: sample map (+ interpolation weights) over the (GH, GW) pixel grid
  const void *plan;         // plan mode: keyed by (pixel of the (GH, GW) grid) * K + slot
  int Cp, SH, SW, K, P, GH, GW, interp, nt;
};

// Gathered columns are accumulated over the taps with packed bf16x2 FMAs (one rounding per tap) by default;
// building with -DSPH_TC_GATHER_FP32 accumulates in fp32 and rounds once.
#ifdef SPH_TC_GATHER_FP32
constexpr bool kAcc32 = true;
#else
constexpr bool kAcc32 = false;
#endif

// Pipeline position kept without division: stage index and phase bit advance together.
struct Ring {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next(int stages) {
    if (++s == stages) { s = 0; ph ^= 1u; }
  }
};

__device__ __forceinline__ void producer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory"); }

// One tap-table entry: byte offset of the source pixel inside its image and the tap weight (fp32 bits, or the
// weight twice as bf16x2).  Unused entries point at the image's zero pixel with weight 0.
struct __align__(8) Tap {
  int off;
  uint32_t w;
};

__device__ __forceinline__ uint32_t tap_weight(float w) {
  return kAcc32 ? __float_as_uint(w) : pack_bf16(w, w);
}

// Taps of map slot (pix, slot) into nt table entries.
template <int INTERP>
__device__ __forceinline__ void fill_taps(const Gather &g, int pix, int slot, Tap *dst) {
  const int PP = g.P > 0 ? g.P : 1;
  const size_t e0 = ((size_t)pix * g.K + slot) * PP;
  const int zero_off = g.SH * g.SW * g.Cp * 2, pitch = g.Cp * 2;
  Taps<float> t;
  int n = 0;
  for (int q = 0; q < PP; q++) {
    decode<float, INTERP>(__ldg(g.map + 2 * (e0 + q)), __ldg(g.map + 2 * (e0 + q) + 1), g.SH, g.SW, t);
    const float wq = g.P > 0 ? __ldg(g.iw + e0 + q) : 1.0f;
#pragma unroll
    for (int i = 0; i < TapCount<INTERP>::value; i++, n++) {
      const bool ok = t.off[i] >= 0;
      dst[n].off = ok ? t.off[i] * pitch : zero_off;
      dst[n].w = tap_weight(ok ? wq * t.w[i] : 0.0f);
    }
  }
}

__device__ __forceinline__ void fill_taps_any(const Gather &g, int pix, int slot, Tap *dst) {
  if (g.map == nullptr) {  // identity gather (dense GEMM over the source grid): one tap, the pixel itself
    dst[0].off = pix * g.Cp * 2;
    dst[0].w = tap_weight(1.0f);
    return;
  }
  SPH_DISPATCH_INTERP(g.interp, fill_taps<INTERP>(g, pix, slot, dst));
}

__device__ __forceinline__ void fill_taps_zero(const Gather &g, Tap *dst) {
  const int zero_off = g.SH * g.SW * g.Cp * 2;
  for (int i = 0; i < g.nt; i++) { dst[i].off = zero_off; dst[i].w = 0u; }
}

// Taps of one unweighted map coordinate (x, y) that is already in registers (P == 0); NT = 1 decodes nearest,
// NT = 4 bilinear or bispherical.  Same entries as fill_taps writes.
template <int NT>
__device__ __forceinline__ void taps_from_xy(const Gather &g, float x, float y, Tap (&dst)[NT]) {
  const int zero_off = g.SH * g.SW * g.Cp * 2, pitch = g.Cp * 2;
  Taps<float> t;
  if (NT == 1) decode<float, SPH_NEAREST>(x, y, g.SH, g.SW, t);
  else if (g.interp == SPH_BISPHERICAL) decode<float, SPH_BISPHERICAL>(x, y, g.SH, g.SW, t);
  else decode<float, SPH_BILINEAR>(x, y, g.SH, g.SW, t);
#pragma unroll
  for (int i = 0; i < NT; i++) {
    const bool ok = t.off[i] >= 0;
    dst[i].off = ok ? t.off[i] * pitch : zero_off;
    dst[i].w = tap_weight(ok ? t.w[i] : 0.0f);
  }
}

// Accumulator of 8 channels: four bf16x2 registers, or eight floats.
struct Acc8 {
  uint32_t h[4];
  float f[8];
};
__device__ __forceinline__ void acc_zero(Acc8 &a) {
  if (kAcc32) {
#pragma unroll
    for (int i = 0; i < 8; i++) a.f[i] = 0.0f;
  } else {
#pragma unroll
    for (int i = 0; i < 4; i++) a.h[i] = 0u;
  }
}
__device__ __forceinline__ uint32_t hfma2_bf16(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ void acc_fma(Acc8 &a, uint32_t w, const uint4 &q) {
  if (kAcc32) {
    const float wf = __uint_as_float(w);
    a.f[0] = fmaf(wf, bf16_lo(q.x), a.f[0]);
    a.f[1] = fmaf(wf, bf16_hi(q.x), a.f[1]);
    a.f[2] = fmaf(wf, bf16_lo(q.y), a.f[2]);
    a.f[3] = fmaf(wf, bf16_hi(q.y), a.f[3]);
    a.f[4] = fmaf(wf, bf16_lo(q.z), a.f[4]);
    a.f[5] = fmaf(wf, bf16_hi(q.z), a.f[5]);
    a.f[6] = fmaf(wf, bf16_lo(q.w), a.f[6]);
    a.f[7] = fmaf(wf, bf16_hi(q.w), a.f[7]);
  } else {
    a.h[0] = hfma2_bf16(w, q.x, a.h[0]);
    a.h[1] = hfma2_bf16(w, q.y, a.h[1]);
    a.h[2] = hfma2_bf16(w, q.z, a.h[2]);
    a.h[3] = hfma2_bf16(w, q.w, a.h[3]);
  }
}
__device__ __forceinline__ uint4 acc_pack(const Acc8 &a) {
  if (kAcc32)
    return make_uint4(pack_bf16(a.f[0], a.f[1]), pack_bf16(a.f[2], a.f[3]), pack_bf16(a.f[4], a.f[5]), pack_bf16(a.f[6], a.f[7]));
  return make_uint4(a.h[0], a.h[1], a.h[2], a.h[3]);
}

__device__ __forceinline__ uint4 ldg16(const char *p) { return __ldg((const uint4 *)p); }

// Two (pixel, slot) items at once: the 2*NT 16-byte loads are issued before any is consumed.  `imgc` is the
// image base advanced to the item's first channel; t0/t1 point at the items' table rows.
template <int NT>
__device__ __forceinline__ void gather_pair(const char *__restrict__ imgc, const char *__restrict__ imgd,
                                            const Tap *__restrict__ t0, const Tap *__restrict__ t1, int nt, Acc8 &a0,
                                            Acc8 &a1) {
  if (NT > 0) {
    uint4 q0[NT > 0 ? NT : 1], q1[NT > 0 ? NT : 1];
    uint32_t w0[NT > 0 ? NT : 1], w1[NT > 0 ? NT : 1];
#pragma unroll
    for (int t = 0; t < NT; t++) {
      const Tap a = t0[t];
      w0[t] = a.w;
      q0[t] = ldg16(imgc + a.off);
    }
#pragma unroll
    for (int t = 0; t < NT; t++) {
      const Tap a = t1[t];
      w1[t] = a.w;
      q1[t] = ldg16(imgd + a.off);
    }
#pragma unroll
    for (int t = 0; t < NT; t++) acc_fma(a0, w0[t], q0[t]);
#pragma unroll
    for (int t = 0; t < NT; t++) acc_fma(a1, w1[t], q1[t]);
  } else {
    for (int t = 0; t < nt; t++) {
      const Tap a = t0[t], b = t1[t];
      const uint4 qa = ldg16(imgc + a.off), qb = ldg16(imgd + b.off);
      acc_fma(a0, a.w, qa);
      acc_fma(a1, b.w, qb);
    }
  }
}

// Plan entries [e0, e1) that did not fit the tap table, straight from the plan.
__device__ __forceinline__ void gather_plan_rest(Acc8 &acc, const char *__restrict__ imgc, const PlanView<float> &pv, int e0,
                                                 int e1, int pitch) {
  for (int e = e0; e < e1; e++) {
    const int sp = __ldg(pv.src + e);
    if (index_ok(sp, pv.n_src)) acc_fma(acc, tap_weight(__ldg(pv.w + e)), ldg16(imgc + (size_t)sp * pitch));
  }
}

// 32 bytes (two neighbouring 16-byte vectors) with one load; the address is 32-byte aligned.
__device__ __forceinline__ void ldg32(const char *p, uint4 &a, uint4 &b) {
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
               : "l"(p));
}

constexpr int kPlanTaps = 4;  // plan entries per (pixel, slot) kept in the shared tap table; the rest is read from the plan

// Pixel of local index l inside tile (ty, tx) of a (GH, GW) grid tiled TH x kTW; -1 if outside.
__device__ __forceinline__ int tile_pixel(int l, int ty, int tx, int TH, int GH, int GW) {
  const int y = ty * TH + (l >> 4), x = tx * kTW + (l & 15);
  return (y < GH && x < GW) ? y * GW + x : -1;
}

// =================================================================================================
// forward-type kernel
// =================================================================================================
constexpr int kTileM = 128, kTH = 8;
constexpr int kAStageBytes = kTileM * 128;
constexpr int kMaxTapBytes = 40 * 1024;

struct TcParams {
  Gather g;
  const __nv_bfloat16 *wp;  // weight tile images: [nblk][nchunks][Npb rows][64] bf16, 128B-swizzled
  const float *bias;        // (Nout) or null
  float *out;               // (B, Nout, GH*GW)
  __nv_bfloat16 *out_h;     // if set: write bf16 rows (B, GH*GW, out_pitch) instead (column buffer of the
  int out_pitch;            // multiply-first adjoint), no bias
  int *status;              // set to 1 if a bounded wait gave up
  int B, Nout, Npb, nblk, nchunks, tiles_x, tiles_y, stages;
  int use_out_map;          // outputs leave through the tensor map passed beside these parameters
  int relu;                 // clamp the outputs at zero (fused activation)
  __nv_bfloat16 *out_cl;    // if set: the outputs are also written as a channels-last bf16 copy (B, GH*GW + 1, cl_pitch)
  int cl_pitch;
};

struct Smem {
  uint8_t *A, *Bw;
  Tap *taps;
  int2 *rest;  // plan mode: [slot][pixel] range of plan entries beyond the table capacity
  uint64_t *full, *empty, *tfull, *tempty;
  uint32_t *tmem_ptr;
  volatile int *abort_flag;
  float *ostage;  // [4 epilogue warps][kOutStageCh channels][32 pixels] output rows on their way to memory
};

constexpr int kOutStageCh = 16;
constexpr int kClStageBytes = kEpilogueWarps * 32 * kOutStageCh * 2;  // channels-last copy: [warp][2 rows][16 px][16 ch] bf16
constexpr int kOutStageBytes = kEpilogueWarps * kOutStageCh * 32 * 4 + kClStageBytes;

inline size_t gemm_smem_bytes(int stages, int Npb, int K, int nt, bool direct) {
  size_t s = 1024;  // alignment slack
  s += (size_t)stages * (kAStageBytes + Npb * 128);
  s += (size_t)K * kTileM * nt * sizeof(Tap);
  if (!direct) s += (size_t)K * kTileM * sizeof(int2);
  s += 8 * (2 * stages + 4) + 16;
  s += kOutStageBytes + 128;
  return s;
}

__device__ inline Smem carve(uint8_t *raw, const TcParams &p, bool direct) {
  Smem s;
  uint8_t *b = (uint8_t *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  s.A = b;
  s.Bw = b + (size_t)p.stages * kAStageBytes;
  uint8_t *q = s.Bw + (size_t)p.stages * p.Npb * 128;
  s.taps = (Tap *)q;
  q += (size_t)p.g.K * kTileM * p.g.nt * sizeof(Tap);
  s.rest = (int2 *)q;
  q += direct ? 0 : (size_t)p.g.K * kTileM * sizeof(int2);
  s.full = (uint64_t *)q;
  s.empty = s.full + p.stages;
  s.tfull = s.empty + p.stages;
  s.tempty = s.tfull + 2;
  s.tmem_ptr = (uint32_t *)(s.tempty + 2);
  s.abort_flag = (volatile int *)(s.tmem_ptr + 1);
  s.ostage = (float *)(((uintptr_t)(s.abort_flag + 1) + 127) & ~(uintptr_t)127);  // tensor stores read 128-byte aligned rows
  return s;
}

constexpr int kRowStep = kProducerThreads / 8;  // pixel rows covered by one pass of all producer threads

// One producer thread's share of a 128-pixel x 64-column tile: 16-byte vector v = pt & 7 of pixels
// (pt >> 3) + kRowStep * r, two pixels at a time.  STRIDE = table entries per (pixel, slot) (0: g.nt),
// NTI = entries actually used (0: g.nt).
template <int STRIDE, int NTI, bool PLAN>
__device__ __forceinline__ void produce_chunk(const Gather &g, const Tap *taps, const int2 *rest, const PlanView<float> &pv,
                                              const char *img, int slot, int c0, int pt, uint8_t *As) {
  const int v = pt & 7, plb = pt >> 3;
  const int stride = STRIDE > 0 ? STRIDE : g.nt;
  const bool valid = slot < g.K;
  const char *imgc = img + c0 * 2;
  const int row0 = (valid ? slot : 0) * kTileM + plb;
  const Tap *trow = taps + (size_t)row0 * stride;
  uint8_t *dst = As + plb * 128 + ((v ^ (plb & 7)) << 4);
  static_assert(128 * 8 / kProducerThreads >= 2 && (128 * 8 / kProducerThreads) % 2 == 0, "items per thread must be even");
#pragma unroll
  for (int r = 0; r < 128 * 8 / kProducerThreads; r += 2) {
    Acc8 a0, a1;
    acc_zero(a0);
    acc_zero(a1);
    if (valid) {
      gather_pair<NTI>(imgc, imgc, trow + (size_t)(r * kRowStep) * stride, trow + (size_t)((r + 1) * kRowStep) * stride, g.nt, a0, a1);
      if (PLAN) {
        const int2 r0 = rest[row0 + r * kRowStep], r1 = rest[row0 + (r + 1) * kRowStep];
        if (r0.x < r0.y) gather_plan_rest(a0, imgc, pv, r0.x, r0.y, g.Cp * 2);
        if (r1.x < r1.y) gather_plan_rest(a1, imgc, pv, r1.x, r1.y, g.Cp * 2);
      }
    }
    *(uint4 *)(dst + r * kRowStep * 128) = acc_pack(a0);
    *(uint4 *)(dst + (r + 1) * kRowStep * 128) = acc_pack(a1);
  }
}

// The same share cut the other way, for Cp >= 16: thread = (pixel pt >> 2, vector pair pt & 3), i.e. one pixel and
// 32 bytes of it per thread.  What limits these kernels is the SM's 128-byte-per-cycle data path into the register
// file, which the gathered bytes share with the tap-table reads and the tensor core's operand reads; taking two
// vectors of one pixel instead of one vector of two pixels halves the tap bytes a thread reads per gathered byte
// (and the load instructions, with 32-byte loads).  c0 is the first channel of the pair.
template <int STRIDE, int NTI, bool PLAN>
__device__ __forceinline__ void produce_chunk_pair(const Gather &g, const Tap *taps, const int2 *rest, const PlanView<float> &pv,
                                                   const char *img, int slot, int c0, int pt, uint8_t *As) {
  static_assert(kProducerThreads == kTileM * 4, "one (pixel, vector pair) per producer thread");
  static_assert(STRIDE > 0 && NTI > 0, "static tap counts only");
  const int vp = pt & 3, pl = pt >> 2;
  const bool valid = slot < g.K;
  const char *imgc = img + c0 * 2;
  const int row = (valid ? slot : 0) * kTileM + pl;
  const Tap *trow = taps + (size_t)row * STRIDE;
  Acc8 a0, a1;
  acc_zero(a0);
  acc_zero(a1);
  if (valid) {
    uint4 qa[NTI], qb[NTI];
    uint32_t w[NTI];
#pragma unroll
    for (int t = 0; t < NTI; t++) {
      const Tap a = trow[t];
      w[t] = a.w;
      ldg32(imgc + a.off, qa[t], qb[t]);
    }
#pragma unroll
    for (int t = 0; t < NTI; t++) {
      acc_fma(a0, w[t], qa[t]);
      acc_fma(a1, w[t], qb[t]);
    }
    if (PLAN) {
      const int2 rr = rest[row];
      for (int e = rr.x; e < rr.y; e++) {
        uint4 xa, xb;
        const int sp = __ldg(pv.src + e);
        if (!index_ok(sp, pv.n_src)) continue;
        ldg32(imgc + (size_t)sp * (g.Cp * 2), xa, xb);
        const uint32_t we = tap_weight(__ldg(pv.w + e));
        acc_fma(a0, we, xa);
        acc_fma(a1, we, xb);
      }
    }
  }
  uint8_t *drow = As + pl * 128;
  *(uint4 *)(drow + (((2 * vp) ^ (pl & 7)) << 4)) = acc_pack(a0);
  *(uint4 *)(drow + (((2 * vp + 1) ^ (pl & 7)) << 4)) = acc_pack(a1);
}

// All chunks of one tile for the common shape (Cp >= 64, static tap count, (pixel, vector pair) threads) with
// the per-chunk instruction count pared down: 32-bit shared-space addresses kept in registers, the tap row and the
// image pointer advanced incrementally with the (channel block, slot) cursor, no generic-address arithmetic.
// Returns false if a wait gave up.
template <int STRIDE, int NTI, bool PLAN>
__device__ __forceinline__ bool produce_tile_lean(const TcParams &p, const Smem &sm, const PlanView<float> &pv, const char *img,
                                                  int nb, int pt, int lane, Ring &ring) {
  static_assert(kProducerThreads == kTileM * 4, "one (pixel, vector pair) per producer thread");
  const Gather &g = p.g;
  const int S = p.stages, vp = pt & 3, pl = pt >> 2;
  const uint32_t tap_slot_bytes = kTileM * STRIDE * sizeof(Tap);
  const uint32_t taps0 = smem_u32(sm.taps) + pl * (STRIDE * (uint32_t)sizeof(Tap));
  const uint32_t a0s = smem_u32(sm.A) + pl * 128 + (((2 * vp) ^ (pl & 7)) << 4);
  const uint32_t a1s = smem_u32(sm.A) + pl * 128 + (((2 * vp + 1) ^ (pl & 7)) << 4);
  const uint32_t full0 = smem_u32(sm.full), empty0 = smem_u32(sm.empty);
  const uint32_t bbytes = (uint32_t)p.Npb * 128;
  const __nv_bfloat16 *wsrc = p.wp + (size_t)nb * p.nchunks * p.Npb * kChunk;
  const char *imgc = img + vp * 32;  // advanced by 128 bytes per channel block
  uint32_t taps_s = taps0;
  int slot = 0;
  uint4 qa[NTI], qb[NTI];
  uint32_t w[NTI];
  // The gather loads roll one chunk ahead: right after a chunk's values are folded into the accumulators, the loads
  // of the next chunk are issued into the same registers - before the tile is stored, fenced and handed over and the
  // next stage waited for - so a thread always has its loads in flight.
  auto issue = [&]() {
    // table entry of (slot, pixel): NTI taps of 8 bytes, read as 16-byte vectors where the entry is 16-byte aligned
    // (STRIDE even), else tap by tap
    uint32_t tw[2 * ((NTI + 1) / 2) * 2];
    if constexpr (STRIDE % 2 == 0) {
#pragma unroll
      for (int i = 0; i < (NTI + 1) / 2; i++) {
        const uint4 t2 = lds128(taps_s + 16 * i);
        tw[4 * i] = t2.x; tw[4 * i + 1] = t2.y; tw[4 * i + 2] = t2.z; tw[4 * i + 3] = t2.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < NTI; i++) {
        const uint2 t1 = lds64(taps_s + 8 * i);
        tw[2 * i] = t1.x; tw[2 * i + 1] = t1.y;
      }
    }
#pragma unroll
    for (int t = 0; t < NTI; t++) {
      w[t] = tw[2 * t + 1];
      ldg32(imgc + (int)tw[2 * t], qa[t], qb[t]);
    }
  };
  // (plan mode keeps the loads inside the chunk: with its overflow loop the rolling form spills registers)
  constexpr bool kRoll = !PLAN;
  if (kRoll) issue();
  for (int chunk = 0; chunk < p.nchunks; chunk++, ring.next(S)) {
    const int s = ring.s;
    if (!mbar_wait_s(empty0 + 8 * s, ring.ph ^ 1u, sm.abort_flag)) return false;
    if (pt == 0) {
      mbar_arrive_expect_tx(sm.full + s, bbytes);
      bulk_copy_g2s(sm.Bw + (size_t)s * bbytes, wsrc + (size_t)chunk * p.Npb * kChunk, bbytes, sm.full + s);
    }
    if (!kRoll) issue();
    Acc8 a0, a1;
    acc_zero(a0);
    acc_zero(a1);
#pragma unroll
    for (int t = 0; t < NTI; t++) {
      acc_fma(a0, w[t], qa[t]);
      acc_fma(a1, w[t], qb[t]);
    }
    if (PLAN) {
      const int2 rr = sm.rest[slot * kTileM + pl];
      for (int e = rr.x; e < rr.y; e++) {
        uint4 xa, xb;
        const int sp = __ldg(pv.src + e);
        if (!index_ok(sp, pv.n_src)) continue;
        ldg32(imgc + (size_t)sp * (g.Cp * 2), xa, xb);
        const uint32_t we = tap_weight(__ldg(pv.w + e));
        acc_fma(a0, we, xa);
        acc_fma(a1, we, xb);
      }
    }
    // cursor: next slot of this channel block, or slot 0 of the next block; its loads go out now
    taps_s += tap_slot_bytes;
    if (++slot == g.K) {
      slot = 0;
      taps_s = taps0;
      imgc += 128;
    }
    if (kRoll && chunk + 1 < p.nchunks) issue();
    sts128(a0s + s * kAStageBytes, acc_pack(a0));
    sts128(a1s + s * kAStageBytes, acc_pack(a1));
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) mbar_arrive_s(full0 + 8 * s);
  }
  return true;
}

// ROWS: the outputs leave as bf16 rows (p.out_h, the column buffer of the multiply-first adjoint) and nothing else; the
// other instantiations carry no code for it.
// LEAN: channel copies of at least 64 padded channels with a static tap count - the producers run the lean per-chunk
// loop and the instantiation carries no code for the general one (and the other way round).
template <int MODE, int NT, bool ROWS = false, bool LEAN = false>
__global__ void __launch_bounds__(kThreads, 1) tc_gemm_kernel(const TcParams p, const __grid_constant__ CUtensorMap out_map,
                                                               const __grid_constant__ CUtensorMap cl_map) {
  extern __shared__ uint8_t smem_raw[];
  const Smem sm = carve(smem_raw, p, MODE == MODE_DIRECT);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.stages;
  const Gather &g = p.g;

  if (tid == 0) {
    for (int s = 0; s < S; s++) {
      mbar_init(sm.full + s, kProducerWarps + 1);
      mbar_init(sm.empty + s, 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(sm.tfull + i, 1);
      mbar_init(sm.tempty + i, kEpilogueWarps);
    }
    *sm.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kEpilogueWarps) {
    tmem_alloc(sm.tmem_ptr, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm.tmem_ptr;
  const int tiles_per_image = p.tiles_x * p.tiles_y;
  const int total_tiles = p.B * tiles_per_image * p.nblk;
  const int npix = g.GH * g.GW;
  const size_t shw = (size_t)g.SH * g.SW;

  if (warp < kEpilogueWarps) {
    // ---------------- epilogue: TMEM -> registers -> (+bias) -> global ----------------
    int tl = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tl++) {
      const int nb = tile % p.nblk, rest = tile / p.nblk;
      const int b = rest / tiles_per_image, t2 = rest % tiles_per_image;
      const int pix = tile_pixel(warp * 32 + lane, t2 / p.tiles_x, t2 % p.tiles_x, kTH, g.GH, g.GW);
      const int buf = tl & 1;
      TC_TIC(t_wait);
      if (!mbar_wait(sm.tfull + buf, (tl >> 1) & 1, sm.abort_flag)) break;
      if (tid == 0) { TC_TOC(t_wait, 5); }
      TC_TIC(t_drain);
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * 256;
      const int ty = t2 / p.tiles_x, tx = t2 % p.tiles_x;
      if (!ROWS && p.use_out_map) {
        // This warp's 32 pixels are two rows of 16.  Sixteen channels at a time go through shared memory as
        // [channel][row][x] and leave as one tiled tensor store (box 16 x 2 x 16 channels) issued by lane 0, so the
        // outputs cost this warp shared-memory stores only; the copy engine writes the 64-byte row segments and
        // clips whatever lies outside the image or beyond the last channel.
        const uint32_t st_s = smem_u32(sm.ostage) + warp * (kOutStageCh * 32 * 4);
        const uint32_t st_lane = st_s + lane * 4;
        // channels-last copy: this lane's pixel is row lane >> 4, column lane & 15 of the warp's 2 x 16 pixels; its 16
        // channels of a pass are 32 consecutive bytes of the [row][pixel][channel] staging block
        const uint32_t cl_s = smem_u32(sm.ostage) + kEpilogueWarps * (kOutStageCh * 32 * 4) + warp * (32 * kOutStageCh * 2);
        const uint32_t cl_lane = cl_s + lane * (kOutStageCh * 2);
        for (int n0 = 0; n0 < p.Npb; n0 += kOutStageCh) {
          uint32_t h[16];
          tmem_ld_32x16(taddr + n0, h);
          float bv[16];
#pragma unroll
          for (int j = 0; j < 16; j++) {
            const int n = nb * p.Npb + n0 + j;
            bv[j] = (p.bias && n < p.Nout) ? __ldg(p.bias + n) : 0.0f;
          }
          tmem_ld_wait();
          if (lane == 0) bulk_wait_read();  // the previous pass has left the staging rows
          __syncwarp();
          float ov[16];
#pragma unroll
          for (int j = 0; j < 16; j++) {
            float o = __uint_as_float(h[j]) + bv[j];
            if (p.relu) o = fmaxf(o, 0.0f);
            ov[j] = o;
            sts32(st_lane + j * 128, __float_as_uint(o));
          }
          if (p.out_cl != nullptr) {
            // the same 16 channels as bf16 (columns beyond Nout are exact zeros); they leave through a second tensor map
            // over the (B, rows, pixels, channels) view of the copy, which clips pixels outside the image and
            // channels beyond the copy's pitch
            sts128(cl_lane, make_uint4(pack_bf16(ov[0], ov[1]), pack_bf16(ov[2], ov[3]), pack_bf16(ov[4], ov[5]), pack_bf16(ov[6], ov[7])));
            sts128(cl_lane + 16, make_uint4(pack_bf16(ov[8], ov[9]), pack_bf16(ov[10], ov[11]), pack_bf16(ov[12], ov[13]), pack_bf16(ov[14], ov[15])));
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            tensor_store_4d(&out_map, st_s, tx * kTW, ty * kTH + 2 * warp, nb * p.Npb + n0, b);
            if (p.out_cl != nullptr) tensor_store_4d(&cl_map, cl_s, nb * p.Npb + n0, tx * kTW, ty * kTH + 2 * warp, b);
            bulk_commit();
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.tempty + buf);
        if (tid == 0) { TC_TOC(t_drain, 6); }
        continue;
      }
      float *orow = p.out + ((size_t)b * p.Nout) * npix + (pix >= 0 ? pix : 0);
      for (int n0 = 0; n0 < p.Npb; n0 += 32) {
        uint32_t r[32];
        if (p.Npb - n0 >= 32) {
          tmem_ld_32x32(taddr + n0, r);
        } else {
          uint32_t h[16];
          tmem_ld_32x16(taddr + n0, h);
#pragma unroll
          for (int j = 0; j < 16; j++) { r[j] = h[j]; r[j + 16] = 0; }
        }
        tmem_ld_wait();
        if constexpr (ROWS) {
          // 32 consecutive columns of every pixel's row, as bf16 (out_pitch and Npb are multiples of 8).  A thread holds
          // its own pixel's 64 bytes; stored directly, one instruction would touch 32 rows with 16 bytes each.  The warp's
          // 32 x 64 bytes go through shared memory (16-byte chunks XOR-swizzled, conflict-free both ways) and leave with
          // eight pixels of 64 contiguous bytes per instruction.
          const uint32_t hs = smem_u32(sm.ostage) + warp * (kOutStageCh * 32 * 4);
          __syncwarp();  // the previous pass has been read
#pragma unroll
          for (int j = 0; j < 4; j++)
            sts128(hs + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4),
                   make_uint4(pack_bf16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                              pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                              pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                              pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]))));
          __syncwarp();
          const int c = lane & 3, col = nb * p.Npb + n0 + c * 8;
#pragma unroll
          for (int it = 0; it < 4; it++) {
            const int pl = it * 8 + (lane >> 2);
            const int ppix = tile_pixel(warp * 32 + pl, ty, tx, kTH, g.GH, g.GW);
            const uint4 v = lds128(hs + pl * 64 + ((c ^ ((pl >> 1) & 3)) << 4));
            if (ppix >= 0 && n0 + c * 8 < p.Npb && col < p.out_pitch)
              *(uint4 *)(p.out_h + ((size_t)b * npix + ppix) * p.out_pitch + col) = v;
          }
        } else if (pix >= 0) {
          float ov[32];
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const int n = nb * p.Npb + n0 + j;
            ov[j] = 0.0f;
            if (n < p.Nout && n0 + j < p.Npb) {
              float o = __uint_as_float(r[j]) + (p.bias ? __ldg(p.bias + n) : 0.0f);
              if (p.relu) o = fmaxf(o, 0.0f);
              ov[j] = o;
              orow[(size_t)n * npix] = o;
            }
          }
          if (p.out_cl != nullptr) {
            __nv_bfloat16 *crow = p.out_cl + ((size_t)b * (npix + 1) + pix) * p.cl_pitch + nb * p.Npb + n0;
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              if (n0 + j < p.Npb && nb * p.Npb + n0 + j + 8 <= p.cl_pitch)
                *(uint4 *)(crow + j) = make_uint4(pack_bf16(ov[j], ov[j + 1]), pack_bf16(ov[j + 2], ov[j + 3]),
                                                  pack_bf16(ov[j + 4], ov[j + 5]), pack_bf16(ov[j + 6], ov[j + 7]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.tempty + buf);
      if (tid == 0) { TC_TOC(t_drain, 6); }
    }
    bulk_wait_all();  // this thread's bulk copies are complete before the CTA may exit
  } else if (warp == kEpilogueWarps) {
    // ---------------- MMA issuer (one thread) ----------------
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16(kTileM, p.Npb, 0, 0);
      int tl = 0;
      Ring ring;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < total_tiles; tile += gridDim.x, tl++) {
        const int buf = tl & 1;
        TC_TIC(t_te);
        if (!mbar_wait(sm.tempty + buf, ((tl >> 1) & 1) ^ 1, sm.abort_flag)) break;
        TC_TOC(t_te, 4);
        tc_fence_after();
        const uint32_t d = tmem_base + buf * 256;
        for (int chunk = 0; chunk < p.nchunks; chunk++, ring.next(S)) {
          const int s = ring.s;
          TC_TIC(t_full);
          if (!mbar_wait(sm.full + s, ring.ph, sm.abort_flag)) { alive = false; break; }
          TC_TOC(t_full, 3);
          tc_fence_after();
          const uint64_t a0 = smem_desc_sw128(smem_u32(sm.A + (size_t)s * kAStageBytes), 16, 1024);
          const uint64_t b0 = smem_desc_sw128(smem_u32(sm.Bw + (size_t)s * p.Npb * 128), 16, 1024);
#pragma unroll
          for (int kk = 0; kk < kChunk / 16; kk++)
            umma_bf16(d, a0 + 2 * kk, b0 + 2 * kk, idesc, (chunk | kk) != 0);
          umma_commit(sm.empty + s);
        }
        if (alive) umma_commit(sm.tfull + buf);
      }
    }
  } else {
    // ---------------- producers: gather Col tiles into swizzled shared memory ----------------
    const int pt = tid - kFirstProducerThread;
    Ring ring;
    bool alive = true;
    PlanView<float> pv{};
    bool plan_ok = true;
    int plan_nti = kPlanTaps;
    if (MODE == MODE_PLAN) {
      pv = plan_view<float>(g.plan, npix * g.K, plan_ok);
      if (plan_ok) plan_nti = min(kPlanTaps, ((const PlanHeader *)g.plan)->max_seg);
    }
    const int pitch = g.Cp * 2, zero_off = (int)shw * pitch;
    // A producer that gave up waiting keeps walking the tile loop and its two barriers (doing no work), so
    // that the named barrier never waits for a thread that left.
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int nb = tile % p.nblk, rest = tile / p.nblk;
      const int b = rest / tiles_per_image, t2 = rest % tiles_per_image;
      const int ty = t2 / p.tiles_x, tx = t2 % p.tiles_x;
      const char *img = (const char *)g.xh + (size_t)b * (shw + 1) * pitch;
      TC_TIC(t_b0);
      producer_bar();  // every producer is done reading the previous tile's taps
      if (pt == 0) { TC_TOC(t_b0, 2); }
      if (!alive) { producer_bar(); continue; }
      TC_TIC(t_fill);
      for (int idx = pt; idx < g.K * kTileM; idx += kProducerThreads) {
        const int slot = idx / kTileM, pl = idx % kTileM;
        const int pix = tile_pixel(pl, ty, tx, kTH, g.GH, g.GW);
        Tap *dst = sm.taps + (size_t)idx * g.nt;
        if (MODE == MODE_DIRECT) {
          if constexpr (NT == 4) {
            if (g.P == 0 && g.map != nullptr) {
              // entry built in registers and stored as two 16-byte vectors (field-by-field stores at this
              // 32-byte stride collide eight ways)
              Tap t[4];
              if (pix >= 0) {
                const float *m = g.map + 2 * ((size_t)pix * g.K + slot);
                taps_from_xy<4>(g, __ldg(m), __ldg(m + 1), t);
              } else {
#pragma unroll
                for (int i = 0; i < 4; i++) { t[i].off = zero_off; t[i].w = 0u; }
              }
              ((uint4 *)dst)[0] = make_uint4((uint32_t)t[0].off, t[0].w, (uint32_t)t[1].off, t[1].w);
              ((uint4 *)dst)[1] = make_uint4((uint32_t)t[2].off, t[2].w, (uint32_t)t[3].off, t[3].w);
              continue;
            }
          }
          if (pix >= 0) fill_taps_any(g, pix, slot, dst);
          else fill_taps_zero(g, dst);
        } else {
          int e0 = 0, e1 = 0;
          if (plan_ok && pix >= 0) {
            e0 = __ldg(pv.offsets + pix * g.K + slot);
            e1 = __ldg(pv.offsets + pix * g.K + slot + 1);
          }
          Tap t[kPlanTaps];
#pragma unroll
          for (int i = 0; i < kPlanTaps; i++) {
            const bool in = e0 + i < e1;
            const int sp = in ? __ldg(pv.src + e0 + i) : 0;
            t[i].off = (in && index_ok(sp, pv.n_src)) ? sp * pitch : zero_off;
            t[i].w = tap_weight(in ? __ldg(pv.w + e0 + i) : 0.0f);
          }
          static_assert(kPlanTaps == 4, "two 16-byte stores per entry");
          ((uint4 *)dst)[0] = make_uint4((uint32_t)t[0].off, t[0].w, (uint32_t)t[1].off, t[1].w);
          ((uint4 *)dst)[1] = make_uint4((uint32_t)t[2].off, t[2].w, (uint32_t)t[3].off, t[3].w);
          sm.rest[idx] = make_int2(min(e0 + kPlanTaps, e1), e1);
        }
      }
      producer_bar();
      if (pt == 0) { TC_TOC(t_fill, 0); TC_COUNT(7); }
      TC_TIC(t_loop);
      if constexpr (LEAN) {  // the common shape: lean per-chunk loop
        if (MODE == MODE_PLAN) {
          if (plan_nti >= 3) alive = produce_tile_lean<kPlanTaps, 4, true>(p, sm, pv, img, nb, pt, lane, ring);
          else if (plan_nti == 2) alive = produce_tile_lean<kPlanTaps, 2, true>(p, sm, pv, img, nb, pt, lane, ring);
          else alive = produce_tile_lean<kPlanTaps, 1, true>(p, sm, pv, img, nb, pt, lane, ring);
        } else {
          alive = produce_tile_lean<(NT > 0 ? NT : 1), (NT > 0 ? NT : 1), false>(p, sm, pv, img, nb, pt, lane, ring);
        }
        if (pt == 0) { TC_TOC(t_loop, 1); }
        continue;
      }
      if constexpr (LEAN) continue;  // (not reached; keeps the general loop out of this instantiation)
      int cslot = 0, cblock = 0;  // Cp >= 64: chunk = cblock * K + cslot, kept incrementally (no division)
      // (pixel, vector pair) threads when a pair lies inside one slot and the tap count is static; else
      // (two pixels, one vector)
      const bool pairs = g.Cp >= 16 && (MODE == MODE_PLAN || NT > 0);
      const int vsel = pairs ? (pt & 3) * 2 : (pt & 7);  // this thread's (first) 16-byte vector of a chunk row
      for (int chunk = 0; alive && chunk < p.nchunks; chunk++, ring.next(S)) {
        const int s = ring.s;
        int slot, c0;
        if (g.Cp >= 64) {
          slot = cslot;
          c0 = cblock * 64 + vsel * 8;
          if (++cslot == g.K) { cslot = 0; cblock++; }
        } else {
          chunk_vec(g.Cp, g.K, chunk, vsel, slot, c0);
        }
        if (!mbar_wait(sm.empty + s, ring.ph ^ 1u, sm.abort_flag)) { alive = false; break; }
        if (pt == 0) {
          const uint32_t bytes = (uint32_t)p.Npb * 128;
          mbar_arrive_expect_tx(sm.full + s, bytes);
          bulk_copy_g2s(sm.Bw + (size_t)s * bytes, p.wp + ((size_t)nb * p.nchunks + chunk) * p.Npb * kChunk, bytes, sm.full + s);
        }
        uint8_t *As = sm.A + (size_t)s * kAStageBytes;
        if (MODE == MODE_DIRECT) {
          if constexpr (NT > 0) {
            if (pairs) produce_chunk_pair<(NT > 0 ? NT : 1), (NT > 0 ? NT : 1), false>(g, sm.taps, nullptr, pv, img, slot, c0, pt, As);
            else produce_chunk<NT, NT, false>(g, sm.taps, nullptr, pv, img, slot, c0, pt, As);
          } else {
            produce_chunk<NT, NT, false>(g, sm.taps, nullptr, pv, img, slot, c0, pt, As);
          }
        } else if (pairs) {
          if (plan_nti >= 3) produce_chunk_pair<kPlanTaps, 4, true>(g, sm.taps, sm.rest, pv, img, slot, c0, pt, As);
          else if (plan_nti == 2) produce_chunk_pair<kPlanTaps, 2, true>(g, sm.taps, sm.rest, pv, img, slot, c0, pt, As);
          else produce_chunk_pair<kPlanTaps, 1, true>(g, sm.taps, sm.rest, pv, img, slot, c0, pt, As);
        } else if (plan_nti >= 3) {
          produce_chunk<kPlanTaps, 4, true>(g, sm.taps, sm.rest, pv, img, slot, c0, pt, As);
        } else if (plan_nti == 2) {
          produce_chunk<kPlanTaps, 2, true>(g, sm.taps, sm.rest, pv, img, slot, c0, pt, As);
        } else {
          produce_chunk<kPlanTaps, 1, true>(g, sm.taps, sm.rest, pv, img, slot, c0, pt, As);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.full + s);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kEpilogueWarps) tmem_dealloc(tmem_base, kTmemCols);
  if (tid == 0 && *sm.abort_flag) {
    *p.status = 1;
    g_wait_status = 1;
  }
}

// =================================================================================================
// weight-gradient kernel
// =================================================================================================
constexpr int kDwPix = 64, kDwTH = 4;      // pixels per reduction step (a 4x16 block)
// A CTA accumulates GRP chunks (of 64 columns) for MBS = 8 / GRP row blocks (of 128 rows): 512 TMEM columns either
// way.  GRP = 4 holds two row blocks and is what the host selects; GRP = 8 (one row block, more map slots per step)
// is kept for experiments.
constexpr int kDwGtBytes = 128 * 128;                  // one 128-row x 64-pixel gradient tile image
constexpr int kDwMaxTapBytes = 20 * 1024;

struct DwParams {
  Gather g;
  const __nv_bfloat16 *gt;  // gradient tile images [b][ptile][mb][128 rows][64 px], 128B-swizzled
  float *partial;           // [splits][mbs_total*128][nchunks*64]
  int *status;
  int B, mbs_total, nchunks, tiles_x, tiles_y, splits, stages, tap_rows;
};

struct DwSmem {
  uint8_t *stage;  // per stage: columns (32 KB) then gradient tiles (mbs * 16 KB)
  Tap *taps;
  uint64_t *full, *empty, *tfull;
  uint32_t *tmem_ptr;
  volatile int *abort_flag;
};

inline size_t dw_stage_bytes(int grp, int mbs) { return (size_t)grp * kDwPix * 128 + (size_t)mbs * kDwGtBytes; }
inline size_t dw_smem_bytes(int stages, int grp, int mbs, int tap_rows, int nt) {
  return 1024 + stages * dw_stage_bytes(grp, mbs) + 2 * (size_t)tap_rows * kDwPix * nt * sizeof(Tap) + 8 * (2 * stages + 1) + 16;
}

// WT selects warp-private taps (unweighted maps, Cp >= 64, NT > 0): every producer warp decodes the taps of its own
// four pixels, one step ahead, into its own slice of the table, so the producers share nothing but the stage
// barriers; otherwise the whole producer group fills one table per step and meets at a named barrier.
template <int NT, int GRP, bool WT>
__global__ void __launch_bounds__(kThreads, 1) tc_dw_kernel(const DwParams p) {
  constexpr int MBS = 8 / GRP;
  constexpr int kDwColBytes = GRP * kDwPix * 128;  // gathered columns per stage
  extern __shared__ uint8_t smem_raw[];
  const Gather &g = p.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.stages;
  const int grp = blockIdx.x, split = blockIdx.y, mb0 = blockIdx.z * MBS;
  const int mbs = min(MBS, p.mbs_total - mb0);
  const int chunk0 = grp * GRP, ncg = min(GRP, p.nchunks - chunk0);
  const size_t stage_bytes = kDwColBytes + (size_t)mbs * kDwGtBytes;

  DwSmem sm;
  {
    uint8_t *b = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    sm.stage = b;
    uint8_t *q = b + (size_t)S * stage_bytes;
    sm.taps = (Tap *)q;
    q += 2 * (size_t)p.tap_rows * kDwPix * g.nt * sizeof(Tap);
    sm.full = (uint64_t *)q;
    sm.empty = sm.full + S;
    sm.tfull = sm.empty + S;
    sm.tmem_ptr = (uint32_t *)(sm.tfull + 1);
    sm.abort_flag = (volatile int *)(sm.tmem_ptr + 1);
  }
  if (tid == 0) {
    for (int s = 0; s < S; s++) {
      mbar_init(sm.full + s, kProducerWarps + 1);
      mbar_init(sm.empty + s, 1);
    }
    mbar_init(sm.tfull, 1);
    *sm.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kEpilogueWarps) {
    tmem_alloc(sm.tmem_ptr, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm.tmem_ptr;

  const int tiles_per_image = p.tiles_x * p.tiles_y;
  const int64_t total_steps = (int64_t)p.B * tiles_per_image;
  const int step_lo = (int)(total_steps * split / p.splits), step_hi = (int)(total_steps * (split + 1) / p.splits);
  const size_t shw = (size_t)g.SH * g.SW;
  const int ncols_total = p.nchunks * kChunk;

  if (warp < kEpilogueWarps) {
    // ---------------- epilogue: TMEM -> partial sums ----------------
    bool have = step_hi > step_lo;
    if (have) have = mbar_wait(sm.tfull, 0, sm.abort_flag);
    tc_fence_after();
    for (int mb = 0; mb < mbs; mb++) {
      const int row = (mb0 + mb) * 128 + warp * 32 + lane;
      float *prow = p.partial + ((size_t)split * p.mbs_total * 128 + row) * ncols_total + (size_t)chunk0 * kChunk;
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + mb * (GRP / 4) * 256;
      for (int n0 = 0; n0 < ncg * kChunk; n0 += 32) {
        uint32_t r[32];
        if (have) {
          tmem_ld_32x32(taddr + n0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++) r[j] = 0;
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *(float4 *)(prow + n0 + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                                   __uint_as_float(r[j + 3]));
      }
    }
    tc_fence_before();
  } else if (warp == kEpilogueWarps) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && step_hi > step_lo) {
      // A (gradient) K-major, B (columns) MN-major; the column group is issued in halves of at most 4 chunks (N <= 256)
      const int nhalves = (ncg + 3) / 4;
      const uint32_t idesc0 = idesc_bf16(128, min(4, ncg) * kChunk, 0, 1);
      const uint32_t idesc1 = idesc_bf16(128, max(1, ncg - 4) * kChunk, 0, 1);
      bool alive = true;
      int it = 0;
      Ring ring;
      for (int step = step_lo; alive && step < step_hi; step++, it++, ring.next(S)) {
        const int s = ring.s;
        if (!mbar_wait(sm.full + s, ring.ph, sm.abort_flag)) { alive = false; break; }
        tc_fence_after();
        uint8_t *st = sm.stage + (size_t)s * stage_bytes;
        for (int mb = 0; mb < mbs; mb++) {
          const uint64_t a0 = smem_desc_sw128(smem_u32(st + kDwColBytes + (size_t)mb * kDwGtBytes), 16, 1024);
          for (int h = 0; h < nhalves; h++) {
            const uint64_t b0 = smem_desc_sw128(smem_u32(st + h * 4 * (kDwPix * 128)), kDwPix * 128, 1024);
            const uint32_t d = tmem_base + (mb * (GRP / 4) + h) * 256;
#pragma unroll
            for (int ks = 0; ks < kDwPix / 16; ks++)
              umma_bf16(d, a0 + 2 * ks, b0 + (uint64_t)(ks * 16 * 128 >> 4), h ? idesc1 : idesc0, (it | ks) != 0);
          }
        }
        umma_commit(sm.empty + s);
      }
      if (alive) umma_commit(sm.tfull);
    }
  } else if constexpr (WT && NT > 0) {
    // ---------------- producers, warp-private taps ----------------
    // Thread = (chunk pair h, pixel pl, vector pair vp): one pixel and 32 bytes of it for two chunks of the group;
    // a warp covers 8 pixels of one chunk pair and decodes exactly the 16 (chunk, pixel) tap entries it reads.
    static_assert(GRP == 4 && kProducerThreads == 2 * kDwPix * 4, "two chunk pairs x 64 pixels x 4 vector pairs");
    const int pt = tid - kFirstProducerThread, pw = pt >> 5;
    const int h = pt >> 8, pl = (pt & 255) >> 2, vp = pt & 3, pxl = lane >> 2;
    constexpr int kEnt = 16;                                   // (chunk of the pair, pixel) entries per warp and step
    constexpr uint32_t kEntBytes = NT * sizeof(Tap);
    const uint32_t wt_s = smem_u32(sm.taps) + pw * (2 * kEnt * kEntBytes);  // this warp's two table halves
    // decoding role: lane e < 16 owns chunk 2h + (e >> 3) of the group and pixel e & 7 of the warp
    const bool dec = lane < kEnt && (2 * h + (lane >> 3)) < ncg;
    const int e_pl = (pw & 7) * 8 + (lane & 7);
    int e_slot = 0;
    if (dec) { int c0; chunk_vec(g.Cp, g.K, chunk0 + 2 * h + (lane >> 3), 0, e_slot, c0); }
    int coff[2];
#pragma unroll
    for (int c = 0; c < 2; c++) {
      int slot = 0, c0 = 0;
      if (2 * h + c < ncg) chunk_vec(g.Cp, g.K, chunk0 + 2 * h + c, 2 * vp, slot, c0);
      coff[c] = c0 * 2;
    }
    const int zero_off = g.SH * g.SW * g.Cp * 2;
    // position (image, tile row, tile column) of the step whose map coordinate is fetched next
    int nb_ = step_lo / tiles_per_image, nty = (step_lo % tiles_per_image) / p.tiles_x, ntx = (step_lo % tiles_per_image) % p.tiles_x;
    int b_dec = 0, pix_dec = -1;
    float mx = 0.0f, my = 0.0f;
    auto fetch = [&]() {  // issue the map loads of the next step; they complete under the current step's gather
      b_dec = nb_;
      pix_dec = tile_pixel(e_pl, nty, ntx, kDwTH, g.GH, g.GW);
      if (++ntx == p.tiles_x) {
        ntx = 0;
        if (++nty == p.tiles_y) { nty = 0; nb_++; }
      }
      if (dec && pix_dec >= 0) {
        const float *m = g.map + 2 * ((size_t)pix_dec * g.K + e_slot);
        mx = __ldg(m);
        my = __ldg(m + 1);
      }
    };
    auto decode_to = [&](uint32_t dst_s) {
      if (lane < kEnt) {
        Tap t[NT];
        if (dec && pix_dec >= 0) taps_from_xy<NT>(g, mx, my, t);
        else {
#pragma unroll
          for (int i = 0; i < NT; i++) { t[i].off = zero_off; t[i].w = 0u; }
        }
        const uint32_t d = dst_s + lane * kEntBytes;
        if constexpr (NT == 4) {
          sts128(d, make_uint4((uint32_t)t[0].off, t[0].w, (uint32_t)t[1].off, t[1].w));
          sts128(d + 16, make_uint4((uint32_t)t[2].off, t[2].w, (uint32_t)t[3].off, t[3].w));
        } else {
#pragma unroll
          for (int i = 0; i < NT; i++) {
            sts32(d + 8 * i, (uint32_t)t[i].off);
            sts32(d + 8 * i + 4, t[i].w);
          }
        }
      }
    };
    int b_cur = 0;
    if (step_lo < step_hi) {
      fetch();
      b_cur = b_dec;
      decode_to(wt_s);
    }
    __syncwarp();
    const uint32_t stage0_s = smem_u32(sm.stage);
    const uint32_t full0 = smem_u32(sm.full), empty0 = smem_u32(sm.empty);
    // this thread's two 16-byte slots of a chunk's row pl (128-byte swizzle)
    const uint32_t d0 = pl * 128 + (((2 * vp) ^ (pl & 7)) << 4), d1 = pl * 128 + (((2 * vp + 1) ^ (pl & 7)) << 4);
    int it = 0;
    Ring ring;
    for (int step = step_lo; step < step_hi; step++, it++, ring.next(S)) {
      const char *img = (const char *)g.xh + (size_t)b_cur * (shw + 1) * g.Cp * 2;
      const uint32_t taps_s = wt_s + (it & 1) * (kEnt * kEntBytes) + pxl * kEntBytes;
      const int s = ring.s;
      const bool ok = mbar_wait_s(empty0 + 8 * s, ring.ph ^ 1u, sm.abort_flag);
      if (!__all_sync(0xffffffffu, ok)) break;  // the whole warp leaves together
      const uint32_t st_s = stage0_s + (uint32_t)(s * stage_bytes);
      if (pt == 0) {
        const uint32_t bytes = (uint32_t)mbs * kDwGtBytes;
        mbar_arrive_expect_tx(sm.full + s, bytes);
        bulk_copy_g2s(sm.stage + (size_t)s * stage_bytes + kDwColBytes, p.gt + ((size_t)step * p.mbs_total + mb0) * (kDwGtBytes / 2),
                      bytes, sm.full + s);
      }
      const bool more = step + 1 < step_hi;
      int b_next = b_cur;
      if (more) {
        fetch();
        b_next = b_dec;
      }
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const int gi = 2 * h + c;
        if (gi >= ncg) break;
        uint4 qa[NT], qb[NT];
        uint32_t w[NT];
        const uint32_t trow = taps_s + c * (8 * kEntBytes);
        if constexpr (NT == 4) {
          const uint4 ta = lds128(trow), tb = lds128(trow + 16);
          w[0] = ta.y; w[1] = ta.w; w[2] = tb.y; w[3] = tb.w;
          const char *ic = img + coff[c];
          ldg32(ic + (int)ta.x, qa[0], qb[0]);
          ldg32(ic + (int)ta.z, qa[1], qb[1]);
          ldg32(ic + (int)tb.x, qa[2], qb[2]);
          ldg32(ic + (int)tb.z, qa[3], qb[3]);
        } else {
#pragma unroll
          for (int t = 0; t < NT; t++) {
            const uint2 tt = lds64(trow + 8 * t);
            w[t] = tt.y;
            ldg32(img + coff[c] + (int)tt.x, qa[t], qb[t]);
          }
        }
        Acc8 a0, a1;
        acc_zero(a0);
        acc_zero(a1);
#pragma unroll
        for (int t = 0; t < NT; t++) {
          acc_fma(a0, w[t], qa[t]);
          acc_fma(a1, w[t], qb[t]);
        }
        sts128(st_s + gi * (kDwPix * 128) + d0, acc_pack(a0));
        sts128(st_s + gi * (kDwPix * 128) + d1, acc_pack(a1));
      }
      if (more) decode_to(wt_s + ((it + 1) & 1) * (kEnt * kEntBytes));
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive_s(full0 + 8 * s);
      b_cur = b_next;
    }
  } else {
    // ---------------- producers, shared tap table ----------------
    const int pt = tid - kFirstProducerThread;
    bool alive = true;
    int it = 0;
    // table row r holds the taps of slot `slot_base + r`
    int slot_base, dummy;
    chunk_vec(g.Cp, g.K, chunk0, 0, slot_base, dummy);
    // The CTA's column group is fixed, so each thread's (slot, first channel, table row) per chunk of the group
    // is computed once.
    int g_coff[GRP], g_trow[GRP];
    bool g_ok[GRP];
#pragma unroll
    for (int gi = 0; gi < GRP; gi++) {
      int slot = g.K, c0 = 0;
      if (gi < ncg) chunk_vec(g.Cp, g.K, chunk0 + gi, pt & 7, slot, c0);
      g_ok[gi] = slot < g.K;
      g_coff[gi] = c0 * 2;
      g_trow[gi] = g_ok[gi] ? ((g.Cp >= 64 ? gi : slot - slot_base) * kDwPix + (pt >> 3)) * (NT > 0 ? NT : g.nt) : 0;
    }
    // The tap table is double buffered: while the columns of one step are gathered from one half, the taps
    // of the next step are decoded into the other half, so the map loads never sit on the critical path.
    const size_t tap_half = (size_t)p.tap_rows * kDwPix * g.nt;
    // position (image, tile row, tile column) of the step whose taps are decoded next, advanced without division
    int nb_ = step_lo / tiles_per_image, nty = (step_lo % tiles_per_image) / p.tiles_x, ntx = (step_lo % tiles_per_image) % p.tiles_x;
    int cur_b = nb_;
    auto fill_step = [&](Tap *table) {
      const int ty = nty, tx = ntx;
      cur_b = nb_;
      if (++ntx == p.tiles_x) {
        ntx = 0;
        if (++nty == p.tiles_y) { nty = 0; nb_++; }
      }
      for (int idx = pt; idx < p.tap_rows * kDwPix; idx += kProducerThreads) {
        const int row = idx / kDwPix, pl = idx % kDwPix;
        int slot;
        if (g.Cp >= 64) { int c0; chunk_vec(g.Cp, g.K, chunk0 + row, 0, slot, c0); }   // one slot per chunk
        else slot = slot_base + row;
        const int pix = tile_pixel(pl, ty, tx, kDwTH, g.GH, g.GW);
        Tap *dst = table + (size_t)idx * g.nt;
        if (pix >= 0 && slot < g.K && (g.Cp < 64 || row < ncg)) fill_taps_any(g, pix, slot, dst);
        else fill_taps_zero(g, dst);
      }
    };
    if (step_lo < step_hi) fill_step(sm.taps);
    producer_bar();
    // A producer that gave up waiting keeps walking the loop and its barriers (doing no work), so that the
    // named barrier never waits for a thread that left.
    Ring ring;
    for (int step = step_lo; step < step_hi; step++, it++, ring.next(S)) {
      const char *img = (const char *)g.xh + (size_t)cur_b * (shw + 1) * g.Cp * 2;  // image of this step
      const Tap *taps = sm.taps + (it & 1) * tap_half;
      const int s = ring.s;
      if (alive && !mbar_wait(sm.empty + s, ring.ph ^ 1u, sm.abort_flag)) alive = false;
      if (!alive) { producer_bar(); continue; }
      uint8_t *st = sm.stage + (size_t)s * stage_bytes;
      if (pt == 0) {
        const uint32_t bytes = (uint32_t)mbs * kDwGtBytes;
        mbar_arrive_expect_tx(sm.full + s, bytes);
        bulk_copy_g2s(st + kDwColBytes, p.gt + ((size_t)step * p.mbs_total + mb0) * (kDwGtBytes / 2), bytes, sm.full + s);
      }
      if (step + 1 < step_hi) fill_step(sm.taps + ((it + 1) & 1) * tap_half);  // also moves cur_b on for the next step
      // thread pt: 16-byte vector v = pt & 7 of pixel pt >> 3, two chunks of the group at a time
      {
        static_assert(kProducerThreads == kDwPix * 8, "one (pixel, vector) per producer thread");
        const int v = pt & 7, pl = pt >> 3;
        uint8_t *dst0 = st + pl * 128 + ((v ^ (pl & 7)) << 4);
#pragma unroll
        for (int gi = 0; gi < GRP; gi += 2) {
          if (gi >= ncg) break;
          Acc8 a0, a1;
          acc_zero(a0);
          acc_zero(a1);
          if (g_ok[gi] || g_ok[gi + 1]) {
            gather_pair<NT>(img + g_coff[gi], img + g_coff[gi + 1], taps + g_trow[gi], taps + g_trow[gi + 1], g.nt, a0, a1);
            if (!g_ok[gi]) acc_zero(a0);
            if (!g_ok[gi + 1]) acc_zero(a1);
          }
          *(uint4 *)(dst0 + gi * (kDwPix * 128)) = acc_pack(a0);
          if (gi + 1 < ncg) *(uint4 *)(dst0 + (gi + 1) * (kDwPix * 128)) = acc_pack(a1);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.full + s);
      producer_bar();  // next table complete, this one no longer read
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kEpilogueWarps) tmem_dealloc(tmem_base, kTmemCols);
  if (tid == 0 && *sm.abort_flag) {
    *p.status = 1;
    g_wait_status = 1;
  }
}

// =================================================================================================
// layout pre-passes
// =================================================================================================

// (B, C, HW) float32 -> (B, HW + 1, Cp) bf16; channels beyond C and the extra pixel HW of every image are
// zero (unused taps point there).  64 pixels x 64 channels per block: 256-byte row segments in, 128-byte
// pixel rows out.
// With `mask` (same shape as x) elements whose mask value is not positive are taken as zero (gradient of a fused ReLU).
__global__ void __launch_bounds__(256) nchw_to_nhwc_bf16_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ y,
                                                                 int C, int Cp, int HW, const float *__restrict__ mask) {
  __shared__ float tile[64][65];
  const int b = blockIdx.z, c0 = blockIdx.y * 64, p0 = blockIdx.x * 64;
  const int tid = threadIdx.x;
  // rows of every channel start 16-byte aligned
  const bool vec_ok = (HW & 3) == 0 && (((uintptr_t)x | (uintptr_t)mask) & 15) == 0;
#pragma unroll
  for (int it = 0; it < 4; it++) {
    const int i = tid + it * 256, c = i >> 4, q = (i & 15) * 4;  // channel row, first of 4 pixels
    float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c0 + c < C) {
      const float *src = x + ((size_t)b * C + c0 + c) * HW + p0 + q;
      const float *msk = mask ? mask + (src - x) : nullptr;
      if (vec_ok && p0 + q + 3 < HW) {
        f = __ldg((const float4 *)src);
        if (msk) {
          const float4 m = __ldg((const float4 *)msk);
          f.x = m.x > 0.0f ? f.x : 0.0f;
          f.y = m.y > 0.0f ? f.y : 0.0f;
          f.z = m.z > 0.0f ? f.z : 0.0f;
          f.w = m.w > 0.0f ? f.w : 0.0f;
        }
      } else {
        if (p0 + q + 0 < HW) f.x = (!msk || __ldg(msk + 0) > 0.0f) ? __ldg(src + 0) : 0.0f;
        if (p0 + q + 1 < HW) f.y = (!msk || __ldg(msk + 1) > 0.0f) ? __ldg(src + 1) : 0.0f;
        if (p0 + q + 2 < HW) f.z = (!msk || __ldg(msk + 2) > 0.0f) ? __ldg(src + 2) : 0.0f;
        if (p0 + q + 3 < HW) f.w = (!msk || __ldg(msk + 3) > 0.0f) ? __ldg(src + 3) : 0.0f;
      }
    }
    tile[c][q + 0] = f.x;
    tile[c][q + 1] = f.y;
    tile[c][q + 2] = f.z;
    tile[c][q + 3] = f.w;
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 2; it++) {
    const int i = tid + it * 256, pp = i >> 3, v = i & 7;
    if (p0 + pp <= HW && c0 + v * 8 < Cp) {
      uint4 o;
      o.x = pack_bf16(tile[v * 8 + 0][pp], tile[v * 8 + 1][pp]);
      o.y = pack_bf16(tile[v * 8 + 2][pp], tile[v * 8 + 3][pp]);
      o.z = pack_bf16(tile[v * 8 + 4][pp], tile[v * 8 + 5][pp]);
      o.w = pack_bf16(tile[v * 8 + 6][pp], tile[v * 8 + 7][pp]);
      *(uint4 *)(y + ((size_t)b * (HW + 1) + p0 + pp) * Cp + c0 + v * 8) = o;
    }
  }
}

// Weights -> bf16 tile images.  Row n of block nb, chunk `chunk`: 64 columns, 16-byte vector v stored at
// position v ^ (n & 7) of the 128-byte row.  The source is addressed W[n*sn + ch*sc + slot*sk].
__global__ void weight_image_kernel(const float *__restrict__ w, __nv_bfloat16 *__restrict__ wp, int Nout, int CH, int Cp,
                                    int K, int Npb, int nblk, int nchunks, int64_t sn, int64_t sc, int64_t sk) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)nblk * nchunks * Npb * kChunk;
  if (i >= total) return;
  const int col = (int)(i % kChunk), n = (int)((i / kChunk) % Npb), chunk = (int)((i / ((int64_t)kChunk * Npb)) % nchunks);
  const int nb = (int)(i / ((int64_t)kChunk * Npb * nchunks));
  int slot, c0;
  chunk_vec(Cp, K, chunk, col >> 3, slot, c0);
  const int ch = c0 + (col & 7), ng = nb * Npb + n;
  const float v = (ng < Nout && slot < K && ch < CH) ? __ldg(w + ng * sn + ch * sc + slot * sk) : 0.0f;
  wp[(((int64_t)nb * nchunks + chunk) * Npb + n) * kChunk + (((col >> 3) ^ (n & 7)) << 3) + (col & 7)] = __float2bfloat16(v);
}

// Gradient (B, N, GH*GW) float32 -> bf16 tile images [b][ptile][mb][128 rows][64 px]; the 64 pixels of a tile
// are a 4x16 block of the (GH, GW) grid; 16-byte vector v (8 pixels) of row r sits at position v ^ (r & 7).
// With `row_part` the kernel also writes the sum of every row over the tile's pixels to
// row_part[(b * tiles + tile) * mbs_total * 128 + row] (first stage of the bias gradient).
// With `cl` the same (masked) values are also written as the channels-last bf16 copy (B, GH*GW + 1, cl_pitch) that the
// input-gradient kernel gathers from, so the gradient is read from memory once for both of its consumers; the extra
// zero pixel of every image is not written here.
constexpr int kClStride = 128 + 8;  // bf16 per staged pixel row: 16-byte aligned rows, shifted banks
__global__ void __launch_bounds__(256) grad_image_kernel(const float *__restrict__ gsrc, __nv_bfloat16 *__restrict__ gt, int N,
                                                          int GH, int GW, int tiles_x, int tiles_y, int mbs_total,
                                                          float *__restrict__ row_part, const float *__restrict__ mask,
                                                          __nv_bfloat16 *__restrict__ cl, int cl_pitch) {
  __shared__ __align__(16) __nv_bfloat16 cls[64 * kClStride];  // [pixel of the 4x16 tile][channel of this 128-row block]
  const int t2 = blockIdx.x, mb = blockIdx.y, b = blockIdx.z;
  const int ty = t2 / tiles_x, tx = t2 % tiles_x;
  const size_t npix = (size_t)GH * GW;
  __nv_bfloat16 *dst = gt + (((size_t)b * tiles_x * tiles_y + t2) * mbs_total + mb) * (128 * 64);
  for (int i = threadIdx.x; i < 128 * 8; i += 256) {
    const int r = i >> 3, v = i & 7, n = mb * 128 + r;
    float f[8];
    {
      // the 8 pixels of vector v are consecutive in one image row: two 16-byte loads when the row segment is
      // inside the image and 16-byte aligned
      const int y = ty * kDwTH + (v >> 1), x0 = tx * kTW + (v & 1) * 8;
      const float *src = gsrc + ((size_t)b * N + n) * npix + (size_t)y * GW + x0;
      const float *msk = mask ? mask + (src - gsrc) : nullptr;  // same shape: a fused ReLU's output
      if (n < N && y < GH && x0 + 8 <= GW && (GW & 3) == 0 && (((uintptr_t)gsrc | (uintptr_t)mask) & 15) == 0) {
        const float4 a = __ldg((const float4 *)src), c = __ldg((const float4 *)src + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = c.x; f[5] = c.y; f[6] = c.z; f[7] = c.w;
        if (msk) {
          const float4 ma = __ldg((const float4 *)msk), mc = __ldg((const float4 *)msk + 1);
          const float mv[8] = {ma.x, ma.y, ma.z, ma.w, mc.x, mc.y, mc.z, mc.w};
#pragma unroll
          for (int e = 0; e < 8; e++) f[e] = mv[e] > 0.0f ? f[e] : 0.0f;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; e++)
          f[e] = (n < N && y < GH && x0 + e < GW && (!msk || __ldg(msk + e) > 0.0f)) ? __ldg(src + e) : 0.0f;
      }
    }
    uint4 o;
    o.x = pack_bf16(f[0], f[1]);
    o.y = pack_bf16(f[2], f[3]);
    o.z = pack_bf16(f[4], f[5]);
    o.w = pack_bf16(f[6], f[7]);
    *(uint4 *)(dst + r * 64 + ((v ^ (r & 7)) << 3)) = o;
    if (cl != nullptr) {
#pragma unroll
      for (int e = 0; e < 8; e++) cls[(v * 8 + e) * kClStride + r] = __float2bfloat16(f[e]);
    }
    if (row_part) {
      float sum = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      if (v == 0) row_part[(((size_t)b * tiles_x * tiles_y + t2) * mbs_total + mb) * 128 + r] = sum;
    }
  }
  if (cl != nullptr) {
    __syncthreads();
    // pixel v * 8 + e of the tile is (row v >> 1, column (v & 1) * 8 + e); 16 threads write one pixel's 128 channels
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int pl = i >> 4, vec = i & 15, v = pl >> 3, e = pl & 7;
      const int y = ty * kDwTH + (v >> 1), x = tx * kTW + (v & 1) * 8 + e, c = mb * 128 + vec * 8;
      if (y < GH && x < GW && c + 8 <= cl_pitch)
        *(uint4 *)(cl + ((size_t)b * (npix + 1) + (size_t)y * GW + x) * cl_pitch + c) = *(const uint4 *)(cls + pl * kClStride + vec * 8);
    }
  }
}

// Second and third stage of the fused bias gradient: fixed-order sums over the (image, tile) blocks.
constexpr int kRowSplits = 64;
__global__ void row_sum_split_kernel(const float *__restrict__ row_part, int64_t nblocks, int rows_total, int C,
                                     float *__restrict__ part2) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, sp = blockIdx.y;
  if (c >= C) return;
  const int64_t lo = nblocks * sp / kRowSplits, hi = nblocks * (sp + 1) / kRowSplits;
  float s = 0.0f;
  for (int64_t i = lo; i < hi; i++) s += __ldg(row_part + i * rows_total + c);
  part2[(size_t)sp * C + c] = s;
}
__global__ void row_sum_final_kernel(const float *__restrict__ part2, int C, float *__restrict__ gb) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.0f;
  for (int sp = 0; sp < kRowSplits; sp++) s += part2[(size_t)sp * C + c];
  gb[c] = s;
}

// Weight image of the multiply-first adjoint: rows n = k * Mp + m (slot-major, so that one map slot's M channels
// are contiguous in the column buffer), columns = source channels; W addressed Wgt[m*sm + ch*sc + k*sk].
__global__ void premul_weight_image_kernel(const float *__restrict__ w, __nv_bfloat16 *__restrict__ wp, int M, int Mp, int K,
                                           int CH, int Npb, int nblk, int nchunks, int64_t sm, int64_t sc, int64_t sk) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)nblk * nchunks * Npb * kChunk;
  if (i >= total) return;
  const int col = (int)(i % kChunk), n = (int)((i / kChunk) % Npb), chunk = (int)((i / ((int64_t)kChunk * Npb)) % nchunks);
  const int nb = (int)(i / ((int64_t)kChunk * Npb * nchunks));
  const int ng = nb * Npb + n, k = ng / Mp, m = ng % Mp, ch = chunk * kChunk + col;
  const float v = (k < K && m < M && ch < CH) ? __ldg(w + m * sm + ch * sc + k * sk) : 0.0f;
  wp[(((int64_t)nb * nchunks + chunk) * Npb + n) * kChunk + (((col >> 3) ^ (n & 7)) << 3) + (col & 7)] = __float2bfloat16(v);
}

// Second half of the multiply-first adjoint (the col2im of the reference, through the plan):
//   Out[b, m, p] = bias[m] + sum_k sum_{e in plan(p*K+k)} w_e * T[b, src_e, k*Mp + m]
// T is the bf16 column buffer (B, n_src, pitch = K*Mp) written by the GEMM on the source grid.  Thread = one
// destination pixel and up to 64 output channels (one 128-byte row segment per plan entry).
__global__ void __launch_bounds__(128)
plan_gather_rows_kernel(const __nv_bfloat16 *__restrict__ T, const void *__restrict__ plan_blob, const float *__restrict__ bias,
                        float *__restrict__ out, int K, int M, int Mp, int n_src, int n_dst) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (p >= n_dst) return;
  bool ok;
  const PlanView<float> pv = plan_view<float>(plan_blob, n_dst * K, ok);
  const int pitch = K * Mp;
  const __nv_bfloat16 *tb = T + (size_t)b * n_src * pitch;
  for (int m0 = 0; m0 < Mp; m0 += 64) {
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; i++) acc[i] = 0.0f;
    if (ok) {
      int e1 = __ldg(pv.offsets + p * K);
      for (int k = 0; k < K; k++) {
        const int e0 = e1;
        e1 = __ldg(pv.offsets + p * K + k + 1);
        for (int e = e0; e < e1; e++) {
          const float w = __ldg(pv.w + e);
          const int sp = __ldg(pv.src + e);
          if (!index_ok(sp, pv.n_src)) continue;
          const __nv_bfloat16 *row = tb + (size_t)sp * pitch + k * Mp + m0;
#pragma unroll
          for (int v = 0; v < 8; v++) {
            if (m0 + v * 8 < Mp) {
              const uint4 q = __ldg((const uint4 *)(row + v * 8));
              acc[v * 8 + 0] = fmaf(w, bf16_lo(q.x), acc[v * 8 + 0]);
              acc[v * 8 + 1] = fmaf(w, bf16_hi(q.x), acc[v * 8 + 1]);
              acc[v * 8 + 2] = fmaf(w, bf16_lo(q.y), acc[v * 8 + 2]);
              acc[v * 8 + 3] = fmaf(w, bf16_hi(q.y), acc[v * 8 + 3]);
              acc[v * 8 + 4] = fmaf(w, bf16_lo(q.z), acc[v * 8 + 4]);
              acc[v * 8 + 5] = fmaf(w, bf16_hi(q.z), acc[v * 8 + 5]);
              acc[v * 8 + 6] = fmaf(w, bf16_lo(q.w), acc[v * 8 + 6]);
              acc[v * 8 + 7] = fmaf(w, bf16_hi(q.w), acc[v * 8 + 7]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 64; i++)
      if (m0 + i < M) out[((size_t)b * M + m0 + i) * n_dst + p] = acc[i] + (bias ? __ldg(bias + m0 + i) : 0.0f);
  }
}

// gw[n*sn + ch*sc + slot*sk] = sum over splits (in order) of partial[split][n][column of (slot, ch)].
__global__ void tc_dw_reduce_kernel(const float *__restrict__ partial, int splits, int rows_total, int ncols_total, int Nout,
                                    int CH, int Cp, int K, int64_t sn, int64_t sc, int64_t sk, float *__restrict__ gw) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= Nout * CH * K) return;
  const int slot = i % K, ch = (i / K) % CH, n = i / (K * CH);
  int col;
  if (Cp >= 64) col = ((ch / 64) * K + slot) * 64 + (ch % 64);
  else col = slot * Cp + ch;
  float s = 0.0f;
  for (int z = 0; z < splits; z++) s += partial[((size_t)z * rows_total + n) * ncols_total + col];
  gw[n * sn + ch * sc + slot * sk] = s;
}

// =================================================================================================
// host side
// =================================================================================================

constexpr int kMaxDevices = 64;

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}

// SM count of the current device (one process may drive several devices).
int sm_count() {
  static int n[kMaxDevices] = {0};
  const int dev = current_device();
  int v = __atomic_load_n(&n[dev], __ATOMIC_RELAXED);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    __atomic_store_n(&n[dev], v, __ATOMIC_RELAXED);
  }
  return v;
}

// Opt a kernel in to `smem` bytes of dynamic shared memory, once per device and kernel (the largest request so far).
template <typename Kernel>
void ensure_dynamic_smem(Kernel kernel, int *granted /* [kMaxDevices], zero-initialised, one array per kernel */, size_t smem) {
  const int dev = current_device();
  if (__atomic_load_n(&granted[dev], __ATOMIC_RELAXED) >= (int)smem) return;
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  __atomic_store_n(&granted[dev], (int)smem, __ATOMIC_RELAXED);
}

struct Geometry {
  int Cp, nchunks, Npb, nblk, nt, stages;
  size_t xh_bytes, wp_bytes, smem;
  bool ok;
};

Geometry geometry(int64_t B, int64_t CH, int64_t SHW, int64_t K, int64_t P, int interp, int64_t Nout, bool direct) {
  Geometry g{};
  const bool map_mode_gather = direct && K > 1;  // (K = 1 is the dense GEMM of the multiply-first adjoint)
  g.ok = true;
  g.Cp = padded_channels(CH);
  g.nchunks = num_chunks(g.Cp, (int)K);
  const int np = (int)align_up((size_t)Nout, 16);
  g.Npb = np > 256 ? 256 : np;
  g.nblk = (np + g.Npb - 1) / g.Npb;
  g.nt = direct ? (int)((P > 0 ? P : 1) * (interp == SPH_NEAREST ? 1 : 4)) : kPlanTaps;
  g.xh_bytes = align_up((size_t)(B * (SHW + 1)) * g.Cp * 2, 256);
  if ((SHW + 1) * g.Cp * 2 >= ((int64_t)1 << 31)) g.ok = false;
  g.wp_bytes = align_up((size_t)g.nblk * g.nchunks * g.Npb * kChunk * 2, 256);
  g.ok = g.ok && (size_t)K * kTileM * g.nt * sizeof(Tap) <= (size_t)kMaxTapBytes;
  // Pipeline depth.  Shared memory and L1 share one 256 KB array whose split moves in steps; a CTA that asks for more
  // than 196 KB leaves 28 KB of L1 for the gather instead of 60 KB, which costs more than a pipeline stage gains
  // (layer-4 input gradient of the encoder: 3 stages at 207 KB 3.97 ms, 2 stages at 158 KB 3.77 ms).  So: as many stages
  // as fit 196 KB, and only if two do not fit, as many as fit the whole array.
  constexpr size_t kSoftLimit = 196 * 1024;
  g.stages = 4;
  while (g.stages > 2 && gemm_smem_bytes(g.stages, g.Npb, (int)K, g.nt, direct) > kSoftLimit) g.stages--;
  if (gemm_smem_bytes(g.stages, g.Npb, (int)K, g.nt, direct) > kSoftLimit) {
    g.stages = 4;
    while (g.stages > 2 && gemm_smem_bytes(g.stages, g.Npb, (int)K, g.nt, direct) > (size_t)kSmemLimit) g.stages--;
  }
  // With at most 128 output columns the MMA of a chunk is short next to its gather, a deeper pipeline buys nothing, and
  // the shared memory two stages leave free goes to L1 (layer-2 forward of the encoder: 4 stages 1.14 ms, 2 stages 1.05 ms).
  if (direct && g.Npb <= 128 && map_mode_gather) g.stages = 2;
  g.smem = gemm_smem_bytes(g.stages, g.Npb, (int)K, g.nt, direct);
  if (g.smem > (size_t)kSmemLimit) g.ok = false;
  return g;
}

void to_nhwc(const void *src, __nv_bfloat16 *xh, int64_t B, int64_t CH, int Cp, int64_t HW, cudaStream_t st,
             const void *mask = nullptr) {
  nchw_to_nhwc_bf16_kernel<<<dim3(cdiv(HW + 1, 64), cdiv(Cp, 64), (unsigned)B), 256, 0, st>>>((const float *)src, xh, (int)CH, Cp, (int)HW,
                                                                                          (const float *)mask);
}

// Tensor map of the float32 output (B, Nout, GH, GW) with the epilogue's box: 16 pixels x 2 rows x kOutStageCh channels.
// Needs rows that start 16-byte aligned; returns false (plain stores are used then) if the map cannot be made.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return (EncodeTiledFn)f;
  }();
  return fn;
}

// The last few encoded maps are kept (a training loop stores to the same activation buffers every step).
struct OutMapSlot {
  float *out;
  int64_t B, Nout, GH, GW;
  CUtensorMap map;
};
constexpr int kOutMapSlots = 16;
thread_local OutMapSlot g_out_maps[kOutMapSlots];
thread_local int g_out_map_next = 0;

bool make_out_map(CUtensorMap *m, float *out, int64_t B, int64_t Nout, int64_t GH, int64_t GW);

bool cached_out_map(CUtensorMap *m, float *out, int64_t B, int64_t Nout, int64_t GH, int64_t GW) {
  for (int i = 0; i < kOutMapSlots; i++) {
    const OutMapSlot &s = g_out_maps[i];
    if (s.out == out && out != nullptr && s.B == B && s.Nout == Nout && s.GH == GH && s.GW == GW) {
      *m = s.map;
      return true;
    }
  }
  if (!make_out_map(m, out, B, Nout, GH, GW)) return false;
  OutMapSlot &s = g_out_maps[g_out_map_next];
  g_out_map_next = (g_out_map_next + 1) % kOutMapSlots;
  s.out = out; s.B = B; s.Nout = Nout; s.GH = GH; s.GW = GW; s.map = *m;
  return true;
}

bool make_out_map(CUtensorMap *m, float *out, int64_t B, int64_t Nout, int64_t GH, int64_t GW) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || out == nullptr || (GW & 3) != 0 || ((uintptr_t)out & 15) != 0) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)GW, (cuuint64_t)GH, (cuuint64_t)Nout, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)GW * 4, (cuuint64_t)GW * GH * 4, (cuuint64_t)Nout * GW * GH * 4};
  const cuuint32_t box[4] = {(cuuint32_t)kTW, 2, (cuuint32_t)kOutStageCh, 1}, estr[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor map of a channels-last bf16 copy (B, GH*GW + 1, pitch) seen as (B, GH, GW, pitch) with the image stride of
// GH*GW + 1 pixels; box = 16 channels x 16 pixels x 2 rows.
bool make_cl_map(CUtensorMap *m, __nv_bfloat16 *cl, int64_t B, int64_t pitch, int64_t GH, int64_t GW) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || cl == nullptr || (pitch & 7) != 0 || ((uintptr_t)cl & 15) != 0) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)pitch, (cuuint64_t)GW, (cuuint64_t)GH, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)pitch * 2, (cuuint64_t)GW * pitch * 2, (cuuint64_t)(GH * GW + 1) * pitch * 2};
  const cuuint32_t box[4] = {(cuuint32_t)kOutStageCh, (cuuint32_t)kTW, 2, 1}, estr[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, cl, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE, int NT, bool ROWS, bool LEAN>
void launch_gemm_l(TcParams p, int grid, size_t smem, cudaStream_t st) {
  CUtensorMap out_map, cl_map;
  memset(&out_map, 0, sizeof(out_map));
  memset(&cl_map, 0, sizeof(cl_map));
  p.use_out_map = (p.out_h == nullptr && cached_out_map(&out_map, p.out, p.B, p.Nout, p.g.GH, p.g.GW)) ? 1 : 0;
  // the copy leaves through its own tensor map when the float32 output does; otherwise with plain stores
  if (p.use_out_map && p.out_cl != nullptr && !make_cl_map(&cl_map, p.out_cl, p.B, p.cl_pitch, p.g.GH, p.g.GW)) p.use_out_map = 0;
  static int granted[kMaxDevices];
  ensure_dynamic_smem(tc_gemm_kernel<MODE, NT, ROWS, LEAN>, granted, smem);
  tc_gemm_kernel<MODE, NT, ROWS, LEAN><<<grid, kThreads, smem, st>>>(p, out_map, cl_map);
}
template <int MODE, int NT, bool ROWS = false>
void launch_gemm(const TcParams &p, int grid, size_t smem, cudaStream_t st) {
  if (p.g.Cp >= 64 && (MODE == MODE_PLAN || NT > 0)) {
    if constexpr (MODE == MODE_PLAN || NT > 0) launch_gemm_l<MODE, NT, ROWS, true>(p, grid, smem, st);
  } else {
    launch_gemm_l<MODE, NT, ROWS, false>(p, grid, smem, st);
  }
}

// ---- multiply-first adjoint -------------------------------------------------------------------------
// When the destination grid of an adjoint (conv dInput, transposed conv forward) is several times larger than the
// source grid (the map down-samples), gathering per destination pixel repeats the channel contraction for every
// destination pixel.  It is cheaper to contract first on the small grid - a dense tcgen05 GEMM that writes the
// bf16 column buffer T[b, o, k*Mp + m] - and then to run the plan gather over rows of T (the reference's own
// order: GEMM, then mapped_col2im, src/cpp/mapped_convolution_layer.cpp:69-86).
struct PremulGeometry {
  Geometry g;     // of the dense GEMM: one slot, CH channels, N = K * Mp
  int Mp;
  size_t t_bytes;
  bool use;
};

PremulGeometry premul_geometry(int64_t B, int64_t CH, int64_t SHW, int64_t K, int64_t M, int64_t n_dst) {
  PremulGeometry q{};
  q.Mp = (int)align_up((size_t)M, 8);
  q.g = geometry(B, CH, SHW, 1, 0, SPH_NEAREST, K * q.Mp, true);
  q.t_bytes = align_up((size_t)(B * SHW) * K * q.Mp * 2, 256);
  q.use = q.g.ok && n_dst >= 3 * SHW && q.t_bytes <= ((size_t)8 << 30) && CH >= 32;
  return q;
}

int tc_adjoint_premul(const PremulGeometry &q, const void *src, const void *plan, int64_t CH, int64_t SH, int64_t SW,
                      int64_t K, int64_t GH, int64_t GW, const void *wgt, int64_t sm_, int64_t sc, int64_t sk, const void *bias,
                      void *out, int64_t M, int64_t B, void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz) {
  const Geometry &g = q.g;
  if (!ws || ws_bytes < 256 + g.xh_bytes + g.wp_bytes + q.t_bytes) return SPH_ERR_WORKSPACE_TOO_SMALL;
  if ((uintptr_t)ws & 255) return SPH_ERR_INVALID_ARGUMENT;  // vector loads and bulk copies assume the alignment
  int *status = (int *)ws;
  __nv_bfloat16 *xh = (__nv_bfloat16 *)((char *)ws + 256);
  __nv_bfloat16 *wp = (__nv_bfloat16 *)((char *)ws + 256 + g.xh_bytes);
  __nv_bfloat16 *T = (__nv_bfloat16 *)((char *)ws + 256 + g.xh_bytes + g.wp_bytes);
  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return SPH_ERR_CUDA;
  if (fz.src_cl != nullptr) xh = (__nv_bfloat16 *)fz.src_cl;  // already converted (and masked) by the caller
  else to_nhwc(src, xh, B, CH, g.Cp, SH * SW, st, fz.mask);   // adjoint: src is grad_output
  const int64_t wtotal = (int64_t)g.nblk * g.nchunks * g.Npb * kChunk;
  premul_weight_image_kernel<<<cdiv(wtotal, 256), 256, 0, st>>>((const float *)wgt, wp, (int)M, q.Mp, (int)K, (int)CH, g.Npb, g.nblk,
                                                                g.nchunks, sm_, sc, sk);
  TcParams p{};
  p.g = Gather{xh, nullptr, nullptr, nullptr, g.Cp, (int)SH, (int)SW, 1, 0, (int)SH, (int)SW, SPH_NEAREST, 1};
  p.out_cl = nullptr; p.cl_pitch = 0;
  p.wp = wp; p.bias = nullptr; p.out = nullptr; p.out_h = T; p.out_pitch = (int)(K * q.Mp); p.status = status;
  p.B = (int)B; p.Nout = (int)(K * q.Mp); p.Npb = g.Npb; p.nblk = g.nblk; p.nchunks = g.nchunks;
  p.tiles_x = cdiv(SW, kTW); p.tiles_y = cdiv(SH, kTH); p.stages = g.stages;
  const int64_t tiles = (int64_t)B * p.tiles_x * p.tiles_y * g.nblk;
  launch_gemm<MODE_DIRECT, 1, true>(p, (int)(tiles < sm_count() ? tiles : sm_count()), g.smem, st);
  plan_gather_rows_kernel<<<dim3(cdiv(GH * GW, 128), (unsigned)B), 128, 0, st>>>(T, plan, (const float *)bias, (float *)out, (int)K,
                                                                                (int)M, q.Mp, (int)(SH * SW), (int)(GH * GW));
  return launch_status(fz.src_cl ? 3 : 4);
}

// Out[b,n,pix] (+bias) on the tensor cores.  src is (B,CH,SH,SW) float32; the GEMM pixels are the (GH,GW) grid.
int tc_gemm(bool use_plan, const void *src, const void *map, const void *iw, const void *plan, int64_t CH, int64_t SH,
            int64_t SW, int64_t K, int64_t P, int64_t GH, int64_t GW, int interp, const void *wgt, int64_t sn, int64_t sc,
            int64_t sk, const void *bias, void *out, int64_t Nout, int64_t B, void *ws, size_t ws_bytes, cudaStream_t st,
            const Fusion &fz = Fusion{}) {
  if (use_plan) {
    const PremulGeometry q = premul_geometry(B, CH, SH * SW, K, Nout, GH * GW);
    if (q.use) return tc_adjoint_premul(q, src, plan, CH, SH, SW, K, GH, GW, wgt, sn, sc, sk, bias, out, Nout, B, ws, ws_bytes, st, fz);
  }
  const Geometry g = geometry(B, CH, SH * SW, K, P, interp, Nout, !use_plan);
  if (!g.ok && (fz.active() || fz.out_cl != nullptr)) return SPH_ERR_UNSUPPORTED;
  if (fz.out_cl != nullptr && (use_plan || Nout % 8 != 0)) return SPH_ERR_UNSUPPORTED;
  if (!g.ok)  // shapes the tile kernel does not cover run on the exact SIMT kernels instead
    return simt_gemm<float>(use_plan, src, map, iw, plan, CH, SH, SW, K, P, GH * GW, interp, wgt, sn, sc, sk, bias, out, Nout, B, st);
  if (!ws || ws_bytes < 256 + g.xh_bytes + g.wp_bytes) return SPH_ERR_WORKSPACE_TOO_SMALL;
  if ((uintptr_t)ws & 255) return SPH_ERR_INVALID_ARGUMENT;  // vector loads and bulk copies assume the alignment
  int *status = (int *)ws;
  __nv_bfloat16 *xh = (__nv_bfloat16 *)((char *)ws + 256);
  __nv_bfloat16 *wp = (__nv_bfloat16 *)((char *)ws + 256 + g.xh_bytes);
  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return SPH_ERR_CUDA;
  if (fz.src_cl != nullptr) xh = (__nv_bfloat16 *)fz.src_cl;  // the caller keeps a channels-last copy of src
  else to_nhwc(src, xh, B, CH, g.Cp, SH * SW, st, use_plan ? fz.mask : nullptr);
  const int64_t wtotal = (int64_t)g.nblk * g.nchunks * g.Npb * kChunk;
  weight_image_kernel<<<cdiv(wtotal, 256), 256, 0, st>>>((const float *)wgt, wp, (int)Nout, (int)CH, g.Cp, (int)K, g.Npb, g.nblk,
                                                         g.nchunks, sn, sc, sk);
  TcParams p{};
  p.g = Gather{xh, (const float *)map, (const float *)iw, plan, g.Cp, (int)SH, (int)SW, (int)K, (int)P, (int)GH, (int)GW, interp, g.nt};
  p.wp = wp; p.bias = (const float *)bias; p.out = (float *)out; p.status = status;
  p.relu = (!use_plan && fz.relu_out) ? 1 : 0;
  p.out_cl = (__nv_bfloat16 *)fz.out_cl;
  p.cl_pitch = fz.out_cl ? padded_channels(Nout) : 0;
  p.B = (int)B; p.Nout = (int)Nout; p.Npb = g.Npb; p.nblk = g.nblk; p.nchunks = g.nchunks;
  p.tiles_x = cdiv(GW, kTW); p.tiles_y = cdiv(GH, kTH); p.stages = g.stages;
  const int64_t tiles = (int64_t)B * p.tiles_x * p.tiles_y * g.nblk;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  if (use_plan) launch_gemm<MODE_PLAN, kPlanTaps>(p, grid, g.smem, st);
  else if (g.nt == 4) launch_gemm<MODE_DIRECT, 4>(p, grid, g.smem, st);
  else if (g.nt == 1) launch_gemm<MODE_DIRECT, 1>(p, grid, g.smem, st);
  else launch_gemm<MODE_DIRECT, 0>(p, grid, g.smem, st);
  return launch_status(fz.src_cl ? 2 : 3);
}

// n_dst > 0: plan mode with that many destination pixels (may select the multiply-first adjoint)
size_t gemm_ws(int64_t B, int64_t CH, int64_t SHW, int64_t K, int64_t P, int interp, int64_t Nout, bool direct,
               int64_t n_dst = 0) {
  if (!direct) {
    const PremulGeometry q = premul_geometry(B, CH, SHW, K, Nout, n_dst);
    if (q.use) return 256 + q.g.xh_bytes + q.g.wp_bytes + q.t_bytes;
  }
  const Geometry g = geometry(B, CH, SHW, K, P, interp, Nout, direct);
  return g.ok ? 256 + g.xh_bytes + g.wp_bytes : 0;
}

struct DwGeometry {
  int Cp, nchunks, ngroups, mbs_total, nt, stages, splits, tap_rows, tiles_x, tiles_y, grp;
  size_t xh_bytes, gt_bytes, partial_bytes, bias_bytes, smem;
  bool ok;
};

DwGeometry dw_geometry(int64_t B, int64_t CH, int64_t SHW, int64_t K, int64_t P, int interp, int64_t Nout, int64_t GH,
                       int64_t GW, int64_t Cbias) {
  DwGeometry d{};
  d.Cp = padded_channels(CH);
  d.nchunks = num_chunks(d.Cp, (int)K);
  // GRP = 8 (one row block, twice the slots per step) leaves room for only two pipeline stages and measured
  // 1.9x slower on the encoder's layers than GRP = 4 with three stages, so it is not selected.
  d.grp = 4;
  d.ngroups = (d.nchunks + d.grp - 1) / d.grp;
  d.mbs_total = (int)((Nout + 127) / 128);
  d.nt = (int)((P > 0 ? P : 1) * (interp == SPH_NEAREST ? 1 : 4));
  d.tap_rows = d.Cp >= 64 ? d.grp : (int)std::min<int64_t>(K, (int64_t)d.grp * (64 / d.Cp));
  d.tiles_x = cdiv(GW, kTW);
  d.tiles_y = cdiv(GH, kDwTH);
  const int mbs_cta = 8 / d.grp;
  const int mbs = d.mbs_total >= mbs_cta ? mbs_cta : 1;
  d.ok = (size_t)d.tap_rows * kDwPix * d.nt * sizeof(Tap) <= (size_t)kDwMaxTapBytes;
  // pipeline depth: as for the forward-type kernel, stay within 196 KB of shared memory if two stages fit there
  // (layer-4 dW of the encoder: 3 stages at 209 KB 3.62 ms, 2 stages at 145 KB 3.32 ms)
  constexpr size_t kSoftLimit = 196 * 1024;
  d.stages = 4;
  while (d.stages > 2 && dw_smem_bytes(d.stages, d.grp, mbs, d.tap_rows, d.nt) > kSoftLimit) d.stages--;
  if (dw_smem_bytes(d.stages, d.grp, mbs, d.tap_rows, d.nt) > kSoftLimit) {
    d.stages = 4;
    while (d.stages > 2 && dw_smem_bytes(d.stages, d.grp, mbs, d.tap_rows, d.nt) > (size_t)kSmemLimit) d.stages--;
  }
  d.smem = dw_smem_bytes(d.stages, d.grp, mbs, d.tap_rows, d.nt);
  if (d.smem > (size_t)kSmemLimit) d.ok = false;
  const int64_t steps = B * d.tiles_x * d.tiles_y;
  const int zdim = (d.mbs_total + mbs_cta - 1) / mbs_cta;
  int64_t s = sm_count() / (d.ngroups * zdim);
  if (s < 1) s = 1;
  if (s > steps) s = steps;
  d.splits = (int)s;
  d.xh_bytes = align_up((size_t)(B * (SHW + 1)) * d.Cp * 2, 256);
  if ((SHW + 1) * d.Cp * 2 >= ((int64_t)1 << 31)) d.ok = false;
  d.gt_bytes = align_up((size_t)steps * d.mbs_total * kDwGtBytes, 256);
  d.partial_bytes = align_up((size_t)d.splits * d.mbs_total * 128 * d.nchunks * kChunk * 4, 256);
  d.bias_bytes = simt_bias_workspace(Cbias, 4) + align_up((size_t)steps * d.mbs_total * 128 * 4, 256) +
                 align_up((size_t)kRowSplits * Cbias * 4, 256);
  return d;
}

template <int NT, int GRP, bool WT>
void launch_dw_g(const DwParams &p, dim3 grid, size_t smem, cudaStream_t st) {
  static int granted[kMaxDevices];
  ensure_dynamic_smem(tc_dw_kernel<NT, GRP, WT>, granted, smem);
  tc_dw_kernel<NT, GRP, WT><<<grid, kThreads, smem, st>>>(p);
}
template <int NT>
void launch_dw(const DwParams &p, int grp, bool warp_taps, dim3 grid, size_t smem, cudaStream_t st) {
  if (grp == 8) launch_dw_g<NT, 8, false>(p, grid, smem, st);
  else if (warp_taps && NT > 0) launch_dw_g<NT, 4, (NT > 0)>(p, grid, smem, st);
  else launch_dw_g<NT, 4, false>(p, grid, smem, st);
}

// gw[n,ch,slot] = sum_{b,pix} A[b,n,pix] * im2col(src)[b,pix,(slot,ch)]; gb = sum of gbias_src over batch and pixels.
int tc_dw(const void *A, const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K,
          int64_t P, int64_t GH, int64_t GW, int interp, int64_t Nout, int64_t B, void *gw, int64_t sn, int64_t sc, int64_t sk,
          const void *gbias_src, int64_t Cbias, int64_t nbias, void *gb, void *ws, size_t ws_bytes, cudaStream_t st,
          const Fusion &fz = Fusion{}) {
  const DwGeometry d = dw_geometry(B, CH, SH * SW, K, P, interp, Nout, GH, GW, Cbias);
  // a masked gradient needs its bias sums from the (masked) imaging pass
  if (fz.active() && (!d.ok || !(gbias_src == A && Cbias == Nout && nbias == GH * GW))) return SPH_ERR_UNSUPPORTED;
  if (!d.ok)
    return simt_dw<float>(A, src, map, iw, CH, SH, SW, K, P, GH * GW, interp, Nout, B, gw, sn, sc, sk, gbias_src, Cbias, nbias, gb,
                          ws, ws_bytes, st);
  if (!ws || ws_bytes < 256 + d.xh_bytes + d.gt_bytes + d.partial_bytes + d.bias_bytes) return SPH_ERR_WORKSPACE_TOO_SMALL;
  if ((uintptr_t)ws & 255) return SPH_ERR_INVALID_ARGUMENT;  // vector loads and bulk copies assume the alignment
  char *w8 = (char *)ws;
  int *status = (int *)w8;
  __nv_bfloat16 *xh = (__nv_bfloat16 *)(w8 + 256);
  __nv_bfloat16 *gt = (__nv_bfloat16 *)(w8 + 256 + d.xh_bytes);
  float *partial = (float *)(w8 + 256 + d.xh_bytes + d.gt_bytes);
  void *bias_ws = w8 + 256 + d.xh_bytes + d.gt_bytes + d.partial_bytes;
  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return SPH_ERR_CUDA;
  if (fz.src_cl != nullptr) xh = (__nv_bfloat16 *)fz.src_cl;  // the caller keeps a channels-last copy of src
  else to_nhwc(src, xh, B, CH, d.Cp, SH * SW, st);
  // When the operand being imaged is also the tensor whose channel sums give the bias gradient (conv dW:
  // both are grad_output), the sums ride along with the imaging pass instead of re-reading the tensor.
  const bool fuse_bias = gbias_src == A && Cbias == Nout && nbias == GH * GW;
  const int64_t nblocks = B * d.tiles_x * d.tiles_y;
  float *row_part = (float *)((char *)bias_ws + simt_bias_workspace(Cbias, 4));
  float *part2 = (float *)((char *)row_part + align_up((size_t)nblocks * d.mbs_total * 128 * 4, 256));
  if (!fz.gt_ready)  // (else the caller's combined pre-pass has filled gt and row_part already)
    grad_image_kernel<<<dim3(d.tiles_x * d.tiles_y, d.mbs_total, (unsigned)B), 256, 0, st>>>(
        (const float *)A, gt, (int)Nout, (int)GH, (int)GW, d.tiles_x, d.tiles_y, d.mbs_total, fuse_bias ? row_part : nullptr,
        (const float *)fz.mask, nullptr, 0);
  DwParams p{};
  p.g = Gather{xh, (const float *)map, (const float *)iw, nullptr, d.Cp, (int)SH, (int)SW, (int)K, (int)P, (int)GH, (int)GW, interp, d.nt};
  p.gt = gt; p.partial = partial; p.status = status;
  p.B = (int)B; p.mbs_total = d.mbs_total; p.nchunks = d.nchunks; p.tiles_x = d.tiles_x; p.tiles_y = d.tiles_y;
  p.splits = d.splits; p.stages = d.stages; p.tap_rows = d.tap_rows;
  dim3 grid(d.ngroups, d.splits, (d.mbs_total + 8 / d.grp - 1) / (8 / d.grp));
  const bool warp_taps = d.Cp >= 64 && P == 0;  // one slot per chunk and one coordinate per slot
  if (d.nt == 4) launch_dw<4>(p, d.grp, warp_taps, grid, d.smem, st);
  else if (d.nt == 1) launch_dw<1>(p, d.grp, warp_taps, grid, d.smem, st);
  else launch_dw<0>(p, d.grp, false, grid, d.smem, st);
  tc_dw_reduce_kernel<<<cdiv(Nout * CH * K, 256), 256, 0, st>>>(partial, d.splits, d.mbs_total * 128, d.nchunks * kChunk, (int)Nout,
                                                               (int)CH, d.Cp, (int)K, sn, sc, sk, (float *)gw);
  note_launches(2 + (fz.src_cl ? 0 : 1) + (fz.gt_ready ? 0 : 1));
  if (fuse_bias) {
    row_sum_split_kernel<<<dim3(cdiv(Cbias, 128), kRowSplits), 128, 0, st>>>(row_part, nblocks, d.mbs_total * 128, (int)Cbias, part2);
    row_sum_final_kernel<<<cdiv(Cbias, 128), 128, 0, st>>>(part2, (int)Cbias, (float *)gb);
    return launch_status(2);
  }
  return simt_bias_grad<float>(gbias_src, B, Cbias, nbias, gb, bias_ws, st);
}

size_t dw_ws(int64_t B, int64_t CH, int64_t SHW, int64_t K, int64_t P, int interp, int64_t Nout, int64_t GH, int64_t GW,
             int64_t Cbias) {
  const DwGeometry d = dw_geometry(B, CH, SHW, K, P, interp, Nout, GH, GW, Cbias);
  if (!d.ok) return simt_dw_workspace(B, GH * GW, Nout, CH, K, Cbias, 4);
  return 256 + d.xh_bytes + d.gt_bytes + d.partial_bytes + d.bias_bytes;
}

}  // namespace

// Tracing aid (sph_trace_phases): events the next combined backward call on this thread records at its phase boundaries.
thread_local cudaEvent_t g_phase_events[4];
thread_local int g_phase_count = 0;

static void mark_phase(int i, cudaStream_t st) {
  if (i < g_phase_count && g_phase_events[i] != nullptr) cudaEventRecord(g_phase_events[i], st);
}

namespace {
#include "conv_tc_thin.cuh"
}  // namespace

int tc_fill_companion(const void *x, void *x_cl, int64_t B, int64_t C, int64_t HW, cudaStream_t st) {
  to_nhwc(x, (__nv_bfloat16 *)x_cl, B, C, padded_channels(C), HW, st);
  return launch_status();
}

bool tc_thin_backward_ok(int64_t CH, int64_t K, int64_t N, int64_t npix) { return thin_bwd_ok(CH, K, N, npix); }
size_t tc_thin_backward_workspace(int64_t B, int64_t CH, int64_t K, int64_t npix, bool with_dx) {
  return thin_bwd_layout(B, CH, K, npix, with_dx).total;
}
int tc_thin_conv_backward(const void *gout, const void *act, const void *x, const void *plan, const void *map, const void *iw,
                          const void *weight, void *gx, void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                          int64_t OH, int64_t OW, int64_t K, int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st) {
  return tc_thin_backward(gout, act, x, plan, map, iw, weight, gx, gw, gb, B, Cin, Cout, IH, IW, OH, OW, K, P, interp, ws, ws_bytes, st);
}

bool tc_thin_forward_ok(int64_t CH, int64_t K, int64_t Nout, int64_t GW) { return thin_fwd_ok(CH, K, Nout, GW); }
size_t tc_thin_forward_workspace(int64_t Nout) { return thin_fwd_workspace(Nout); }
int tc_thin_conv_forward(const void *x, const void *map, const void *iw, const void *weight, const void *bias, void *out, int64_t B,
                         int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int interp,
                         void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz) {
  return tc_thin_forward(x, map, iw, Cin, IH, IW, K, P, OH, OW, interp, weight, Cin * K, K, 1, bias, out, Cout, B, ws, ws_bytes, st, fz);
}

size_t tc_workspace_bytes(int op, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                          int64_t K, int64_t P, int interp) {
  switch (op) {
    case SPH_CONV_FORWARD: return gemm_ws(B, Cin, IH * IW, K, P, interp, Cout, true);
    case SPH_CONV_BACKWARD_INPUT: return gemm_ws(B, Cout, OH * OW, K, 0, 0, Cin, false, IH * IW);
    case SPH_CONV_BACKWARD_WEIGHT: return dw_ws(B, Cin, IH * IW, K, P, interp, Cout, OH, OW, Cout);
    case SPH_TCONV_FORWARD: return gemm_ws(B, Cin, IH * IW, K, 0, 0, Cout, false, OH * OW);
    case SPH_TCONV_BACKWARD_INPUT: return gemm_ws(B, Cout, OH * OW, K, P, interp, Cin, true);
    case SPH_TCONV_BACKWARD_WEIGHT: return dw_ws(B, Cout, OH * OW, K, P, interp, Cin, IH, IW, Cout);
    default: return 0;
  }
}

int tc_conv_forward(const void *x, const void *map, const void *iw, const void *weight, const void *bias, void *out,
                    int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                    int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz) {
  return tc_gemm(false, x, map, iw, nullptr, Cin, IH, IW, K, P, OH, OW, interp, weight, Cin * K, K, 1, bias, out, Cout, B, ws,
                 ws_bytes, st, fz);
}

int tc_conv_backward_input(const void *gout, const void *plan, const void *weight, void *gx, int64_t B, int64_t Cin,
                           int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, void *ws,
                           size_t ws_bytes, cudaStream_t st, const Fusion &fz) {
  return tc_gemm(true, gout, nullptr, nullptr, plan, Cout, OH, OW, K, 0, IH, IW, 0, weight, K, Cin * K, 1, nullptr, gx, Cin, B, ws,
                 ws_bytes, st, fz);
}

int tc_conv_backward_weight(const void *gout, const void *x, const void *map, const void *iw, void *gw, void *gb,
                            int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                            int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz) {
  return tc_dw(gout, x, map, iw, Cin, IH, IW, K, P, OH, OW, interp, Cout, B, gw, Cin * K, K, 1, gout, Cout, OH * OW, gb, ws,
               ws_bytes, st, fz);
}

// Combined backward of one convolution.  grad_output feeds two kernels in two layouts - channels-last bf16 for the
// input-gradient gather, 128-row tile images for the weight-gradient MMA - and, with a fused ReLU, has to be masked
// for both.  One pre-pass reads it (and the mask) once and writes both, where the separate entry points read it
// twice; the reference likewise computes all three gradients in one call
// (ext_modules/include/layers/mapped_convolution_layer.h:89-134).  Workspace: the input-gradient part first, then
// the weight-gradient part, each laid out as its own operator expects.
size_t tc_conv_backward_workspace(int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                                  int64_t K, int64_t P, int interp) {
  const size_t a = gemm_ws(B, Cout, OH * OW, K, 0, 0, Cin, false, IH * IW);
  const DwGeometry d = dw_geometry(B, Cin, IH * IW, K, P, interp, Cout, OH, OW, Cout);
  if (a == 0 || !d.ok) return 0;
  return align_up(a, 256) + dw_ws(B, Cin, IH * IW, K, P, interp, Cout, OH, OW, Cout);
}

int tc_conv_backward(const void *gout, const void *x, const void *plan, const void *map, const void *iw, const void *weight,
                     void *gx, void *gw, void *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH,
                     int64_t OW, int64_t K, int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz) {
  const size_t dx_bytes = gemm_ws(B, Cout, OH * OW, K, 0, 0, Cin, false, IH * IW);
  const DwGeometry d = dw_geometry(B, Cin, IH * IW, K, P, interp, Cout, OH, OW, Cout);
  if (dx_bytes == 0 || !d.ok) return SPH_ERR_UNSUPPORTED;  // one of the two runs on other kernels: use the separate entry points
  const size_t dw_bytes = dw_ws(B, Cin, IH * IW, K, P, interp, Cout, OH, OW, Cout);
  if (!ws || ws_bytes < align_up(dx_bytes, 256) + dw_bytes) return SPH_ERR_WORKSPACE_TOO_SMALL;
  if ((uintptr_t)ws & 255) return SPH_ERR_INVALID_ARGUMENT;
  char *ws_dx = (char *)ws, *ws_dw = (char *)ws + align_up(dx_bytes, 256);
  // where the two operators expect their operands (see tc_gemm / tc_adjoint_premul and tc_dw)
  const int cp_go = padded_channels(Cout);
  __nv_bfloat16 *go_cl = (__nv_bfloat16 *)(ws_dx + 256);
  __nv_bfloat16 *gt = (__nv_bfloat16 *)(ws_dw + 256 + d.xh_bytes);
  char *bias_ws = ws_dw + 256 + d.xh_bytes + d.gt_bytes + d.partial_bytes;
  float *row_part = (float *)(bias_ws + simt_bias_workspace(Cout, 4));
  const size_t npix = (size_t)(OH * OW);
  struct PhaseScope {  // the event list is consumed by this call, whatever its outcome
    ~PhaseScope() { g_phase_count = 0; }
  } phase_scope;
  mark_phase(0, st);
  // the zero pixel behind every image of the channels-last copy (unused taps point there)
  if (cudaMemset2DAsync((char *)go_cl + npix * cp_go * 2, (npix + 1) * cp_go * 2, 0, (size_t)cp_go * 2, (size_t)B, st) != cudaSuccess)
    return SPH_ERR_CUDA;
  grad_image_kernel<<<dim3(d.tiles_x * d.tiles_y, d.mbs_total, (unsigned)B), 256, 0, st>>>(
      (const float *)gout, gt, (int)Cout, (int)OH, (int)OW, d.tiles_x, d.tiles_y, d.mbs_total, row_part, (const float *)fz.mask,
      go_cl, cp_go);
  note_launches(1);
  mark_phase(1, st);
  // channels between mbs_total * 128 and cp_go do not exist (cp_go <= mbs_total * 128), so the copy is complete
  Fusion fx;
  fx.src_cl = go_cl;  // already masked
  int rc = tc_gemm(true, gout, nullptr, nullptr, plan, Cout, OH, OW, K, 0, IH, IW, 0, weight, K, Cin * K, 1, nullptr, gx, Cin, B,
                   ws_dx, dx_bytes, st, fx);
  if (rc != SPH_OK) return rc;
  mark_phase(2, st);
  Fusion fw;
  fw.src_cl = fz.src_cl;  // channels-last copy of x, if the caller keeps one
  fw.gt_ready = true;
  rc = tc_dw(gout, x, map, iw, Cin, IH, IW, K, P, OH, OW, interp, Cout, B, gw, Cin * K, K, 1, gout, Cout, OH * OW, gb, ws_dw,
             dw_bytes, st, fw);
  mark_phase(3, st);
  return rc;
}

int tc_tconv_forward(const void *x, const void *plan, const void *weight, const void *bias, void *out, int64_t B,
                     int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, void *ws,
                     size_t ws_bytes, cudaStream_t st) {
  return tc_gemm(true, x, nullptr, nullptr, plan, Cin, IH, IW, K, 0, OH, OW, 0, weight, K, Cout * K, 1, bias, out, Cout, B, ws,
                 ws_bytes, st);
}

int tc_tconv_backward_input(const void *gout, const void *map, const void *iw, const void *weight, void *gx, int64_t B,
                            int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                            int interp, void *ws, size_t ws_bytes, cudaStream_t st) {
  return tc_gemm(false, gout, map, iw, nullptr, Cout, OH, OW, K, P, IH, IW, interp, weight, Cout * K, K, 1, nullptr, gx, Cin, B,
                 ws, ws_bytes, st);
}

int tc_tconv_backward_weight(const void *gout, const void *x, const void *map, const void *iw, void *gw, void *gb,
                             int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                             int64_t K, int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st) {
  return tc_dw(x, gout, map, iw, Cout, OH, OW, K, P, IH, IW, interp, Cin, B, gw, Cout * K, K, 1, gout, Cout, OH * OW, gb, ws,
               ws_bytes, st);
}

}  // namespace sph

// ---- device status and the bounded-wait self check ---------------------------------------------------------
namespace sph {
namespace {
// One CTA allocates tensor memory, then every thread waits on an mbarrier that nothing ever arrives at.  The wait is
// the same bounded wait the convolution kernels use, with the caller's (short) limit: it must run out, the CTA must
// free its tensor memory and return normally, and the give-up must show in *status and in the sticky device word.
__global__ void __launch_bounds__(128) bounded_wait_check_kernel(unsigned long long limit_ns, int *status) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_ptr;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 0) {
    tc::tmem_alloc(&tmem_ptr, 32);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t taddr = tmem_ptr;
  const bool done = tc::mbar_wait(&bar, 0, &abort_flag, limit_ns);
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(taddr, 32);
  if (tid == 0) {
    *status = (abort_flag && !done) ? 1 : 0;
    if (abort_flag) g_wait_status = 1;
  }
}
}  // namespace
}  // namespace sph

SPH_TU_STATUS(conv_tc)
#ifdef SPH_BOUNDS_CHECK
extern "C" {
int sph_tu_status_resample(int);
int sph_tu_status_plan(int);
int sph_tu_status_pool(int);
int sph_tu_status_conv_simt(int);
int sph_tu_status_conv_small(int);
}
#endif

extern "C" int sph_device_status(int *status, int reset) {
  if (!status) return SPH_ERR_INVALID_ARGUMENT;
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, sph::g_wait_status, sizeof(int)) != cudaSuccess) return SPH_ERR_CUDA;
  if (reset && v) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(sph::g_wait_status, &zero, sizeof(int)) != cudaSuccess) return SPH_ERR_CUDA;
  }
  v = v ? 1 : 0;
#ifdef SPH_BOUNDS_CHECK
  // checked build: bit 1 = some kernel met an index outside its range (and skipped the access)
  int (*const parts[])(int) = {sph_tu_status_resample, sph_tu_status_plan, sph_tu_status_pool, sph_tu_status_conv_simt,
                               sph_tu_status_conv_small, sph_tu_status_conv_tc};
  for (auto f : parts) {
    const int r = f(reset);
    if (r < 0) return SPH_ERR_CUDA;
    if (r) v |= 2;
  }
#endif
  *status = v;
  return SPH_OK;
}

extern "C" int sph_build_is_checked(void) {
#ifdef SPH_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

extern "C" int sph_trace_phases(void **events, int n_events) {
  if (n_events < 0 || n_events > 4 || (n_events > 0 && !events)) return SPH_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < n_events; i++) sph::g_phase_events[i] = (cudaEvent_t)events[i];
  sph::g_phase_count = n_events;
  return SPH_OK;
}

extern "C" int sph_debug_bounded_wait(unsigned long long limit_ns, int *status, void *stream) {
  if (!status || limit_ns == 0 || limit_ns > 1000000000ull) return SPH_ERR_INVALID_ARGUMENT;
  sph::bounded_wait_check_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(limit_ns, status);
  return sph::launch_status();
}

#ifdef SPH_TC_TIMING
// out[16]: accumulated counters of tc_gemm_kernel (0 fill, 1 chunk loop, 2 tile barrier, 3 MMA wait for operands,
// 4 MMA wait for a free accumulator, 5 epilogue wait for the accumulator, 6 epilogue drain, 7 tiles); reset != 0 clears.
extern "C" int sph_debug_tc_timing(unsigned long long *out, int reset) {
  if (out && cudaMemcpyFromSymbol(out, sph::g_tc_timing, sizeof(unsigned long long) * 16) != cudaSuccess) return 1;
  if (reset) {
    unsigned long long z[16] = {0};
    if (cudaMemcpyToSymbol(sph::g_tc_timing, z, sizeof(z)) != cudaSuccess) return 1;
  }
  return 0;
}
#endif
