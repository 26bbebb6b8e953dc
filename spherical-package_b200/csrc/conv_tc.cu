// bf16 tensor-core path of the mapped convolution family (float32 tensors,
// bf16 operands, fp32 accumulation in tensor memory).
//
// One persistent, warp-specialised kernel computes
//     Out[b, n, pix] = sum_{slot, ch} Col[b, pix, (slot, ch)] * Wt[n, (slot, ch)]  (+ bias[n])
// for a tile of 128 pixels at a time.  Col is never written to HBM: eight
// producer warps gather it (through the sample map's taps, or through a scatter
// plan for the adjoint direction) from a channels-last bf16 copy of the source
// image straight into the 128-byte-swizzled shared-memory layout tcgen05.mma
// reads; the matching weight tile arrives by one bulk async copy per stage from a
// pre-swizzled bf16 image of the weights; one thread issues the MMAs into a
// double-buffered TMEM accumulator; four epilogue warps read TMEM, add the bias
// and store coalesced NCHW rows.  The reference does the same work per image as
// im2col kernel + cuBLAS SGEMM + bias kernel with a (Cin*K, OH*OW) column buffer
// in HBM (src/cuda/mapped_convolution_layer.cu:16-74).
#include <cuda_bf16.h>

#include "common.cuh"
#include "conv_internal.h"
#include "tc_common.cuh"

namespace sph {
namespace {

using namespace tc;

constexpr int kTileM = 128;          // pixels per tile = TMEM lanes
constexpr int kChunk = 64;           // GEMM-K columns per pipeline stage (one 128-byte swizzle row)
constexpr int kAStageBytes = kTileM * 128;
constexpr int kEpilogueWarps = 4, kProducerWarps = 8;
constexpr int kProducerThreads = 32 * kProducerWarps;
constexpr int kThreads = 32 * (kEpilogueWarps + 1 + kProducerWarps);
constexpr int kFirstProducerThread = 32 * (kEpilogueWarps + 1);
constexpr int kMaxTapBytes = 40 * 1024;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kTmemCols = 512;

enum { MODE_DIRECT = 0, MODE_PLAN = 1 };

struct TcParams {
  const __nv_bfloat16 *xh;  // (B, SH*SW, Cp) channels-last bf16 source
  const __nv_bfloat16 *wp;  // weight tile images: [nblk][nchunks][Npb rows][64] bf16, 128B-swizzled
  const float *bias;        // (Nout) or null
  float *out;               // (B, Nout, npix)
  const float *map, *iw;    // direct mode: sample map (+ interpolation weights)
  const void *plan;         // plan mode
  int *status;              // set to 1 if a bounded wait gave up
  int B, Cp, SH, SW, K, P, npix, Nout, Npb, nblk, nchunks, KC, tiles_per_image, interp, nt, stages;
};

struct Smem {
  uint8_t *A, *Bw;
  int *tap_off;
  float *tap_w;
  uint64_t *full, *empty, *tfull, *tempty;
  uint32_t *tmem_ptr;
  volatile int *abort_flag;
};

__host__ __device__ inline size_t smem_bytes(int stages, int Npb, int K, int nt, bool direct) {
  size_t s = 1024;  // alignment slack
  s += (size_t)stages * (kAStageBytes + Npb * 128);
  if (direct) s += (size_t)K * kTileM * nt * 8;
  s += 8 * (2 * stages + 4) + 16;
  return s;
}

__device__ inline Smem carve(uint8_t *raw, const TcParams &p, bool direct) {
  Smem s;
  uint8_t *b = (uint8_t *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  s.A = b;
  s.Bw = b + (size_t)p.stages * kAStageBytes;
  uint8_t *q = s.Bw + (size_t)p.stages * p.Npb * 128;
  s.tap_off = (int *)q;
  s.tap_w = (float *)(q + (direct ? (size_t)p.K * kTileM * p.nt * 4 : 0));
  q += direct ? (size_t)p.K * kTileM * p.nt * 8 : 0;
  s.full = (uint64_t *)q;
  s.empty = s.full + p.stages;
  s.tfull = s.empty + p.stages;
  s.tempty = s.tfull + 2;
  s.tmem_ptr = (uint32_t *)(s.tempty + 2);
  s.abort_flag = (volatile int *)(s.tmem_ptr + 1);
  return s;
}

__device__ __forceinline__ void producer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory"); }

// acc[0..7] += w * (8 bf16 channels in q)
__device__ __forceinline__ void fma8(float (&acc)[8], float w, const uint4 &q) {
  acc[0] = fmaf(w, bf16_lo(q.x), acc[0]);
  acc[1] = fmaf(w, bf16_hi(q.x), acc[1]);
  acc[2] = fmaf(w, bf16_lo(q.y), acc[2]);
  acc[3] = fmaf(w, bf16_hi(q.y), acc[3]);
  acc[4] = fmaf(w, bf16_lo(q.z), acc[4]);
  acc[5] = fmaf(w, bf16_hi(q.z), acc[5]);
  acc[6] = fmaf(w, bf16_lo(q.w), acc[6]);
  acc[7] = fmaf(w, bf16_hi(q.w), acc[7]);
}

// Taps of map slot (pix, slot) into the shared tap table (nt entries; unused ones get weight 0).
template <int INTERP>
__device__ __forceinline__ void fill_taps(const TcParams &p, int pix, int slot, int *off, float *w) {
  const int PP = p.P > 0 ? p.P : 1;
  const size_t e0 = ((size_t)pix * p.K + slot) * PP;
  Taps<float> t;
  int n = 0;
  for (int q = 0; q < PP; q++) {
    decode<float, INTERP>(__ldg(p.map + 2 * (e0 + q)), __ldg(p.map + 2 * (e0 + q) + 1), p.SH, p.SW, t);
    const float wq = p.P > 0 ? __ldg(p.iw + e0 + q) : 1.0f;
#pragma unroll
    for (int i = 0; i < TapCount<INTERP>::value; i++, n++) {
      const bool ok = t.off[i] >= 0;
      off[n] = ok ? t.off[i] : 0;
      w[n] = ok ? wq * t.w[i] : 0.0f;
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1) tc_gemm_kernel(const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const Smem sm = carve(smem_raw, p, MODE == MODE_DIRECT);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.stages;

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
  const int total_tiles = p.B * p.tiles_per_image * p.nblk;
  const size_t shw = (size_t)p.SH * p.SW;

  if (warp < kEpilogueWarps) {
    // ---------------- epilogue: TMEM -> registers -> (+bias) -> global ----------------
    int tl = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tl++) {
      const int nb = tile % p.nblk, rest = tile / p.nblk;
      const int b = rest / p.tiles_per_image, pix = (rest % p.tiles_per_image) * kTileM + warp * 32 + lane;
      const int buf = tl & 1;
      if (!mbar_wait(sm.tfull + buf, (tl >> 1) & 1, sm.abort_flag)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * 256;
      float *orow = p.out + ((size_t)b * p.Nout) * p.npix + pix;
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
        if (pix < p.npix) {
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const int n = nb * p.Npb + n0 + j;
            if (n < p.Nout && n0 + j < p.Npb)
              orow[(size_t)n * p.npix] = __uint_as_float(r[j]) + (p.bias ? __ldg(p.bias + n) : 0.0f);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.tempty + buf);
    }
  } else if (warp == kEpilogueWarps) {
    // ---------------- MMA issuer (one thread) ----------------
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16(kTileM, p.Npb, 0, 0);
      int it = 0, tl = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < total_tiles; tile += gridDim.x, tl++) {
        const int buf = tl & 1;
        if (!mbar_wait(sm.tempty + buf, ((tl >> 1) & 1) ^ 1, sm.abort_flag)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + buf * 256;
        for (int chunk = 0; chunk < p.nchunks; chunk++, it++) {
          const int s = it % S;
          if (!mbar_wait(sm.full + s, (it / S) & 1, sm.abort_flag)) { alive = false; break; }
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
    int it = 0;
    bool alive = true;
    PlanView<float> pv{};
    bool plan_ok = true;
    if (MODE == MODE_PLAN) pv = plan_view<float>(p.plan, p.npix * p.K, plan_ok);
    for (int tile = blockIdx.x; alive && tile < total_tiles; tile += gridDim.x) {
      const int nb = tile % p.nblk, rest = tile / p.nblk;
      const int b = rest / p.tiles_per_image, pix0 = (rest % p.tiles_per_image) * kTileM;
      const __nv_bfloat16 *img = p.xh + (size_t)b * shw * p.Cp;
      if (MODE == MODE_DIRECT) {
        producer_bar();  // every producer is done reading the previous tile's taps
        for (int idx = pt; idx < p.K * kTileM; idx += kProducerThreads) {
          const int slot = idx / kTileM, pl = idx % kTileM, pix = pix0 + pl;
          int *off = sm.tap_off + (size_t)idx * p.nt;
          float *w = sm.tap_w + (size_t)idx * p.nt;
          if (pix < p.npix) {
            SPH_DISPATCH_INTERP(p.interp, fill_taps<INTERP>(p, pix, slot, off, w));
          } else {
            for (int i = 0; i < p.nt; i++) { off[i] = 0; w[i] = 0.0f; }
          }
        }
        producer_bar();
      }
      for (int chunk = 0; chunk < p.nchunks; chunk++, it++) {
        const int s = it % S;
        if (!mbar_wait(sm.empty + s, ((it / S) & 1) ^ 1, sm.abort_flag)) { alive = false; break; }
        if (pt == 0) {
          const uint32_t bytes = (uint32_t)p.Npb * 128;
          mbar_arrive_expect_tx(sm.full + s, bytes);
          bulk_copy_g2s(sm.Bw + (size_t)s * bytes, p.wp + ((size_t)nb * p.nchunks + chunk) * p.Npb * kChunk, bytes, sm.full + s);
        }
        uint8_t *As = sm.A + (size_t)s * kAStageBytes;
#pragma unroll 2
        for (int r = 0; r < kTileM * 8 / kProducerThreads; r++) {
          const int idx = pt + r * kProducerThreads, pl = idx >> 3, v = idx & 7;
          const int j = chunk * kChunk + v * 8;
          float acc[8];
#pragma unroll
          for (int i = 0; i < 8; i++) acc[i] = 0.0f;
          if (j < p.KC) {
            const int slot = j / p.Cp, c0 = j - slot * p.Cp;
            if (MODE == MODE_DIRECT) {
              const int *off = sm.tap_off + (size_t)(slot * kTileM + pl) * p.nt;
              const float *w = sm.tap_w + (size_t)(slot * kTileM + pl) * p.nt;
              for (int t = 0; t < p.nt; t++) {
                const float wt = w[t];
                if (wt != 0.0f) fma8(acc, wt, __ldg((const uint4 *)(img + (size_t)off[t] * p.Cp + c0)));
              }
            } else if (plan_ok && pix0 + pl < p.npix) {
              const int key = (pix0 + pl) * p.K + slot;
              const int e0 = __ldg(pv.offsets + key), e1 = __ldg(pv.offsets + key + 1);
              for (int e = e0; e < e1; e++)
                fma8(acc, __ldg(pv.w + e), __ldg((const uint4 *)(img + (size_t)__ldg(pv.src + e) * p.Cp + c0)));
            }
          }
          uint4 o;
          o.x = pack_bf16(acc[0], acc[1]);
          o.y = pack_bf16(acc[2], acc[3]);
          o.z = pack_bf16(acc[4], acc[5]);
          o.w = pack_bf16(acc[6], acc[7]);
          *(uint4 *)(As + pl * 128 + ((v ^ (pl & 7)) << 4)) = o;
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
  if (tid == 0 && *sm.abort_flag) *p.status = 1;
}

// (B, C, HW) float32 -> (B, HW, Cp) bf16, channels beyond C zero.  32 pixels x 64 channels per block.
__global__ void __launch_bounds__(256) nchw_to_nhwc_bf16_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ y,
                                                                 int C, int Cp, int HW) {
  __shared__ float tile[64][33];
  const int b = blockIdx.z, c0 = blockIdx.y * 64, p0 = blockIdx.x * 32;
  const int tid = threadIdx.x;
  for (int i = tid; i < 64 * 32; i += 256) {
    const int c = i >> 5, pp = i & 31;
    tile[c][pp] = (c0 + c < C && p0 + pp < HW) ? __ldg(x + ((size_t)b * C + c0 + c) * HW + p0 + pp) : 0.0f;
  }
  __syncthreads();
  const int pp = tid >> 3, v = tid & 7;
  if (p0 + pp < HW && c0 + v * 8 < Cp) {
    uint4 o;
    o.x = pack_bf16(tile[v * 8 + 0][pp], tile[v * 8 + 1][pp]);
    o.y = pack_bf16(tile[v * 8 + 2][pp], tile[v * 8 + 3][pp]);
    o.z = pack_bf16(tile[v * 8 + 4][pp], tile[v * 8 + 5][pp]);
    o.w = pack_bf16(tile[v * 8 + 6][pp], tile[v * 8 + 7][pp]);
    *(uint4 *)(y + ((size_t)b * HW + p0 + pp) * Cp + c0 + v * 8) = o;
  }
}

// Weights -> bf16 tile images.  Element (n, j = slot*Cp + ch) of block nb, chunk j/64 sits at row n, 16-byte
// chunk ((j%64)/8) ^ (n&7) of a 128-byte row.  The source is addressed W[n*sn + ch*sc + slot*sk].
__global__ void weight_image_kernel(const float *__restrict__ w, __nv_bfloat16 *__restrict__ wp, int Nout, int CH, int Cp,
                                    int K, int Npb, int nblk, int nchunks, int64_t sn, int64_t sc, int64_t sk) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)nblk * nchunks * Npb * kChunk;
  if (i >= total) return;
  const int col = (int)(i % kChunk), n = (int)((i / kChunk) % Npb), chunk = (int)((i / ((int64_t)kChunk * Npb)) % nchunks);
  const int nb = (int)(i / ((int64_t)kChunk * Npb * nchunks));
  const int j = chunk * kChunk + col, slot = j / Cp, ch = j % Cp, ng = nb * Npb + n;
  const float v = (ng < Nout && slot < K && ch < CH) ? __ldg(w + ng * sn + ch * sc + slot * sk) : 0.0f;
  const int v16 = col >> 3, e = col & 7;
  wp[(((int64_t)nb * nchunks + chunk) * Npb + n) * kChunk + ((v16 ^ (n & 7)) << 3) + e] = __float2bfloat16(v);
}

struct Geometry {
  int Cp, KC, nchunks, Npb, nblk, nt, stages;
  size_t xh_bytes, wp_bytes, smem;
  bool ok;
};

Geometry geometry(int64_t B, int64_t CH, int64_t SHW, int64_t K, int64_t P, int interp, int64_t Nout, bool direct) {
  Geometry g{};
  g.Cp = (int)align_up((size_t)CH, 8);
  if (g.Cp > 64) g.Cp = (int)align_up((size_t)CH, 64);
  else while (64 % g.Cp) g.Cp += 8;            // a 16-byte vector never straddles two slots and slots tile a chunk
  g.KC = (int)(K * g.Cp);
  g.nchunks = (g.KC + kChunk - 1) / kChunk;
  const int np = (int)align_up((size_t)Nout, 16);
  g.Npb = np > 256 ? 256 : np;
  g.nblk = (np + g.Npb - 1) / g.Npb;
  g.nt = (int)((P > 0 ? P : 1) * (interp == SPH_NEAREST ? 1 : 4));
  g.xh_bytes = align_up((size_t)(B * SHW) * g.Cp * 2, 256);
  g.wp_bytes = align_up((size_t)g.nblk * g.nchunks * g.Npb * kChunk * 2, 256);
  g.ok = !direct || (size_t)K * kTileM * g.nt * 8 <= (size_t)kMaxTapBytes;
  g.stages = 4;
  while (g.stages > 2 && smem_bytes(g.stages, g.Npb, (int)K, g.nt, direct) > (size_t)kSmemLimit) g.stages--;
  g.smem = smem_bytes(g.stages, g.Npb, (int)K, g.nt, direct);
  if (g.smem > (size_t)kSmemLimit) g.ok = false;
  return g;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

// Out[b,n,pix] (+bias) on the tensor cores.  src is (B,CH,SH,SW) float32.
int tc_gemm(bool use_plan, const void *src, const void *map, const void *iw, const void *plan, int64_t CH, int64_t SH,
            int64_t SW, int64_t K, int64_t P, int64_t npix, int interp, const void *wgt, int64_t sn, int64_t sc, int64_t sk,
            const void *bias, void *out, int64_t Nout, int64_t B, void *ws, size_t ws_bytes, cudaStream_t st) {
  const Geometry g = geometry(B, CH, SH * SW, K, P, interp, Nout, !use_plan);
  if (!g.ok)  // shapes the tile kernel does not cover run on the exact SIMT kernels instead
    return simt_gemm<float>(use_plan, src, map, iw, plan, CH, SH, SW, K, P, npix, interp, wgt, sn, sc, sk, bias, out, Nout, B, st);
  if (!ws || ws_bytes < 256 + g.xh_bytes + g.wp_bytes) return SPH_ERR_WORKSPACE_TOO_SMALL;
  int *status = (int *)ws;
  __nv_bfloat16 *xh = (__nv_bfloat16 *)((char *)ws + 256);
  __nv_bfloat16 *wp = (__nv_bfloat16 *)((char *)ws + 256 + g.xh_bytes);
  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return SPH_ERR_CUDA;
  const int HW = (int)(SH * SW);
  nchw_to_nhwc_bf16_kernel<<<dim3(cdiv(HW, 32), cdiv(g.Cp, 64), (unsigned)B), 256, 0, st>>>((const float *)src, xh, (int)CH, g.Cp, HW);
  const int64_t wtotal = (int64_t)g.nblk * g.nchunks * g.Npb * kChunk;
  weight_image_kernel<<<cdiv(wtotal, 256), 256, 0, st>>>((const float *)wgt, wp, (int)Nout, (int)CH, g.Cp, (int)K, g.Npb, g.nblk,
                                                         g.nchunks, sn, sc, sk);
  TcParams p{};
  p.xh = xh; p.wp = wp; p.bias = (const float *)bias; p.out = (float *)out;
  p.map = (const float *)map; p.iw = (const float *)iw; p.plan = plan; p.status = status;
  p.B = (int)B; p.Cp = g.Cp; p.SH = (int)SH; p.SW = (int)SW; p.K = (int)K; p.P = (int)P; p.npix = (int)npix;
  p.Nout = (int)Nout; p.Npb = g.Npb; p.nblk = g.nblk; p.nchunks = g.nchunks; p.KC = g.KC;
  p.tiles_per_image = cdiv(npix, kTileM); p.interp = interp; p.nt = g.nt; p.stages = g.stages;
  const int64_t tiles = (int64_t)B * p.tiles_per_image * g.nblk;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  if (use_plan) {
    cudaFuncSetAttribute(tc_gemm_kernel<MODE_PLAN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
    tc_gemm_kernel<MODE_PLAN><<<grid, kThreads, g.smem, st>>>(p);
  } else {
    cudaFuncSetAttribute(tc_gemm_kernel<MODE_DIRECT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
    tc_gemm_kernel<MODE_DIRECT><<<grid, kThreads, g.smem, st>>>(p);
  }
  return launch_status(3);
}

size_t gemm_ws(int64_t B, int64_t CH, int64_t SHW, int64_t K, int64_t P, int interp, int64_t Nout, bool direct) {
  const Geometry g = geometry(B, CH, SHW, K, P, interp, Nout, direct);
  return g.ok ? 256 + g.xh_bytes + g.wp_bytes : 0;
}

}  // namespace

size_t tc_workspace_bytes(int op, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                          int64_t K, int64_t P, int interp) {
  switch (op) {
    case SPH_CONV_FORWARD: return gemm_ws(B, Cin, IH * IW, K, P, interp, Cout, true);
    case SPH_CONV_BACKWARD_INPUT: return gemm_ws(B, Cout, OH * OW, K, 0, 0, Cin, false);
    case SPH_CONV_BACKWARD_WEIGHT: return simt_dw_workspace(B, OH * OW, Cout, Cin, K, Cout, 4);
    case SPH_TCONV_FORWARD: return gemm_ws(B, Cin, IH * IW, K, 0, 0, Cout, false);
    case SPH_TCONV_BACKWARD_INPUT: return gemm_ws(B, Cout, OH * OW, K, P, interp, Cin, true);
    case SPH_TCONV_BACKWARD_WEIGHT: return simt_dw_workspace(B, IH * IW, Cin, Cout, K, Cout, 4);
    default: return 0;
  }
}

int tc_conv_forward(const void *x, const void *map, const void *iw, const void *weight, const void *bias, void *out,
                    int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                    int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st) {
  return tc_gemm(false, x, map, iw, nullptr, Cin, IH, IW, K, P, OH * OW, interp, weight, Cin * K, K, 1, bias, out, Cout, B, ws,
                 ws_bytes, st);
}

int tc_conv_backward_input(const void *gout, const void *plan, const void *weight, void *gx, int64_t B, int64_t Cin,
                           int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, void *ws,
                           size_t ws_bytes, cudaStream_t st) {
  return tc_gemm(true, gout, nullptr, nullptr, plan, Cout, OH, OW, K, 0, IH * IW, 0, weight, K, Cin * K, 1, nullptr, gx, Cin, B,
                 ws, ws_bytes, st);
}

int tc_conv_backward_weight(const void *gout, const void *x, const void *map, const void *iw, void *gw, void *gb,
                            int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K,
                            int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st) {
  return simt_dw<float>(gout, x, map, iw, Cin, IH, IW, K, P, OH * OW, interp, Cout, B, gw, Cin * K, K, 1, gout, Cout, OH * OW, gb,
                        ws, ws_bytes, st);
}

int tc_tconv_forward(const void *x, const void *plan, const void *weight, const void *bias, void *out, int64_t B,
                     int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, void *ws,
                     size_t ws_bytes, cudaStream_t st) {
  return tc_gemm(true, x, nullptr, nullptr, plan, Cin, IH, IW, K, 0, OH * OW, 0, weight, K, Cout * K, 1, bias, out, Cout, B, ws,
                 ws_bytes, st);
}

int tc_tconv_backward_input(const void *gout, const void *map, const void *iw, const void *weight, void *gx, int64_t B,
                            int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                            int interp, void *ws, size_t ws_bytes, cudaStream_t st) {
  return tc_gemm(false, gout, map, iw, nullptr, Cout, OH, OW, K, P, IH * IW, interp, weight, Cout * K, K, 1, nullptr, gx, Cin, B,
                 ws, ws_bytes, st);
}

int tc_tconv_backward_weight(const void *gout, const void *x, const void *map, const void *iw, void *gw, void *gb,
                             int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH, int64_t OW,
                             int64_t K, int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st) {
  return simt_dw<float>(x, gout, map, iw, Cout, OH, OW, K, P, IH * IW, interp, Cin, B, gw, Cout * K, K, 1, gout, Cout, OH * OW, gb,
                        ws, ws_bytes, st);
}

}  // namespace sph
