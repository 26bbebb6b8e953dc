// Thin contractions on the tensor cores (bf16 precision): convolutions whose gathered side has so few channels that
// all its columns (channels x K <= 63) fit one 64-column operand row, e.g. an RGB first layer.  The general
// tensor-core kernels spend a tile's fixed work on two chunks there, and the exact register-tiled kernels are bound
// by instruction issue; here a tile is ONE 128 x 64 operand block gathered straight from the float32 planes (exact
// float32 interpolation, one rounding to bf16), one group of MMAs against a weight block that stays in shared
// memory for the CTA's lifetime, and the same tensor-map epilogue as the general kernel.
//
// Included by conv_tc.cu inside its anonymous namespace (uses its epilogue constants, tensor maps and launch helpers).
#pragma once

constexpr int kThinProducerWarps = 8;  // two groups of four warps, each group gathers whole tiles into its own stage
constexpr int kThinThreads = 32 * (kEpilogueWarps + 1 + kThinProducerWarps);
constexpr int kThinFirstProducer = 32 * (kEpilogueWarps + 1);
constexpr int kThinMaxCols = 63;       // gathered columns (channels x K); one more column may carry ones

struct ThinFwdParams {
  const float *src;          // (B, CH, SH, SW)
  const float *map, *iw;     // sample map over the (GH, GW) grid (+ interpolation weights)
  const __nv_bfloat16 *wp;   // weight block [Npb rows][64 columns] bf16, 128B-swizzled; column j = slot * CH + channel
  const float *bias;
  int *status;
  int B, CH, SH, SW, K, P, GH, GW, Nout, Npb, tiles_x, tiles_y, relu, has_cl, tmem_cols;
};

inline size_t thin_fwd_smem(int Npb) {
  return 1024 + 2 * (size_t)kAStageBytes + (size_t)Npb * 128 + (((size_t)Npb * 4 + 127) & ~(size_t)127) + kOutStageBytes + 8 * 8 + 16;
}

// One producer thread's pixel: columns j = slot * CH + c, interpolated in float32 from the planes and stored as bf16
// into row `l` of the 128-byte-swizzled operand block.
template <int INTERP>
__device__ __forceinline__ void thin_gather_row(const ThinFwdParams &p, const float *__restrict__ img, int pix, uint32_t row_s,
                                                int l) {
  const size_t plane = (size_t)p.SH * p.SW;
  const int PP = p.P > 0 ? p.P : 1;
  int j = 0;
  for (int k = 0; k < p.K; k++) {
    const float *m = p.map + 2 * ((size_t)pix * p.K + k) * PP;
    if (p.P == 0) {
      Taps<float> t;
      decode<float, INTERP>(__ldg(m), __ldg(m + 1), p.SH, p.SW, t);
      for (int c = 0; c < p.CH; c++, j++) {
        const float v = gather<float, INTERP>(img + c * plane, t);
        const uint32_t a = row_s + ((((uint32_t)j >> 3) ^ ((uint32_t)l & 7u)) << 4) + (((uint32_t)j & 7u) << 1);
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(a), "h"(__bfloat16_as_ushort(__float2bfloat16(v))) : "memory");
      }
    } else {
      const float *w = p.iw + ((size_t)pix * p.K + k) * PP;
      for (int c = 0; c < p.CH; c++, j++) {
        const float v = gather_slot<float, INTERP, true>(img + c * plane, m, w, p.P, p.SH, p.SW);
        const uint32_t a = row_s + ((((uint32_t)j >> 3) ^ ((uint32_t)l & 7u)) << 4) + (((uint32_t)j & 7u) << 1);
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(a), "h"(__bfloat16_as_ushort(__float2bfloat16(v))) : "memory");
      }
    }
  }
}

// The common case spelled out: bilinear, one point per slot, CHT (1..4) channels.  Slots are taken two at a time so
// that their 2 * CHT values leave as aligned bf16 pairs; the interpolation uses fused multiply-adds (the value is
// rounded to bf16 anyway) and 32-bit offsets; the map coordinates of the next slot pair are loaded a pair ahead.
__device__ __forceinline__ void thin_store_pair(uint32_t row_s, int l, int j, float a, float b) {
  const uint32_t addr = row_s + ((((uint32_t)j >> 3) ^ ((uint32_t)l & 7u)) << 4) + (((uint32_t)j & 7u) << 1);
  sts32(addr, pack_bf16(a, b));
}
__device__ __forceinline__ void thin_store_one(uint32_t row_s, int l, int j, float a) {
  const uint32_t addr = row_s + ((((uint32_t)j >> 3) ^ ((uint32_t)l & 7u)) << 4) + (((uint32_t)j & 7u) << 1);
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(__bfloat16_as_ushort(__float2bfloat16(a))) : "memory");
}
template <int CHT>
__device__ __forceinline__ void thin_bilinear_slot(const float *__restrict__ img, int plane, int SH, int SW, float2 xy, float (&v)[CHT]) {
  const float xf = floorf(xy.x), yf = floorf(xy.y);
  const int x1 = (int)xf, y1 = (int)yf;
  const float C = xy.x - xf, D = xy.y - yf, B = (xf + 1.0f) - xy.x, A = (yf + 1.0f) - xy.y;
  const bool sane = fabsf(xy.x) < 1e9f && fabsf(xy.y) < 1e9f;
  const bool vx1 = sane && (unsigned)x1 < (unsigned)SW, vx2 = sane && (unsigned)(x1 + 1) < (unsigned)SW;
  const bool vy1 = (unsigned)y1 < (unsigned)SH, vy2 = (unsigned)(y1 + 1) < (unsigned)SH;
  const int o00 = y1 * SW + x1;
  const bool p0 = vx1 && vy1, p1 = vx2 && vy1, p2 = vx1 && vy2, p3 = vx2 && vy2;
  // (a NaN, infinite or astronomically large coordinate has no tap: zero weights, or NaN * 0 would reach the sum)
  const float w0 = sane ? A * B : 0.0f, w1 = sane ? A * C : 0.0f, w2 = sane ? D * B : 0.0f, w3 = sane ? D * C : 0.0f;
#pragma unroll
  for (int c = 0; c < CHT; c++) {
    const float *pc = img + c * plane;
    const float a0 = (p0 && index_ok(o00, plane)) ? __ldg(pc + o00) : 0.0f;
    const float a1 = (p1 && index_ok(o00 + 1, plane)) ? __ldg(pc + o00 + 1) : 0.0f;
    const float a2 = (p2 && index_ok(o00 + SW, plane)) ? __ldg(pc + o00 + SW) : 0.0f;
    const float a3 = (p3 && index_ok(o00 + SW + 1, plane)) ? __ldg(pc + o00 + SW + 1) : 0.0f;
    v[c] = fmaf(w3, a3, fmaf(w2, a2, fmaf(w1, a1, w0 * a0)));
  }
}
template <int CHT>
__device__ __forceinline__ void thin_gather_row_bilinear(const ThinFwdParams &p, const float *__restrict__ img, int pix, uint32_t row_s,
                                                         int l) {
  const int plane = p.SH * p.SW;
  const float2 *m = (const float2 *)p.map + (size_t)pix * p.K;
  int k = 0;
  float2 c0 = __ldg(m), c1 = p.K > 1 ? __ldg(m + 1) : make_float2(0.0f, 0.0f);
  for (; k + 1 < p.K; k += 2) {
    const float2 n0 = k + 2 < p.K ? __ldg(m + k + 2) : make_float2(0.0f, 0.0f);
    const float2 n1 = k + 3 < p.K ? __ldg(m + k + 3) : make_float2(0.0f, 0.0f);
    float v[2 * CHT];
    thin_bilinear_slot<CHT>(img, plane, p.SH, p.SW, c0, *(float(*)[CHT])(v));
    thin_bilinear_slot<CHT>(img, plane, p.SH, p.SW, c1, *(float(*)[CHT])(v + CHT));
#pragma unroll
    for (int i = 0; i < CHT; i++) thin_store_pair(row_s, l, k * CHT + 2 * i, v[2 * i], v[2 * i + 1]);
    c0 = n0;
    c1 = n1;
  }
  if (k < p.K) {  // odd K: the last slot alone
    float v[CHT];
    thin_bilinear_slot<CHT>(img, plane, p.SH, p.SW, c0, v);
    const int j0 = k * CHT;  // even when k is even
#pragma unroll
    for (int i = 0; i + 1 < CHT; i += 2) thin_store_pair(row_s, l, j0 + i, v[i], v[i + 1]);
    if (CHT & 1) thin_store_one(row_s, l, j0 + CHT - 1, v[CHT - 1]);
  }
}

// Row of one pixel, by the fastest form that covers the call.
template <int INTERP>
__device__ __forceinline__ void thin_row(const ThinFwdParams &p, const float *__restrict__ img, int pix, uint32_t row_s, int l) {
  if constexpr (INTERP == SPH_BILINEAR) {
    if (p.P == 0 && p.SH * p.SW < (1 << 30)) {
      switch (p.CH) {
        case 1: thin_gather_row_bilinear<1>(p, img, pix, row_s, l); return;
        case 2: thin_gather_row_bilinear<2>(p, img, pix, row_s, l); return;
        case 3: thin_gather_row_bilinear<3>(p, img, pix, row_s, l); return;
        case 4: thin_gather_row_bilinear<4>(p, img, pix, row_s, l); return;
        default: break;
      }
    }
  }
  thin_gather_row<INTERP>(p, img, pix, row_s, l);
}

template <int INTERP>
__global__ void __launch_bounds__(kThinThreads, 2) tc_thin_fwd_kernel(const ThinFwdParams p, const __grid_constant__ CUtensorMap out_map,
                                                                       const __grid_constant__ CUtensorMap cl_map) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *base = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *A = base;                                   // two operand stages, one per producer group
  uint8_t *Bw = A + 2 * kAStageBytes;                  // weight block, resident
  float *bias_s = (float *)(Bw + (size_t)p.Npb * 128);  // bias (zeros if there is none), padded to 128 bytes
  float *ostage = (float *)((uint8_t *)bias_s + (((size_t)p.Npb * 4 + 127) & ~(size_t)127));  // epilogue staging (128-byte aligned)
  uint64_t *full = (uint64_t *)((uint8_t *)ostage + kOutStageBytes);
  uint64_t *empty = full + 2, *tfull = empty + 2, *tempty = tfull + 2;
  uint32_t *tmem_ptr = (uint32_t *)(tempty + 2);
  volatile int *abort_flag = (volatile int *)(tmem_ptr + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < 2; s++) {
      mbar_init(full + s, kThinProducerWarps / 2);
      mbar_init(empty + s, 1);
      mbar_init(tfull + s, 1);
      mbar_init(tempty + s, kEpilogueWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  // operand stages start as zeros (the padding columns are never written again); the weight block is copied once
  for (int i = tid; i < 2 * kAStageBytes / 16; i += kThinThreads) ((uint4 *)A)[i] = make_uint4(0, 0, 0, 0);
  for (int i = tid; i < p.Npb * 8; i += kThinThreads) ((uint4 *)Bw)[i] = __ldg((const uint4 *)p.wp + i);
  for (int i = tid; i < p.Npb; i += kThinThreads) bias_s[i] = (p.bias && i < p.Nout) ? __ldg(p.bias + i) : 0.0f;
  fence_proxy_async();
  if (warp == kEpilogueWarps) {
    tmem_alloc(tmem_ptr, (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const int tiles_per_image = p.tiles_x * p.tiles_y;
  const int total_tiles = p.B * tiles_per_image;
  const int buf_cols = p.tmem_cols / 2;

  if (warp < kEpilogueWarps) {
    // ---------------- epilogue: TMEM -> (+bias, ReLU) -> shared staging -> tensor-map stores ----------------
    const uint32_t st_s = smem_u32(ostage) + warp * (kOutStageCh * 32 * 4);
    const uint32_t st_lane = st_s + lane * 4;
    const uint32_t cl_s = smem_u32(ostage) + kEpilogueWarps * (kOutStageCh * 32 * 4) + warp * (32 * kOutStageCh * 2);
    const uint32_t cl_lane = cl_s + lane * (kOutStageCh * 2);
    int tl = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tl++) {
      const int b = tile / tiles_per_image, t2 = tile % tiles_per_image;
      const int ty = t2 / p.tiles_x, tx = t2 % p.tiles_x;
      const int buf = tl & 1;
      if (!mbar_wait(tfull + buf, (tl >> 1) & 1, abort_flag)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * buf_cols;
      for (int n0 = 0; n0 < p.Npb; n0 += kOutStageCh) {
        uint32_t h[16];
        tmem_ld_32x16(taddr + n0, h);
        float bv[16];
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          const float4 t = *(const float4 *)(bias_s + n0 + j);
          bv[j] = t.x; bv[j + 1] = t.y; bv[j + 2] = t.z; bv[j + 3] = t.w;
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
        if (p.has_cl) {
          sts128(cl_lane, make_uint4(pack_bf16(ov[0], ov[1]), pack_bf16(ov[2], ov[3]), pack_bf16(ov[4], ov[5]), pack_bf16(ov[6], ov[7])));
          sts128(cl_lane + 16, make_uint4(pack_bf16(ov[8], ov[9]), pack_bf16(ov[10], ov[11]), pack_bf16(ov[12], ov[13]), pack_bf16(ov[14], ov[15])));
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          tensor_store_4d(&out_map, st_s, tx * kTW, ty * kTH + 2 * warp, n0, b);
          if (p.has_cl) tensor_store_4d(&cl_map, cl_s, n0, tx * kTW, ty * kTH + 2 * warp, b);
          bulk_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty + buf);
    }
    bulk_wait_all();  // this thread's bulk copies are complete before the CTA may exit
  } else if (warp == kEpilogueWarps) {
    // ---------------- MMA issuer (one thread): one 128 x Npb x 64 product per tile ----------------
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16(kTileM, p.Npb, 0, 0);
      const uint64_t b0 = smem_desc_sw128(smem_u32(Bw), 16, 1024);
      int tl = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tl++) {
        const int s = tl & 1;
        if (!mbar_wait(tempty + s, ((tl >> 1) & 1) ^ 1, abort_flag)) break;
        if (!mbar_wait(full + s, (tl >> 1) & 1, abort_flag)) break;
        tc_fence_after();
        const uint64_t a0 = smem_desc_sw128(smem_u32(A + (size_t)s * kAStageBytes), 16, 1024);
        const uint32_t d = tmem_base + s * buf_cols;
#pragma unroll
        for (int kk = 0; kk < kChunk / 16; kk++) umma_bf16(d, a0 + 2 * kk, b0 + 2 * kk, idesc, kk != 0);
        umma_commit(empty + s);
        umma_commit(tfull + s);
      }
    }
  } else {
    // ---------------- producers: group g gathers every second tile of the CTA into stage g ----------------
    const int pt = tid - kThinFirstProducer, grp = pt >> 7, l = pt & 127;
    const uint32_t row_s = smem_u32(A) + grp * kAStageBytes + l * 128;
    int n = 0;  // uses of this group's stage so far
    for (int tile = blockIdx.x + grp * gridDim.x; tile < total_tiles; tile += 2 * gridDim.x, n++) {
      const int b = tile / tiles_per_image, t2 = tile % tiles_per_image;
      const int pix = tile_pixel(l, t2 / p.tiles_x, t2 % p.tiles_x, kTH, p.GH, p.GW);
      const bool ok = mbar_wait(empty + grp, (n & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) break;  // the whole warp leaves together
      if (pix >= 0) thin_row<INTERP>(p, p.src + (size_t)b * p.CH * p.SH * p.SW, pix, row_s, l);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(full + grp);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kEpilogueWarps) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  if (tid == 0 && *abort_flag) {
    *p.status = 1;
    g_wait_status = 1;
  }
}

// Weight block of the thin forward: wp[n][j] = w[n*sn + c*sc + k*sk] for column j = k * CH + c, zero elsewhere.
__global__ void thin_weight_image_kernel(const float *__restrict__ w, __nv_bfloat16 *__restrict__ wp, int Nout, int CH, int K, int Npb,
                                         int64_t sn, int64_t sc, int64_t sk) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= Npb * kChunk) return;
  const int col = i % kChunk, n = i / kChunk;
  float v = 0.0f;
  if (n < Nout && col < CH * K) {
    const int k = col / CH, c = col % CH;
    v = w[n * sn + c * sc + k * sk];
  }
  wp[(size_t)n * kChunk + (((col >> 3) ^ (n & 7)) << 3) + (col & 7)] = __float2bfloat16(v);
}

// Shapes the thin tensor-core forward covers; `out` decides whether the tensor-map epilogue applies.
inline bool thin_fwd_ok(int64_t CH, int64_t K, int64_t Nout, int64_t GW) {
  return CH * K <= kThinMaxCols && Nout % 16 == 0 && Nout <= 128 && (GW & 3) == 0;
}
inline size_t thin_fwd_workspace(int64_t Nout) { return 256 + align_up((size_t)Nout * kChunk * 2, 256); }

template <int INTERP>
void launch_thin_fwd(const ThinFwdParams &p, const CUtensorMap &out_map, const CUtensorMap &cl_map, int grid, size_t smem, cudaStream_t st) {
  static int granted[kMaxDevices];
  ensure_dynamic_smem(tc_thin_fwd_kernel<INTERP>, granted, smem);
  tc_thin_fwd_kernel<INTERP><<<grid, kThinThreads, smem, st>>>(p, out_map, cl_map);
}

// Out[b, n, pix] = bias[n] + sum_j Col[b, pix, j] * W[n, j] (+ ReLU, + channels-last bf16 copy) for a thin gathered side.
// Returns SPH_ERR_UNSUPPORTED if the output cannot leave through a tensor map (the caller then uses other kernels).
int tc_thin_forward(const void *src, const void *map, const void *iw, int64_t CH, int64_t SH, int64_t SW, int64_t K, int64_t P,
                    int64_t GH, int64_t GW, int interp, const void *wgt, int64_t sn, int64_t sc, int64_t sk, const void *bias,
                    void *out, int64_t Nout, int64_t B, void *ws, size_t ws_bytes, cudaStream_t st, const Fusion &fz) {
  if (!thin_fwd_ok(CH, K, Nout, GW)) return SPH_ERR_UNSUPPORTED;
  if (!ws || ws_bytes < thin_fwd_workspace(Nout)) return SPH_ERR_WORKSPACE_TOO_SMALL;
  if ((uintptr_t)ws & 255) return SPH_ERR_INVALID_ARGUMENT;
  CUtensorMap out_map, cl_map;
  memset(&out_map, 0, sizeof(out_map));
  memset(&cl_map, 0, sizeof(cl_map));
  if (!cached_out_map(&out_map, (float *)out, B, Nout, GH, GW)) return SPH_ERR_UNSUPPORTED;
  if (fz.out_cl != nullptr && !make_cl_map(&cl_map, (__nv_bfloat16 *)fz.out_cl, B, padded_channels(Nout), GH, GW)) return SPH_ERR_UNSUPPORTED;
  int *status = (int *)ws;
  __nv_bfloat16 *wp = (__nv_bfloat16 *)((char *)ws + 256);
  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return SPH_ERR_CUDA;
  ThinFwdParams p{};
  p.src = (const float *)src; p.map = (const float *)map; p.iw = (const float *)iw; p.wp = wp; p.bias = (const float *)bias;
  p.status = status;
  p.B = (int)B; p.CH = (int)CH; p.SH = (int)SH; p.SW = (int)SW; p.K = (int)K; p.P = (int)P; p.GH = (int)GH; p.GW = (int)GW;
  p.Nout = (int)Nout; p.Npb = (int)Nout; p.tiles_x = cdiv(GW, kTW); p.tiles_y = cdiv(GH, kTH);
  p.relu = fz.relu_out ? 1 : 0; p.has_cl = fz.out_cl != nullptr ? 1 : 0;
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * p.Npb) p.tmem_cols *= 2;
  thin_weight_image_kernel<<<cdiv(p.Npb * kChunk, 256), 256, 0, st>>>((const float *)wgt, wp, (int)Nout, (int)CH, (int)K, p.Npb, sn, sc, sk);
  const int64_t tiles = (int64_t)B * p.tiles_x * p.tiles_y;
  const int grid = (int)std::min<int64_t>(tiles, 2 * (int64_t)sm_count());
  const size_t smem = thin_fwd_smem(p.Npb);
  SPH_DISPATCH_INTERP(interp, launch_thin_fwd<INTERP>(p, out_map, cl_map, grid, smem, st));
  return launch_status(2);
}

// =================================================================================================
// thin backward: weight gradient, bias gradient and the multiply-first half of the input gradient in one pass
// =================================================================================================
// A step is 64 consecutive pixels of one image's flattened (GH*GW) grid.  Per step the producers build two operand
// blocks: G[o][px] = grad_output (masked by the saved activation) as bf16, rows = output channel, and Col[px][j] =
// the gathered columns (plus a column of ones at j = CH*K for the bias gradient), rows = pixel.  G serves twice:
//   D1[o, j]  += G (K-major A: M = o, K = px) x Col (MN-major B: K = px, N = j)          -> dW and dBias, kept in TMEM
//   D2[j, px]  = Wt (K-major A: M = j, K = o, resident) x G (MN-major B: K = o, N = px)  -> sum_o W[o, j] g[o, px]
// D2 is drained every step, transposed through shared memory and written as the bf16 column buffer T2[b][px][k][c]
// (per pixel one 8-byte vector per slot), which the plan gather of the input gradient reads - so grad_output and the
// activation are read from memory exactly once for all three gradients.
constexpr int kThinBwdTeams = 4;                 // producer teams of two warps; team t fills stage t
constexpr int kThinBwdPix = 64;                  // pixels per step
constexpr int kThinBwdStage = 2 * kThinBwdPix * 128;  // G (64 rows) then Col (64 rows), 128 bytes per row
constexpr int kThinBwdTmemCols = 256;            // D1: columns 0-63, D2: 64-127 and 128-191

struct ThinBwdParams {
  const float *gout, *act;   // (B, N, npix) grad_output and, if set, the activation output whose sign masks it
  const float *src;          // (B, CH, SH, SW) input of the convolution
  const float *map, *iw;
  const __nv_bfloat16 *wt;   // [128 rows j][64 columns o] bf16, 128B-swizzled: W[o, c, k] at row j = k*CH + c
  __nv_bfloat16 *t2;         // (B, npix, t2_pitch bytes) out: per pixel K slots of four bf16 (channels 0..CH-1, then zeros)
  int t2_pitch;
  float *partial;            // [grid][64 rows o][64 columns j] fp32 out
  int *status;
  int B, N, CH, SH, SW, K, P, npix, steps_per_image;
  int do_dw, do_dx;          // which of the two products run (a caller may want only one of the gradients)
  long long total_steps;
};

inline size_t thin_bwd_smem() { return 1024 + (size_t)kThinBwdTeams * kThinBwdStage + 128 * 128 + 64 * 33 * 4 + 8 * 16 + 16; }

// 16 bytes that are read once: kept out of L1, which the gather needs
__device__ __forceinline__ float4 ldg_stream(const float *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 thin_mask_pack(const float4 &g0, const float4 &g1, const float4 &a0, const float4 &a1) {
  return make_uint4(pack_bf16(a0.x > 0.0f ? g0.x : 0.0f, a0.y > 0.0f ? g0.y : 0.0f), pack_bf16(a0.z > 0.0f ? g0.z : 0.0f, a0.w > 0.0f ? g0.w : 0.0f),
                    pack_bf16(a1.x > 0.0f ? g1.x : 0.0f, a1.y > 0.0f ? g1.y : 0.0f), pack_bf16(a1.z > 0.0f ? g1.z : 0.0f, a1.w > 0.0f ? g1.w : 0.0f));
}

template <int INTERP>
__global__ void __launch_bounds__(kThinThreads, 2) tc_thin_bwd_kernel(const ThinBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *base = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *stages = base;
  uint8_t *Wt = stages + kThinBwdTeams * kThinBwdStage;
  uint32_t *tr = (uint32_t *)(Wt + 128 * 128);  // [64 rows][33 words]: D2 rows on their way to the pixel-major T2
  uint64_t *full = (uint64_t *)(tr + 64 * 33);  // 8448 bytes on: still 8-byte aligned
  uint64_t *empty = full + kThinBwdTeams, *t2full = empty + kThinBwdTeams, *t2empty = t2full + 2, *d1full = t2empty + 2;
  uint32_t *tmem_ptr = (uint32_t *)(d1full + 1);
  volatile int *abort_flag = (volatile int *)(tmem_ptr + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ncols = p.CH * p.K;                      // real columns; column ncols carries ones
  const int t2_warps = (ncols + 31) / 32;            // epilogue warps that hold rows of D2

  if (tid == 0) {
    for (int s = 0; s < kThinBwdTeams; s++) {
      mbar_init(full + s, 2);
      mbar_init(empty + s, 1);
    }
    for (int u = 0; u < 2; u++) {
      mbar_init(t2full + u, 1);
      mbar_init(t2empty + u, t2_warps);
    }
    mbar_init(d1full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // stages start as zeros (rows of G beyond N and the padding columns of Col are never written); Wt is copied once
  for (int i = tid; i < kThinBwdTeams * kThinBwdStage / 16; i += kThinThreads) ((uint4 *)stages)[i] = make_uint4(0, 0, 0, 0);
  for (int i = tid; i < 128 * 8; i += kThinThreads) ((uint4 *)Wt)[i] = __ldg((const uint4 *)p.wt + i);
  fence_proxy_async();
  if (warp == kEpilogueWarps) {
    tmem_alloc(tmem_ptr, kThinBwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const long long step_lo = p.total_steps * blockIdx.x / gridDim.x, step_hi = p.total_steps * (blockIdx.x + 1) / gridDim.x;
  const int nsteps = (int)(step_hi - step_lo);

  if (warp < kEpilogueWarps) {
    // ---------------- epilogue: D2 of every step -> T2; D1 at the end -> partial sums ----------------
    if (p.do_dx && warp < t2_warps) {
      const int j = warp * 32 + lane;
      const uint32_t tr_s = smem_u32(tr);
      auto epi_sync = [&]() {
        if (t2_warps == 1) __syncwarp();
        else asm volatile("bar.sync 2, 64;" ::: "memory");
      };
      for (int i = 0; i < nsteps; i++) {
        const int u = i & 1;
        if (!mbar_wait(t2full + u, (i >> 1) & 1, abort_flag)) break;
        tc_fence_after();
        const long long step = step_lo + i;
        const int b = (int)(step / p.steps_per_image), px0 = (int)(step % p.steps_per_image) * kThinBwdPix;
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + 64 + u * 64;
        uint4 q[8];  // this row's 64 pixels as bf16
        {
          uint32_t r[32];
          tmem_ld_32x32(taddr, r);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 4; c++)
            q[c] = make_uint4(pack_bf16(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                              pack_bf16(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                              pack_bf16(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                              pack_bf16(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7])));
          tmem_ld_32x32(taddr + 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 4; c++)
            q[4 + c] = make_uint4(pack_bf16(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                                  pack_bf16(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                                  pack_bf16(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                                  pack_bf16(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7])));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(t2empty + u);  // the accumulator is in registers: the next product may overwrite it
        // Row j of D2 holds one column for 64 pixels; T2 wants, per pixel, the CH values of every slot side by side
        // (one 8-byte vector per slot).  The rows go through shared memory ([j][33 words]: conflict-free both ways) and
        // come back pixel by pixel.
        epi_sync();  // the previous step's rows have been read
#pragma unroll
        for (int c = 0; c < 8; c++) {
          const uint32_t a = tr_s + (uint32_t)(j * 33 + 4 * c) * 4;
          sts32(a, q[c].x); sts32(a + 4, q[c].y); sts32(a + 8, q[c].z); sts32(a + 12, q[c].w);
        }
        epi_sync();
        for (int px = warp * 32 + lane; px < kThinBwdPix; px += 32 * t2_warps) {
          if (px0 + px >= p.npix) continue;
          char *row = (char *)p.t2 + ((size_t)b * p.npix + px0 + px) * p.t2_pitch;
          const uint32_t col_s = tr_s + (uint32_t)(px >> 1) * 4 + (px & 1) * 2;
          for (int k = 0; k < p.K; k++) {
            uint32_t h[4] = {0, 0, 0, 0};
#pragma unroll
            for (int c = 0; c < 4; c++)
              if (c < p.CH) {
                unsigned short t;
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(t) : "r"(col_s + (uint32_t)((k * p.CH + c) * 33) * 4));
                h[c] = t;
              }
            *(uint2 *)(row + k * 8) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
          }
        }
      }
    }
    if (p.do_dw && warp < 2) {  // D1 rows o = lane index 0..63
      bool have = nsteps > 0;
      if (have) have = mbar_wait(d1full, 0, abort_flag);
      tc_fence_after();
      float *prow = p.partial + ((size_t)blockIdx.x * 64 + warp * 32 + lane) * 64;
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
      for (int n0 = 0; n0 < 64; n0 += 32) {
        uint32_t r[32];
        if (have) {
          tmem_ld_32x32(taddr + n0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int q = 0; q < 32; q++) r[q] = 0;
        }
#pragma unroll
        for (int q = 0; q < 32; q += 4)
          *(float4 *)(prow + n0 + q) = make_float4(__uint_as_float(r[q]), __uint_as_float(r[q + 1]), __uint_as_float(r[q + 2]),
                                                   __uint_as_float(r[q + 3]));
      }
      tc_fence_before();
    }
  } else if (warp == kEpilogueWarps) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && nsteps > 0) {
      const uint32_t idesc = idesc_bf16(128, 64, 0, 1);  // A K-major, B MN-major, for both products
      const uint64_t wt0 = smem_desc_sw128(smem_u32(Wt), 16, 1024);
      bool alive = true;
      for (int i = 0; alive && i < nsteps; i++) {
        const int s = i % kThinBwdTeams, n = i / kThinBwdTeams, u = i & 1;
        if (!mbar_wait(full + s, n & 1, abort_flag)) { alive = false; break; }
        if (p.do_dx && !mbar_wait(t2empty + u, ((i >> 1) & 1) ^ 1, abort_flag)) { alive = false; break; }
        tc_fence_after();
        const uint32_t g_s = smem_u32(stages + (size_t)s * kThinBwdStage), col_s = g_s + kThinBwdPix * 128;
        const uint64_t ga = smem_desc_sw128(g_s, 16, 1024);                  // G as K-major A (rows 64-127 = Col: unread lanes)
        const uint64_t cb = smem_desc_sw128(col_s, kThinBwdPix * 128, 1024); // Col as MN-major B
        const uint64_t gb = smem_desc_sw128(g_s, kThinBwdPix * 128, 1024);   // G as MN-major B
        if (p.do_dw) {
#pragma unroll
          for (int ks = 0; ks < kThinBwdPix / 16; ks++)
            umma_bf16(tmem_base, ga + 2 * ks, cb + (uint64_t)(ks * 16 * 128 >> 4), idesc, (i | ks) != 0);
        }
        if (p.do_dx) {
#pragma unroll
          for (int ks = 0; ks < 64 / 16; ks++)
            umma_bf16(tmem_base + 64 + u * 64, wt0 + 2 * ks, gb + (uint64_t)(ks * 16 * 128 >> 4), idesc, ks != 0);
        }
        umma_commit(empty + s);
        if (p.do_dx) umma_commit(t2full + u);
      }
      if (alive && p.do_dw) umma_commit(d1full);
    }
  } else {
    // ---------------- producers: team t builds G and Col of every fourth step in stage t ----------------
    const int pt = tid - kThinFirstProducer, team = pt >> 6, lt = pt & 63;
    const uint32_t g_s = smem_u32(stages) + team * kThinBwdStage, col_s = g_s + kThinBwdPix * 128;
    const uint32_t row_s = col_s + lt * 128;
    const int nchunks = p.N * 8;  // 16-byte chunks of G: 8 pixels of one channel
    int n = 0;
    for (int i = team; i < nsteps; i += kThinBwdTeams, n++) {
      const long long step = step_lo + i;
      const int b = (int)(step / p.steps_per_image), px0 = (int)(step % p.steps_per_image) * kThinBwdPix;
      const bool ok = mbar_wait(empty + team, (n & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) break;  // the whole warp leaves together
      // G: chunk q = (channel o = q >> 3, pixels 8 * (q & 7) ...), consecutive threads on consecutive chunks
      const float *gb_ = p.gout + (size_t)b * p.N * p.npix + px0;
      const float *ab_ = p.act ? p.act + (size_t)b * p.N * p.npix + px0 : nullptr;
      const float4 one = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
      for (int q = lt; q < nchunks; q += 128) {  // two chunks' loads in flight
        const int q2 = q + 64;
        const int o = q >> 3, c = q & 7, o2 = q2 >> 3;  // (q2 & 7 == c)
        const bool in = px0 + 8 * c < p.npix, in2 = in && q2 < nchunks;  // npix is a multiple of 8: whole chunks
        float4 g0 = make_float4(0, 0, 0, 0), g1 = g0, h0 = g0, h1 = g0, a0 = one, a1 = one, e0 = one, e1 = one;
        if (in) {
          g0 = ldg_stream(gb_ + (size_t)o * p.npix + 8 * c); g1 = ldg_stream(gb_ + (size_t)o * p.npix + 8 * c + 4);
          if (ab_) { a0 = ldg_stream(ab_ + (size_t)o * p.npix + 8 * c); a1 = ldg_stream(ab_ + (size_t)o * p.npix + 8 * c + 4); }
        }
        if (in2) {
          h0 = ldg_stream(gb_ + (size_t)o2 * p.npix + 8 * c); h1 = ldg_stream(gb_ + (size_t)o2 * p.npix + 8 * c + 4);
          if (ab_) { e0 = ldg_stream(ab_ + (size_t)o2 * p.npix + 8 * c); e1 = ldg_stream(ab_ + (size_t)o2 * p.npix + 8 * c + 4); }
        }
        sts128(g_s + o * 128 + ((c ^ (o & 7)) << 4), thin_mask_pack(g0, g1, a0, a1));
        if (q2 < nchunks) sts128(g_s + o2 * 128 + ((c ^ (o2 & 7)) << 4), thin_mask_pack(h0, h1, e0, e1));
      }
      // Col: this thread's pixel, then the ones column
      const int pix = px0 + lt;
      const bool valid = pix < p.npix;
      if (!p.do_dw) {
        // (the block stays zero; the first product does not run)
      } else if (valid) {
        ThinFwdParams f{};
        f.map = p.map; f.iw = p.iw; f.CH = p.CH; f.SH = p.SH; f.SW = p.SW; f.K = p.K; f.P = p.P;
        thin_row<INTERP>(f, p.src + (size_t)b * p.CH * p.SH * p.SW, pix, row_s, lt);
      } else {
        for (int c = 0; c < 8; c++) sts128(row_s + (c << 4), make_uint4(0, 0, 0, 0));
      }
      if (p.do_dw) {
        const uint32_t a = row_s + ((((uint32_t)ncols >> 3) ^ ((uint32_t)lt & 7u)) << 4) + (((uint32_t)ncols & 7u) << 1);
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(a), "h"((unsigned short)(valid ? 0x3F80 : 0)) : "memory");
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(full + team);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kEpilogueWarps) tmem_dealloc(tmem_base, kThinBwdTmemCols);
  if (tid == 0 && *abort_flag) {
    *p.status = 1;
    g_wait_status = 1;
  }
}

// Wt[j][o] = w[o*so + c*sc + k*sk] for row j = k * CH + c (zero elsewhere), 128 rows x 64 columns, 128B-swizzled.
__global__ void thin_wt_image_kernel(const float *__restrict__ w, __nv_bfloat16 *__restrict__ wt, int N, int CH, int K, int64_t so,
                                     int64_t sc, int64_t sk) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 128 * kChunk) return;
  const int o = i % kChunk, j = i / kChunk;
  float v = 0.0f;
  if (o < N && j < CH * K) v = w[o * so + (j % CH) * sc + (j / CH) * sk];
  wt[(size_t)j * kChunk + (((o >> 3) ^ (j & 7)) << 3) + (o & 7)] = __float2bfloat16(v);
}

// gw[o, c, k] and gb[o] from the per-CTA partial sums.  One warp per output element: lane l adds the parts l, l + 32,
// ... in order, then the 32 lane sums are combined by a fixed shuffle tree - the same order on every run.
__global__ void __launch_bounds__(256) thin_dw_reduce_kernel(const float *__restrict__ partial, int nparts, int N, int CH, int K,
                                                             int64_t so, int64_t sc, int64_t sk, float *__restrict__ gw,
                                                             float *__restrict__ gb) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int ncols = CH * K;
  if (i >= N * (ncols + 1)) return;  // whole warps leave together
  const int j = i % (ncols + 1), o = i / (ncols + 1);
  float s = 0.0f;
  for (int z = lane; z < nparts; z += 32) s += partial[((size_t)z * 64 + o) * 64 + j];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  if (lane != 0) return;
  if (j == ncols) gb[o] = s;
  else gw[o * so + (j % CH) * sc + (j / CH) * sk] = s;
}

// gx[b, c, q] = sum over the plan entries (p, k, w) of destination pixel q of w * T2[b][p][k][c], in plan order.
// Thread = destination pixel x IMG images: per entry one 8-byte load per image fetches all channels of the slot.
template <int IMG>
__global__ void __launch_bounds__(256) thin_plan_gather_kernel(const __nv_bfloat16 *__restrict__ t2, int t2_pitch,
                                                               const void *__restrict__ plan_blob, float *__restrict__ gx, int B, int CH,
                                                               int K, int n_src, int n_dst) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x, b0 = blockIdx.y * IMG;
  if (q >= n_dst) return;
  bool ok;
  const PlanView<float> pv = plan_view<float>(plan_blob, n_dst * K, ok);
  const int nimg = min(IMG, B - b0);
  const size_t img_stride = (size_t)n_src * t2_pitch;
  const char *base = (const char *)t2 + (size_t)b0 * img_stride;
  float acc[IMG][4];
#pragma unroll
  for (int bi = 0; bi < IMG; bi++)
#pragma unroll
    for (int c = 0; c < 4; c++) acc[bi][c] = 0.0f;
  if (ok) {
    int e1 = __ldg(pv.offsets + (size_t)q * K);
    for (int k = 0; k < K; k++) {
      const int e0 = e1;
      e1 = __ldg(pv.offsets + (size_t)q * K + k + 1);
      for (int e = e0; e < e1; e++) {
        const int sp = __ldg(pv.src + e);
        if (!index_ok(sp, pv.n_src)) continue;
        const float w = __ldg(pv.w + e);
        const char *pe = base + (size_t)sp * t2_pitch + k * 8;
        uint2 v[IMG];
#pragma unroll
        for (int bi = 0; bi < IMG; bi++) v[bi] = bi < nimg ? __ldg((const uint2 *)(pe + bi * img_stride)) : make_uint2(0, 0);
#pragma unroll
        for (int bi = 0; bi < IMG; bi++) {
          acc[bi][0] = fmaf(w, bf16_lo(v[bi].x), acc[bi][0]);
          acc[bi][1] = fmaf(w, bf16_hi(v[bi].x), acc[bi][1]);
          acc[bi][2] = fmaf(w, bf16_lo(v[bi].y), acc[bi][2]);
          acc[bi][3] = fmaf(w, bf16_hi(v[bi].y), acc[bi][3]);
        }
      }
    }
  }
#pragma unroll
  for (int bi = 0; bi < IMG; bi++)
    if (bi < nimg)
#pragma unroll
      for (int c = 0; c < 4; c++)
        if (c < CH) gx[((size_t)(b0 + bi) * CH + c) * n_dst + q] = acc[bi][c];
}

// Shapes the thin tensor-core backward covers.
inline bool thin_bwd_ok(int64_t CH, int64_t K, int64_t N, int64_t npix) {
  return CH * K <= kThinMaxCols && CH <= 4 && N % 8 == 0 && N <= 64 && npix % 8 == 0;
}
inline size_t thin_t2_pitch(int64_t K) { return align_up((size_t)K * 8, 16); }  // bytes of T2 per pixel
struct ThinBwdLayout {
  size_t off_wt, off_partial, off_t2, total;
  int grid;
};
inline ThinBwdLayout thin_bwd_layout(int64_t B, int64_t CH, int64_t K, int64_t npix, bool with_t2 = true) {
  ThinBwdLayout L{};
  const int64_t steps = B * ((npix + kThinBwdPix - 1) / kThinBwdPix);
  L.grid = (int)std::max<int64_t>(1, std::min<int64_t>(steps, 2 * (int64_t)sm_count()));
  size_t o = 256;
  L.off_wt = o;      o = align_up(o + 128 * kChunk * 2, 256);
  L.off_partial = o; o = align_up(o + (size_t)L.grid * 64 * 64 * 4, 256);
  L.off_t2 = o;      o = align_up(o + (with_t2 ? (size_t)(B * npix) * thin_t2_pitch(K) : 0), 256);
  L.total = o;
  return L;
}

template <int INTERP>
void launch_thin_bwd(const ThinBwdParams &p, int grid, cudaStream_t st) {
  static int granted[kMaxDevices];
  const size_t smem = thin_bwd_smem();
  ensure_dynamic_smem(tc_thin_bwd_kernel<INTERP>, granted, smem);
  tc_thin_bwd_kernel<INTERP><<<grid, kThinThreads, smem, st>>>(p);
}

// Gradients of a convolution with a thin input side: gx (B, CH, SH, SW) and / or gw (N, CH, K) with gb (N); a null gx
// or gw leaves that gradient out (its product does not run, its scratch is not needed).
int tc_thin_backward(const void *gout, const void *act, const void *x, const void *plan, const void *map, const void *iw,
                     const void *weight, void *gx, void *gw, void *gb, int64_t B, int64_t CH, int64_t N, int64_t SH, int64_t SW,
                     int64_t GH, int64_t GW, int64_t K, int64_t P, int interp, void *ws, size_t ws_bytes, cudaStream_t st) {
  const int64_t npix = GH * GW;
  if (!thin_bwd_ok(CH, K, N, npix) || (((uintptr_t)gout | (uintptr_t)act) & 15) != 0) return SPH_ERR_UNSUPPORTED;
  const bool do_dx = gx != nullptr, do_dw = gw != nullptr && gb != nullptr;
  if (!do_dx && !do_dw) return SPH_ERR_INVALID_ARGUMENT;
  const ThinBwdLayout L = thin_bwd_layout(B, CH, K, npix, do_dx);
  if (!ws || ws_bytes < L.total) return SPH_ERR_WORKSPACE_TOO_SMALL;
  if ((uintptr_t)ws & 255) return SPH_ERR_INVALID_ARGUMENT;
  char *w8 = (char *)ws;
  int *status = (int *)w8;
  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return SPH_ERR_CUDA;
  ThinBwdParams p{};
  p.gout = (const float *)gout; p.act = (const float *)act; p.src = (const float *)x; p.map = (const float *)map; p.iw = (const float *)iw;
  p.wt = (const __nv_bfloat16 *)(w8 + L.off_wt); p.t2 = (__nv_bfloat16 *)(w8 + L.off_t2); p.partial = (float *)(w8 + L.off_partial);
  p.status = status;
  p.B = (int)B; p.N = (int)N; p.CH = (int)CH; p.SH = (int)SH; p.SW = (int)SW; p.K = (int)K; p.P = (int)P; p.npix = (int)npix;
  p.steps_per_image = (int)((npix + kThinBwdPix - 1) / kThinBwdPix);
  p.total_steps = (long long)B * p.steps_per_image;
  p.do_dw = do_dw ? 1 : 0; p.do_dx = do_dx ? 1 : 0;
  p.t2_pitch = (int)thin_t2_pitch(K);
  struct PhaseScope {  // the event list is consumed by this call, whatever its outcome
    ~PhaseScope() { g_phase_count = 0; }
  } phase_scope;
  mark_phase(0, st);
  if (do_dx)
    thin_wt_image_kernel<<<cdiv(128 * kChunk, 256), 256, 0, st>>>((const float *)weight, (__nv_bfloat16 *)(w8 + L.off_wt), (int)N, (int)CH,
                                                                (int)K, CH * K, K, 1);
  mark_phase(1, st);
  SPH_DISPATCH_INTERP(interp, launch_thin_bwd<INTERP>(p, L.grid, st));
  if (do_dw)
    thin_dw_reduce_kernel<<<cdiv(N * (CH * K + 1) * 32, 256), 256, 0, st>>>(p.partial, L.grid, (int)N, (int)CH, (int)K, CH * K, K, 1, (float *)gw,
                                                                      (float *)gb);
  mark_phase(2, st);
  constexpr int kImg = 8;
  const dim3 grid(cdiv(SH * SW, 256), (unsigned)cdiv(B, kImg));
  if (do_dx)
    thin_plan_gather_kernel<kImg><<<grid, 256, 0, st>>>(p.t2, p.t2_pitch, plan, (float *)gx, (int)B, (int)CH, (int)K, (int)npix, (int)(SH * SW));
  mark_phase(3, st);
  return launch_status(1 + (do_dx ? 2 : 0) + (do_dw ? 1 : 0));
}
