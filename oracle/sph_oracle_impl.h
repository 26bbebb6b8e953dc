/* CPU restatement of the mapped-operator path -- TEST INFRASTRUCTURE ONLY.
 *
 * This header is included twice by sph_oracle.c, once with T = float and once
 * with T = double.  It restates, in plain C, the arithmetic of the reference's
 * CPU path so that the CUDA library can be checked against it; it is never
 * linked into, imported by or called from the product library.
 *
 * Each function names the reference file:line whose behaviour it follows
 * (paths are relative to the reference project's root).
 */

/* ---- leaf interpolation (ext_modules/include/core/interpolation.h) ------ */

/* core/interpolation.h:17-33: the four products are formed as (A*B)*v and
 * summed left to right; no fused multiply-add (built with -ffp-contract=off). */
static inline T FN(bilerp)(T x, T y, int64_t x1, int64_t x2, int64_t y1, int64_t y2,
                           T v11, T v21, T v12, T v22) {
  const T A = (T)y2 - y, B = (T)x2 - x, C = x - (T)x1, D = y - (T)y1;
  const T a = A * B * v11, b = A * C * v21, c = D * B * v12, d = D * C * v22;
  return a + b + c + d;
}

/* core/interpolation.h:97-115 (nearest: llround in double, zero outside). */
static inline T FN(gather_nearest)(const T *p, T x, T y, int64_t H, int64_t W) {
  const int64_t xi = llround((double)x), yi = llround((double)y);
  return (xi >= 0 && xi <= W - 1 && yi >= 0 && yi <= H - 1) ? p[yi * W + xi] : (T)0;
}

/* core/interpolation.h:137-162 (bilinear, zero padding per corner). */
static inline T FN(gather_bilinear)(const T *p, T x, T y, int64_t H, int64_t W) {
  const int64_t x1 = (int64_t)floor(x), y1 = (int64_t)floor(y), x2 = x1 + 1, y2 = y1 + 1;
  const int vx1 = x1 >= 0 && x1 <= W - 1, vx2 = x2 >= 0 && x2 <= W - 1;
  const int vy1 = y1 >= 0 && y1 <= H - 1, vy2 = y2 >= 0 && y2 <= H - 1;
  const T v11 = (vx1 && vy1) ? p[y1 * W + x1] : (T)0, v21 = (vx2 && vy1) ? p[y1 * W + x2] : (T)0;
  const T v12 = (vx1 && vy2) ? p[y2 * W + x1] : (T)0, v22 = (vx2 && vy2) ? p[y2 * W + x2] : (T)0;
  return FN(bilerp)(x, y, x1, x2, y1, y2, v11, v21, v12, v22);
}

static inline int64_t FN(negmod)(int64_t a, int64_t m) { return ((a % m) + m) % m; } /* core/util.h:59-62 */

/* core/interpolation.h:191-218 (x wraps, only y is range checked, weights
 * come from the unwrapped integers). */
static inline T FN(gather_bispherical)(const T *p, T x, T y, int64_t H, int64_t W) {
  const int64_t x1 = (int64_t)floor(x), y1 = (int64_t)floor(y), x2 = x1 + 1, y2 = y1 + 1;
  const int64_t x1w = FN(negmod)(x1, W), x2w = FN(negmod)(x2, W);
  const int vy1 = y1 >= 0 && y1 <= H - 1, vy2 = y2 >= 0 && y2 <= H - 1;
  const T v11 = vy1 ? p[y1 * W + x1w] : (T)0, v21 = vy1 ? p[y1 * W + x2w] : (T)0;
  const T v12 = vy2 ? p[y2 * W + x1w] : (T)0, v22 = vy2 ? p[y2 * W + x2w] : (T)0;
  return FN(bilerp)(x, y, x1, x2, y1, y2, v11, v21, v12, v22);
}

/* core/resample.h:63-89 (switch; anything unknown falls to NEAREST). */
static inline T FN(gather)(const T *p, const T *m, int64_t H, int64_t W, int interp) {
  switch (interp) {
    case 1: return FN(gather_bilinear)(p, m[0], m[1], H, W);
    case 2: return FN(gather_bispherical)(p, m[0], m[1], H, W);
    default: return FN(gather_nearest)(p, m[0], m[1], H, W);
  }
}

/* core/resample.h:143-161: sum over the P points, each itself interpolated. */
static inline T FN(gather_w)(const T *p, const T *m, const T *iw, int64_t P, int64_t H, int64_t W, int interp) {
  T acc = (T)0;
  for (int64_t i = 0; i < P; i++) acc += iw[i] * FN(gather)(p, m + 2 * i, H, W, interp);
  return acc;
}

/* adjoint leaf: core/interpolation.h:36-61,117-134,165-188,221-247 and
 * core/resample.h:35-60.  Serial here, so the sum order is the loop order
 * (the reference uses an OpenMP atomic: any order). */
static inline void FN(scatter)(T v, const T *m, int64_t H, int64_t W, int interp, T *dst) {
  const T x = m[0], y = m[1];
  if (interp != 1 && interp != 2) {
    const int64_t xi = llround((double)x), yi = llround((double)y);
    if (xi >= 0 && xi <= W - 1 && yi >= 0 && yi <= H - 1) dst[yi * W + xi] += v;
    return;
  }
  const int64_t x1 = (int64_t)floor(x), y1 = (int64_t)floor(y), x2 = x1 + 1, y2 = y1 + 1;
  const T A = (T)y2 - y, B = (T)x2 - x, C = x - (T)x1, D = y - (T)y1;
  const int vy1 = y1 >= 0 && y1 <= H - 1, vy2 = y2 >= 0 && y2 <= H - 1;
  int vx1, vx2;
  int64_t xa = x1, xb = x2;
  if (interp == 2) { xa = FN(negmod)(x1, W); xb = FN(negmod)(x2, W); vx1 = vx2 = 1; }
  else { vx1 = x1 >= 0 && x1 <= W - 1; vx2 = x2 >= 0 && x2 <= W - 1; }
  if (vx1 && vy1) dst[y1 * W + xa] += A * B * v;
  if (vx2 && vy1) dst[y1 * W + xb] += A * C * v;
  if (vx1 && vy2) dst[y2 * W + xa] += D * B * v;
  if (vx2 && vy2) dst[y2 * W + xb] += D * C * v;
}

/* core/resample.h:127-141 */
static inline void FN(scatter_w)(T v, const T *m, const T *iw, int64_t P, int64_t H, int64_t W, int interp, T *dst) {
  for (int64_t i = 0; i < P; i++) FN(scatter)(iw[i] * v, m + 2 * i, H, W, interp, dst);
}

/* ---- resample_from_map / resample_to_map --------------------------------
 * common/resample.h:11-107, src/cpp/resample_layer.cpp:7-69 (+ weighted
 * twins).  P == 0 means "no interpolation weights" (map is MH x MW x 2);
 * P >= 1 means map MH x MW x P x 2 with weights MH x MW x P. */
void FN(sph_o_resample_from_map)(const T *x, const T *map, const T *iw, T *y, int64_t B, int64_t C,
                                 int64_t H, int64_t W, int64_t MH, int64_t MW, int64_t P, int interp) {
  const int64_t n = MH * MW;
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++) {
    const T *plane = x + bc * H * W;
    for (int64_t i = 0; i < n; i++)
      y[bc * n + i] = P ? FN(gather_w)(plane, map + i * P * 2, iw + i * P, P, H, W, interp)
                        : FN(gather)(plane, map + i * 2, H, W, interp);
  }
}

void FN(sph_o_resample_to_map)(const T *x, const T *map, const T *iw, T *out, int64_t B, int64_t C,
                               int64_t MH, int64_t MW, int64_t OH, int64_t OW, int64_t P, int interp) {
  const int64_t n = MH * MW;
  memset(out, 0, sizeof(T) * (size_t)(B * C * OH * OW));
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++) {
    T *plane = out + bc * OH * OW;
    for (int64_t i = 0; i < n; i++) {
      if (P) FN(scatter_w)(x[bc * n + i], map + i * P * 2, iw + i * P, P, OH, OW, interp, plane);
      else FN(scatter)(x[bc * n + i], map + i * 2, OH, OW, interp, plane);
    }
  }
}

/* ---- mapped max pool -----------------------------------------------------
 * common/mapped_max_pool.h:13-57 (plain) and :81-133 (weighted);
 * src/cpp/mapped_max_pooling_layer.cpp:8-42.  The running maximum starts at
 * the smallest positive normal number on the CPU build (line 30) and at
 * -FLT_MAX on the CUDA build (line 28); `cuda_sentinel` selects which.  The
 * index is the offset of the winning entry's x coordinate in the flattened
 * sample map, or -1 when nothing beat the sentinel. */
void FN(sph_o_max_pool)(const T *x, const T *map, const T *iw, T *out, int64_t *idx, int64_t B, int64_t C,
                        int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int interp,
                        int cuda_sentinel) {
  const int64_t n = OH * OW, PP = P ? P : 1;
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++) {
    const T *plane = x + bc * IH * IW;
    for (int64_t o = 0; o < n; o++) {
      T best = cuda_sentinel ? (T)(-FLT_MAX) : (T)TMIN;
      int64_t bi = -1;
      for (int64_t k = 0; k < K; k++) {
        const int64_t e = (o * K + k) * PP;
        const T v = P ? FN(gather_w)(plane, map + e * 2, iw + e, P, IH, IW, interp)
                      : FN(gather)(plane, map + e * 2, IH, IW, interp);
        if (v > best) { best = v; bi = e * 2; }
      }
      out[bc * n + o] = best;
      idx[bc * n + o] = bi;
    }
  }
}

/* common/mapped_max_pool.h:60-78 and :136-171; src/cpp/...:44-75.  Entries
 * with idx < 0 are skipped here (the reference would read out of bounds). */
void FN(sph_o_max_unpool)(const T *g, const int64_t *idx, const T *map, const T *iw, T *gin, int64_t B,
                          int64_t C, int64_t IH, int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P,
                          int interp) {
  const int64_t n = OH * OW;
  (void)K;
  memset(gin, 0, sizeof(T) * (size_t)(B * C * IH * IW));
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++) {
    T *plane = gin + bc * IH * IW;
    for (int64_t o = 0; o < n; o++) {
      const int64_t s = idx[bc * n + o];
      if (s < 0) continue;
      if (P) FN(scatter_w)(g[bc * n + o], map + s, iw + s / 2, P, IH, IW, interp, plane);
      else FN(scatter)(g[bc * n + o], map + s, IH, IW, interp, plane);
    }
  }
}

/* ---- mapped im2col / col2im ----------------------------------------------
 * common/mapped_im2col.h:11-41,80-116 (gather) and :44-77,119-158 (scatter).
 * col is (C*K) x N with row index c*K + k; one image. */
void FN(sph_o_im2col)(const T *im, const T *map, const T *iw, T *col, int64_t C, int64_t H, int64_t W,
                      int64_t N, int64_t K, int64_t P, int interp) {
  const int64_t PP = P ? P : 1;
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < C; c++)
    for (int64_t k = 0; k < K; k++)
      for (int64_t o = 0; o < N; o++) {
        const int64_t e = (o * K + k) * PP;
        col[(c * K + k) * N + o] = P ? FN(gather_w)(im + c * H * W, map + e * 2, iw + e, P, H, W, interp)
                                     : FN(gather)(im + c * H * W, map + e * 2, H, W, interp);
      }
}

void FN(sph_o_col2im)(const T *col, const T *map, const T *iw, T *im, int64_t C, int64_t H, int64_t W,
                      int64_t N, int64_t K, int64_t P, int interp) {
  const int64_t PP = P ? P : 1;
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < C; c++)
    for (int64_t o = 0; o < N; o++)
      for (int64_t k = 0; k < K; k++) {
        const int64_t e = (o * K + k) * PP;
        const T v = col[(c * K + k) * N + o];
        if (P) FN(scatter_w)(v, map + e * 2, iw + e, P, H, W, interp, im + c * H * W);
        else FN(scatter)(v, map + e * 2, H, W, interp, im + c * H * W);
      }
}

/* C(M x N) (+)= A(M x K) * B(K x N), row major; ta/tb read A or B transposed.
 * Stands in for the at::mm calls of the reference's layer files. */
static void FN(gemm)(int ta, int tb, int64_t M, int64_t N, int64_t K, const T *A, const T *Bm, T *Cm, int accumulate) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; i++) {
    T *crow = Cm + i * N;
    if (!accumulate) for (int64_t j = 0; j < N; j++) crow[j] = (T)0;
    if (!tb) {
      for (int64_t k = 0; k < K; k++) {
        const T a = ta ? A[k * M + i] : A[i * K + k];
        const T *brow = Bm + k * N;
        for (int64_t j = 0; j < N; j++) crow[j] += a * brow[j];
      }
    } else {
      for (int64_t j = 0; j < N; j++) {
        T s = (T)0;
        for (int64_t k = 0; k < K; k++) s += (ta ? A[k * M + i] : A[i * K + k]) * Bm[j * K + k];
        crow[j] += s;
      }
    }
  }
}

/* ---- mapped convolution --------------------------------------------------
 * src/cpp/mapped_convolution_layer.cpp:8-51 (forward), :53-89 (grad input),
 * :91-133 (grad weight); bias gradient = sum over (b, y, x) of grad_output
 * (include/layers/mapped_convolution_layer.h:130).  weight is (Cout,Cin,K). */
void FN(sph_o_conv_forward)(const T *x, const T *map, const T *iw, const T *w, const T *bias, T *out,
                            int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH,
                            int64_t OW, int64_t K, int64_t P, int interp) {
  const int64_t N = OH * OW;
  T *col = (T *)malloc(sizeof(T) * (size_t)(Cin * K * N));
  for (int64_t b = 0; b < B; b++) {
    FN(sph_o_im2col)(x + b * Cin * IH * IW, map, iw, col, Cin, IH, IW, N, K, P, interp);
    FN(gemm)(0, 0, Cout, N, Cin * K, w, col, out + b * Cout * N, 0);
    for (int64_t co = 0; co < Cout; co++)
      for (int64_t o = 0; o < N; o++) out[(b * Cout + co) * N + o] += bias[co];
  }
  free(col);
}

void FN(sph_o_conv_backward)(const T *go, const T *x, const T *map, const T *iw, const T *w, T *gx, T *gw,
                             T *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                             int64_t OH, int64_t OW, int64_t K, int64_t P, int interp) {
  const int64_t N = OH * OW;
  T *col = (T *)malloc(sizeof(T) * (size_t)(Cin * K * N));
  memset(gx, 0, sizeof(T) * (size_t)(B * Cin * IH * IW));
  memset(gw, 0, sizeof(T) * (size_t)(Cout * Cin * K));
  for (int64_t co = 0; co < Cout; co++) gb[co] = (T)0;
  for (int64_t b = 0; b < B; b++) {
    const T *gob = go + b * Cout * N;
    FN(gemm)(1, 0, Cin * K, N, Cout, w, gob, col, 0);                 /* col = W^T * dO[b] */
    FN(sph_o_col2im)(col, map, iw, gx + b * Cin * IH * IW, Cin, IH, IW, N, K, P, interp);
    FN(sph_o_im2col)(x + b * Cin * IH * IW, map, iw, col, Cin, IH, IW, N, K, P, interp);
    FN(gemm)(0, 1, Cout, Cin * K, N, gob, col, gw, 1);                /* dW += dO[b] * col^T */
    for (int64_t co = 0; co < Cout; co++)
      for (int64_t o = 0; o < N; o++) gb[co] += gob[co * N + o];
  }
  free(col);
}

/* ---- mapped transposed convolution ---------------------------------------
 * src/cpp/mapped_transposed_convolution_layer.cpp:8-47 (forward), :49-89
 * (grad input), :91-131 (grad weight).  weight is (Cin,Cout,K); the map has
 * the INPUT's spatial size and points into the output grid. */
void FN(sph_o_tconv_forward)(const T *x, const T *map, const T *iw, const T *w, const T *bias, T *out,
                             int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW, int64_t OH,
                             int64_t OW, int64_t K, int64_t P, int interp) {
  const int64_t N = IH * IW;
  T *col = (T *)malloc(sizeof(T) * (size_t)(Cout * K * N));
  memset(out, 0, sizeof(T) * (size_t)(B * Cout * OH * OW));
  for (int64_t b = 0; b < B; b++) {
    FN(gemm)(1, 0, Cout * K, N, Cin, w, x + b * Cin * N, col, 0);     /* col = W^T * x[b] */
    FN(sph_o_col2im)(col, map, iw, out + b * Cout * OH * OW, Cout, OH, OW, N, K, P, interp);
    for (int64_t co = 0; co < Cout; co++)
      for (int64_t o = 0; o < OH * OW; o++) out[(b * Cout + co) * OH * OW + o] += bias[co];
  }
  free(col);
}

void FN(sph_o_tconv_backward)(const T *go, const T *x, const T *map, const T *iw, const T *w, T *gx, T *gw,
                              T *gb, int64_t B, int64_t Cin, int64_t Cout, int64_t IH, int64_t IW,
                              int64_t OH, int64_t OW, int64_t K, int64_t P, int interp) {
  const int64_t N = IH * IW;
  T *col = (T *)malloc(sizeof(T) * (size_t)(Cout * K * N));
  memset(gw, 0, sizeof(T) * (size_t)(Cout * Cin * K));
  for (int64_t co = 0; co < Cout; co++) gb[co] = (T)0;
  for (int64_t b = 0; b < B; b++) {
    const T *gob = go + b * Cout * OH * OW;
    FN(sph_o_im2col)(gob, map, iw, col, Cout, OH, OW, N, K, P, interp);
    FN(gemm)(0, 0, Cin, N, Cout * K, w, col, gx + b * Cin * N, 0);    /* dX[b] = W * col */
    FN(gemm)(0, 1, Cin, Cout * K, N, x + b * Cin * N, col, gw, 1);    /* dW += x[b] * col^T */
    for (int64_t co = 0; co < Cout; co++)
      for (int64_t o = 0; o < OH * OW; o++) gb[co] += gob[co * OH * OW + o];
  }
  free(col);
}

/* ---- mapped average pool --------------------------------------------------
 * common/mapped_avg_pool.h:12-39 (plain) and :71-107 (weighted): the K slot
 * values are added in slot order and the sum is divided by kernel_size;
 * src/cpp/mapped_avg_pooling_layer.cpp:8-38. */
void FN(sph_o_avg_pool)(const T *x, const T *map, const T *iw, T *out, int64_t B, int64_t C, int64_t IH,
                        int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int interp) {
  const int64_t n = OH * OW, PP = P ? P : 1;
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++) {
    const T *plane = x + bc * IH * IW;
    for (int64_t o = 0; o < n; o++) {
      T acc = (T)0;
      for (int64_t k = 0; k < K; k++) {
        const int64_t e = (o * K + k) * PP;
        acc += P ? FN(gather_w)(plane, map + e * 2, iw + e, P, IH, IW, interp)
                 : FN(gather)(plane, map + e * 2, IH, IW, interp);
      }
      out[bc * n + o] = acc / (T)K;
    }
  }
}

/* common/mapped_avg_pool.h:41-69 and :109-143: grad / kernel_size goes back
 * through every slot; src/cpp/mapped_avg_pooling_layer.cpp:40-72. */
void FN(sph_o_avg_unpool)(const T *g, const T *map, const T *iw, T *gin, int64_t B, int64_t C, int64_t IH,
                          int64_t IW, int64_t OH, int64_t OW, int64_t K, int64_t P, int interp) {
  const int64_t n = OH * OW, PP = P ? P : 1;
  memset(gin, 0, sizeof(T) * (size_t)(B * C * IH * IW));
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++) {
    T *plane = gin + bc * IH * IW;
    for (int64_t o = 0; o < n; o++) {
      const T v = g[bc * n + o] / (T)K;
      for (int64_t k = 0; k < K; k++) {
        const int64_t e = (o * K + k) * PP;
        if (P) FN(scatter_w)(v, map + e * 2, iw + e, P, IH, IW, interp, plane);
        else FN(scatter)(v, map + e * 2, IH, IW, interp, plane);
      }
    }
  }
}

/* ---- UV-map resampling (tangent-image textures) ---------------------------
 * common/resample.h:133-159 (gather) and :161-187 (scatter);
 * src/cpp/uv_resample_layer.cpp:8-72.  tex is (B,C,NT,TH,TW); quad (IH,IW)
 * names the texture of every image pixel, uv (IH,IW,2) the position inside
 * it in texel units.  A quad index outside [0,NT) contributes nothing here
 * (the reference would address out of bounds). */
void FN(sph_o_resample_from_uv)(const T *tex, const int64_t *quad, const T *uv, T *out, int64_t B, int64_t C,
                                int64_t NT, int64_t TH, int64_t TW, int64_t IH, int64_t IW, int interp) {
  const int64_t n = IH * IW;
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++)
    for (int64_t i = 0; i < n; i++) {
      const int64_t q = quad[i];
      out[bc * n + i] = (q >= 0 && q < NT) ? FN(gather)(tex + (bc * NT + q) * TH * TW, uv + 2 * i, TH, TW, interp) : (T)0;
    }
}

void FN(sph_o_resample_to_uv)(const T *x, const int64_t *quad, const T *uv, T *tex, int64_t B, int64_t C,
                              int64_t NT, int64_t TH, int64_t TW, int64_t IH, int64_t IW, int interp) {
  const int64_t n = IH * IW;
  memset(tex, 0, sizeof(T) * (size_t)(B * C * NT * TH * TW));
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; bc++)
    for (int64_t i = 0; i < n; i++) {
      const int64_t q = quad[i];
      if (q >= 0 && q < NT) FN(scatter)(x[bc * n + i], uv + 2 * i, TH, TW, interp, tex + (bc * NT + q) * TH * TW);
    }
}
