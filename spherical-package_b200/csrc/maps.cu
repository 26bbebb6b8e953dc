// Sample maps of the equirectangular kernels, built on the device: for every (strided) pixel of an H x W
// equirectangular image, the kh x kw kernel grid laid out around it and expressed in fractional pixel coordinates of
// the same image.  These are the maps the mapped convolution / pooling layers of a spherical network consume; the
// reference builds them on the host with tensor expressions (layers/util/mapping_functions.py:16-163, with
// layers/util/grids.py:5-25 and layers/util/conversions.py:24-53).  Arithmetic is done in float64 and rounded to
// the map's type once.
#include <math.h>

#include "common.cuh"

namespace sph {

constexpr double kPi = 3.14159265358979323846;

template <typename T>
__global__ void __launch_bounds__(256)
kernel_map_kernel(T *__restrict__ out, int H, int W, int kh, int kw, int stride, int dilation, int kind, int OH, int OW) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int KK = kh * kw;
  if (i >= (int64_t)OH * OW * KK) return;
  const int k = (int)(i % KK), ox = (int)((i / KK) % OW), oy = (int)(i / ((int64_t)KK * OW));
  const int x = ox * stride, y = oy * stride;
  // grids.py:5-25: longitudes -pi + x * 2pi/W (W + 1 points, the last dropped), latitudes -pi/2 ... pi/2 over H points
  const double res_lon = 2.0 * kPi / W, res_lat = H > 1 ? kPi / (H - 1) : 0.0;
  const double lon = -kPi + x * res_lon, lat = -kPi / 2 + y * res_lat;
  // mapping_functions.py:16-41: kernel differentials; +y is down, so the latitude step is negated
  const int ki = k / kw, kj = k % kw;
  const double dlon = (double)((kj - kw / 2) * dilation) * res_lon, dlat = (double)((ki - kh / 2) * dilation) * -res_lat;
  double mlon, mlat;
  if (kind == SPH_MAP_GRID) {                       // :44-75  plain offsets on the lat/lon grid, no wrap
    mlat = lat + dlat;
    mlon = lon + dlon;
  } else if (kind == SPH_MAP_INVERSE_GNOMONIC) {    // :78-120 tangent-plane grid projected back onto the sphere
    // The reference overwrites slot kh*kw/2 with the pixel itself (:107-109), which is the zero differential for odd
    // kernels; for even kernels the zero differential sits elsewhere and evaluates to 0/0 = NaN there - here it is
    // the pixel itself as well.
    const double rho = sqrt(dlon * dlon + dlat * dlat);
    if (k == KK / 2 || rho == 0.0) {
      mlat = lat;
      mlon = lon;
    } else {
      const double nu = atan(rho);
      mlat = asin(cos(nu) * sin(lat) + dlat * sin(nu) * cos(lat) / rho);
      mlon = lon + atan2(dlon * sin(nu), rho * cos(lat) * cos(nu) - dlat * sin(lat) * sin(nu));
    }
    mlon = mlon + kPi;
    mlon = mlon - floor(mlon / (2.0 * kPi)) * (2.0 * kPi) - kPi;   // ((lon + pi) mod 2pi) - pi, modulo with the sign of the divisor
  } else {                                          // :123-163 inverse equirectangular projection
    mlat = lat + dlat;
    mlon = lon + dlon / cos(mlat);
    mlon = mlon + kPi;
    mlon = mlon - floor(mlon / (2.0 * kPi)) * (2.0 * kPi) - kPi;
  }
  // conversions.py:33-53: x = W * (lon + pi) / (2 pi), y = (H - 1) * (lat + pi/2) / pi
  out[2 * i] = (T)((double)W * (mlon + kPi) / (2.0 * kPi));
  out[2 * i + 1] = (T)((double)(H - 1) * (mlat + kPi / 2) / kPi);
}

}  // namespace sph

using namespace sph;

extern "C" int sph_build_kernel_map(void *map, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t stride, int64_t dilation,
                                    int kind, int dtype, void *stream) {
  SPH_RANGE("sph_build_kernel_map");
  if (!map || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || dilation <= 0 || kind < 0 || kind > 2)
    return SPH_ERR_INVALID_ARGUMENT;
  if (dtype != SPH_F32 && dtype != SPH_F64) return SPH_ERR_UNSUPPORTED;
  const int64_t OH = (H + stride - 1) / stride, OW = (W + stride - 1) / stride, total = OH * OW * kh * kw;
  if (H >= ((int64_t)1 << 30) || W >= ((int64_t)1 << 30) || kh * kw >= 65536 || total >= ((int64_t)1 << 40)) return SPH_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == SPH_F32)
    kernel_map_kernel<float><<<blocks, 256, 0, st>>>((float *)map, (int)H, (int)W, (int)kh, (int)kw, (int)stride, (int)dilation,
                                                     kind, (int)OH, (int)OW);
  else
    kernel_map_kernel<double><<<blocks, 256, 0, st>>>((double *)map, (int)H, (int)W, (int)kh, (int)kw, (int)stride,
                                                      (int)dilation, kind, (int)OH, (int)OW);
  return launch_status();
}
