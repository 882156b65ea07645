// Quantization parameter arithmetic shared by host code and device kernels.
#pragma once
#include <cfloat>
#include <cmath>
#include <stdint.h>

namespace glowb200 {

// chooseQuantizationParams without calibration (lib/Quantization/Base/Base.cpp:433-565) for the
// signed quantized range [qmin, qmax] and the schemas Asymmetric (0), Symmetric (1) and
// SymmetricWithUnsigned (2).  Plain IEEE double / float arithmetic with no product-sum pairs, so
// host and device agree bit for bit.
__host__ __device__ inline void choose_quantization_params_basic(float min, float max, int schema, int64_t qmin, int64_t qmax,
                                                                 double &scale_out, int32_t &offset_out) {
  min = min < 0.f ? min : 0.f;
  max = max > 0.f ? max : 0.f;
  if (schema == 2) {
    if (!(min >= 0.f)) schema = 1;
  }
  if (schema == 1 || schema == 3) {
    const double rmin = min / (double)qmin;
    const double rmax = max / (double)qmax;
    if (rmin > rmax) max = (float)(rmin * qmax);
    else min = (float)(rmax * qmin);
  }
  min = min > -FLT_MAX ? min : -FLT_MAX;
  max = max < FLT_MAX ? max : FLT_MAX;
  double scale = ((double)max - min) / ((double)qmax - qmin);
  if (scale == 0) scale = 0.1;
  const double zp_from_min = qmin - min / scale;
  const double zp_from_max = qmax - max / scale;
  const double err_min = fabs((double)qmin) + fabs(min / scale);
  const double err_max = fabs((double)qmax) + fabs(max / scale);
  double zp = err_min < err_max ? zp_from_min : zp_from_max;
  const float difference = fabsf(max + min);
  if (difference <= FLT_EPSILON) zp = 0;
  int32_t nudged;
  if (zp < qmin) nudged = (int32_t)qmin;
  else if (zp > qmax) nudged = (int32_t)qmax;
  else nudged = static_cast<int32_t>(round(zp));
  scale_out = scale;
  offset_out = nudged;
}

}  // namespace glowb200
