// Host-side derivation of the integer requantisation parameters, done once per network at
// load time (Glow does it while emitting code, with the results baked into the JIT-ed call).
// Float types and operation order follow the reference exactly, because the kernels' int8
// results depend on every bit of these integers.
#include <cmath>

#include "common.cuh"

namespace glowb200 {

// quantizeScaleOffset32To8 (lib/Quantization/Base/Base.cpp:234-359; isFloatPowerOf2 and
// getFloat2Exp :793-799).  The scale stays an fp32 variable; doubling it is exact.
void quantize_scale_32to8(float scale, int32_t &pre, int32_t &post, int32_t &iscale) {
  int e = 0;
  if (std::fabs(std::frexp(scale, &e)) == 0.5f) {  // a power of two
    const int ex = std::ilogb(scale);
    pre = 0;
    if (ex > 0) { post = 0; iscale = static_cast<int>(scale); }
    else        { post = -ex; iscale = 1; }
    return;
  }
  int pre_shift = 0, post_shift = 0;
  while (scale < 0.5 || (scale < 256 && post_shift < 15)) { scale *= 2; post_shift++; }
  while (scale < 255 && pre_shift < (post_shift / 2)) { scale *= 2; pre_shift++; }
  pre = pre_shift;
  post = post_shift;
  iscale = static_cast<int32_t>(std::round(scale));
}

}  // namespace glowb200

extern "C" void glowb200_quantize_scale_offset_32to8(float scale, int32_t *pre, int32_t *post, int32_t *integer_scale) {
  glowb200::quantize_scale_32to8(scale, *pre, *post, *integer_scale);
}

extern "C" int glowb200_rowwise_requant_params(const float *row_scales, int64_t n, float in_scale,
                                               const float *bias_scales, int64_t num_bias_scales, float out_scale,
                                               int32_t *bias_pre, int32_t *bias_post, int32_t *bias_scale,
                                               int32_t *out_pre, int32_t *out_post, int32_t *out_scale_int) {
  GLOWB200_REQUIRE(n >= 0 && (num_bias_scales == 1 || num_bias_scales == n), "bias scales: one, or one per row");
  for (int64_t j = 0; j < n; j++) {
    // lib/LLVMIRCodeGen/LLVMIRGen.cpp:2245-2251 (rowwise FC), :2726-2730 (channelwise conv)
    const float mat_mul_scale = in_scale * row_scales[j];
    const float b = bias_scales[num_bias_scales == 1 ? 0 : j];
    glowb200::quantize_scale_32to8(b / mat_mul_scale, bias_pre[j], bias_post[j], bias_scale[j]);
    glowb200::quantize_scale_32to8(mat_mul_scale / out_scale, out_pre[j], out_post[j], out_scale_int[j]);
  }
  return GLOWB200_OK;
}
