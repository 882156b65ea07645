// Host-side derivation of the integer requantisation parameters, done once per network at
// load time (Glow does it while emitting code, with the results baked into the JIT-ed call).
// Float types and operation order follow the reference exactly, because the kernels' int8
// results depend on every bit of these integers.
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstring>
#include <limits>

#include "common.cuh"
#include "quant_math.cuh"

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

namespace glowb200 {

// chooseQuantizationParams without calibration (lib/Quantization/Base/Base.cpp:433-565) for a
// signed quantized range [qmin, qmax].  schema: 0 Asymmetric, 1 Symmetric, 2 SymmetricWithUnsigned,
// 3 SymmetricWithPower2Scale (include/glow/Quantization/Base/Base.h Schema).
void choose_quantization_params(float min, float max, int schema, int64_t qmin, int64_t qmax, float &scale_out,
                                int32_t &offset_out) {
  double scale;
  choose_quantization_params_basic(min, max, schema, qmin, qmax, scale, offset_out);
  if (schema == 3) scale = std::exp2(std::ceil(std::log2(scale)));
  scale_out = static_cast<float>(scale);
}

// quantization::quantize<int8_t> (include/glow/Quantization/Base/Base.h:322-329)
static inline int8_t quantize_i8(float x, float scale, int32_t offset) {
  const float r = x / scale + (float)offset;
  int64_t v = (int64_t)std::nearbyintf(r);
  v = v < -128 ? -128 : (v > 127 ? 127 : v);
  return (int8_t)v;
}

}  // namespace glowb200

extern "C" void glowb200_choose_quantization_params(float min, float max, int schema, int quantized_bits, float *scale,
                                                    int32_t *offset) {
  // int8 / int16 use their full range; int32 is limited to 30 bits (getQuantizedRange, Base.cpp:361-403)
  int64_t qmin = -128, qmax = 127;
  if (quantized_bits == 16) { qmin = -32768; qmax = 32767; }
  if (quantized_bits == 32) { qmin = (int64_t)INT32_MIN >> 2; qmax = (int64_t)INT32_MAX >> 2; }
  glowb200::choose_quantization_params(min, max, schema, qmin, qmax, *scale, *offset);
}

// tensorRowwiseQuantization<float, int32_t, int8_t> (include/glow/Quantization/Base/Base.h:522-576):
// every row gets its own (scale, offset) from its min/max.  HOST arrays.
extern "C" int glowb200_tensor_rowwise_quantize_i8(const float *in, int64_t rows, int64_t cols, int schema, int8_t *out,
                                                   float *scales, int32_t *offsets) {
  GLOWB200_REQUIRE(rows >= 0 && cols > 0 && in && out && scales && offsets, "bad arguments");
  for (int64_t i = 0; i < rows; i++) {
    const float *r = in + i * cols;
    float mn = r[0], mx = r[0];
    for (int64_t j = 1; j < cols; j++) { mn = r[j] < mn ? r[j] : mn; mx = r[j] > mx ? r[j] : mx; }
    float scale;
    int32_t offset;
    glowb200::choose_quantization_params(mn, mx, schema, -128, 127, scale, offset);
    for (int64_t j = 0; j < cols; j++) out[i * cols + j] = glowb200::quantize_i8(r[j], scale, offset);
    scales[i] = scale;
    offsets[i] = offset;
  }
  return GLOWB200_OK;
}

// quantization::quantize<int32_t>-style bias quantisation with a given scale/offset
// (quantizeTensor, lib/Quantization/Base/Base.cpp; the int32 range is the 30-bit one).
extern "C" int glowb200_quantize_bias_i32(const float *in, int64_t n, float scale, int32_t offset, int32_t *out) {
  GLOWB200_REQUIRE(n >= 0 && (n == 0 || (in && out)), "bad arguments");
  const int64_t qmin = (int64_t)INT32_MIN >> 2, qmax = (int64_t)INT32_MAX >> 2;
  for (int64_t i = 0; i < n; i++) {
    const float r = in[i] / scale + (float)offset;
    int64_t v = (int64_t)std::nearbyintf(r);
    out[i] = (int32_t)(v < qmin ? qmin : (v > qmax ? qmax : v));
  }
  return GLOWB200_OK;
}

// Host-side constant preparation of Function::createChannelwiseQuantizedConv
// (lib/Graph/Graph.cpp:3525-3700) for a float filter and a float bias with an int8 filter and an
// int32 bias: per-output-channel filter parameters (getTensorQuantizationParams along
// dimension 0), per-channel bias parameters specialised with
// specializeBiasWeightsQuantizationParams (lib/Quantization/Base/Base.cpp:595-629: the bias
// offset is forced to 0 and its scale to in_scale * filter_scale, widening the filter scale when
// that would saturate the bias), then both tensors quantized with the final parameters.
// filter is [out_channels, k] (k = kH*kW*inC/group).  HOST arrays.
extern "C" int glowb200_channelwise_conv_prepare(const float *filter, const float *bias, int64_t out_channels, int64_t k,
                                                 float in_scale, int schema, int8_t *filter_q, float *filter_scales,
                                                 int32_t *filter_offsets, int32_t *bias_q, float *bias_scales,
                                                 int32_t *bias_offsets) {
  GLOWB200_REQUIRE(out_channels >= 0 && k > 0 && filter && bias && filter_q && filter_scales && filter_offsets && bias_q &&
                       bias_scales && bias_offsets, "bad arguments");
  const int64_t qmin32 = (int64_t)INT32_MIN >> 2, qmax32 = (int64_t)INT32_MAX >> 2;
  for (int64_t c = 0; c < out_channels; c++) {
    const float *f = filter + c * k;
    float mn = f[0], mx = f[0];
    for (int64_t j = 1; j < k; j++) { mn = f[j] < mn ? f[j] : mn; mx = f[j] > mx ? f[j] : mx; }
    float w_scale, b_scale;
    int32_t w_off, b_off;
    glowb200::choose_quantization_params(mn, mx, schema, -128, 127, w_scale, w_off);
    glowb200::choose_quantization_params(bias[c], bias[c], schema, qmin32, qmax32, b_scale, b_off);
    b_off = 0;
    const bool bias_zero = bias[c] == 0.f;
    if (in_scale * w_scale >= b_scale || bias_zero) {
      b_scale = in_scale * w_scale;
    } else {
      w_scale = b_scale / in_scale;
      b_scale = in_scale * w_scale;
    }
    for (int64_t j = 0; j < k; j++) filter_q[c * k + j] = glowb200::quantize_i8(f[j], w_scale, w_off);
    filter_scales[c] = w_scale;
    filter_offsets[c] = w_off;
    const float r = bias[c] / b_scale + (float)b_off;
    int64_t v = (int64_t)std::nearbyintf(r);
    bias_q[c] = (int32_t)(v < qmin32 ? qmin32 : (v > qmax32 ? qmax32 : v));
    bias_scales[c] = b_scale;
    bias_offsets[c] = b_off;
  }
  return GLOWB200_OK;
}

// tensorFusedRowwiseQuantization<T> (include/glow/Quantization/Base/Base.h:598-678) on the host:
// per row scale = (max - min) / range in double (1 when max - min < 1e-10), offset = min;
// values quantized with the fp32 scale/offset (quantizeWithFloatOffset, :361-379), which the
// fp16 kinds then store rounded to fp16 (Tensor.h:1585-1607).  The fp16 rounding is cuda_fp16's
// host-side round-to-nearest-even conversion.
extern "C" int glowb200_fused_rowwise_quantize(const float *in, int64_t rows, int64_t cols, int kind, uint8_t *out,
                                               int64_t out_line_size) {
  GLOWB200_REQUIRE(kind >= 0 && kind <= 3, "unknown fused kind %d", kind);
  GLOWB200_REQUIRE(rows >= 0 && cols > 0, "rows / cols out of range");
  const bool four = kind >= 2, so16 = (kind & 1) != 0;
  GLOWB200_REQUIRE(!four || cols % 2 == 0, "4-bit fused quantization needs an even number of columns");
  const int64_t want = (four ? cols / 2 : cols) + (so16 ? 4 : 8);
  GLOWB200_REQUIRE(out_line_size == want, "out_line_size must be %lld for %lld columns of kind %d", (long long)want,
                   (long long)cols, kind);
  if (rows == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(in != nullptr && out != nullptr, "NULL tensor pointer");
  const float range = four ? 15.0f : 255.0f;
  for (int64_t i = 0; i < rows; i++) {
    const float *src = in + i * cols;
    uint8_t *dst = out + i * out_line_size;
    const auto mm = std::minmax_element(src, src + cols);
    const float mn = *mm.first, mx = *mm.second;
    const float scale = ((mx - mn) < 1e-10f) ? 1.0f : (float)(((double)mx - (double)mn) / range);
    const float offset = mn;
    if (!four) {
      for (int64_t j = 0; j < cols; j++) dst[j] = (uint8_t)(uint16_t)std::round((src[j] - offset) / scale);
    } else {
      for (int64_t b = 0; b < cols / 2; b++) {
        const int lo = std::max(0, std::min((int)std::round((src[2 * b] - offset) / scale), 15));
        const int hi = std::max(0, std::min((int)std::round((src[2 * b + 1] - offset) / scale), 15));
        dst[b] = (uint8_t)(lo | (hi << 4));
      }
    }
    uint8_t *tail = dst + out_line_size;
    if (so16) {
      const __half s = __float2half_rn(scale), o = __float2half_rn(offset);
      memcpy(tail - 4, &s, 2);
      memcpy(tail - 2, &o, 2);
    } else {
      memcpy(tail - 8, &scale, 4);
      memcpy(tail - 4, &offset, 4);
    }
  }
  return GLOWB200_OK;
}
