/*
 * TEST INFRASTRUCTURE ONLY -- NOT PART OF THE PRODUCT.
 *
 * A plain-C restatement, on the CPU, of the arithmetic of pytorch/glow's quantized
 * inference kernels.  It exists so the CUDA kernels can be checked against it and so the
 * benchmark has a CPU baseline to time.  Only tests, the smoke check and the benchmark's
 * CPU-baseline leg may load this library; the product never does.
 *
 * Parity pin: every function here is checked (tests/test_oracle_*.py) against
 *   (1) the hand-computed expected tensors in the reference's own unit tests
 *       (tests/unittests/OperatorTest.cpp, QuantizationTest.cpp), and
 *   (2) the reference's own kernel sources (lib/LLVMIRCodeGen/libjit/*.cpp) compiled
 *       unmodified into oracle/_ref/libjit_strict.so, bit for bit on seeded inputs.
 * The 4-bit / fp16 paths exist only in the reference's Interpreter (which cannot be
 * compiled without LLVM); those are pinned by (1) only.
 *
 * Each function cites the reference file:line (paths inside pytorch/glow) it follows.
 * All float arithmetic is written as separate multiply and add steps and the file is
 * built with -ffp-contract=off so no FMA is formed: that is the canonical operation
 * order of the reference's C++ source.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------ */
/* fp16 <-> fp32.  The reference converts with the FP16 library's                        */
/* fp16_ieee_from_fp32_value / fp16_ieee_to_fp32_value (include/glow/Support/Float16.h:  */
/* 38,81; un-vendored submodule Maratyszcza/FP16, no pinned version): IEEE binary16,     */
/* round-to-nearest-even, subnormals kept, overflow to infinity.  Written out on bits.   */
/* ------------------------------------------------------------------------------------ */
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

ORC_API uint16_t orc_f32_to_f16(float f) {
  uint32_t x = f32_bits(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7fffffffu;
  if (absx > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);       /* NaN */
  if (absx >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);      /* >= 65536 -> inf (also inf) */
  if (absx < 0x38800000u) {                                        /* below 2^-14: subnormal half */
    if (absx < 0x33000000u) return (uint16_t)sign;                 /* < 2^-25 rounds to 0 */
    /* value = m * 2^(e-150) with the implicit bit; target unit is 2^-24 */
    uint32_t e = absx >> 23;
    uint32_t m = (absx & 0x7fffffu) | 0x800000u;
    uint32_t shift = 126u - e;                                     /* 14..24 */
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1u);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | q);
  }
  /* normal half (possibly rounding up into infinity) */
  uint32_t e = (absx >> 23) - 112u;
  uint32_t m = absx & 0x7fffffu;
  uint32_t h = (e << 10) | (m >> 13);
  uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
  return (uint16_t)(sign | h);
}

ORC_API float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1fu;
  uint32_t m = h & 0x3ffu;
  if (e == 0x1fu) return bits_f32(sign | 0x7f800000u | (m << 13));
  if (e == 0) {
    float v = (float)m * 5.9604644775390625e-08f;                  /* m * 2^-24, exact */
    return sign ? -v : v;
  }
  return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* ------------------------------------------------------------------------------------ */
/* Integer requantisation.                                                               */
/* ------------------------------------------------------------------------------------ */

/* libjit_scale<int32_t,int32_t>: lib/LLVMIRCodeGen/libjit/libjit_defs.h:158-173.
 * Arithmetic right shifts, wrapping 32-bit multiply and add (done on uint32 here so the
 * wrap is defined in C), rounding term only when post > 0, offset added last. */
ORC_API int32_t orc_scale32(int32_t input, int32_t pre, int32_t post, int32_t scale,
                            int32_t offset) {
  int32_t rtn = (post > 0) ? (int32_t)(1u << (post - 1)) : 0;
  int32_t a = input >> pre;
  int32_t b = (int32_t)((uint32_t)a * (uint32_t)scale);
  int32_t c = (int32_t)((uint32_t)b + (uint32_t)rtn);
  return (int32_t)((uint32_t)(c >> post) + (uint32_t)offset);
}

/* libjit_clip_i8: libjit_defs.h:146-148. */
ORC_API int8_t orc_clip_i8(int32_t v) { return (int8_t)(v < -128 ? -128 : (v > 127 ? 127 : v)); }

/* libjit_div_round_i32: libjit_defs.h:238-244. */
static inline int32_t div_round_i32(int32_t input, int32_t divider) {
  int32_t rnd = divider >> 1;
  return (input > 0) ? ((input + rnd) / divider) : ((input - rnd) / divider);
}

/* libjit_activation_i32: libjit_defs.h:206-233 (0 none, 1 relu, 2 clip, 5 leaky relu). */
static inline int32_t activation_i32(int32_t x, int32_t offset, int32_t actType,
                                     const int32_t *actArgs) {
  if (actType == 0) return x;
  if (actType == 1) return x > offset ? x : offset;
  if (actType == 2) { int32_t t = x > actArgs[0] ? x : actArgs[0]; return t < actArgs[1] ? t : actArgs[1]; }
  if (actType == 3 || actType == 4) return x;
  return (x >= offset) ? x : orc_scale32(x - offset, actArgs[0], actArgs[1], actArgs[2], offset);
}

/* quantizeScaleOffset32To8: lib/Quantization/Base/Base.cpp:234-359, with
 * isFloatPowerOf2 / getFloat2Exp (:793-799).  `scale` stays a float throughout. */
ORC_API void orc_quantize_scale_offset_32to8(float scale, int32_t *pre, int32_t *post,
                                             int32_t *iscale) {
  int e;
  float mant = frexpf(scale, &e);
  if (fabsf(mant) == 0.5f) {
    int ex = ilogbf(scale);
    if (ex > 0) { *pre = 0; *post = 0; *iscale = (int)scale; }
    else        { *pre = 0; *post = -ex; *iscale = 1; }
    return;
  }
  int preShift = 0, postShift = 0;
  while (scale < 0.5 || (scale < 256 && postShift < 15)) { scale *= 2; postShift++; }
  while (scale < 255 && preShift < (postShift / 2)) { scale *= 2; preShift++; }
  *pre = preShift; *post = postShift; *iscale = (int)roundf(scale);
}

/* Per-row triples of RowwiseQuantizedFullyConnected and per-channel triples of
 * ChannelwiseQuantizedConvolution: lib/LLVMIRCodeGen/LLVMIRGen.cpp:2245-2251 and
 * :2726-2730.  matMulScale = inScale * wScale[j] in fp32; bias from biasScale[j]/matMul,
 * output from matMul/outScale.  bias_scales has n entries, or 1 (bias_scales_n == 1) for
 * the rowwise FC whose bias has one type-level scale. */
ORC_API void orc_rowwise_requant_params(const float *w_scales, int64_t n, float in_scale,
                                        const float *bias_scales, int64_t bias_scales_n,
                                        float out_scale, int32_t *bias_pre, int32_t *bias_post,
                                        int32_t *bias_scale, int32_t *out_pre, int32_t *out_post,
                                        int32_t *out_scale_i) {
  for (int64_t j = 0; j < n; j++) {
    float mm = in_scale * w_scales[j];
    float bs = bias_scales[bias_scales_n == 1 ? 0 : j];
    orc_quantize_scale_offset_32to8(bs / mm, &bias_pre[j], &bias_post[j], &bias_scale[j]);
    orc_quantize_scale_offset_32to8(mm / out_scale, &out_pre[j], &out_post[j], &out_scale_i[j]);
  }
}

/* ------------------------------------------------------------------------------------ */
/* Fused-rowwise tables.                                                                 */
/* kind: 0 UInt8FusedQTy (fp32 scale/offset), 1 UInt8FusedFP16QTy, 2 UInt4FusedQTy,      */
/*       3 UInt4FusedFP16QTy   (include/glow/Base/Type.h:424-433).                       */
/* ------------------------------------------------------------------------------------ */
static inline int kind_is4(int kind) { return kind >= 2; }
static inline int kind_fp16so(int kind) { return kind & 1; }

/* Scale/offset sit in the last 2*sizeof(T) bytes of a row: include/glow/Base/Tensor.h:1585-1607. */
static inline void row_scale_offset(const uint8_t *row_end, int kind, float *scale, float *offset) {
  if (kind_fp16so(kind)) {
    uint16_t s, o;
    memcpy(&s, row_end - 4, 2); memcpy(&o, row_end - 2, 2);
    *scale = orc_f16_to_f32(s); *offset = orc_f16_to_f32(o);
  } else {
    memcpy(scale, row_end - 8, 4); memcpy(offset, row_end - 4, 4);
  }
}

/* tensorFusedRowwiseQuantization<T>: include/glow/Quantization/Base/Base.h:598-678 with
 * quantizeWithFloatOffset / quantize4BitsWithFloatOffset (:361-379).  in: fp32 [rows, cols];
 * out: uint8 [rows, out_line] where out_line = cols (+8 or +4) or cols/2 (+8 or +4). */
ORC_API void orc_fused_rowwise_quantize(const float *in, int64_t rows, int64_t cols, int kind,
                                        uint8_t *out, int64_t out_line) {
  const float range = kind_is4(kind) ? 15.0f : 255.0f;
  for (int64_t i = 0; i < rows; i++) {
    const float *src = in + i * cols;
    uint8_t *dst = out + i * out_line;
    float mn = src[0], mx = src[0];
    for (int64_t j = 1; j < cols; j++) { if (src[j] < mn) mn = src[j]; if (src[j] > mx) mx = src[j]; }
    const float scale = ((mx - mn) < 1e-10f) ? 1.0f : (float)(((double)mx - (double)mn) / range);
    const float offset = mn;
    for (int64_t j = 0; j < cols; j++) {
      float r = roundf((src[j] - offset) / scale);
      if (!kind_is4(kind)) {
        dst[j] = (uint8_t)(uint16_t)r;
      } else {
        int q = (int)r; q = q < 0 ? 0 : (q > 15 ? 15 : q);
        if ((j & 1) == 0) dst[j / 2] = (uint8_t)q; else dst[j / 2] |= (uint8_t)(q << 4);
      }
    }
    uint8_t *tail = dst + out_line;
    if (kind_fp16so(kind)) {
      uint16_t s = orc_f32_to_f16(scale), o = orc_f32_to_f16(offset);
      memcpy(tail - 4, &s, 2); memcpy(tail - 2, &o, 2);
    } else {
      memcpy(tail - 8, &scale, 4); memcpy(tail - 4, &offset, 4);
    }
  }
}

static inline int64_t load_index(const void *indices, int idx64, int64_t i) {
  return idx64 ? ((const int64_t *)indices)[i] : (int64_t)((const int32_t *)indices)[i];
}

/* libjit_fused_rowwise_quantized_sparse_lengths_weighted_sum_generic (and its _f_u / _f_i32
 * entry points): lib/LLVMIRCodeGen/libjit/libjit.cpp:1253-1276, :2416-2452.
 * UInt8FusedQTy table, fp32 weights, fp32 result. */
ORC_API void orc_frwq_slws_u8_f32(float *dest, const uint8_t *data, const float *weights,
                                  const void *indices, int idx64, const int32_t *lengths,
                                  int64_t segments, int64_t in_line, int64_t out_line) {
  memset(dest, 0, (size_t)(segments * out_line) * sizeof(float));
  int64_t cur = 0;
  for (int64_t i = 0; i < segments; i++) {
    for (int32_t j = 0, e = lengths[i]; j < e; j++) {
      const float weight = weights[cur];
      const int64_t line = load_index(indices, idx64, cur);
      const uint8_t *row = data + line * in_line;
      float scale, offset;
      memcpy(&scale, row + in_line - 8, 4);
      memcpy(&offset, row + in_line - 4, 4);
      for (int64_t k = 0; k < out_line; k++) {
        const float fData = (scale * (float)row[k]) + offset;
        dest[i * out_line + k] += weight * fData;
      }
      cur++;
    }
  }
}

/* One bag of the Interpreter's kernel, shared by the lengths and the offsets forms:
 * lib/Backends/Interpreter/InterpreterNodes.cpp:5797-5840 (and :5936-5978), with
 * dequantizeWithFloatOffset / dequantize4BitWithFloatOffset
 * (include/glow/Quantization/Base/Base.h:385-406) and the float16 class
 * (include/glow/Support/Float16.h:34-88).
 *   out_fp16 : result and weights are fp16 (T = float16_t) instead of fp32
 *   fp16_acc : AccumT = float16_t -- the addend d*w is rounded to fp16, added to the fp16
 *              running sum in fp32, and the sum rounded to fp16, at every step.        */
static void interp_bag(void *dest_row, const uint8_t *data, int kind, const void *weights,
                       const void *indices, int idx64, int64_t begin, int64_t end,
                       int64_t in_line, int64_t out_line, int out_fp16, int fp16_acc,
                       float *accum_f, uint16_t *accum_h) {
  if (fp16_acc) memset(accum_h, 0, (size_t)out_line * 2);   /* float16(0.0f) has bits 0 */
  else for (int64_t k = 0; k < out_line; k++) accum_f[k] = 0.0f;
  for (int64_t c = begin; c < end; c++) {
    const float weight = out_fp16 ? orc_f16_to_f32(((const uint16_t *)weights)[c])
                                  : ((const float *)weights)[c];
    const int64_t rowIdx = load_index(indices, idx64, c);
    const uint8_t *row = data + rowIdx * in_line;
    float scale, offset;
    row_scale_offset(row + in_line, kind, &scale, &offset);
    for (int64_t k = 0; k < out_line; k++) {
      float q;
      if (!kind_is4(kind)) {
        q = (float)row[k];
      } else {
        uint8_t b = row[k / 2];
        if (k & 1) b >>= 4;
        q = (float)(b & 0x0f);
      }
      const float d = (q * scale) + offset;
      const float p = d * weight;
      if (fp16_acc) {
        const float addend = orc_f16_to_f32(orc_f32_to_f16(p));
        accum_h[k] = orc_f32_to_f16(orc_f16_to_f32(accum_h[k]) + addend);
      } else {
        accum_f[k] += p;
      }
    }
  }
  for (int64_t k = 0; k < out_line; k++) {
    if (out_fp16) ((uint16_t *)dest_row)[k] = fp16_acc ? accum_h[k] : orc_f32_to_f16(accum_f[k]);
    else ((float *)dest_row)[k] = accum_f[k];
  }
}

/* fwdFusedRowwiseQuantizedSparseLengthsWeightedSumImpl<T,AccumT,TI> and its dispatcher:
 * InterpreterNodes.cpp:5764-5889.  All four fused kinds; fp32 or fp16 result. */
ORC_API void orc_frwq_slws_interp(void *dest, const uint8_t *data, int kind, const void *weights,
                                  const void *indices, int idx64, const int32_t *lengths,
                                  int64_t segments, int64_t in_line, int64_t out_line,
                                  int out_fp16, int fp16_acc) {
  /* the dispatcher only accumulates in fp16 for an fp16 result on an fp16-scale table */
  if (!(out_fp16 && kind_fp16so(kind))) fp16_acc = 0;
  float *accum_f = (float *)malloc((size_t)(out_line > 0 ? out_line : 1) * sizeof(float));
  uint16_t *accum_h = (uint16_t *)malloc((size_t)(out_line > 0 ? out_line : 1) * 2);
  const size_t esz = out_fp16 ? 2 : 4;
  int64_t cur = 0;
  for (int64_t i = 0; i < segments; i++) {
    int64_t len = lengths[i];
    interp_bag((char *)dest + (size_t)(i * out_line) * esz, data, kind, weights, indices, idx64,
               cur, cur + len, in_line, out_line, out_fp16, fp16_acc, accum_f, accum_h);
    cur += len;
  }
  free(accum_f); free(accum_h);
}

/* libjit_embedding_bag_byte_rowwise_offsets_f: libjit.cpp:2454-2481 (int32 indices/offsets on
 * the CPU backend), and fwdEmbeddingBagByteRowwiseOffsetsImpl: InterpreterNodes.cpp:5896-5986.
 * `segments` counts the entries of `offsets` (so it includes the end offset when present).
 * A segment whose start is not below its end contributes nothing. */
ORC_API void orc_embedding_bag_byte_rowwise_offsets(void *dest, const uint8_t *data, int kind,
                                                    const void *weights, const void *indices,
                                                    const void *offsets, int idx64,
                                                    int64_t segments, int64_t num_indices,
                                                    int64_t in_line, int64_t out_line,
                                                    int has_end_offset, int out_fp16,
                                                    int fp16_acc) {
  if (!(out_fp16 && kind_fp16so(kind))) fp16_acc = 0;
  if (has_end_offset) --segments;
  float *accum_f = (float *)malloc((size_t)(out_line > 0 ? out_line : 1) * sizeof(float));
  uint16_t *accum_h = (uint16_t *)malloc((size_t)(out_line > 0 ? out_line : 1) * 2);
  const size_t esz = out_fp16 ? 2 : 4;
  for (int64_t i = 0; i < segments; i++) {
    int64_t start = load_index(offsets, idx64, i);
    int64_t end = (!has_end_offset && i == segments - 1) ? num_indices : load_index(offsets, idx64, i + 1);
    if (end < start) end = start;
    interp_bag((char *)dest + (size_t)(i * out_line) * esz, data, kind, weights, indices, idx64,
               start, end, in_line, out_line, out_fp16, fp16_acc, accum_f, accum_h);
  }
  free(accum_f); free(accum_h);
}

/* libjit_sparse_lengths_weighted_sum_generic: libjit.cpp:1182-1198 (fp32 table). */
ORC_API void orc_sparse_lengths_weighted_sum_f32(float *dest, const float *data,
                                                 const float *weights, const void *indices,
                                                 int idx64, const int32_t *lengths,
                                                 int64_t segments, int64_t line) {
  memset(dest, 0, (size_t)(segments * line) * sizeof(float));
  int64_t cur = 0;
  for (int64_t i = 0; i < segments; i++)
    for (int32_t j = 0; j < lengths[i]; j++, cur++) {
      const float w = weights[cur];
      const int64_t r = load_index(indices, idx64, cur);
      for (int64_t k = 0; k < line; k++) dest[i * line + k] += w * data[r * line + k];
    }
}

/* libjit_sparse_lengths_sum_generic: libjit.cpp:1164-1180 (fp32 table, rows added as they are). */
ORC_API void orc_sparse_lengths_sum_f32(float *dest, const float *data, const void *indices, int idx64,
                                        const int32_t *lengths, int64_t segments, int64_t line) {
  memset(dest, 0, (size_t)(segments * line) * sizeof(float));
  int64_t cur = 0;
  for (int64_t i = 0; i < segments; i++)
    for (int32_t j = 0; j < lengths[i]; j++, cur++) {
      const int64_t r = load_index(indices, idx64, cur);
      for (int64_t k = 0; k < line; k++) dest[i * line + k] += data[r * line + k];
    }
}

/* libjit_rowwise_quantized_sparse_lengths_weighted_sum_generic: libjit.cpp:1232-1251
 * (uint8 table, per-row fp32 scale and offset in separate vectors). */
ORC_API void orc_rowwise_quantized_slws_f32(float *dest, const uint8_t *data, const float *scales,
                                            const float *offsets, const float *weights,
                                            const void *indices, int idx64, const int32_t *lengths,
                                            int64_t segments, int64_t line) {
  memset(dest, 0, (size_t)(segments * line) * sizeof(float));
  int64_t cur = 0;
  for (int64_t i = 0; i < segments; i++)
    for (int32_t j = 0; j < lengths[i]; j++, cur++) {
      const float w = weights[cur];
      const int64_t r = load_index(indices, idx64, cur);
      const float scale = scales[r], offset = offsets[r];
      for (int64_t k = 0; k < line; k++) {
        const float f = scale * (float)data[r * line + k] + offset;
        dest[i * line + k] += w * f;
      }
    }
}

/* fwdIntNBitSplitEmbeddingWeightedBagsImpl: InterpreterNodes.cpp:6664-6738, with the row helpers
 * of InterpreterNodes.cpp:42-114 (table-batched embedding bags: T tables of mixed element types
 * in one byte buffer).
 *   weights_tys[t] : 0 fp32, 1 fp16, 2 int8, 3 int4 elements (Nodes.h:302-309)
 *   row layout     : int8 / int4 rows START with their scale and offset (two fp16, or two fp32
 *                    when so_fp32), columns follow; rows are padded to row_alignment bytes
 *   placements[t]  : 3 (HOST) reads dev_weights, anything else uvm_weights
 *   offsets        : T*B+1 entries, bag (t, b) = offsets[t*B+b] .. offsets[t*B+b+1]
 *   result         : [B, total_dims], element (b, dim_offsets[t]+d); accumulated in the RESULT
 *                    type (an fp16 result is rounded to fp16 after every row); mean pooling
 *                    divides by the bag length converted to the result type
 *   indice_weights : NULL = 1.0; fp32 or fp16 (iw_fp16)                                        */
ORC_API void orc_int_nbit_split_embedding_bags(
    void *dest, const uint8_t *dev_weights, const uint8_t *uvm_weights, const int32_t *placements,
    const void *weights_offsets, int wo64, const uint8_t *weights_tys, const int32_t *dim_offsets,
    int64_t num_tables, int64_t total_dims, const void *indices, const void *offsets, int idx64,
    int64_t num_bags_per_table, int pooling_mode, const void *indice_weights, int iw_fp16,
    int out_fp16, int so_fp32, int row_alignment) {
  const size_t esz = out_fp16 ? 2 : 4;
  memset(dest, 0, (size_t)(num_bags_per_table * total_dims) * esz);
  const int so = so_fp32 ? 4 : 2;
  for (int64_t t = 0; t < num_tables; t++) {
    const int32_t dim_start = dim_offsets[t], num_dims = dim_offsets[t + 1] - dim_offsets[t];
    const uint8_t *w = placements[t] == 3 ? dev_weights : uvm_weights;
    const int ty = weights_tys[t];
    const int64_t wo = load_index(weights_offsets, wo64, t);
    int32_t unpadded = ty == 0 ? num_dims * 4 : ty == 1 ? num_dims * 2
                     : ty == 2 ? num_dims + 2 * so : num_dims / 2 + 2 * so;
    const int64_t row_bytes = ((unpadded + row_alignment - 1) / row_alignment) * (int64_t)row_alignment;
    for (int64_t b = 0; b < num_bags_per_table; b++) {
      const int64_t start = load_index(offsets, idx64, t * num_bags_per_table + b);
      const int64_t end = load_index(offsets, idx64, t * num_bags_per_table + b + 1);
      for (int32_t d = 0; d < num_dims; d++) {
        float sum_f = 0.0f;          /* OutputTy sum: fp32, or fp16 kept as its fp32 value */
        for (int64_t i = start; i < end; i++) {
          const uint8_t *row = w + wo + load_index(indices, idx64, i) * row_bytes;
          const float weight = !indice_weights ? 1.0f
                             : iw_fp16 ? orc_f16_to_f32(((const uint16_t *)indice_weights)[i])
                                       : ((const float *)indice_weights)[i];
          float v;
          if (ty == 0) { memcpy(&v, row + (size_t)d * 4, 4); }
          else if (ty == 1) { uint16_t h; memcpy(&h, row + (size_t)d * 2, 2); v = orc_f16_to_f32(h); }
          else {
            float scale, offset;
            if (so_fp32) { memcpy(&scale, row, 4); memcpy(&offset, row + 4, 4); }
            else { uint16_t hs, ho; memcpy(&hs, row, 2); memcpy(&ho, row + 2, 2);
                   scale = orc_f16_to_f32(hs); offset = orc_f16_to_f32(ho); }
            const uint8_t byte = ty == 2 ? row[2 * so + d] : row[2 * so + d / 2];
            const uint8_t q = ty == 2 ? byte : ((d & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xF));
            volatile float prod = (float)q * scale;   /* two roundings: no contraction */
            v = prod + offset;
          }
          volatile float addend = weight * v;
          const float s = sum_f + addend;
          sum_f = out_fp16 ? orc_f16_to_f32(orc_f32_to_f16(s)) : s;
        }
        if (pooling_mode == 1 && end > start) {
          const float n = out_fp16 ? orc_f16_to_f32(orc_f32_to_f16((float)(end - start)))
                                   : (float)(end - start);
          sum_f = sum_f / n;
          if (out_fp16) sum_f = orc_f16_to_f32(orc_f32_to_f16(sum_f));
        }
        const int64_t o = b * total_dims + dim_start + d;
        if (out_fp16) ((uint16_t *)dest)[o] = orc_f32_to_f16(sum_f);
        else ((float *)dest)[o] = sum_f;
      }
    }
  }
}

/* ------------------------------------------------------------------------------------ */
/* Dense int8 layers.  Integer arithmetic wraps mod 2^32 like the reference's int32.      */
/* Callers that want more host threads split the batch rows over them (oracle.py).       */
/* ------------------------------------------------------------------------------------ */

/* libjit_rowwise_quantized_fc_generic<int8_t,int32_t>: libjit_matmul.cpp:284-316.
 * in [M,K], weights [N,K] (not transposed), out [M,N]. */
ORC_API void orc_rowwise_quantized_fc_i8_i32(
    int8_t *out, const int8_t *in, const int8_t *w, const int32_t *bias,
    const int32_t *w_offsets, const int32_t *bias_pre, const int32_t *bias_post,
    const int32_t *bias_scale, const int32_t *out_pre, const int32_t *out_post,
    const int32_t *out_scale, int64_t M, int64_t K, int64_t N, int32_t out_offset,
    int32_t in_offset, int32_t bias_offset) {
  for (int64_t i = 0; i < M; i++) {
    for (int64_t j = 0; j < N; j++) {
      uint32_t sum = 0;
      const int32_t wo = w_offsets[j];
      for (int64_t k = 0; k < K; k++)
        sum += (uint32_t)(((int32_t)w[j * K + k] - wo) * ((int32_t)in[i * K + k] - in_offset));
      int32_t B = orc_scale32(bias[j] - bias_offset, bias_pre[j], bias_post[j], bias_scale[j], 0);
      sum += (uint32_t)B;
      out[i * N + j] = orc_clip_i8(orc_scale32((int32_t)sum, out_pre[j], out_post[j], out_scale[j], out_offset));
    }
  }
}

/* libjit_fc_generic<int8_t,int32_t>: libjit_matmul.cpp:254-280.  weights [K,N]. */
ORC_API void orc_fc_i8_i32(int8_t *out, const int8_t *in, const int8_t *w, const int32_t *bias,
                           int64_t M, int64_t K, int64_t N, int32_t out_offset, int32_t in_offset,
                           int32_t w_offset, int32_t bias_offset, int32_t bias_pre,
                           int32_t bias_post, int32_t bias_scale, int32_t out_pre,
                           int32_t out_post, int32_t out_scale) {
  for (int64_t i = 0; i < M; i++) {
    for (int64_t j = 0; j < N; j++) {
      uint32_t sum = (uint32_t)orc_scale32(bias[j] - bias_offset, bias_pre, bias_post, bias_scale, 0);
      for (int64_t k = 0; k < K; k++)
        sum += (uint32_t)(((int32_t)in[i * K + k] - in_offset) * ((int32_t)w[k * N + j] - w_offset));
      out[i * N + j] = orc_clip_i8(orc_scale32((int32_t)sum, out_pre, out_post, out_scale, out_offset));
    }
  }
}

/* libjit_matmul_i8: libjit_matmul.cpp:353-371.  lhs [M,K], rhs [K,N]. */
ORC_API void orc_matmul_i8(int8_t *out, const int8_t *lhs, const int8_t *rhs, int64_t M, int64_t K,
                           int64_t N, int32_t out_offset, int32_t lhs_offset, int32_t rhs_offset,
                           int32_t out_pre, int32_t out_post, int32_t out_scale) {
  for (int64_t x = 0; x < M; x++) {
    for (int64_t y = 0; y < N; y++) {
      uint32_t sum = 0;
      for (int64_t i = 0; i < K; i++)
        sum += (uint32_t)(((int32_t)lhs[x * K + i] - lhs_offset) * ((int32_t)rhs[i * N + y] - rhs_offset));
      out[x * N + y] = orc_clip_i8(orc_scale32((int32_t)sum, out_pre, out_post, out_scale, out_offset));
    }
  }
}

/* libjit_channelwise_quantized_conv2d_generic<int8_t,int32_t>: libjit_conv.cpp:151-239, and
 * (per_channel == 0, every array of length 1) libjit_quantized_conv2d_generic: :49-147.
 * NHWC input, filter [outC,kH,kW,inC/group], taps outside the input are skipped, only
 * pads[0] (top) and pads[1] (left) are read. */
ORC_API void orc_conv2d_i8_i32(
    int8_t *out, const int8_t *in, const int8_t *filter, const int32_t *bias,
    const int64_t *out_dims, const int64_t *in_dims, const int64_t *filter_dims,
    const int64_t *kernels, const int64_t *strides, const int64_t *pads, int64_t group,
    const int64_t *dilation, int32_t out_offset, int32_t in_offset, int per_channel,
    const int32_t *filter_offsets, const int32_t *bias_offsets, const int32_t *bias_pre,
    const int32_t *bias_post, const int32_t *bias_scale, const int32_t *out_pre,
    const int32_t *out_post, const int32_t *out_scale, int32_t act_type,
    const int32_t *act_args) {
  const int64_t inC = in_dims[3], outC = out_dims[3];
  const int64_t inCperG = inC / group, outCperG = outC / group;
  const int64_t IH = in_dims[1], IW = in_dims[2], OH = out_dims[1], OW = out_dims[2];
  const int64_t kh = kernels[0], kw = kernels[1];
  const int64_t fstride = filter_dims[1] * filter_dims[2] * filter_dims[3];
  for (int64_t n = 0; n < in_dims[0]; n++) {
    for (int64_t ax = 0; ax < OH; ax++) {
      const int64_t x = ax * strides[0] - pads[0];
      for (int64_t ay = 0; ay < OW; ay++) {
        const int64_t y = ay * strides[1] - pads[1];
        for (int64_t d = 0; d < outC; d++) {
          const int64_t g = d / outCperG;
          const int64_t c = per_channel ? d : 0;
          const int32_t fo = filter_offsets[c];
          uint32_t sum = (uint32_t)orc_scale32(bias[d] - bias_offsets[c], bias_pre[c], bias_post[c], bias_scale[c], 0);
          for (int64_t fx = 0; fx < kh; fx++) {
            for (int64_t fy = 0; fy < kw; fy++) {
              const int64_t ox = x + fx * dilation[0], oy = y + fy * dilation[1];
              if (ox < 0 || oy < 0 || ox >= IH || oy >= IW) continue;
              const int8_t *ip = in + ((n * IH + ox) * IW + oy) * inC + g * inCperG;
              const int8_t *fp = filter + d * fstride + (fx * filter_dims[2] + fy) * filter_dims[3];
              for (int64_t fd = 0; fd < inCperG; fd++)
                sum += (uint32_t)(((int32_t)fp[fd] - fo) * ((int32_t)ip[fd] - in_offset));
            }
          }
          int32_t s = orc_scale32((int32_t)sum, out_pre[c], out_post[c], out_scale[c], out_offset);
          s = activation_i32(s, out_offset, act_type, act_args);
          out[((n * OH + ax) * OW + ay) * outC + d] = orc_clip_i8(s);
        }
      }
    }
  }
}

/* ------------------------------------------------------------------------------------ */
/* Int8 glue operators of a quantized network.                                           */
/* ------------------------------------------------------------------------------------ */

/* libjit_element_add_kernel_i8 (DEFINE_DATA_PARALLEL_KERNEL_QUANTIZED): libjit.cpp:1593-1603. */
ORC_API void orc_element_add_i8(int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                                int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset,
                                int32_t lhs_pre, int32_t lhs_post, int32_t lhs_scale,
                                int32_t rhs_pre, int32_t rhs_post, int32_t rhs_scale) {
  for (int64_t i = 0; i < n; i++) {
    int32_t l = orc_scale32(lhs[i] - lhs_offset, lhs_pre, lhs_post, lhs_scale, 0);
    int32_t r = orc_scale32(rhs[i] - rhs_offset, rhs_pre, rhs_post, rhs_scale, 0);
    dest[i] = orc_clip_i8(l + r + dest_offset);
  }
}

/* libjit_element_{sub,max,min}_kernel_i8 (DEFINE_DATA_PARALLEL_KERNEL_QUANTIZED): libjit.cpp:1593-1603,
 * 1677-1682.  op 0 add, 1 sub, 2 max, 3 min. */
ORC_API void orc_element_binary_i8(int op, int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                                   int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset,
                                   int32_t lhs_pre, int32_t lhs_post, int32_t lhs_scale,
                                   int32_t rhs_pre, int32_t rhs_post, int32_t rhs_scale) {
  for (int64_t i = 0; i < n; i++) {
    int32_t l = orc_scale32(lhs[i] - lhs_offset, lhs_pre, lhs_post, lhs_scale, 0);
    int32_t r = orc_scale32(rhs[i] - rhs_offset, rhs_pre, rhs_post, rhs_scale, 0);
    int32_t v = op == 0 ? (int32_t)((uint32_t)l + (uint32_t)r) : op == 1 ? (int32_t)((uint32_t)l - (uint32_t)r)
              : op == 2 ? (l > r ? l : r) : (l < r ? l : r);
    dest[i] = orc_clip_i8((int32_t)((uint32_t)v + (uint32_t)dest_offset));
  }
}

/* libjit_element_mul_kernel_i8 / libjit_element_div_kernel_i8 (DEFINE_DATA_PARALLEL_KERNEL_QUANTIZED_M):
 * libjit.cpp:1610-1619, 1683-1684.  A zero divisor is given the quotient 0 (the reference traps). */
ORC_API void orc_element_muldiv_i8(int is_div, int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                                   int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset,
                                   int32_t pre, int32_t post, int32_t scale) {
  for (int64_t i = 0; i < n; i++) {
    int32_t l = lhs[i] - lhs_offset, r = rhs[i] - rhs_offset;
    int32_t v = is_div ? (r == 0 ? 0 : l / r) : (int32_t)((uint32_t)l * (uint32_t)r);
    dest[i] = orc_clip_i8(orc_scale32(v, pre, post, scale, dest_offset));
  }
}

/* libjit_batchedadd_quantized: libjit.cpp:997-1015 (libjit_batchedadd_i8, libjit_batchedadd_i32_i8). */
ORC_API void orc_batched_add_i8(int8_t *dest, const int8_t *batch, const void *slice, int slice_is_i32,
                                int64_t num_slices, int64_t slice_size, int32_t dest_offset,
                                int32_t batch_offset, int32_t slice_offset, int32_t batch_pre,
                                int32_t batch_post, int32_t batch_scale, int32_t slice_pre,
                                int32_t slice_post, int32_t slice_scale) {
  for (int64_t n = 0; n < num_slices; n++)
    for (int64_t i = 0; i < slice_size; i++) {
      int32_t b = batch[n * slice_size + i] - batch_offset;
      int32_t sv = slice_is_i32 ? ((const int32_t *)slice)[i] : ((const int8_t *)slice)[i];
      int32_t s = (int32_t)((uint32_t)sv - (uint32_t)slice_offset);
      int32_t x = orc_scale32(b, batch_pre, batch_post, batch_scale, 0);
      int32_t y = orc_scale32(s, slice_pre, slice_post, slice_scale, 0);
      dest[n * slice_size + i] = orc_clip_i8((int32_t)((uint32_t)x + (uint32_t)y + (uint32_t)dest_offset));
    }
}

/* libjit_element_relu_i8: libjit.cpp:1850-1858: max(x, srcOffset) then rescale. */
ORC_API void orc_element_relu_i8(int8_t *dest, const int8_t *src, int64_t n, int32_t src_offset,
                                 int32_t dest_offset, int32_t pre, int32_t post, int32_t scale) {
  for (int64_t i = 0; i < n; i++) {
    int32_t v = src[i] > src_offset ? src[i] : src_offset;
    dest[i] = orc_clip_i8(orc_scale32(v - src_offset, pre, post, scale, dest_offset));
  }
}

/* libjit_element_maxsplat_kernel_i8: lib/Backends/CPU/libjit_cpu/libjit_cpu.cpp:39-44. */
ORC_API void orc_element_maxsplat_i8(int8_t *dest, const int8_t *src, int64_t n, int8_t splat) {
  for (int64_t i = 0; i < n; i++) dest[i] = src[i] > splat ? src[i] : splat;
}

/* libjit_element_rescale_kernel_i8: libjit.cpp:3030-3038. */
ORC_API void orc_element_rescale_i8(int8_t *dest, const int8_t *src, int64_t n, int32_t out_offset,
                                    int32_t in_offset, int32_t pre, int32_t post, int32_t scale) {
  for (int64_t i = 0; i < n; i++)
    dest[i] = orc_clip_i8(orc_scale32(src[i] - in_offset, pre, post, scale, out_offset));
}

/* libjit_element_quantize_kernel_i8: libjit.cpp:2997-3002 (nearbyintf, round-half-even). */
ORC_API void orc_element_quantize_i8(int8_t *dest, const float *src, int64_t n, float scale,
                                     int32_t offset) {
  for (int64_t i = 0; i < n; i++) {
    float t = src[i] / scale;
    t = t + (float)offset;
    dest[i] = orc_clip_i8((int32_t)nearbyintf(t));
  }
}

/* libjit_element_dequantize_kernel_i8: libjit.cpp:3014-3018. */
ORC_API void orc_element_dequantize_i8(float *dest, const int8_t *src, int64_t n, float scale,
                                       int32_t offset) {
  for (int64_t i = 0; i < n; i++) dest[i] = scale * (float)(src[i] - offset);
}

/* libjit_max_pool_generic<int8_t>: libjit.cpp:811-860 via libjit_max_pool_i8 :2592-2597.
 * NHWC; window cells outside the input are skipped; an empty window yields the output
 * offset (the `defaultValue`). */
ORC_API void orc_max_pool_i8(const int8_t *in, int8_t *out, const int64_t *in_dims,
                             const int64_t *out_dims, const int64_t *kernels,
                             const int64_t *strides, const int64_t *pads, int32_t out_offset) {
  const int64_t IH = in_dims[1], IW = in_dims[2], C = in_dims[3], OH = out_dims[1], OW = out_dims[2];
  for (int64_t n = 0; n < in_dims[0]; n++)
    for (int64_t oh = 0; oh < OH; oh++)
      for (int64_t ow = 0; ow < OW; ow++)
        for (int64_t c = 0; c < C; c++) {
          int first = 1; int8_t best = (int8_t)out_offset;
          for (int64_t fh = 0; fh < kernels[0]; fh++)
            for (int64_t fw = 0; fw < kernels[1]; fw++) {
              int64_t ih = oh * strides[0] - pads[0] + fh, iw = ow * strides[1] - pads[1] + fw;
              if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
              int8_t v = in[((n * IH + ih) * IW + iw) * C + c];
              if (first || v > best) { best = v; first = 0; }
            }
          out[((n * OH + oh) * OW + ow) * C + c] = best;
        }
}

/* libjit_avg_pool_i8: libjit.cpp:2812-2897. */
ORC_API void orc_avg_pool_i8(const int8_t *in, int8_t *out, const int64_t *in_dims,
                             const int64_t *out_dims, const int64_t *kernels,
                             const int64_t *strides, const int64_t *pads, int count_include_pads,
                             int32_t out_offset, int32_t in_offset, int32_t out_pre,
                             int32_t out_post, int32_t out_scale) {
  const int64_t IH = in_dims[1], IW = in_dims[2], C = in_dims[3], OH = out_dims[1], OW = out_dims[2];
  for (int64_t n = 0; n < in_dims[0]; n++)
    for (int64_t oh = 0; oh < OH; oh++)
      for (int64_t ow = 0; ow < OW; ow++)
        for (int64_t c = 0; c < C; c++) {
          int32_t sum = 0, area = 0;
          for (int64_t fh = 0; fh < kernels[0]; fh++)
            for (int64_t fw = 0; fw < kernels[1]; fw++) {
              int64_t ih = oh * strides[0] - pads[0] + fh, iw = ow * strides[1] - pads[1] + fw;
              if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
              sum += in[((n * IH + ih) * IW + iw) * C + c] - in_offset;
              area++;
            }
          int8_t r;
          if (count_include_pads) {
            r = orc_clip_i8(orc_scale32(sum, out_pre, out_post, out_scale, out_offset));
          } else if (area == 0) {
            r = (int8_t)out_offset;
          } else {
            int32_t s = orc_scale32(sum, out_pre, out_post, out_scale, 0);
            r = orc_clip_i8(div_round_i32(s, area) + out_offset);
          }
          out[((n * OH + oh) * OW + ow) * C + c] = r;
        }
}

/* ------------------------------------------------------------------------------------ */
/* Host-side weight preparation.                                                         */
/* ------------------------------------------------------------------------------------ */

/* chooseQuantizationParams, Calibration::None: lib/Quantization/Base/Base.cpp:433-565.
 * schema 0 Asymmetric, 1 Symmetric, 2 SymmetricWithUnsigned, 3 SymmetricWithPower2Scale. */
ORC_API void orc_choose_quantization_params(float min, float max, int schema, int64_t qmin, int64_t qmax,
                                            float *scale_out, int32_t *offset_out) {
  if (min > 0.f) min = 0.f;
  if (max < 0.f) max = 0.f;
  if (schema == 2 && !(min >= 0.f)) schema = 1;
  if (schema == 1 || schema == 3) {
    double rmin = min / (double)qmin, rmax = max / (double)qmax;
    if (rmin > rmax) max = (float)(rmin * qmax); else min = (float)(rmax * qmin);
  }
  double scale = ((double)max - min) / ((double)qmax - qmin);
  if (scale == 0) scale = 0.1;
  double zmin = qmin - min / scale, zmax = qmax - max / scale;
  double emin = fabs((double)qmin) + fabs(min / scale), emax = fabs((double)qmax) + fabs(max / scale);
  double zp = emin < emax ? zmin : zmax;
  if (fabsf(max + min) <= 1.1920928955078125e-07f) zp = 0;
  int32_t nudged;
  if (zp < qmin) nudged = (int32_t)qmin; else if (zp > qmax) nudged = (int32_t)qmax; else nudged = (int32_t)round(zp);
  if (schema == 3) scale = exp2(ceil(log2(scale)));
  *scale_out = (float)scale;
  *offset_out = nudged;
}

/* tensorRowwiseQuantization<float,int32_t,int8_t>: include/glow/Quantization/Base/Base.h:522-576,
 * with quantization::quantize (:322-329). */
ORC_API void orc_tensor_rowwise_quantize_i8(const float *in, int64_t rows, int64_t cols, int schema, int8_t *out,
                                            float *scales, int32_t *offsets) {
  for (int64_t i = 0; i < rows; i++) {
    const float *r = in + i * cols;
    float mn = r[0], mx = r[0];
    for (int64_t j = 1; j < cols; j++) { if (r[j] < mn) mn = r[j]; if (r[j] > mx) mx = r[j]; }
    orc_choose_quantization_params(mn, mx, schema, -128, 127, &scales[i], &offsets[i]);
    for (int64_t j = 0; j < cols; j++) {
      float t = r[j] / scales[i] + (float)offsets[i];
      int64_t v = (int64_t)nearbyintf(t);
      out[i * cols + j] = (int8_t)(v < -128 ? -128 : (v > 127 ? 127 : v));
    }
  }
}

/* fwdDynRowwiseQuantizedFullyConnectedInstPreimpl / ...InstImpl: InterpreterNodes.cpp:4677-4749
 * (and fwdDynamicQuantizedFullyConnectedInst, :4766-4790, which repeats the weights' type-level
 * scale and offset for every column).  in [M,K] fp16, weights [K,N] int8, out [M,N] fp16.
 * Every input row is quantized on its own: Symmetric int8 parameters from its min and max, then
 * quantization::quantize (Base.h:322-329). */
ORC_API void orc_dynamic_rowwise_quantized_fc(uint16_t *out, const uint16_t *in, const int8_t *w, const float *bias,
                                              const float *scales, const int32_t *offsets, int64_t M, int64_t K,
                                              int64_t N) {
  int8_t *q = (int8_t *)malloc((size_t)(K > 0 ? K : 1));
  for (int64_t i = 0; i < M; i++) {
    float mn = orc_f16_to_f32(in[i * K]), mx = mn;
    for (int64_t k = 1; k < K; k++) {
      const float v = orc_f16_to_f32(in[i * K + k]);
      if (v < mn) mn = v;
      if (v > mx) mx = v;
    }
    float in_scale;
    int32_t in_offset;
    orc_choose_quantization_params(mn, mx, 1, -128, 127, &in_scale, &in_offset);
    for (int64_t k = 0; k < K; k++) {
      const float t = orc_f16_to_f32(in[i * K + k]) / in_scale + (float)in_offset;
      const int64_t v = (int64_t)nearbyintf(t);
      q[k] = (int8_t)(v < -128 ? -128 : (v > 127 ? 127 : v));
    }
    for (int64_t j = 0; j < N; j++) {
      const float mm = in_scale * scales[j];
      int32_t sum = 0;
      for (int64_t k = 0; k < K; k++)
        sum = (int32_t)((uint32_t)sum + (uint32_t)(((int32_t)w[k * N + j] - offsets[j]) * ((int32_t)q[k] - in_offset)));
      volatile float prod = (float)sum * mm;   /* product and sum rounded separately */
      out[i * N + j] = orc_f32_to_f16(prod + bias[j]);
    }
  }
  free(q);
}

/* libjit_quantization_profile: libjit.cpp:3440-3523 (generateTensorHistogram, Profile.cpp:36-112).
 * comp_info = {running min, running max}; hist has `bins` float counters. */
static uint64_t orc_get_bin(uint64_t bins, float width, float minv, float v) {
  if (width == 0.0f) return 0;
  uint64_t b = (uint64_t)((v - minv) / width);
  return b < bins - 1 ? b : bins - 1;
}
ORC_API void orc_quantization_profile(const float *x, int64_t n, float *comp_info, float *hist, int64_t bins) {
  float mn = comp_info[0], mx = comp_info[1];
  float min_in = x[0], max_in = x[0];
  for (int64_t i = 1; i < n; i++) { if (x[i] < min_in) min_in = x[i]; if (x[i] > max_in) max_in = x[i]; }
  const float new_min = min_in < mn ? min_in : mn, new_max = max_in > mx ? max_in : mx;
  comp_info[0] = new_min;
  comp_info[1] = new_max;
  if (bins == 0) return;
  int all_zero = 1;
  for (int64_t i = 0; i < bins; i++) if (hist[i] != 0) { all_zero = 0; break; }
  if (all_zero) { mn = min_in; mx = max_in; }
  if (new_min < mn || new_max > mx) {
    const float dest_w = (new_max - new_min) / (float)(uint64_t)bins, src_w = (mx - mn) / (float)(uint64_t)bins;
    float *scaled = (float *)calloc((size_t)bins, sizeof(float));
    for (int64_t i = 0; i < bins; i++) {
      if (hist[i] == 0) continue;
      const float src_begin = mn + src_w * (float)(uint64_t)i;
      const uint64_t dest_bin = (uint64_t)((src_begin - new_min) / dest_w);
      const float dest_end = new_min + dest_w * (float)(dest_bin + 1);
      const float rounded = (float)round((double)((dest_end - src_begin) / src_w * hist[i]));
      const uint64_t cnt = (uint64_t)(rounded < hist[i] ? rounded : hist[i]);
      scaled[orc_get_bin((uint64_t)bins, dest_w, new_min, src_begin)] += (float)cnt;
      if ((float)cnt < hist[i])
        scaled[orc_get_bin((uint64_t)bins, dest_w, new_min, src_begin + dest_w)] += hist[i] - (float)cnt;
    }
    memcpy(hist, scaled, (size_t)bins * sizeof(float));
    free(scaled);
    mn = new_min;
    mx = new_max;
  }
  const float width = (mx - mn) / (float)(uint64_t)bins;
  for (int64_t i = 0; i < n; i++) hist[orc_get_bin((uint64_t)bins, width, mn, x[i])] += 1.0f;
}

/* Pairwise-dot feature interaction of the benchmark's recommendation model: no single kernel in
 * the reference (it composes Concat/Reshape/BatchMatMul, tests/unittests/
 * RecommendationSystemTest.cpp:640-680); this restates the definition the CUDA kernel
 * implements: out[b] = [v_0 | v_i.v_j for j < i, row-major], every dot product a sequential
 * fp32 FMA chain over the components. */
ORC_API void orc_pairwise_dot_interaction(const float *dense, const float *pooled, int64_t batch, int64_t tables,
                                          int64_t dim, float *out) {
  const int64_t n = tables + 1, width = dim + n * (n - 1) / 2;
  for (int64_t b = 0; b < batch; b++) {
    float *o = out + b * width;
    for (int64_t k = 0; k < dim; k++) o[k] = dense[b * dim + k];
    int64_t p = dim;
    for (int64_t i = 1; i < n; i++)
      for (int64_t j = 0; j < i; j++) {
        const float *a = pooled + (b * tables + (i - 1)) * dim;
        const float *c = j == 0 ? dense + b * dim : pooled + (b * tables + (j - 1)) * dim;
        float acc = 0.0f;
        for (int64_t k = 0; k < dim; k++) acc = fmaf(a[k], c[k], acc);
        o[p++] = acc;
      }
  }
}
