// Gather-pool over tables that are not fused-rowwise:
//   * fp32 tables -- SparseLengthsSum / SparseLengthsWeightedSum
//     (libjit_sparse_lengths_sum_generic, libjit_sparse_lengths_weighted_sum_generic:
//      lib/LLVMIRCodeGen/libjit/libjit.cpp:1164-1198);
//   * uint8 tables with per-row scale and offset in separate vectors --
//     RowwiseQuantizedSparseLengthsWeightedSum
//     (libjit_rowwise_quantized_sparse_lengths_weighted_sum_generic: libjit.cpp:1232-1251).
//
// A group of lanes owns a bag and walks its rows in index order, every lane keeping the sums of
// its own columns, so each result element is accumulated in exactly the reference's order; the
// multiply and the add are kept apart (no FMA contraction), which makes the result bit-identical
// to the reference kernel compiled without fast-math.  Several rows are requested before the
// first is consumed: the loop is bound by random row fetches from HBM, like the fused kernel.
#include "common.cuh"

namespace glowb200 {
namespace {

struct UnfusedLaunch {
  void *dest;
  const void *data;
  const float *scales, *offsets;  // rowwise-quantized tables only
  const float *weights;           // nullptr: every weight is 1
  const void *indices;
  const int64_t *seg_begin;
  int32_t *status;
  int64_t rows, segments;
  int32_t line;  // columns of a row (and of a result row)
  int32_t lpr_log2;
};

constexpr int kThreads = 256;
constexpr int kTiles = 4;   // column tiles a lane carries
constexpr int kRows = 4;    // rows in flight

// SRC 0: fp32 rows; SRC 1: uint8 rows + scale/offset vectors.  VEC: 4 columns per lane per tile
// through 16-byte (fp32) or 4-byte (uint8) loads; otherwise one column per lane per tile.
template <int SRC, typename IdxT, bool VEC>
__global__ void __launch_bounds__(kThreads) slws_unfused_kernel(const __grid_constant__ UnfusedLaunch p) {
  constexpr int W = VEC ? 4 : 1;
  const int lpr = 1 << p.lpr_log2;
  const int gl = threadIdx.x & (lpr - 1);
  const int64_t bag = (int64_t)blockIdx.x * (kThreads >> p.lpr_log2) + (threadIdx.x >> p.lpr_log2);
  if (bag >= p.segments) return;
  const int64_t begin = p.seg_begin[bag], end = p.seg_begin[bag + 1];
  const IdxT *indices = reinterpret_cast<const IdxT *>(p.indices);
  const int D = p.line;
  const int span = lpr * W * kTiles;
  int32_t flags = 0;

  for (int base = 0; base < D; base += span) {
    int col[kTiles];
    bool has[kTiles];
#pragma unroll
    for (int t = 0; t < kTiles; t++) {
      col[t] = base + (t * lpr + gl) * W;
      has[t] = col[t] < D;
    }
    float acc[kTiles][W];
#pragma unroll
    for (int t = 0; t < kTiles; t++)
#pragma unroll
      for (int i = 0; i < W; i++) acc[t][i] = 0.0f;

    for (int64_t j = begin; j < end; j += kRows) {
      int64_t r[kRows];
      float w[kRows], scale[kRows], offset[kRows];
      float x[kRows][kTiles][W];
#pragma unroll
      for (int u = 0; u < kRows; u++) {
        r[u] = -1;
        w[u] = 1.0f;
        if (j + u < end) {
          const int64_t v = (int64_t)indices[j + u];
          if (v < 0 || v >= p.rows) flags |= GLOWB200_STATUS_INDEX_OUT_OF_RANGE;
          else r[u] = v;
          if (p.weights != nullptr) w[u] = p.weights[j + u];
        }
      }
#pragma unroll
      for (int u = 0; u < kRows; u++) {
        if (r[u] < 0) continue;
        if constexpr (SRC == 1) {
          scale[u] = p.scales[r[u]];
          offset[u] = p.offsets[r[u]];
        }
#pragma unroll
        for (int t = 0; t < kTiles; t++) {
          if (!has[t]) continue;
          if constexpr (SRC == 0) {
            const float *row = reinterpret_cast<const float *>(p.data) + r[u] * D + col[t];
            if constexpr (VEC) {
              const float4 q = __ldg(reinterpret_cast<const float4 *>(row));
              x[u][t][0] = q.x; x[u][t][1] = q.y; x[u][t][2] = q.z; x[u][t][3] = q.w;
            } else {
              x[u][t][0] = __ldg(row);
            }
          } else {
            const uint8_t *row = reinterpret_cast<const uint8_t *>(p.data) + r[u] * D + col[t];
            if constexpr (VEC) {
              const uint32_t q = __ldg(reinterpret_cast<const uint32_t *>(row));
#pragma unroll
              for (int i = 0; i < 4; i++) x[u][t][i] = (float)((q >> (8 * i)) & 0xFFu);
            } else {
              x[u][t][0] = (float)__ldg(row);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kRows; u++) {
        if (r[u] < 0) continue;
#pragma unroll
        for (int t = 0; t < kTiles; t++) {
          if (!has[t]) continue;
#pragma unroll
          for (int i = 0; i < W; i++) {
            float d = x[u][t][i];
            if constexpr (SRC == 1) d = __fadd_rn(__fmul_rn(scale[u], d), offset[u]);
            // SparseLengthsSum adds the row itself; the weighted forms add weight * value
            acc[t][i] = __fadd_rn(acc[t][i], p.weights != nullptr ? __fmul_rn(w[u], d) : d);
          }
        }
      }
    }

    float *out = reinterpret_cast<float *>(p.dest) + bag * D;
#pragma unroll
    for (int t = 0; t < kTiles; t++) {
      if (!has[t]) continue;
      if constexpr (VEC) *reinterpret_cast<float4 *>(out + col[t]) = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
      else out[col[t]] = acc[t][0];
    }
  }
  if (p.status != nullptr && flags != 0) atomicOr(p.status, flags);
}

template <int SRC, typename IdxT>
void launch_vec(const UnfusedLaunch &L, bool vec, unsigned blocks, cudaStream_t s) {
  if (vec) slws_unfused_kernel<SRC, IdxT, true><<<blocks, kThreads, 0, s>>>(L);
  else slws_unfused_kernel<SRC, IdxT, false><<<blocks, kThreads, 0, s>>>(L);
}

int run(int src, void *dest, const void *data, const float *scales, const float *offsets, int64_t rows,
        const float *weights, const void *indices, int idx64, const int32_t *lengths, int64_t segments,
        int64_t num_indices, int64_t line, void *workspace, size_t workspace_bytes, int32_t *status,
        cudaStream_t s) {
  GLOWB200_REQUIRE(segments >= 0 && segments < (1ll << 31), "segments out of range");
  GLOWB200_REQUIRE(rows >= 0 && num_indices >= 0 && line > 0 && line < (1ll << 24), "rows / num_indices / line_size out of range");
  if (segments == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(dest != nullptr && (num_indices == 0 || (data != nullptr && indices != nullptr)), "NULL tensor pointer");
  GLOWB200_REQUIRE(src == 0 || num_indices == 0 || (scales != nullptr && offsets != nullptr), "scales / offsets is NULL");
  if (int rc = launch_segments_from_lengths(lengths, segments, num_indices, workspace, workspace_bytes, status, s)) return rc;
  const uintptr_t da = reinterpret_cast<uintptr_t>(data), oa = reinterpret_cast<uintptr_t>(dest);
  const bool vec = (line % 4 == 0) && (oa % 16 == 0) && (da % (src == 0 ? 16 : 4) == 0);
  const int64_t per_lane = vec ? 4 : 1;
  int lpr_log2 = 0;
  while (lpr_log2 < 5 && ((int64_t)1 << lpr_log2) * per_lane * kTiles < line) lpr_log2++;
  UnfusedLaunch L{};
  L.dest = dest;
  L.data = data;
  L.scales = scales;
  L.offsets = offsets;
  L.weights = weights;
  L.indices = indices;
  L.seg_begin = reinterpret_cast<const int64_t *>(workspace);
  L.status = status;
  L.rows = rows;
  L.segments = segments;
  L.line = (int32_t)line;
  L.lpr_log2 = lpr_log2;
  const int64_t bags_per_block = kThreads >> lpr_log2;
  const unsigned blocks = (unsigned)((segments + bags_per_block - 1) / bags_per_block);
  if (src == 0) {
    if (idx64) launch_vec<0, int64_t>(L, vec, blocks, s);
    else launch_vec<0, int32_t>(L, vec, blocks, s);
  } else {
    if (idx64) launch_vec<1, int64_t>(L, vec, blocks, s);
    else launch_vec<1, int32_t>(L, vec, blocks, s);
  }
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

}  // namespace
}  // namespace glowb200

extern "C" int glowb200_sparse_lengths_weighted_sum_f32(float *dest, const float *data, int64_t rows,
                                                         const float *weights, const void *indices,
                                                         int indices_are_int64, const int32_t *lengths,
                                                         int64_t segments, int64_t num_indices, int64_t line_size,
                                                         void *workspace, size_t workspace_bytes, int32_t *status,
                                                         glowb200_stream_t stream) {
  return glowb200::run(0, dest, data, nullptr, nullptr, rows, weights, indices, indices_are_int64, lengths, segments,
                       num_indices, line_size, workspace, workspace_bytes, status, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int glowb200_rowwise_quantized_sparse_lengths_weighted_sum_f32(
    float *dest, const uint8_t *data, const float *scales, const float *offsets, int64_t rows, const float *weights,
    const void *indices, int indices_are_int64, const int32_t *lengths, int64_t segments, int64_t num_indices,
    int64_t line_size, void *workspace, size_t workspace_bytes, int32_t *status, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(weights != nullptr || num_indices == 0 || segments == 0, "weights is NULL");
  return glowb200::run(1, dest, data, scales, offsets, rows, weights, indices, indices_are_int64, lengths, segments,
                       num_indices, line_size, workspace, workspace_bytes, status, reinterpret_cast<cudaStream_t>(stream));
}
