// Table-batched embedding bags: IntNBitSplitEmbeddingBags / IntNBitSplitEmbeddingWeightedBags.
//
// Reference: fwdIntNBitSplitEmbeddingWeightedBagsImpl and the row helpers of
// lib/Backends/Interpreter/InterpreterNodes.cpp:42-114, 6593-6738 (the CPU backend has no kernel
// for this node).  T tables of mixed element type (fp32, fp16, int8, int4) live in one byte
// buffer; int8 / int4 rows start with their scale and offset, rows are padded to a byte
// alignment; the request holds T*B bags, bag (t, b) = offsets[t*B+b] .. offsets[t*B+b+1], and
// the result is [B, total_dims] with table t's columns at dim_offsets[t].
//
// One launch pools every bag of every table.  blockIdx.y is the table; inside a table a group of
// lanes (as many as a row has 16-byte chunks, 8-byte ones for tables off 16-byte boundaries) owns a bag and walks its
// rows in index order, each lane keeping the sums of the columns of its own chunk: every result
// element is accumulated in the reference's order and in the result's type (an fp16 result is
// rounded after every row, as the reference's float16 sum is), with the multiply and the add
// kept apart, so results are bit-identical to the Interpreter's.  Four rows are requested before
// the first is consumed; the loop is bound by random row fetches from HBM.
//
// A lane's chunk is cut from the row start, not from the first column: for int8 / int4 rows the
// first lane's chunk begins with the scale/offset header, so all loads stay aligned to the chunk
// size although the columns start 4 (or 8) bytes into the row.
#include "common.cuh"

namespace glowb200 {
namespace {

struct SplitLaunch {
  void *dest;
  const uint8_t *dev_weights, *uvm_weights;
  int64_t dev_bytes, uvm_bytes;
  const int32_t *placements;
  const void *weights_offsets;
  const uint8_t *weights_tys;
  const int32_t *dim_offsets;
  const void *indices, *offsets;
  const void *indice_weights;
  int32_t *status;
  int64_t num_indices, bags_per_table, total_dims;
  int32_t wo64, iw16, so_fp32, row_alignment, pooling_mode;
};

constexpr int kThreads = 256;
#ifndef GLOWB200_TBE_MIN_BLOCKS
#define GLOWB200_TBE_MIN_BLOCKS 4
#endif
#ifndef GLOWB200_TBE_I4_WIDE
#define GLOWB200_TBE_I4_WIDE 1
#endif
#ifndef GLOWB200_TBE_ROWS
#define GLOWB200_TBE_ROWS 4
#endif
constexpr int kRows = GLOWB200_TBE_ROWS;  // rows in flight per lane

enum : int { TY_F32 = 0, TY_F16 = 1, TY_I8 = 2, TY_I4 = 3 };

// The bytes [at, at + 4*CW) of a table as CW words.  A chunk that is aligned and lies inside
// the buffer is one vector load; the last chunk of a buffer that ends with an unpadded row, and
// tables at odd addresses, are put together from single bytes (bytes past the end read as 0).
template <int CW>
__device__ __forceinline__ void load_chunk(const uint8_t *base, int64_t at, int64_t limit, bool vec, uint32_t (&q)[CW]) {
  if (vec && at + 4 * CW <= limit) {
    if constexpr (CW == 4) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(base + at));
      q[0] = v.x; q[1] = v.y; q[2] = v.z; q[3] = v.w;
    } else {
      const uint2 v = __ldg(reinterpret_cast<const uint2 *>(base + at));
      q[0] = v.x; q[1] = v.y;
    }
  } else {
#pragma unroll
    for (int w = 0; w < CW; w++) {
      uint32_t word = 0;
#pragma unroll
      for (int b = 0; b < 4; b++) {
        const int64_t o = at + 4 * w + b;
        if (o < limit) word |= (uint32_t)__ldg(base + o) << (8 * b);
      }
      q[w] = word;
    }
  }
}

// float(h) for the fp16 number in the low half of `h`, through the mixed-precision add of sm_100
// (adding -0 keeps every value, the sign of a zero included) instead of a conversion
// instruction: conversions issue at an eighth of the rate of adds, and this kernel would be
// bound by them.
__device__ __forceinline__ float add_f32_f16(uint16_t h, float c) {
  float d;
  asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(h), "f"(c));
  return d;
}
__device__ __forceinline__ float half_bits_to_float(uint32_t h) { return add_f32_f16((uint16_t)(h & 0xFFFFu), -0.0f); }
#ifndef GLOWB200_TBE_X2
#define GLOWB200_TBE_X2 1
#endif
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpack2f(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// Two floats rounded to fp16 (round to nearest even), packed {lo, hi}: one conversion for two.
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// Pools the bag [begin, end) of one table for the lanes of one group.
//   TY   element type of the table; CW words per lane chunk (2 or 4); SO32: fp32 row headers
//   gl / lpr  lane within the group / lanes of the group
// Slots (the elements of a lane's chunk) are handled in pairs.  An fp16 result keeps its running
// sums as fp16 pairs: per row the sum is widened, added to in fp32 and rounded back
// (float16::operator+ of the reference, include/glow/Support/Float16.h:47-49).
// Quantized elements become floats without a conversion instruction: byte or nibble q is merged
// into the mantissa of the fp16 number 1024 (0x6400 | q = 1024 + q) and 1024 is subtracted in the
// mixed-precision add.  With fp16 headers q * scale is exact in fp32 (8 + 11 significant bits), so
// one fused multiply-add gives the reference's separately rounded q * scale + offset.
template <int TY, int CW, bool OUT16, bool WEIGHTED, bool SO32, typename IdxT>
__device__ __forceinline__ int32_t pool_bag(const SplitLaunch &p, const uint8_t *base, int64_t limit, int64_t table_at,
                                            int32_t row_bytes, int32_t touched, int32_t num_dims, bool vec,
                                            int64_t begin, int64_t end, int gl, int lpr, void *out_row) {
  constexpr int CB = 4 * CW;                                           // chunk bytes
  constexpr int SLOTS = TY == TY_F32 ? CW : TY == TY_F16 ? 2 * CW : TY == TY_I8 ? 4 * CW : 8 * CW;
  constexpr int PAIRS = SLOTS / 2;
  constexpr int H = (TY == TY_I8 || TY == TY_I4) ? (SO32 ? 8 : 4) : 0;  // header bytes of a row
  const IdxT *indices = reinterpret_cast<const IdxT *>(p.indices);
  int32_t flags = 0;
  // the two slots of pair i: neighbours, except for nibbles, where one mask takes nibbles k and k + 4 of a word
  auto slot_a = [](int i) { return TY == TY_I4 ? 8 * (i >> 2) + (i & 3) : 2 * i; };
  auto slot_b = [](int i) { return TY == TY_I4 ? 8 * (i >> 2) + (i & 3) + 4 : 2 * i + 1; };
  // rows whose touched bytes all lie inside the buffer (InterpreterNodes.cpp:6720): 0 .. max_row
  int64_t max_row = -1;
  if (table_at >= 0 && table_at + touched <= limit) max_row = (limit - touched - table_at) / row_bytes;
  if (max_row > 0x7FFFFFFEll) max_row = 0x7FFFFFFEll;

  for (int32_t cbase = 0; cbase < touched; cbase += lpr * CB) {
    const int32_t at = cbase + gl * CB;          // byte of the row this lane's chunk starts at
    const bool has = at < touched;
    // column of slot 0 (negative inside the header)
    const int32_t col0 = TY == TY_F32 ? at / 4 : TY == TY_F16 ? at / 2 : TY == TY_I8 ? at - H : 2 * (at - H);
    float acc[OUT16 ? 1 : SLOTS];      // fp32 result: the sums
    uint32_t acch[OUT16 ? PAIRS : 1];  // fp16 result: the sums as fp16 pairs {slot_a, slot_b}
#pragma unroll
    for (int s = 0; s < (OUT16 ? 1 : SLOTS); s++) acc[s] = 0.0f;
#pragma unroll
    for (int s = 0; s < (OUT16 ? PAIRS : 1); s++) acch[s] = 0u;

    // The indices (and weights) of the next kRows rows are requested while the current rows are
    // in flight: an index fetch and the row fetch that depends on it would otherwise add their
    // latencies in every trip of the loop.  A row is kept as a 32-bit number: -2 none, -1 refused.
    int32_t next_r[kRows];
    float next_w[kRows];
    auto request = [&](int64_t j) {
#pragma unroll
      for (int u = 0; u < kRows; u++) {
        next_r[u] = -2;
        next_w[u] = 1.0f;
        if (j + u < end) {
          const int64_t r = (int64_t)indices[j + u];
          next_r[u] = (r < 0 || r > max_row) ? -1 : (int32_t)r;
          if constexpr (WEIGHTED)
            next_w[u] = p.iw16 ? __half2float(reinterpret_cast<const __half *>(p.indice_weights)[j + u])
                               : reinterpret_cast<const float *>(p.indice_weights)[j + u];
        }
      }
    };
    request(begin);
    for (int64_t j = begin; j < end; j += kRows) {
      bool live[kRows];
      float w[kRows];
      uint32_t q[kRows][CW];
      uint32_t hdr[kRows][2];
#pragma unroll
      for (int u = 0; u < kRows; u++) {
        w[u] = next_w[u];
        live[u] = next_r[u] >= 0 && has;
        if (next_r[u] == -1) flags |= GLOWB200_STATUS_INDEX_OUT_OF_RANGE;
        if (!live[u]) continue;
        const int64_t row_at = table_at + (int64_t)next_r[u] * row_bytes;
        load_chunk<CW>(base, row_at + at, limit, vec, q[u]);
        if constexpr (TY == TY_I8 || TY == TY_I4) {
          // all lanes of the group read the same header word(s): one transaction
          if (vec) {
            hdr[u][0] = __ldg(reinterpret_cast<const uint32_t *>(base + row_at));
            hdr[u][1] = SO32 ? __ldg(reinterpret_cast<const uint32_t *>(base + row_at + 4)) : 0u;
          } else {
            uint32_t h2[2];
            load_chunk<2>(base, row_at, limit, false, h2);
            hdr[u][0] = h2[0];
            hdr[u][1] = h2[1];
          }
        }
      }
      request(j + kRows);
#pragma unroll
      for (int u = 0; u < kRows; u++) {
        if (!live[u]) continue;
        float scale = 0.0f, offset = 0.0f;
        if constexpr (TY == TY_I8 || TY == TY_I4) {
          if constexpr (SO32) {
            scale = __uint_as_float(hdr[u][0]);
            offset = __uint_as_float(hdr[u][1]);
          } else {
            scale = half_bits_to_float(hdr[u][0]);
            offset = half_bits_to_float(hdr[u][0] >> 16);
          }
        }
        // Pairs of fp32 values go through the two-lane fp32 instructions of sm_100 (each lane
        // rounds like the scalar instruction, subnormals included) for the dequantising FMA and
        // for the sums of unweighted quantized rows.  The weight multiply and the add behind it
        // stay scalar: issued as a two-lane multiply followed by a two-lane add they did not
        // reproduce the reference's two roundings on its own unit vectors, whereas scalar
        // mul.rn / add.rn are never contracted.
        auto dequant2 = [&](uint32_t h2, float &ta, float &tb) {  // h2 = two fp16 numbers 1024 + q
          const float fa = add_f32_f16((uint16_t)(h2 & 0xFFFFu), -1024.0f), fb = add_f32_f16((uint16_t)(h2 >> 16), -1024.0f);
          if constexpr (SO32) {
            ta = __fadd_rn(__fmul_rn(fa, scale), offset);
            tb = __fadd_rn(__fmul_rn(fb, scale), offset);
          } else if constexpr (GLOWB200_TBE_X2) {
            uint64_t v2;
            asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(v2) : "l"(pack2f(fa, fb)), "l"(pack2f(scale, scale)), "l"(pack2f(offset, offset)));
            unpack2f(v2, ta, tb);
          } else {
            ta = __fmaf_rn(fa, scale, offset);
            tb = __fmaf_rn(fb, scale, offset);
          }
        };
#pragma unroll
        for (int i = 0; i < PAIRS; i++) {
          float ta, tb;  // the values of the pair's slots in this row
          if constexpr (TY == TY_F32) {
            ta = __uint_as_float(q[u][2 * i]);
            tb = __uint_as_float(q[u][2 * i + 1]);
          } else if constexpr (TY == TY_F16) {
            ta = half_bits_to_float(q[u][i]);
            tb = half_bits_to_float(q[u][i] >> 16);
          } else if constexpr (TY == TY_I8) {
            dequant2(__byte_perm(q[u][i >> 1], 0x64646464u, (i & 1) ? 0x4342u : 0x4140u), ta, tb);
          } else {  // even column = low nibble, odd column = high nibble (InterpreterNodes.cpp:104-109)
            dequant2(((q[u][i >> 2] >> (4 * (i & 3))) & 0x000F000Fu) | 0x64006400u, ta, tb);
          }
          if constexpr (WEIGHTED) {  // (an unweighted bag multiplies by 1.0)
            ta = __fmul_rn(w[u], ta);
            tb = __fmul_rn(w[u], tb);
          }
          if constexpr (OUT16) {
            // (keeping fp32 copies of the sums and converting both ways every row was tried: half the speed)
            const float lo = add_f32_f16((uint16_t)(acch[i] & 0xFFFFu), ta);
            const float hi = add_f32_f16((uint16_t)(acch[i] >> 16), tb);
            acch[i] = pack_f16x2(lo, hi);
          } else if constexpr (GLOWB200_TBE_X2 && !WEIGHTED && !SO32 && (TY == TY_I8 || TY == TY_I4)) {
            uint64_t s2;
            asm("add.rn.f32x2 %0, %1, %2;" : "=l"(s2) : "l"(pack2f(acc[slot_a(i)], acc[slot_b(i)])), "l"(pack2f(ta, tb)));
            unpack2f(s2, acc[slot_a(i)], acc[slot_b(i)]);
          } else {
            acc[slot_a(i)] = __fadd_rn(acc[slot_a(i)], ta);
            acc[slot_b(i)] = __fadd_rn(acc[slot_b(i)], tb);
          }
        }
      }
    }

    if (!has) continue;
    const bool mean = p.pooling_mode == 1 && end > begin;
    float n = 1.0f;
    if (mean) {
      n = (float)(end - begin);
      if (OUT16) n = __half2float(__float2half_rn(n));
    }
#pragma unroll
    for (int i = 0; i < PAIRS; i++) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int slot = e ? slot_b(i) : slot_a(i);
        const int32_t c = col0 + slot;
        if (c < 0 || c >= num_dims) continue;
        if constexpr (OUT16) {
          const __half h = __ushort_as_half((unsigned short)((acch[i] >> (16 * e)) & 0xFFFFu));
          reinterpret_cast<__half *>(out_row)[c] = mean ? __float2half_rn(__fdiv_rn(__half2float(h), n)) : h;
        } else {
          reinterpret_cast<float *>(out_row)[c] = mean ? __fdiv_rn(acc[slot], n) : acc[slot];
        }
      }
    }
  }
  return flags;
}

template <bool OUT16, typename IdxT>
__global__ void __launch_bounds__(kThreads, GLOWB200_TBE_MIN_BLOCKS) split_embedding_bags_kernel(const __grid_constant__ SplitLaunch p) {
  const int t = blockIdx.y;
  const int32_t dim_start = p.dim_offsets[t], num_dims = p.dim_offsets[t + 1] - dim_start;
  const int ty = p.weights_tys[t];
  const int32_t placement = p.placements[t];
  if (num_dims <= 0) return;
  if (ty > TY_I4 || placement == 0 || dim_start < 0 || (int64_t)dim_start + num_dims > p.total_dims || num_dims > (1 << 27)) {
    // int2 rows and tables placed in device-only memory are not supported by the reference
    // either (InterpreterNodes.cpp:6696, 6704): the table's columns stay 0
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, GLOWB200_STATUS_UNSUPPORTED_TABLE);
    return;
  }
  const int so = p.so_fp32 ? 4 : 2;
  const int32_t unpadded = ty == TY_F32 ? num_dims * 4 : ty == TY_F16 ? num_dims * 2
                         : ty == TY_I8 ? num_dims + 2 * so : num_dims / 2 + 2 * so;
  const int32_t row_bytes = (unpadded + p.row_alignment - 1) / p.row_alignment * p.row_alignment;
  // bytes of a row the reference touches: the last column of an int4 row with an odd column
  // count sits in the byte after the counted payload (column d reads byte d / 2)
  const int32_t touched = ty == TY_I4 ? (num_dims + 1) / 2 + 2 * so : unpadded;
  const uint8_t *base = placement == 3 ? p.dev_weights : p.uvm_weights;
  const int64_t limit = placement == 3 ? p.dev_bytes : p.uvm_bytes;
  const int64_t table_at = p.wo64 ? reinterpret_cast<const int64_t *>(p.weights_offsets)[t]
                                  : (int64_t)reinterpret_cast<const int32_t *>(p.weights_offsets)[t];
  // 16-byte chunks where the table allows them (rows at 16-byte boundaries), else 8-byte chunks.
  // A bag takes as many lanes as its rows have chunks (32 at most; wider rows take several
  // passes), not a power of two: a 132-byte int8 row is 9 lanes, three bags to a warp.
  const uint64_t addr = reinterpret_cast<uintptr_t>(base) + (uint64_t)table_at;
  const bool wide = (addr % 16) == 0 && (row_bytes % 16) == 0;
  // (int4 rows with an fp32 result keep 8-byte chunks: 32 fp32 sums per lane spill, 16.0 against 12.9 G rows/s)
  const bool wide_i4 = GLOWB200_TBE_I4_WIDE && OUT16;
  const int cb = (wide && (ty != TY_I4 || wide_i4)) ? 16 : 8;
  const bool vec = wide || ((addr % 8) == 0 && (row_bytes % 8) == 0);
  const int chunks = (touched + cb - 1) / cb;
  int lpr = chunks > 32 ? 32 : chunks;
  // Rows of a little more than half a warp (17 chunks: a 260-byte int8 row) would leave the other
  // half idle: half as many lanes then walk the bag twice, one half of the row per pass, when that
  // puts over 2.4 times as many bags into the warp.
  if (chunks <= 32 && 32 / ((chunks + 1) / 2) * 5 > 32 / lpr * 12) lpr = (chunks + 1) / 2;
  const int bags_per_warp = 32 / lpr;
  const int lane = threadIdx.x & 31;
  if (lane >= bags_per_warp * lpr) return;
  const int64_t b = ((int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * bags_per_warp + lane / lpr;
  if (b >= p.bags_per_table) return;
  const int gl = lane % lpr;

  const IdxT *offsets = reinterpret_cast<const IdxT *>(p.offsets);
  int64_t begin = (int64_t)offsets[(int64_t)t * p.bags_per_table + b];
  int64_t end = (int64_t)offsets[(int64_t)t * p.bags_per_table + b + 1];
  int32_t flags = 0;
  if (begin < 0 || end < begin || end > p.num_indices) {
    if (end >= begin) flags |= GLOWB200_STATUS_BAD_OFFSETS;  // a start above its end is an empty bag
    begin = end = 0;
  }
  void *out_row = reinterpret_cast<char *>(p.dest) + ((size_t)(b * p.total_dims + dim_start)) * (OUT16 ? 2 : 4);

#define GLOWB200_POOL3(TY, CW, WEIGHTED, SO32)                                                                     \
  flags |= pool_bag<TY, CW, OUT16, WEIGHTED, SO32, IdxT>(p, base, limit, table_at, row_bytes, touched, num_dims, vec, \
                                                         begin, end, gl, lpr, out_row)
#define GLOWB200_POOL2(TY, CW, SO32) \
  do { if (p.indice_weights != nullptr) GLOWB200_POOL3(TY, CW, true, SO32); else GLOWB200_POOL3(TY, CW, false, SO32); } while (0)
#define GLOWB200_POOLQ(TY, CW) \
  do { if (p.so_fp32) GLOWB200_POOL2(TY, CW, true); else GLOWB200_POOL2(TY, CW, false); } while (0)
  switch (ty) {
    case TY_F32: if (wide) GLOWB200_POOL2(TY_F32, 4, false); else GLOWB200_POOL2(TY_F32, 2, false); break;
    case TY_F16: if (wide) GLOWB200_POOL2(TY_F16, 4, false); else GLOWB200_POOL2(TY_F16, 2, false); break;
    case TY_I8: if (wide) GLOWB200_POOLQ(TY_I8, 4); else GLOWB200_POOLQ(TY_I8, 2); break;
    default: if (wide && wide_i4) GLOWB200_POOLQ(TY_I4, 4); else GLOWB200_POOLQ(TY_I4, 2); break;
  }
#undef GLOWB200_POOLQ
#undef GLOWB200_POOL2
#undef GLOWB200_POOL3
  if (p.status != nullptr && flags != 0) atomicOr(p.status, flags);
}

}  // namespace
}  // namespace glowb200

using namespace glowb200;

extern "C" int glowb200_int_nbit_split_embedding_bags(
    void *dest, const void *dev_weights, int64_t dev_weights_bytes, const void *uvm_weights,
    int64_t uvm_weights_bytes, const int32_t *weights_placements, const void *weights_offsets,
    int weights_offsets_are_int64, const uint8_t *weights_tys, const int32_t *dim_offsets, int64_t num_tables,
    int64_t total_dims, const void *indices, const void *offsets, int indices_are_int64, int64_t num_indices,
    int64_t bags_per_table, int pooling_mode, const void *indice_weights, int indice_weights_are_fp16,
    int out_is_fp16, int scale_offset_is_fp32, int row_alignment, int32_t *status, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(num_tables >= 0 && num_tables <= 65535, "num_tables must be in [0, 65535]");
  GLOWB200_REQUIRE(bags_per_table >= 0 && bags_per_table < (1ll << 31), "bags_per_table out of range");
  GLOWB200_REQUIRE(total_dims >= 0 && total_dims < (1ll << 31) && num_indices >= 0, "total_dims / num_indices out of range");
  GLOWB200_REQUIRE(pooling_mode >= 0 && pooling_mode <= 2, "pooling_mode must be 0 (sum), 1 (mean) or 2 (none)");
  GLOWB200_REQUIRE(row_alignment > 0 && row_alignment <= 4096, "row_alignment must be in [1, 4096]");
  GLOWB200_REQUIRE(dev_weights_bytes >= 0 && uvm_weights_bytes >= 0, "negative weights size");
  if (bags_per_table == 0 || total_dims == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(dest != nullptr, "dest is NULL");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the reference clears the result first (InterpreterNodes.cpp:6672); columns no table covers stay 0
  GLOWB200_CUDA_OK(cudaMemsetAsync(dest, 0, (size_t)(bags_per_table * total_dims) * (out_is_fp16 ? 2 : 4), s));
  if (num_tables == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(weights_placements != nullptr && weights_offsets != nullptr && weights_tys != nullptr &&
                       dim_offsets != nullptr && offsets != nullptr,
                   "NULL table description or offsets");
  GLOWB200_REQUIRE(num_indices == 0 || indices != nullptr, "indices is NULL");
  SplitLaunch L{};
  L.dest = dest;
  L.dev_weights = reinterpret_cast<const uint8_t *>(dev_weights);
  L.uvm_weights = reinterpret_cast<const uint8_t *>(uvm_weights);
  L.dev_bytes = dev_weights != nullptr ? dev_weights_bytes : 0;
  L.uvm_bytes = uvm_weights != nullptr ? uvm_weights_bytes : 0;
  L.placements = weights_placements;
  L.weights_offsets = weights_offsets;
  L.weights_tys = weights_tys;
  L.dim_offsets = dim_offsets;
  L.indices = indices;
  L.offsets = offsets;
  L.indice_weights = indice_weights;
  L.status = status;
  L.num_indices = num_indices;
  L.bags_per_table = bags_per_table;
  L.total_dims = total_dims;
  L.wo64 = weights_offsets_are_int64 ? 1 : 0;
  L.iw16 = indice_weights_are_fp16 ? 1 : 0;
  L.so_fp32 = scale_offset_is_fp32 ? 1 : 0;
  L.row_alignment = row_alignment;
  L.pooling_mode = pooling_mode;
  // a block holds 8 bags of the widest kind of table (32 lanes a bag); tables with narrower
  // rows put more bags into a block and their surplus blocks leave at once
  dim3 grid((unsigned)((bags_per_table + 7) / 8), (unsigned)num_tables);
  if (out_is_fp16) {
    if (indices_are_int64) split_embedding_bags_kernel<true, int64_t><<<grid, kThreads, 0, s>>>(L);
    else split_embedding_bags_kernel<true, int32_t><<<grid, kThreads, 0, s>>>(L);
  } else {
    if (indices_are_int64) split_embedding_bags_kernel<false, int64_t><<<grid, kThreads, 0, s>>>(L);
    else split_embedding_bags_kernel<false, int32_t><<<grid, kThreads, 0, s>>>(L);
  }
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}
