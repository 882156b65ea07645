// Embedding gather-pool kernels for fused-rowwise quantized tables on sm_100a:
// FusedRowwiseQuantizedSparseLengthsWeightedSum (uint8 and 4-bit rows, fp32 or fp16
// scale/offset, fp32 or fp16 result) and EmbeddingBagByteRowwiseOffsets.
//
// The work is a random gather of short rows out of HBM, so the design goal is bytes in
// flight, not arithmetic:
//   * a "segments" kernel turns lengths (or offsets) into validated bag boundaries in the
//     caller's workspace, one int64 array per table;
//   * the gather kernel gives each bag to a group of `lpr` lanes (a power of two, 1..32).
//     A lane owns P chunks of 8 columns; chunk c of a row is one 8-byte (uint8 rows) or
//     4-byte (4-bit rows) read-only load, and the lanes of a group read consecutive chunks,
//     so one load instruction covers a contiguous piece of the row.  Indices and weights
//     are read coalesced, `lpr` at a time, and handed round inside the group by shuffles;
//     kUnroll rows are requested before the first is consumed.
//
// Arithmetic.  The reference computes dest[k] += w * (scale * q[k] + offset) row by row
// (lib/LLVMIRCodeGen/libjit/libjit.cpp:1253-1276; InterpreterNodes.cpp:5797-5836).  With
// fp32 accumulation this kernel evaluates the same sum as
//     sum_j (w_j*scale_j) * q_jk  +  sum_j (w_j*offset_j)
// with one FMA per element: the reference's CPU backend is itself compiled with fast-math,
// so its float result is defined only up to reassociation (tolerance 1e-5 relative).
// With fp16 accumulation the reference rounds at every step, and the kernel does exactly
// that, step by step.
#include "common.cuh"

#include <climits>
#include <mutex>

namespace glowb200 {
namespace {

// Threads of a gather block.  A block's SM slots stay taken until its slowest warp is done, and
// bags differ a lot in length (power-law pooling factors), so blocks are kept small: against
// 256 threads, 64 pool the 256-table launch 4.7 % faster (329 us), the recommendation model's
// 64 skewed tables 9.5 % and one rank's eight of them 11 %.  (A persistent form -- warps taking
// pieces of work from a counter -- was tried first: the loop round both mappings cost 250 bytes
// of spills a thread and the launch 60 %.)
#ifndef GLOWB200_SLWS_THREADS
#define GLOWB200_SLWS_THREADS 64
#endif
constexpr int kGatherThreads = GLOWB200_SLWS_THREADS;
constexpr int kGatherBlockScale = 256 / kGatherThreads;  // blocks per SM scale with it
constexpr int kSegThreads = 1024;

struct SlwsLaunch {
  const glowb200_slws_job *jobs;  // device array, or nullptr when `single` is the only job
  glowb200_slws_job single;
  int64_t *seg_begin;  // workspace: per job an int64 [segments + 1] array
  int64_t seg_stride;  // int64 elements between the arrays of consecutive jobs
  int64_t max_segments;  // bags a table's array has room for (a descriptor naming more is cut short)
  int32_t *status;
  int32_t in_line, out_line;
  int32_t lpr_log2;
  // 1: the gather kernel picks, per table, the thread-to-bag mapping its bag-length profile
  // favours (a word the segments kernel leaves behind the table's boundaries);
  // 0: the group-per-bag mapping for every table.
  int32_t select;
  // 1: the tables are row-range shards (row_begin / global_rows of the descriptors are honoured)
  int32_t sharded;
  int32_t warp_per_bag;  // every table of the launch takes the warp-per-run mapping
  int32_t inline_lengths;  // single table, few bags: no boundary array, see slws_gather_small_kernel
};

// Bags of a table as the kernels walk them: never more than its boundary array has room for.
__device__ __forceinline__ int64_t bags_of(const SlwsLaunch &p, const glowb200_slws_job *jp) {
  return jp->segments < p.max_segments ? jp->segments : p.max_segments;
}

__device__ __forceinline__ void raise(int32_t *status, int32_t bits) {
  if (status != nullptr && bits != 0) atomicOr(status, bits);
}

// Tuning knobs, with the values measured best on B200 for 72-byte rows (256 tables x 1M rows):
// 3 resident blocks per SM (<= 85 registers) pooled 2278 GB/s, 2 blocks 2096, 4 blocks (64
// registers, spills) 1486; letting the row loads allocate in L1 or not, and prefetching the
// next index chunk or not, changed nothing measurable.
// Two other structures were built and measured on the same 256-table launch (346 us as it is):
//  * one 16-byte load per lane over the aligned window of a row (a single request per row, the
//    scale/offset pair handed round by shuffle): 8 lanes a row instead of 4 halves the rows a
//    warp has in flight -- 522 us;
//  * rows copied by cp.async.bulk into a per-warp shared-memory ring two blocks of 32 indices
//    ahead, pooled out of shared memory in index order: the copies alone (no pooling) take
//    344 us, the pooling alone 288 us, both in one warp 420 us.  The fetch side of that kernel
//    runs at the rate this one reaches with everything included, which is the evidence that
//    24 G rows/s is what the memory system gives 72-byte rows at 8-byte boundaries.
#ifndef GLOWB200_SLWS_L1_NOALLOC
#define GLOWB200_SLWS_L1_NOALLOC 0
#endif
#ifndef GLOWB200_SLWS_MIN_BLOCKS
#define GLOWB200_SLWS_MIN_BLOCKS 3
#endif
#ifndef GLOWB200_SLWS_MIN_BLOCKS_P4
#define GLOWB200_SLWS_MIN_BLOCKS_P4 2
#endif
#ifndef GLOWB200_SLWS_P4_FROM
#define GLOWB200_SLWS_P4_FROM 16
#endif
#ifndef GLOWB200_SLWS_FORCE_WARP
#define GLOWB200_SLWS_FORCE_WARP 0
#endif
#ifndef GLOWB200_SLWS_MAX_BPW
#define GLOWB200_SLWS_MAX_BPW 8
#endif
#ifndef GLOWB200_SLWS_UNROLL_P2
#define GLOWB200_SLWS_UNROLL_P2 4
#endif
__device__ __forceinline__ uint32_t ldg_stream_u32(const void *p) {
  uint32_t v;
#if GLOWB200_SLWS_L1_NOALLOC
  asm("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
#else
  asm("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
#endif
  return v;
}
__device__ __forceinline__ uint2 ldg_stream_u64(const void *p) {
  uint2 v;
#if GLOWB200_SLWS_L1_NOALLOC
  asm("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
#else
  asm("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
#endif
  return v;
}

// ------------------------------------------------------------------------------------------
// Bag boundaries.  One block per table.
//   lengths form : seg_begin[i] = min(sum(max(lengths[0..i), 0)), num_indices)
//   offsets form : seg_begin[i] = clamp(offsets[i], 0, num_indices); the closing entry is
//                  offsets[segments] when an end offset is present, else num_indices
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t *warp_tot, int64_t &block_total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int64_t t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int64_t w = (lane < (int)(blockDim.x >> 5)) ? warp_tot[lane] : 0;
    int64_t winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int64_t t = __shfl_up_sync(0xffffffffu, winc, d);
      if (lane >= d) winc += t;
    }
    warp_tot[lane] = winc - w;  // exclusive prefix of warp totals
    if (lane == 31) warp_tot[32] = winc;
  }
  __syncthreads();
  const int64_t res = warp_tot[warp] + inc - v;
  block_total = warp_tot[32];
  __syncthreads();
  return res;
}

__global__ void __launch_bounds__(kSegThreads) slws_segments_from_lengths_kernel(const __grid_constant__ SlwsLaunch p) {
  pdl_wait();               // the gather before this one may still read the boundaries this kernel rewrites
  pdl_launch_dependents();  // this launch's gather may take its place on the SMs (it waits before reading them)
  __shared__ int64_t warp_tot[33];
  const glowb200_slws_job job = p.jobs ? p.jobs[blockIdx.x] : p.single;
  int64_t *out = p.seg_begin + (int64_t)blockIdx.x * p.seg_stride;
  int32_t flags = 0;
  int64_t S = job.segments;
  if (S > p.max_segments) { S = p.max_segments; flags |= GLOWB200_STATUS_BAD_OFFSETS; }
  const int64_t N = job.num_indices;
  constexpr int kItems = 4;
  int64_t carry = 0;
  int64_t longest = 0;
  for (int64_t tile = 0; tile < S; tile += (int64_t)kSegThreads * kItems) {
    const int64_t first = tile + (int64_t)threadIdx.x * kItems;
    int64_t v[kItems], sum = 0;
#pragma unroll
    for (int i = 0; i < kItems; i++) {
      int64_t l = (first + i < S) ? (int64_t)job.lengths[first + i] : 0;
      if (l < 0) { l = 0; flags |= GLOWB200_STATUS_NEGATIVE_LENGTH; }
      v[i] = l;
      sum += l;
      longest = l > longest ? l : longest;
    }
    int64_t tile_total;
    int64_t run = carry + block_exclusive_scan(sum, warp_tot, tile_total);
#pragma unroll
    for (int i = 0; i < kItems; i++) {
      if (first + i < S) out[first + i] = run < N ? run : N;
      run += v[i];
    }
    carry += tile_total;
  }
  // longest bag of the table (block-wide maximum through the scan's scratch)
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const int64_t o = __shfl_xor_sync(0xffffffffu, longest, d);
    longest = o > longest ? o : longest;
  }
  if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = longest;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) longest = warp_tot[w] > longest ? warp_tot[w] : longest;
    if (carry > N) flags |= GLOWB200_STATUS_LENGTHS_OVERRUN;
    out[S] = carry < N ? carry : N;
    // Bag-length profile: when the longest bag is more than 2.5 times the mean, bags that
    // share a warp in lock step would wait for each other -- such a table goes to the kernel
    // that gives every bag a whole warp.
    out[S + 1] = (S > 0 && 2 * longest * S > 5 * carry) ? 1 : 0;
  }
  raise(p.status, flags);
}

template <typename IdxT>
__global__ void __launch_bounds__(256) slws_segments_from_offsets_kernel(const __grid_constant__ SlwsLaunch p,
                                                                           const IdxT *offsets, int has_end) {
  const int64_t S = p.single.segments, N = p.single.num_indices;
  int32_t flags = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i <= S; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t v = (i < S || has_end) ? (int64_t)offsets[i] : N;
    if (v < 0) { v = 0; flags |= GLOWB200_STATUS_BAD_OFFSETS; }
    if (v > N) { v = N; flags |= GLOWB200_STATUS_BAD_OFFSETS; }
    p.seg_begin[i] = v;
  }
  raise(p.status, flags);
}

// 1: pool uint8 rows with the packed two-lane fp32 instructions of sm_100
#ifndef GLOWB200_SLWS_F32X2
#define GLOWB200_SLWS_F32X2 1
#endif
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// ------------------------------------------------------------------------------------------
// Row decoding
// ------------------------------------------------------------------------------------------
template <int BITS, bool SO16>
struct RowLoad {
  // 8-byte loads need 8-byte aligned rows: only the uint8 / fp32-scale layout (D + 8 bytes,
  // D a multiple of 8) guarantees that.
  static constexpr bool kWide = (BITS == 8) && !SO16;

  struct Chunk { uint32_t lo, hi; };

  __device__ static __forceinline__ Chunk payload(const uint8_t *row, int chunk) {
    Chunk c;
    if constexpr (BITS == 4) {
      c.lo = ldg_stream_u32(row + chunk * 4);
      c.hi = 0;
    } else if constexpr (kWide) {
      uint2 v = ldg_stream_u64(row + chunk * 8);
      c.lo = v.x; c.hi = v.y;
    } else {
      c.lo = ldg_stream_u32(row + chunk * 8);
      c.hi = ldg_stream_u32(row + chunk * 8 + 4);
    }
    return c;
  }

  // raw scale/offset words from the end of the row
  __device__ static __forceinline__ uint2 tail(const uint8_t *row_end) {
    if constexpr (SO16) {
      return make_uint2(ldg_stream_u32(row_end - 4), 0u);
    } else if constexpr (kWide) {
      return ldg_stream_u64(row_end - 8);
    } else {
      return make_uint2(ldg_stream_u32(row_end - 8), ldg_stream_u32(row_end - 4));
    }
  }

  __device__ static __forceinline__ void scale_offset(uint2 t, float &scale, float &offset) {
    if constexpr (SO16) {
      const __half2 h = *reinterpret_cast<const __half2 *>(&t.x);
      scale = __low2float(h);
      offset = __high2float(h);
    } else {
      scale = __uint_as_float(t.x);
      offset = __uint_as_float(t.y);
    }
  }

  // Column i (0..7) of a chunk as an exact float: the byte / nibble is dropped into the
  // mantissa of 2^23 and 2^23 is subtracted.  4-bit rows keep column 2m in the low nibble of
  // byte m and column 2m+1 in the high nibble (include/glow/Quantization/Base/Base.h:399-406).
  __device__ static __forceinline__ float column(const Chunk &c, int i) {
    uint32_t m;
    if constexpr (BITS == 8) {
      const uint32_t w = i < 4 ? c.lo : c.hi;
      m = __byte_perm(w, 0x4B000000u, 0x7440 + (i & 3));  // {byte i, 0, 0, 0x4B}
    } else {
      m = ((c.lo >> (4 * i)) & 0xFu) | 0x4B000000u;
    }
    return __uint_as_float(m) - 8388608.0f;
  }

  // fp32 pooling of one chunk: acc[i] += (w*scale) * q_i.
  //  * uint8 rows: q_i as above (byte into the mantissa of 2^23, minus 2^23), one FMA each.
  //  * 4-bit rows are bound by instruction issue, not by memory, so the conversion is made
  //    cheaper: the nibbles are spread into bytes 0x8q (three logic ops per 8 columns), a byte
  //    permute drops each into bits 16..23 of 0x3F80'0000, which reads as m = 1 + q/128, and
  //    acc[i] += (128*w*scale) * m.  The surplus sum_j 128*w_j*scale_j is the same for every
  //    column and is taken out once per row through the shared offset sum (row_term).
  //    m is exact; the products are about 8-128 times larger than the wanted a*q, which costs
  //    at most 7 of the 24 mantissa bits -- inside the fp32 tolerance.
  __device__ static __forceinline__ float scale_for_pooling(float a) { return BITS == 4 ? a * 128.0f : a; }
  __device__ static __forceinline__ float row_term(float w, float offset, float a_eff, float sum) {
    // sum += w*offset (and, 4-bit, minus the surplus a_eff)
    sum = fmaf(w, offset, sum);
    return BITS == 4 ? sum - a_eff : sum;
  }
  __device__ static __forceinline__ void pool(const Chunk &c, float a_eff, float *acc) {
    if constexpr (BITS == 8) {
#if GLOWB200_SLWS_F32X2
      // two columns per instruction: sm_100's packed fp32 add and fma (the same roundings as
      // the scalar forms, element by element)
      const uint64_t a2 = pack2(a_eff, a_eff), magic2 = pack2(-8388608.0f, -8388608.0f);
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        const uint32_t w = i < 4 ? c.lo : c.hi;
        const uint32_t m0 = __byte_perm(w, 0x4B000000u, 0x7440 + (i & 3));  // {byte i, 0, 0, 0x4B} = 2^23 + q
        const uint32_t m1 = __byte_perm(w, 0x4B000000u, 0x7440 + ((i + 1) & 3));
        uint64_t q2, s2;
        asm("mov.b64 %0, {%1, %2};" : "=l"(q2) : "r"(m0), "r"(m1));
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(q2) : "l"(q2), "l"(magic2));
        s2 = pack2(acc[i], acc[i + 1]);
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(s2) : "l"(a2), "l"(q2), "l"(s2));
        unpack2(s2, acc[i], acc[i + 1]);
      }
#else
#pragma unroll
      for (int i = 0; i < 8; i++) acc[i] = fmaf(a_eff, column(c, i), acc[i]);
#endif
    } else {
      const uint32_t lo = (c.lo & 0x0F0F0F0Fu) | 0x80808080u;         // columns 0,2,4,6 as bytes 0x8q
      const uint32_t hi = ((c.lo >> 4) & 0x0F0F0F0Fu) | 0x80808080u;  // columns 1,3,5,7
#pragma unroll
      for (int b = 0; b < 4; b++) {
        const float m0 = __uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7044 + (b << 8)));  // {0, 0, byte b, 0x3F}
        const float m1 = __uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7044 + (b << 8)));
        acc[2 * b] = fmaf(a_eff, m0, acc[2 * b]);
        acc[2 * b + 1] = fmaf(a_eff, m1, acc[2 * b + 1]);
      }
    }
  }
};

template <bool OUT16>
__device__ __forceinline__ float load_weight(const void *weights, int64_t i) {
  if constexpr (OUT16) return __half2float(reinterpret_cast<const __half *>(weights)[i]);
  else return reinterpret_cast<const float *>(weights)[i];
}

// ------------------------------------------------------------------------------------------
// Gather-pool.  grid = (ceil(max_segments / bags_per_block), num_jobs).
// ------------------------------------------------------------------------------------------
template <int BITS, bool SO16, bool OUT16, bool ACC16, typename IdxT, int P, int kUnroll, bool SHARD = false>
__device__ __forceinline__ void gather_group_body(const SlwsLaunch &p) {
  using RL = RowLoad<BITS, SO16>;
  const int job_id = blockIdx.y;
  const glowb200_slws_job *jp = p.jobs ? (p.jobs + job_id) : &p.single;
  const int64_t segments = bags_of(p, jp);
  const int lpr = 1 << p.lpr_log2;
  const int gl = threadIdx.x & (lpr - 1);
  const int64_t bag = (int64_t)blockIdx.x * (kGatherThreads >> p.lpr_log2) + (threadIdx.x >> p.lpr_log2);
  if (bag >= segments) return;  // whole groups leave together

  const uint8_t *data = reinterpret_cast<const uint8_t *>(jp->data);
  const IdxT *indices = reinterpret_cast<const IdxT *>(jp->indices);
  const void *weights = jp->weights;
  const int64_t rows = jp->rows;
  const int64_t *sb = p.seg_begin + (int64_t)job_id * p.seg_stride;
  const int64_t in_line = p.in_line;
  const int chunks = p.out_line >> 3;

  const unsigned lane = threadIdx.x & 31u;
  const unsigned gmask = (lpr == 32) ? 0xffffffffu : (((1u << lpr) - 1u) << (lane & ~(unsigned)(lpr - 1)));

  int64_t begin = sb[bag], end = sb[bag + 1];
  int32_t flags = 0;
  if (end < begin) { end = begin; flags |= GLOWB200_STATUS_BAD_OFFSETS; }

  bool has[P];
#pragma unroll
  for (int c = 0; c < P; c++) has[c] = (c * lpr + gl) < chunks;

  float acc[P][8];
#pragma unroll
  for (int c = 0; c < P; c++)
#pragma unroll
    for (int i = 0; i < 8; i++) acc[c][i] = 0.0f;
  float bias_sum = 0.0f;  // sum_j w_j * offset_j (fp32 accumulation only)

  // Row numbers travel as int32 inside the group (-1 = skip): tables have fewer than 2^31 rows
  // (checked on the host).  The next `lpr` indices are requested before the current ones are
  // consumed, so the index fetch overlaps the row fetches.  Asking for an index (`request`) and
  // looking at it (`resolve`: range check, narrowing) are kept apart: nothing may depend on the
  // loaded value -- not even a branch -- until the rows of the chunk before it are on their
  // way, or the warp would sit out the index latency first and the row latency after it.
  auto request = [&](int64_t pos, IdxT &v, float &w) {
    v = 0;
    w = 0.0f;
    if (pos < end) {
      v = indices[pos];
      w = load_weight<OUT16>(weights, pos);
    }
  };
  auto resolve = [&](int64_t pos, IdxT raw) -> int32_t {
    if (pos >= end) return -1;
    const int64_t g = (int64_t)raw;
    int64_t v = g;
    if constexpr (SHARD) v -= jp->row_begin;
    if (v >= 0 && v < rows) return (int32_t)v;
    if (!SHARD || g < 0 || g >= jp->global_rows) flags |= GLOWB200_STATUS_INDEX_OUT_OF_RANGE;  // else: another shard's row
    return -1;
  };
  int32_t r_mine;
  IdxT v_next;
  float w_mine, w_next;
  request(begin + gl, v_next, w_mine);
  r_mine = resolve(begin + gl, v_next);
  for (int64_t base = begin; base < end; base += lpr) {
    request(base + lpr + gl, v_next, w_next);
    const int n = (int)((end - base) < (int64_t)lpr ? (end - base) : (int64_t)lpr);
    for (int t = 0; t < n; t += kUnroll) {
      int32_t r[kUnroll];
      float w[kUnroll];
      typename RL::Chunk pay[kUnroll][P];
      uint2 tl[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        r[u] = __shfl_sync(gmask, r_mine, t + u, lpr);
        w[u] = __shfl_sync(gmask, w_mine, t + u, lpr);
        if (t + u >= n) r[u] = -1;
      }
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        if (r[u] >= 0) {
          const uint8_t *row = data + (int64_t)r[u] * in_line;
#pragma unroll
          for (int c = 0; c < P; c++)
            if (has[c]) pay[u][c] = RL::payload(row, c * lpr + gl);
          tl[u] = RL::tail(row + in_line);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        if (r[u] >= 0) {
          float scale, offset;
          RL::scale_offset(tl[u], scale, offset);
          if constexpr (ACC16) {
            // AccumT = float16 (InterpreterNodes.cpp:5799,5832; Float16.h:38-56): the addend
            // d*w is rounded to fp32 then to fp16, the fp16 sum is widened, added and rounded.
            // q*scale is exact in fp32 for an fp16 scale, so the FMA equals multiply-then-add.
#pragma unroll
            for (int c = 0; c < P; c++)
              if (has[c]) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                  const float d = __fmaf_rn(RL::column(pay[u][c], i), scale, offset);
                  const float addend = __half2float(__float2half_rn(__fmul_rn(d, w[u])));
                  acc[c][i] = __half2float(__float2half_rn(__fadd_rn(acc[c][i], addend)));
                }
              }
          } else {
            const float a = RL::scale_for_pooling(w[u] * scale);
            bias_sum = RL::row_term(w[u], offset, a, bias_sum);
#pragma unroll
            for (int c = 0; c < P; c++)
              if (has[c]) RL::pool(pay[u][c], a, acc[c]);
          }
        }
      }
    }
    r_mine = resolve(base + lpr + gl, v_next);
    w_mine = w_next;
  }

  // Every bag writes its row, empty bags write zeros (the reference zero-fills dest first).
  const int64_t dest_stride = jp->dest_stride;
  void *dest_base = jp->dest;
  int64_t dest_row = bag;
  if (jp->bags_per_dest > 0) {  // scatter over several (possibly remote) destination buffers
    const int64_t which = bag / jp->bags_per_dest;
    dest_base = jp->dests[which];
    dest_row = bag - which * jp->bags_per_dest;
  }
#pragma unroll
  for (int c = 0; c < P; c++) {
    if (!has[c]) continue;
    const int64_t col = (int64_t)(c * lpr + gl) * 8;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = ACC16 ? acc[c][i] : (acc[c][i] + bias_sum);
    if constexpr (OUT16) {
      __half *d = reinterpret_cast<__half *>(dest_base) + dest_row * dest_stride + col;
      __half2 h[4];
#pragma unroll
      for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(o[2 * i], o[2 * i + 1]);
      if ((reinterpret_cast<uintptr_t>(d) & 15u) == 0) {
        *reinterpret_cast<uint4 *>(d) = *reinterpret_cast<const uint4 *>(h);
      } else {
#pragma unroll
        for (int i = 0; i < 4; i++) *reinterpret_cast<__half2 *>(d + 2 * i) = h[i];
      }
    } else {
      float *d = reinterpret_cast<float *>(dest_base) + dest_row * dest_stride + col;
      if ((reinterpret_cast<uintptr_t>(d) & 15u) == 0) {
        *reinterpret_cast<float4 *>(d) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4 *>(d + 4) = make_float4(o[4], o[5], o[6], o[7]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) d[i] = o[i];
      }
    }
  }
  raise(p.status, flags);
}

template <int BITS, bool SO16, bool OUT16, bool ACC16, typename IdxT, int P, int U>
__global__ void __launch_bounds__(kGatherThreads, kGatherBlockScale * (P == 4 ? GLOWB200_SLWS_MIN_BLOCKS_P4 : GLOWB200_SLWS_MIN_BLOCKS)) slws_gather_kernel(const __grid_constant__ SlwsLaunch p) {
  gather_group_body<BITS, SO16, OUT16, ACC16, IdxT, P, U>(p);
}

// ------------------------------------------------------------------------------------------
// Gather-pool, a WARP per run of consecutive bags (fp32 accumulation).
//
// The bags of a table are consecutive in its index array, so a warp that owns `bags_per_warp`
// consecutive bags simply streams one contiguous piece of that array: 32 indices (one per
// lane) are in hand, the next 32 are already requested, and bag boundaries only decide where
// the running sums are reduced and stored.  The 32 lanes form 32/lpr row slots of lpr lanes;
// the rows of a bag are dealt round-robin to the slots and the slots are summed with shuffles
// when the bag ends.  Every lane of the warp works on the same bag, so bags of very different
// lengths (power-law pooling factors) do not hold each other up the way they do when several
// bags share a warp in lock step.  The summation order differs from the sequential one (inside
// the fp32 tolerance); fp16 accumulation, whose rounding is defined step by step, stays on the
// group-per-bag kernel above.
// grid = (ceil(ceil(max_segments / bags_per_warp) / 8), num_jobs), 8 warps per block.
// ------------------------------------------------------------------------------------------
// INLINE_LEN: no bag-boundary array exists; the warp adds up the lengths before its run itself
// (for requests of a few thousand bags, where that costs less than a launch of its own).
template <int BITS, bool SO16, bool OUT16, typename IdxT, int P, int kUnroll, bool SHARD = false, bool INLINE_LEN = false>
__device__ __forceinline__ void gather_warp_body(const SlwsLaunch &p, int bags_per_warp) {
  using RL = RowLoad<BITS, SO16>;
  constexpr int V = 8 * P;  // sums a lane carries
  const int job_id = blockIdx.y;
  const glowb200_slws_job *jp = p.jobs ? (p.jobs + job_id) : &p.single;
  const int64_t segments = bags_of(p, jp);
  const int64_t first_bag = ((int64_t)blockIdx.x * (kGatherThreads >> 5) + (threadIdx.x >> 5)) * bags_per_warp;
  if (first_bag >= segments) return;  // whole warps leave together
  const int n_bags = (int)((first_bag + bags_per_warp < segments ? first_bag + bags_per_warp : segments) - first_bag);
  const int lane = threadIdx.x & 31;
  const int lpr = 1 << p.lpr_log2, slots = 32 >> p.lpr_log2;
  const int gl = lane & (lpr - 1), slot = lane >> p.lpr_log2;

  const uint8_t *data = reinterpret_cast<const uint8_t *>(jp->data);
  const int64_t rows = jp->rows;
  const int64_t *sb = INLINE_LEN ? nullptr : p.seg_begin + (int64_t)job_id * p.seg_stride + first_bag;
  int32_t flags = 0;
  int64_t prefix = 0;  // INLINE_LEN: sum of the (non-negative) lengths before the bag in hand, not clamped
  if constexpr (INLINE_LEN) {
    for (int64_t i = threadIdx.x & 31; i < first_bag; i += 32) {
      const int32_t l = jp->lengths[i];
      prefix += l > 0 ? l : 0;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) prefix += __shfl_xor_sync(0xffffffffu, prefix, d);
  }
  // end of bag `b` of the run, as seg_begin would hold it: min(sum of lengths, num_indices)
  auto end_of_bag = [&](int b) -> int64_t {
    if constexpr (INLINE_LEN) {
      int32_t l = jp->lengths[first_bag + b];
      if (l < 0) { l = 0; flags |= GLOWB200_STATUS_NEGATIVE_LENGTH; }
      prefix += l;
      if (prefix > jp->num_indices) flags |= GLOWB200_STATUS_LENGTHS_OVERRUN;
      return prefix < jp->num_indices ? prefix : jp->num_indices;
    } else {
      return sb[b + 1];
    }
  };
  const int64_t run0 = INLINE_LEN ? (prefix < jp->num_indices ? prefix : jp->num_indices) : sb[0];
  // positions below are relative to run0 (a warp's run is far shorter than 2^31 indices)
  const IdxT *indices = reinterpret_cast<const IdxT *>(jp->indices) + run0;
  const void *weights = OUT16 ? (const void *)(reinterpret_cast<const __half *>(jp->weights) + run0)
                              : (const void *)(reinterpret_cast<const float *>(jp->weights) + run0);
  const int avail = (int)((jp->num_indices - run0) < (int64_t)INT32_MAX ? (jp->num_indices - run0) : (int64_t)INT32_MAX);
  const int in_line = p.in_line;
  const int chunks = p.out_line >> 3;

  bool has[P];
#pragma unroll
  for (int c = 0; c < P; c++) has[c] = (c * lpr + gl) < chunks;
  float acc[V];
  float bias_sum;
  auto reset = [&]() {
    bias_sum = 0.0f;
#pragma unroll
    for (int i = 0; i < V; i++) acc[i] = 0.0f;
  };
  reset();

  // Row numbers travel as int32 (tables have fewer than 2^31 rows); -1 marks an index outside
  // the table, which is reported only if a bag really uses it (indices past the last bag are
  // never looked at); -3 marks a row of another shard of a row-range sharded table.
  auto fetch = [&](int at, int32_t &r, float &w) {
    r = -1;
    w = 0.0f;
    if (at < avail) {
      const int64_t g = (int64_t)indices[at];
      int64_t v = g;
      if constexpr (SHARD) v -= jp->row_begin;
      w = load_weight<OUT16>(weights, at);
      if (v >= 0 && v < rows) r = (int32_t)v;
      else if (SHARD && g >= 0 && g < jp->global_rows) r = -3;
    }
  };

  // Reduce the row slots and store the bag's row (the sums are consumed: reset() follows).
  // Recursive halving: in every round a lane hands half of its values to its partner and keeps
  // the other half, so after log2(slots) rounds the 8*P sums of a column group are spread over
  // the slots (rounds that would go below one value per lane fall back to exchange-and-add).
  auto flush = [&](int64_t bag) {
    float bsum = bias_sum;
    int first = 0, owned = V;
#pragma unroll
    for (int round = 0; round < 5; round++) {
      const int off = 16 >> round;
      if (off >= lpr) {
        bsum += __shfl_xor_sync(0xffffffffu, bsum, off);
        constexpr int kV = V;
        const int nv = kV >> (round + 1);  // compile-time per round
        const bool upper = (lane & off) != 0;
        if (nv >= 1) {
#pragma unroll
          for (int i = 0; i < (nv > 0 ? nv : 1); i++) {
            const float keep = upper ? acc[i + nv] : acc[i];
            const float send = upper ? acc[i] : acc[i + nv];
            acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
          }
          first += upper ? nv : 0;
          owned = nv;
        } else {
          acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], off);
          if (upper) owned = 0;
        }
      }
    }
    if (owned > 0) {
      const int64_t dest_stride = jp->dest_stride;
      void *dest_base = jp->dest;
      int64_t dest_row = bag;
      if (jp->bags_per_dest > 0) {  // scatter over several (possibly remote) destination buffers
        const int64_t which = bag / jp->bags_per_dest;
        dest_base = jp->dests[which];
        dest_row = bag - which * jp->bags_per_dest;
      }
      const int c_first = first >> 3, i_first = first & 7;
      if (owned >= 8) {  // whole chunks
#pragma unroll
        for (int c = 0; c < P; c++) {
          if (c * 8 >= owned) break;
          const int chunk = (c_first + c) * lpr + gl;
          if (chunk >= chunks) continue;
          const int64_t col = (int64_t)chunk * 8;
          if constexpr (OUT16) {
            __half *d = reinterpret_cast<__half *>(dest_base) + dest_row * dest_stride + col;
            __half2 h[4];
#pragma unroll
            for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(acc[c * 8 + 2 * i] + bsum, acc[c * 8 + 2 * i + 1] + bsum);
            if ((reinterpret_cast<uintptr_t>(d) & 15u) == 0) {
              *reinterpret_cast<uint4 *>(d) = *reinterpret_cast<const uint4 *>(h);
            } else {
#pragma unroll
              for (int i = 0; i < 4; i++) *reinterpret_cast<__half2 *>(d + 2 * i) = h[i];
            }
          } else {
            float *d = reinterpret_cast<float *>(dest_base) + dest_row * dest_stride + col;
            if ((reinterpret_cast<uintptr_t>(d) & 15u) == 0) {
              *reinterpret_cast<float4 *>(d) = make_float4(acc[c * 8] + bsum, acc[c * 8 + 1] + bsum, acc[c * 8 + 2] + bsum, acc[c * 8 + 3] + bsum);
              *reinterpret_cast<float4 *>(d + 4) = make_float4(acc[c * 8 + 4] + bsum, acc[c * 8 + 5] + bsum, acc[c * 8 + 6] + bsum, acc[c * 8 + 7] + bsum);
            } else {
#pragma unroll
              for (int i = 0; i < 8; i++) d[i] = acc[c * 8 + i] + bsum;
            }
          }
        }
      } else {  // a piece of one chunk: 4, 2 or 1 consecutive columns
        const int chunk = c_first * lpr + gl;
        if (chunk < chunks) {
          const int64_t col = (int64_t)chunk * 8 + i_first;
#pragma unroll
          for (int i = 0; i < 4; i++) {
            if (i >= owned) break;
            if constexpr (OUT16) reinterpret_cast<__half *>(dest_base)[dest_row * dest_stride + col + i] = __float2half_rn(acc[i] + bsum);
            else reinterpret_cast<float *>(dest_base)[dest_row * dest_stride + col + i] = acc[i] + bsum;
          }
        }
      }
    }
  };

  // The run is walked in blocks of 32 positions (the indices in hand).  Within a block the rows
  // of the current bag are dealt to the slots kUnroll steps at a time: their loads are issued
  // together, then pooled.  When the bag ends its sums are flushed and the next bag continues
  // in the same block.
  // A row's slot is its index within the bag modulo the slot count, wherever the bag begins in
  // its block and however many bags the run holds: every slot then adds the same rows in the
  // same order for any launch size, and a table pooled alone gives the same bits as the table
  // pooled beside others.
  int bag = 0;
  int pos = 0, bag_start = 0, bag_end = (int)(end_of_bag(0) - run0);
  int blk = 0;  // the 32 indices in hand are positions blk .. blk + 31
  int32_t r_mine, r_next;
  float w_mine, w_next;
  fetch(lane, r_mine, w_mine);
  fetch(32 + lane, r_next, w_next);
  while (true) {
    const int lim = bag_end < blk + 32 ? bag_end : blk + 32;
    const int q0 = pos - blk, n = lim - blk;
    const int rot = (slot - (pos - bag_start)) & (slots - 1);  // this slot's first row of the piece, counted from q0
    for (int k = 0; q0 + k * slots < n; k += kUnroll) {
      int32_t r[kUnroll];
      float w[kUnroll];
      typename RL::Chunk pay[kUnroll][P];
      uint2 tl[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        const int src = q0 + (k + u) * slots + rot;  // position of this slot's row in the block
        r[u] = __shfl_sync(0xffffffffu, r_mine, src & 31);
        w[u] = __shfl_sync(0xffffffffu, w_mine, src & 31);
        if (src >= n) r[u] = -2;                       // no row for this slot in this step
        else if (r[u] == -1) flags |= GLOWB200_STATUS_INDEX_OUT_OF_RANGE;
      }
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        if (r[u] >= 0) {
          const uint8_t *row = data + (int64_t)r[u] * in_line;
#pragma unroll
          for (int c = 0; c < P; c++)
            if (has[c]) pay[u][c] = RL::payload(row, c * lpr + gl);
          tl[u] = RL::tail(row + in_line);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; u++) {
        if (r[u] >= 0) {
          float scale, offset;
          RL::scale_offset(tl[u], scale, offset);
          const float a = RL::scale_for_pooling(w[u] * scale);
          bias_sum = RL::row_term(w[u], offset, a, bias_sum);
#pragma unroll
          for (int c = 0; c < P; c++)
            if (has[c]) RL::pool(pay[u][c], a, acc + c * 8);
        }
      }
    }
    pos = lim;
    if (pos == bag_end) {  // the bag is complete
      flush(first_bag + bag);
      if (bag == n_bags - 1) break;
      reset();
      bag++;
      bag_start = pos;
      bag_end = (int)(end_of_bag(bag) - run0);  // bags of a lengths array are back to back: the next one starts at pos
    }
    if (pos == blk + 32) {  // the block is used up: the prefetched one becomes current
      blk += 32;
      r_mine = r_next;
      w_mine = w_next;
      fetch(blk + 32 + lane, r_next, w_next);
    }
  }
  raise(p.status, flags);
}

// The warp-per-run mapping alone, bag boundaries computed in place: the whole of a small request
// in one launch.
template <int BITS, bool SO16, bool OUT16, typename IdxT, int P, int U>
__global__ void __launch_bounds__(kGatherThreads, kGatherBlockScale * GLOWB200_SLWS_MIN_BLOCKS)
slws_gather_small_kernel(const __grid_constant__ SlwsLaunch p) {
  gather_warp_body<BITS, SO16, OUT16, IdxT, P, U, false, true>(p, 1);
}

// One launch, two thread-to-bag mappings: every table is pooled by the mapping its bag-length
// profile favours (the word the segments kernel leaves behind the table's boundaries).
// grid.x covers the larger of the two mappings' block counts; surplus blocks leave at once.
// MINB: blocks of 256 threads' worth per SM the register allocation must allow.  Three (85 registers)
// is best for narrow rows in uniform bags (four, 64 registers: 360 against 335 us on 72-byte rows);
// four for uint8 rows of 128 columns and more, whose lane groups are wide and whose tables in the
// recommendation model are skewed (one rank's share of eight 177 -> 172 us, the whole model +3 %).
template <int BITS, bool SO16, bool OUT16, typename IdxT, int P, int U, bool SHARD = false,
          int MINB = (P == 4 ? GLOWB200_SLWS_MIN_BLOCKS_P4 : GLOWB200_SLWS_MIN_BLOCKS)>
__global__ void __launch_bounds__(kGatherThreads, kGatherBlockScale * MINB)
slws_gather_select_kernel(const __grid_constant__ SlwsLaunch p, int bags_per_warp) {
  pdl_wait();
  pdl_launch_dependents();
  const glowb200_slws_job *jp = p.jobs ? (p.jobs + blockIdx.y) : &p.single;
  const bool skewed = GLOWB200_SLWS_FORCE_WARP || p.warp_per_bag != 0 ||
                      p.seg_begin[(int64_t)blockIdx.y * p.seg_stride + bags_of(p, jp) + 1] != 0;
  if (skewed) gather_warp_body<BITS, SO16, OUT16, IdxT, P, U, SHARD>(p, bags_per_warp);
  else gather_group_body<BITS, SO16, OUT16, false, IdxT, P, U, SHARD>(p);
}

// ------------------------------------------------------------------------------------------
// Any-shape gather-pool: rows of any width and alignment (a column count that is not a
// multiple of 8, a table that is not 8-byte aligned).  One warp per bag, byte loads, column
// tiles of 128; the row-by-row arithmetic of the reference in its order, without FMA
// contraction.  Correct for everything, fast for nothing -- real tables take the kernel above.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) slws_gather_any_kernel(const __grid_constant__ SlwsLaunch p, int bits,
                                                               int so16, int out16, int acc16, int idx64) {
  const int job_id = blockIdx.y;
  const glowb200_slws_job *jp = p.jobs ? (p.jobs + job_id) : &p.single;
  const int64_t bag = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (bag >= bags_of(p, jp)) return;
  const int lane = threadIdx.x & 31;
  const uint8_t *data = reinterpret_cast<const uint8_t *>(jp->data);
  const int64_t *sb = p.seg_begin + (int64_t)job_id * p.seg_stride;
  int64_t begin = sb[bag], end = sb[bag + 1];
  int32_t flags = 0;
  if (end < begin) { end = begin; flags |= GLOWB200_STATUS_BAD_OFFSETS; }
  const int64_t in_line = p.in_line;
  const int D = p.out_line;
  for (int tile = 0; tile < D; tile += 128) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t j = begin; j < end; j++) {
      int64_t r = idx64 ? reinterpret_cast<const int64_t *>(jp->indices)[j]
                        : (int64_t) reinterpret_cast<const int32_t *>(jp->indices)[j];
      const int64_t g = r;
      if (p.sharded) r -= jp->row_begin;
      if (r < 0 || r >= jp->rows) {
        if (!p.sharded || g < 0 || g >= jp->global_rows) flags |= GLOWB200_STATUS_INDEX_OUT_OF_RANGE;
        continue;
      }
      const float w = out16 ? __half2float(reinterpret_cast<const __half *>(jp->weights)[j])
                            : reinterpret_cast<const float *>(jp->weights)[j];
      const uint8_t *row = data + r * in_line;
      float scale, offset;
      if (so16) {
        const uint8_t *t = row + in_line - 4;
        scale = __half2float(__ushort_as_half((unsigned short)(t[0] | (t[1] << 8))));
        offset = __half2float(__ushort_as_half((unsigned short)(t[2] | (t[3] << 8))));
      } else {
        const uint8_t *t = row + in_line - 8;
        scale = __uint_as_float(t[0] | (t[1] << 8) | (t[2] << 16) | ((uint32_t)t[3] << 24));
        offset = __uint_as_float(t[4] | (t[5] << 8) | (t[6] << 16) | ((uint32_t)t[7] << 24));
      }
#pragma unroll
      for (int s = 0; s < 4; s++) {
        const int k = tile + s * 32 + lane;
        if (k < D) {
          uint32_t q;
          if (bits == 8) q = row[k];
          else { q = row[k >> 1]; q = (k & 1) ? (q >> 4) : (q & 0xFu); }
          const float d = __fadd_rn(__fmul_rn((float)q, scale), offset);
          const float prod = __fmul_rn(d, w);
          if (acc16) acc[s] = __half2float(__float2half_rn(__fadd_rn(acc[s], __half2float(__float2half_rn(prod)))));
          else acc[s] = __fadd_rn(acc[s], prod);
        }
      }
    }
#pragma unroll
    for (int s = 0; s < 4; s++) {
      const int k = tile + s * 32 + lane;
      if (k < D) {
        void *dest_base = jp->dest;
        int64_t dest_row = bag;
        if (jp->bags_per_dest > 0) {
          const int64_t which = bag / jp->bags_per_dest;
          dest_base = jp->dests[which];
          dest_row = bag - which * jp->bags_per_dest;
        }
        if (out16) reinterpret_cast<__half *>(dest_base)[dest_row * jp->dest_stride + k] = __float2half_rn(acc[s]);
        else reinterpret_cast<float *>(dest_base)[dest_row * jp->dest_stride + k] = acc[s];
      }
    }
  }
  raise(p.status, flags);
}

// ------------------------------------------------------------------------------------------
// Host dispatch
// ------------------------------------------------------------------------------------------
struct GatherConfig {
  int kind, idx64, out16, acc16;
};

#ifndef GLOWB200_SLWS_WARP_PER_BAG
#define GLOWB200_SLWS_WARP_PER_BAG 1
#endif


// (P, U) pairs that exist: chunks per lane P, rows requested per lane before the first is
// consumed U (4 everywhere but the tuning macro of P = 2).
template <int BITS, bool SO16, bool OUT16, bool ACC16, typename IdxT, int P, int U>
cudaError_t launch_gather_pu(const SlwsLaunch &L, dim3 grid, cudaStream_t s) {
#if GLOWB200_SLWS_WARP_PER_BAG
  if constexpr (!ACC16) {
    if (L.select) {
      // fp32 accumulation with lengths: the kernel that picks a mapping per table.  The
      // warp-per-run mapping takes runs of up to 8 bags once that still leaves every SM a few
      // waves of warps; single bags for small launches.
      if (L.inline_lengths) {  // one warp per bag, boundaries computed by the warps: a single launch
        const unsigned blocks = (unsigned)((L.single.segments + (kGatherThreads >> 5) - 1) / (kGatherThreads >> 5));
        slws_gather_small_kernel<BITS, SO16, OUT16, IdxT, P, U><<<blocks, kGatherThreads, 0, s>>>(L);
        return cudaGetLastError();
      }
      const int64_t max_segments = (int64_t)grid.x * (kGatherThreads >> L.lpr_log2);
      // (measured on the recommendation model's power-law bags: 262 144 bags in a launch pool
      // fastest in runs of 4, 32 768 -- one rank's share of eight -- in single bags; the sums do
      // not depend on the choice)
      const int64_t total = max_segments * grid.y, want = (int64_t)sm_count() * 24 * 16;
      int bpw = (int)(total / want);
      bpw = bpw < 1 ? 1 : (bpw > GLOWB200_SLWS_MAX_BPW ? GLOWB200_SLWS_MAX_BPW : bpw);
      const int64_t warps = (max_segments + bpw - 1) / bpw;
      const unsigned wblocks = (unsigned)((warps + (kGatherThreads >> 5) - 1) / (kGatherThreads >> 5));
      dim3 sgrid(wblocks > grid.x ? wblocks : grid.x, grid.y);
      if constexpr (!OUT16) {  // shards give fp32 partial sums (checked by the entry point)
        if (L.sharded) {
          return launch_pdl(slws_gather_select_kernel<BITS, SO16, OUT16, IdxT, P, U, true>, sgrid, kGatherThreads, 0, s, L, bpw);
        }
      }
      if constexpr (P == 2 && BITS == 8) {
        if (L.lpr_log2 >= 3)
          return launch_pdl(slws_gather_select_kernel<BITS, SO16, OUT16, IdxT, P, U, false, 4>, sgrid, kGatherThreads, 0, s, L, bpw);
      }
      return launch_pdl(slws_gather_select_kernel<BITS, SO16, OUT16, IdxT, P, U, false>, sgrid, kGatherThreads, 0, s, L, bpw);
    }
  }
#endif
  slws_gather_kernel<BITS, SO16, OUT16, ACC16, IdxT, P, U><<<grid, kGatherThreads, 0, s>>>(L);
  return cudaGetLastError();
}

template <int BITS, bool SO16, bool OUT16, bool ACC16, typename IdxT>
cudaError_t launch_gather_p(const SlwsLaunch &L, int P, dim3 grid, cudaStream_t s) {
  switch (P) {
    case 1: return launch_gather_pu<BITS, SO16, OUT16, ACC16, IdxT, 1, 4>(L, grid, s);
    case 2: return launch_gather_pu<BITS, SO16, OUT16, ACC16, IdxT, 2, GLOWB200_SLWS_UNROLL_P2>(L, grid, s);
    // (8 rows in flight per lane were tried for 4-bit rows of 256 and 512 columns: 6 % slower)
    default: return launch_gather_pu<BITS, SO16, OUT16, ACC16, IdxT, 4, 4>(L, grid, s);
  }
}

template <int BITS, bool SO16, bool OUT16, bool ACC16>
cudaError_t launch_gather_idx(const SlwsLaunch &L, int idx64, int P, dim3 grid, cudaStream_t s) {
  return idx64 ? launch_gather_p<BITS, SO16, OUT16, ACC16, int64_t>(L, P, grid, s)
               : launch_gather_p<BITS, SO16, OUT16, ACC16, int32_t>(L, P, grid, s);
}

template <int BITS, bool SO16>
cudaError_t launch_gather_out(const SlwsLaunch &L, const GatherConfig &g, int P, dim3 grid, cudaStream_t s) {
  if (g.out16) {
    if constexpr (SO16) {
      if (g.acc16) return launch_gather_idx<BITS, SO16, true, true>(L, g.idx64, P, grid, s);
    }
    return launch_gather_idx<BITS, SO16, true, false>(L, g.idx64, P, grid, s);
  }
  return launch_gather_idx<BITS, SO16, false, false>(L, g.idx64, P, grid, s);
}

int payload_bytes(int kind, int64_t out_line) { return (int)(kind >= 2 ? out_line / 2 : out_line); }
int tail_bytes(int kind) { return (kind & 1) ? 4 : 8; }

// Validates the shape arguments shared by every entry point and decides between the vector
// kernel (P > 0, lpr_log2 set) and the any-shape kernel (P == 0).
int plan(int kind, int64_t in_line, int64_t out_line, bool pointers_aligned, int &P, int &lpr_log2) {
  GLOWB200_REQUIRE(kind >= 0 && kind <= 3, "unknown fused table kind %d", kind);
  GLOWB200_REQUIRE(out_line >= 0 && in_line > 0 && in_line < (1 << 30), "bad line sizes");
  GLOWB200_REQUIRE(kind < 2 || (out_line % 2) == 0, "4-bit rows need an even column count");
  // Rows may be wider than payload + scale/offset: the columns come first, the scale/offset
  // pair is the LAST bytes of the row (where the reference kernel looks for it,
  // libjit.cpp:1263-1264), and whatever lies between is padding -- a table stored with its rows
  // padded to a memory-friendly stride is pooled as it is.
  GLOWB200_REQUIRE(in_line >= payload_bytes(kind, out_line) + tail_bytes(kind),
                   "in_line_size %lld is too small for %lld columns of kind %d", (long long)in_line,
                   (long long)out_line, kind);
  P = 0;
  lpr_log2 = 0;
  const int align = (kind == GLOWB200_UINT8_FUSED) ? 8 : 4;
  if (out_line == 0 || (out_line % 8) != 0 || (in_line % align) != 0 || !pointers_aligned) return GLOWB200_OK;
  const int chunks = (int)(out_line / 8);
  if (chunks > 128) return GLOWB200_OK;  // > 1024 columns: any-shape kernel
  // Two chunks per lane once a row has 8 or more chunks: halves the per-row bookkeeping per
  // byte. Four when 32 lanes cannot cover the row otherwise, and for 4-bit rows of 128 or more
  // columns, where a chunk is only 4 payload bytes and a lane's load would otherwise be 8 bytes
  // (measured on the 4-bit sweep: +12 % at 128 columns, +15 % at 256; at 64 and 32 columns four
  // chunks per lane leave too few lanes per row and lose 20-25 %).
  P = chunks > 64 || (kind >= 2 && chunks >= GLOWB200_SLWS_P4_FROM) ? 4 : (chunks >= 8 ? 2 : 1);
  int lpr = 1;
  while (lpr * P < chunks) lpr <<= 1;
  lpr_log2 = 0;
  while ((1 << lpr_log2) < lpr) lpr_log2++;
  return GLOWB200_OK;
}

int run_gather(SlwsLaunch &L, const GatherConfig &g, int P, int64_t max_segments, int64_t num_jobs,
               cudaStream_t s) {
  if (max_segments == 0 || num_jobs == 0) return GLOWB200_OK;
  cudaError_t e;
  if (P == 0) {
    dim3 grid((unsigned)((max_segments + 7) / 8), (unsigned)num_jobs);
    slws_gather_any_kernel<<<grid, 256, 0, s>>>(L, g.kind >= 2 ? 4 : 8, g.kind & 1, g.out16, g.acc16, g.idx64);
    e = cudaGetLastError();
  } else {
    const int bags_per_block = kGatherThreads >> L.lpr_log2;
    dim3 grid((unsigned)((max_segments + bags_per_block - 1) / bags_per_block), (unsigned)num_jobs);
    switch (g.kind) {
      case GLOWB200_UINT8_FUSED: e = launch_gather_out<8, false>(L, g, P, grid, s); break;
      case GLOWB200_UINT8_FUSED_FP16: e = launch_gather_out<8, true>(L, g, P, grid, s); break;
      case GLOWB200_UINT4_FUSED: e = launch_gather_out<4, false>(L, g, P, grid, s); break;
      default: e = launch_gather_out<4, true>(L, g, P, grid, s); break;
    }
  }
  if (e != cudaSuccess) return set_error(GLOWB200_ERR_CUDA, "gather-pool launch failed: %s", cudaGetErrorString(e));
  return GLOWB200_OK;
}

size_t seg_stride_elems(int64_t max_segments) { return align_up((size_t)(max_segments + 2) * 8, 256) / 8; }

bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace
}  // namespace glowb200

int glowb200::launch_segments_from_lengths(const int32_t *lengths, int64_t segments, int64_t num_indices,
                                           void *workspace, size_t workspace_bytes, int32_t *status,
                                           cudaStream_t stream) {
  GLOWB200_REQUIRE(segments >= 0 && segments < (1ll << 31) && num_indices >= 0, "segments / num_indices out of range");
  if (segments == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(lengths != nullptr, "lengths is NULL");
  const size_t need = seg_stride_elems(segments) * 8;
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(GLOWB200_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  GLOWB200_REQUIRE(aligned_to(workspace, 8), "workspace must be 8-byte aligned");
  SlwsLaunch L{};
  L.single.lengths = lengths;
  L.single.segments = segments;
  L.single.num_indices = num_indices;
  L.seg_begin = reinterpret_cast<int64_t *>(workspace);
  L.seg_stride = (int64_t)seg_stride_elems(segments);
  L.max_segments = segments;
  L.status = status;
  slws_segments_from_lengths_kernel<<<1, kSegThreads, 0, stream>>>(L);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

using namespace glowb200;

extern "C" size_t glowb200_slws_workspace_bytes(int64_t max_segments, int64_t num_jobs) {
  if (max_segments < 0 || num_jobs <= 0) return 0;
  return seg_stride_elems(max_segments) * 8 * (size_t)num_jobs;
}

namespace {
int run_batched(const glowb200_slws_job *jobs, int64_t num_jobs, int64_t max_segments, int kind, int indices_are_int64,
                int64_t in_line_size, int64_t out_line_size, int out_is_fp16, int use_fp16_accumulation,
                void *workspace, size_t workspace_bytes, int32_t *status, glowb200_stream_t stream, bool sharded) {
  GLOWB200_REQUIRE(num_jobs >= 0 && num_jobs <= 65535, "num_jobs must be in [0, 65535]");
  GLOWB200_REQUIRE(max_segments >= 0 && max_segments < (1ll << 31), "max_segments out of range");
  if (num_jobs == 0 || max_segments == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(jobs != nullptr, "jobs is NULL");
  int P, lpr_log2;
  // Table / result pointers of a batched launch live in device memory: the descriptors are
  // required to hold 16-byte aligned tables, which every cudaMalloc'ed slab offset that keeps
  // Glow's 64-byte TensorAlignment satisfies.
  if (int rc = plan(kind, in_line_size, out_line_size, true, P, lpr_log2)) return rc;
  const size_t need = glowb200_slws_workspace_bytes(max_segments, num_jobs);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(GLOWB200_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  GLOWB200_REQUIRE(aligned_to(workspace, 8), "workspace must be 8-byte aligned");
  SlwsLaunch L{};
  L.jobs = jobs;
  L.seg_begin = reinterpret_cast<int64_t *>(workspace);
  L.seg_stride = (int64_t)seg_stride_elems(max_segments);
  L.max_segments = max_segments;
  L.status = status;
  L.in_line = (int32_t)in_line_size;
  L.out_line = (int32_t)out_line_size;
  L.lpr_log2 = lpr_log2;
  GatherConfig g{kind, indices_are_int64 ? 1 : 0, out_is_fp16 ? 1 : 0,
                 (use_fp16_accumulation && out_is_fp16 && (kind & 1)) ? 1 : 0};
  L.select = (P != 0 && !g.acc16) ? 1 : 0;
  L.sharded = sharded ? 1 : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  GLOWB200_CUDA_OK(launch_pdl(slws_segments_from_lengths_kernel, dim3((unsigned)num_jobs), kSegThreads, 0, s, L));
  return run_gather(L, g, P, max_segments, num_jobs, s);
}
}  // namespace

extern "C" int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_batched(
    const glowb200_slws_job *jobs, int64_t num_jobs, int64_t max_segments, int kind, int indices_are_int64,
    int64_t in_line_size, int64_t out_line_size, int out_is_fp16, int use_fp16_accumulation, void *workspace,
    size_t workspace_bytes, int32_t *status, glowb200_stream_t stream) {
  return run_batched(jobs, num_jobs, max_segments, kind, indices_are_int64, in_line_size, out_line_size, out_is_fp16,
                     use_fp16_accumulation, workspace, workspace_bytes, status, stream, false);
}

extern "C" int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_row_sharded(
    const glowb200_slws_job *jobs, int64_t num_jobs, int64_t max_segments, int kind, int indices_are_int64,
    int64_t in_line_size, int64_t out_line_size, void *workspace, size_t workspace_bytes, int32_t *status,
    glowb200_stream_t stream) {
  return run_batched(jobs, num_jobs, max_segments, kind, indices_are_int64, in_line_size, out_line_size, 0, 0,
                     workspace, workspace_bytes, status, stream, true);
}

namespace {
int fill_single(SlwsLaunch &L, GatherConfig &g, int &P, void *dest, const void *data, int kind, int64_t rows,
                const void *weights, const void *indices, int idx64, const int32_t *lengths, int64_t segments,
                int64_t num_indices, int64_t in_line, int64_t out_line, int out16, int acc16, void *workspace,
                size_t workspace_bytes, int32_t *status) {
  GLOWB200_REQUIRE(segments >= 0 && segments < (1ll << 31), "segments out of range");
  GLOWB200_REQUIRE(rows >= 0 && rows < (1ll << 31) && num_indices >= 0, "rows must be in [0, 2^31), num_indices >= 0");
  GLOWB200_REQUIRE(segments == 0 || (dest && (num_indices == 0 || (data && weights && indices))),
                   "NULL tensor pointer");
  const bool al = aligned_to(data, kind == GLOWB200_UINT8_FUSED ? 8 : 4) && aligned_to(dest, out16 ? 2 : 4) &&
                  aligned_to(weights, out16 ? 2 : 4) && aligned_to(indices, idx64 ? 8 : 4);
  int lpr_log2;
  if (int rc = plan(kind, in_line, out_line, al, P, lpr_log2)) return rc;
  const size_t need = glowb200_slws_workspace_bytes(segments, 1);
  if (segments > 0 && (workspace == nullptr || workspace_bytes < need))
    return set_error(GLOWB200_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  GLOWB200_REQUIRE(aligned_to(workspace, 8), "workspace must be 8-byte aligned");
  L = SlwsLaunch{};
  L.jobs = nullptr;
  L.single.data = data;
  L.single.weights = weights;
  L.single.indices = indices;
  L.single.lengths = lengths;
  L.single.dest = dest;
  L.single.rows = rows;
  L.single.num_indices = num_indices;
  L.single.dest_stride = out_line;
  L.single.segments = segments;
  L.seg_begin = reinterpret_cast<int64_t *>(workspace);
  L.seg_stride = (int64_t)seg_stride_elems(segments);
  L.max_segments = segments;
  L.status = status;
  L.in_line = (int32_t)in_line;
  L.out_line = (int32_t)out_line;
  L.lpr_log2 = lpr_log2;
  g = GatherConfig{kind, idx64 ? 1 : 0, out16 ? 1 : 0, (acc16 && out16 && (kind & 1)) ? 1 : 0};
  return GLOWB200_OK;
}
}  // namespace

extern "C" int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum(
    void *dest, const void *data, int kind, int64_t rows, const void *weights, const void *indices,
    int indices_are_int64, const int32_t *lengths, int64_t segments, int64_t num_indices, int64_t in_line_size,
    int64_t out_line_size, int out_is_fp16, int use_fp16_accumulation, void *workspace, size_t workspace_bytes,
    int32_t *status, glowb200_stream_t stream) {
  SlwsLaunch L;
  GatherConfig g;
  int P;
  if (int rc = fill_single(L, g, P, dest, data, kind, rows, weights, indices, indices_are_int64, lengths, segments,
                           num_indices, in_line_size, out_line_size, out_is_fp16, use_fp16_accumulation, workspace,
                           workspace_bytes, status))
    return rc;
  if (segments == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(lengths != nullptr, "lengths is NULL");
  L.select = (P != 0 && !g.acc16) ? 1 : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  slws_segments_from_lengths_kernel<<<1, kSegThreads, 0, s>>>(L);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return run_gather(L, g, P, segments, 1, s);
}

extern "C" int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_low_latency(
    void *dest, const void *data, int kind, int64_t rows, const void *weights, const void *indices,
    int indices_are_int64, const int32_t *lengths, int64_t segments, int64_t num_indices, int64_t in_line_size,
    int64_t out_line_size, int out_is_fp16, void *workspace, size_t workspace_bytes, int32_t *status,
    glowb200_stream_t stream) {
  SlwsLaunch L;
  GatherConfig g;
  int P;
  if (int rc = fill_single(L, g, P, dest, data, kind, rows, weights, indices, indices_are_int64, lengths, segments,
                           num_indices, in_line_size, out_line_size, out_is_fp16, 0, workspace, workspace_bytes, status))
    return rc;
  if (segments == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(lengths != nullptr, "lengths is NULL");
  L.select = (P != 0) ? 1 : 0;
  L.warp_per_bag = 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // up to 2048 bags every warp adds up the lengths before its bag itself (at most 64 loads a lane)
  L.inline_lengths = (P != 0 && segments <= 2048) ? 1 : 0;
  if (!L.inline_lengths) {
    slws_segments_from_lengths_kernel<<<1, kSegThreads, 0, s>>>(L);
    GLOWB200_CUDA_OK(cudaGetLastError());
  }
  return run_gather(L, g, P, segments, 1, s);
}

extern "C" int glowb200_embedding_bag_byte_rowwise_offsets(
    void *dest, const void *data, int kind, int64_t rows, const void *weights, const void *indices,
    const void *offsets, int indices_are_int64, int64_t num_offsets, int64_t num_indices, int64_t in_line_size,
    int64_t out_line_size, int has_end_offset, int out_is_fp16, int use_fp16_accumulation, void *workspace,
    size_t workspace_bytes, int32_t *status, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(num_offsets >= 0, "negative num_offsets");
  const int64_t segments = has_end_offset ? num_offsets - 1 : num_offsets;
  if (segments <= 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(offsets != nullptr, "offsets is NULL");
  SlwsLaunch L;
  GatherConfig g;
  int P;
  if (int rc = fill_single(L, g, P, dest, data, kind, rows, weights, indices, indices_are_int64, nullptr, segments,
                           num_indices, in_line_size, out_line_size, out_is_fp16, use_fp16_accumulation, workspace,
                           workspace_bytes, status))
    return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((segments + 1 + 255) / 256 < 1024 ? (segments + 1 + 255) / 256 : 1024);
  if (indices_are_int64)
    slws_segments_from_offsets_kernel<int64_t><<<blocks, 256, 0, s>>>(L, reinterpret_cast<const int64_t *>(offsets), has_end_offset ? 1 : 0);
  else
    slws_segments_from_offsets_kernel<int32_t><<<blocks, 256, 0, s>>>(L, reinterpret_cast<const int32_t *>(offsets), has_end_offset ? 1 : 0);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return run_gather(L, g, P, segments, 1, s);
}

// ------------------------------------------------------------------------------------------
// Pooling with no caller-provided workspace and no allocation of any kind.
//
// Who needs this: code that serves requests after all device memory has been handed out.  A
// Glow DeviceManager sizes its slabs when a network is loaded and accounts every byte against
// the device's budget; on its request thread a cudaMalloc could fail against that budget and,
// succeed or fail, stalls every stream of the device while the driver takes its allocator
// lock.  A plug-in that is only ever handed buffers by its host has no allocator at all.  Such
// callers cannot size a workspace per request either, so the bag boundaries go into a fixed
// array that is part of the library image.
//
// The array costs kStaticScratchMaxSegments * 8 bytes (+ padding) of device memory on every
// GPU that loads the library, for the life of the process.
// ------------------------------------------------------------------------------------------
namespace glowb200 {
namespace {
constexpr int64_t kStaticScratchMaxSegments = 65536;
constexpr size_t kStaticScratchBytes = ((kStaticScratchMaxSegments + 2) * 8 + 255) / 256 * 256;
constexpr int kStaticScratchMaxDevices = 64;
}  // namespace
}  // namespace glowb200

// Device storage.  In host code this name is only a handle for the runtime's symbol lookup --
// it is NOT a device address and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned char g_slws_static_scratch[glowb200::kStaticScratchBytes];

namespace glowb200 {
namespace {
// Device address of g_slws_static_scratch on the CURRENT device, looked up once per device.
int static_scratch_address(void **out) {
  static void *cached[kStaticScratchMaxDevices] = {nullptr};
  static bool known[kStaticScratchMaxDevices] = {false};
  static std::mutex lock;
  int dev = -1;
  GLOWB200_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kStaticScratchMaxDevices)
    return set_error(GLOWB200_ERR_UNSUPPORTED, "device ordinal %d is beyond the %d this entry point tracks", dev,
                     kStaticScratchMaxDevices);
  std::lock_guard<std::mutex> guard(lock);
  if (!known[dev]) {
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_slws_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return set_error(GLOWB200_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d failed: %s", dev,
                       cudaGetErrorString(e));
    cached[dev] = ptr;
    known[dev] = true;
  }
  *out = cached[dev];
  return GLOWB200_OK;
}
}  // namespace
}  // namespace glowb200

extern "C" int64_t glowb200_slws_static_scratch_max_segments(void) { return glowb200::kStaticScratchMaxSegments; }

extern "C" int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_static_scratch(
    void *dest, const void *data, int kind, int64_t rows, const void *weights, const void *indices,
    int indices_are_int64, const int32_t *lengths, int64_t segments, int64_t num_indices, int64_t in_line_size,
    int64_t out_line_size, int out_is_fp16, int use_fp16_accumulation, int32_t *status, glowb200_stream_t stream) {
  if (segments > kStaticScratchMaxSegments)
    return set_error(GLOWB200_ERR_UNSUPPORTED,
                     "%lld bags exceed the %lld the built-in scratch array holds; use the entry point that takes a "
                     "workspace", (long long)segments, (long long)kStaticScratchMaxSegments);
  if (segments <= 0) {
    GLOWB200_REQUIRE(segments == 0, "segments out of range");
    return GLOWB200_OK;
  }
  void *scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  SlwsLaunch L;
  GatherConfig g;
  int P;
  if (int rc = fill_single(L, g, P, dest, data, kind, rows, weights, indices, indices_are_int64, lengths, segments,
                           num_indices, in_line_size, out_line_size, out_is_fp16, use_fp16_accumulation, scratch,
                           kStaticScratchBytes, status))
    return rc;
  GLOWB200_REQUIRE(lengths != nullptr, "lengths is NULL");
  L.select = (P != 0 && !g.acc16) ? 1 : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // The segments kernel rewrites everything this call reads (segments + 1 boundaries and the
  // table's profile word); nothing in the array has to start at zero, and whatever an earlier
  // call left beyond them is never read.
  slws_segments_from_lengths_kernel<<<1, kSegThreads, 0, s>>>(L);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return run_gather(L, g, P, segments, 1, s);
}
