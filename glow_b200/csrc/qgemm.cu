// Int8 contraction for Glow's quantized dense layers on the sm_100a tensor cores:
// RowwiseQuantizedFullyConnected, FullyConnected (int8) and MatMul (int8).
//
//   out[i,j] = clip8( scale32( sum_k (A[i,k]-aOff)*(B[j,k]-bOff_j) + biasTerm_j ,
//                              outPre_j, outPost_j, outScale_j, outOffset ) )
//
// The tensor cores contract the raw int8 values (tcgen05.mma kind::i8, int32 accumulators in
// tensor memory); the offsets are folded in afterwards, exactly, in 32-bit wrapping arithmetic:
//   sum_k (A-a0)(B-b0) = sum_k A*B - a0*rowsum(B_j) - b0_j*rowsum(A_i) + K*a0*b0_j .
// The epilogue then applies Glow's integer requantisation (libjit_scale, libjit_clip_i8).
//
// Persistent CTAs (one per SM) walk 128 x BLOCK_N output tiles.  Warp 0 feeds shared memory
// with TMA (128-byte swizzled K-major tiles of 128 bytes of K), warp 1 issues the MMAs and owns
// the tensor-memory allocation, warps 2-5 build each tile's per-column constants and drain its
// accumulators (tcgen05.ld), requantise and store int8 -- overlapped with the next tile's main
// loop through two accumulator buffers in tensor memory.
//
// Every wait on an mbarrier is bounded: when it runs out the kernel raises
// GLOWB200_STATUS_WAIT_TIMEOUT, all roles leave their loops, tensor memory is released and the
// kernel returns.
#include <cuda.h>

#include <cstdlib>
#include <cstdio>
#include <mutex>
#include <type_traits>

#include "common.cuh"

#include <climits>
#include "qgemm.cuh"

namespace glowb200 {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockK = 128;          // bytes of K per pipeline stage = one 128B swizzle atom
constexpr int kUmmaK = 32;            // K per tcgen05.mma for 8-bit operands
constexpr int kEpilogueWarps = 16;    // 4 per tensor-memory lane quarter: enough warps per scheduler to hide ALU latency
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kGemmThreads = 64 + kEpilogueThreads;  // TMA warp, MMA warp, epilogue warps
constexpr long long kWaitCycles = 2000000000ll;  // ~1 s: far beyond any legitimate wait

// Per output column, built once per column block in shared memory and read back with one
// 16-byte load per record.
struct __align__(16) ColParams {
  int32_t c;        // bias term - aOff*rowsum(B_j) + K*aOff*bOff_j
  int32_t scale;    // integer multiplier of the output rescale
  int32_t shifts;   // pre | post << 8
  int32_t b_off;    // weight offset
};

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when it gave up (or another role already did).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          long long limit = kWaitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    for (int i = 0; i < 64; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) {
      *abort_flag = 1;
      return false;
    }
  }
}

// The bounded wait, exercised on its own: one warp waits on a barrier that nothing will ever
// complete, with a short limit; it must give up, say so through the status word and return, and
// the other warp, polling the shared flag the way the kernel's other roles do, must leave too.
__global__ void __launch_bounds__(64) wait_limit_selftest_kernel(long long limit, int32_t *status, int32_t *gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag_storage;
  volatile int *abort_flag = &abort_flag_storage;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag_storage = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    ok = mbar_wait(&bar, 0, abort_flag, limit);  // phase 0 never completes: nobody arrives
  } else if (threadIdx.x == 32) {
    ok = mbar_wait(&bar, 0, abort_flag, 4 * limit);  // leaves as soon as the first waiter gave up
  }
  if (!ok) {
    atomicAdd(gave_up, 1);
    if (status != nullptr) atomicOr(status, GLOWB200_STATUS_WAIT_TIMEOUT);
  }
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

// ---- CTA pairs (a cluster of two CTAs issuing one MMA over both SMs, cta_group::2) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (a shared-memory address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void *p, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
  return a;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A load into this CTA's shared memory whose bytes are counted on a barrier of the pair's even CTA
// (every CTA loads its own tiles).
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int c0, int c1, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// One MMA over the pair: 256 rows (128 per CTA, each from its own shared memory and into its own
// tensor memory) by N columns, whose right operand is split by rows between the two CTAs.
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this address in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[N]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// rows 16 lanes from the address's lane on, 16 columns: see the drain of the int8 result for the layout
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, uint32_t *r) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): 8-row groups are 1024
// bytes apart (stride byte offset), the leading byte offset is unused and set to 16 bytes,
// descriptor version 1 (sm_100), layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// The same for a K-major tile of 32-byte rows in the 32-byte swizzle (CU_TENSOR_MAP_SWIZZLE_32B):
// 8-row groups are 256 bytes apart, layout type 6.
__device__ __forceinline__ uint64_t smem_desc_sw32(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(256 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)6 << 61;
  return d;
}

// Instruction descriptor for kind::i8: D = s32, A = B = signed 8-bit, both K-major, dense.
__host__ __device__ constexpr uint32_t idesc_i8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// The tensor pipe's own int8 rate, measured rather than quoted: every CTA (one per SM) issues
// `mmas` 128 x 256 x 32 int8 MMAs back to back on operand tiles that already sit in shared
// memory (their contents do not matter to the timing), into two alternating accumulators in
// tensor memory, then waits -- bounded -- for the last one.  Nothing is loaded, drained or
// stored, so the time of a launch is what the MMA pipe itself needs under full load at the
// clocks the GPU holds: the ceiling a contraction kernel is measured against.
__global__ void __launch_bounds__(128) i8_mma_issue_probe_kernel(int mmas, int32_t *status) {
  extern __shared__ __align__(1024) uint8_t probe_smem[];
  __shared__ uint64_t done_bar;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag_storage;
  volatile int *abort_flag = &abort_flag_storage;
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(probe_smem) + 1023) & ~(uintptr_t)1023);
  constexpr int kN = 256;
  if (threadIdx.x == 0) {
    mbar_init(&done_bar, 1);
    abort_flag_storage = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // defined operand bytes (the values are irrelevant, but nothing reads uninitialised memory)
  for (int i = threadIdx.x; i < (kBlockM + kN) * kBlockK / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(tiles)[i] = 0x01020304u * (uint32_t)(i + 1);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x < 32) {
    tmem_alloc(&tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  bool ok = true;
  if (threadIdx.x == 0) {
    const uint32_t a_addr = smem_u32(tiles), b_addr = a_addr + kBlockM * kBlockK;
    const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(b_addr);
    constexpr uint32_t idesc = idesc_i8(kBlockM, kN);
    for (int i = 0; i < mmas; i++) {
      const int k = i & 3;  // the four 32-byte k steps of the 128-byte tile rows
      umma_i8(tmem_base + (uint32_t)((i >> 2) & 1) * kN, a_desc + (uint64_t)(k * kUmmaK >> 4), b_desc + (uint64_t)(k * kUmmaK >> 4),
              idesc, k != 0);
    }
    umma_commit(&done_bar);
    ok = mbar_wait(&done_bar, 0, abort_flag);
    if (!ok && status != nullptr) atomicOr(status, GLOWB200_STATUS_WAIT_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem_base, 512);
}

// Byte offset of 16-byte piece q16 of row r (0..31) in a quarter's staging area of PITCH-byte rows.
// The piece index is xor-ed with the row's position among the rows that share 128 bytes of banks, so
// eight lanes writing the same piece of eight consecutive rows, and eight lanes reading consecutive
// pieces of one row (or of neighbouring short rows), each cover all 32 banks once.
template <int PITCH>
__device__ __forceinline__ int stage_offset(int r, int q16) {
  constexpr int n = PITCH / 16;
  const int x = n >= 8 ? (r & 7) : ((r / (8 / n)) & (n - 1));
  return r * PITCH + 16 * (q16 ^ x);
}

// Optional tracing for tuning builds (python -m glow_b200.build -DGLOWB200_GEMM_TRACE): every CTA
// stamps %globaltimer (ns) at entry and exit -- entries 2b and 2b + 1 of a device buffer -- and
// CTA 0 its clock64 at the same two points (entries 510, 511), from which the SM clock a launch really
// ran at follows; CTA 0 also stamps the phases of its first tile (entries 496 + slot).
// glowb200_debug_gemm_trace copies the 512 entries out.  Compiled out by default.
#ifdef GLOWB200_GEMM_TRACE
__device__ unsigned long long g_gemm_trace[512];
__device__ __forceinline__ void trace(int slot) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  if ((slot == 0 || slot == 6) && blockIdx.x < 248) {
    g_gemm_trace[2 * blockIdx.x + (slot == 6)] = t;
    if (blockIdx.x == 0) g_gemm_trace[510 + (slot == 6)] = (unsigned long long)clock64();
  }
  if (blockIdx.x == 0 && slot < 14) g_gemm_trace[496 + slot] = t;
}
#define GEMM_TRACE(slot, cond) do { if (cond) trace(slot); } while (0)
#else
#define GEMM_TRACE(slot, cond) do { } while (0)
#endif

// ---------------------------------------------------------------------------------------
// The tile kernel
// ---------------------------------------------------------------------------------------
template <int BLOCK_N, int STAGES, int PAIR = 0>
struct GemmSmem {
  static constexpr int kABytes = kBlockM * kBlockK;
  static constexpr int kBBytes = (PAIR ? BLOCK_N / 2 : BLOCK_N) * kBlockK;  // a pair's CTAs hold half of the rows each
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTileBytes = STAGES * kStageBytes;
  static constexpr int kColBytes = BLOCK_N * (int)sizeof(ColParams);
  // The int8 result of a tile on its way out: 128 rows of kOutPitch bytes, then the output row of each.
  static constexpr int kOutPitch = BLOCK_N <= 32 ? 32 : BLOCK_N <= 64 ? 64 : BLOCK_N <= 128 ? 128 : 256;
  static constexpr int kOutBytes = kBlockM * kOutPitch + kBlockM * 4;
  static constexpr int kTotal = kTileBytes + kColBytes + kOutBytes + 256 /*barriers*/ + 1024 /*alignment slack*/;
  static_assert(kTotal <= 232448, "more shared memory than a CTA can have");
};

// Persistent: gridDim.x CTAs walk the tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...
// (column-tile-major, so CTAs running together share weight tiles in L2).  The accumulators are
// double-buffered in tensor memory: while the epilogue warps drain tile i, the MMA warp is
// already accumulating tile i+1 into the other buffer.
// MODE 0: no input row sums take part (every weight offset is 0) and the activation is none or
// Relu -- the common case, whose drain has neither the row-sum term nor the activation switch;
// MODE 1: everything else with an int8 result; MODE 2: the floating-point result of the
// dynamically quantized layers (GemmParams::float_out).  One drain body per kernel keeps the
// register allocation inside the 96 registers a 576-thread CTA leaves.
// PAIR: the grid is clusters of two CTAs and a tile is 256 rows -- 128 per CTA, whose tensor core
// reads its own rows of the left operand and HALF of the right operand's rows from its own shared
// memory and the other half from its partner's (tcgen05.mma.cta_group::2, issued by the even CTA
// for both), so every SM loads and reads a third fewer operand bytes per MMA.
// Barriers: full[] of the even CTA counts the bytes of both CTAs' loads; empty[] and acc_full[] are
// signalled in both CTAs by multicast commits; acc_empty[] of the even CTA collects the epilogue
// warps of both.
template <int BLOCK_N, int STAGES, int MODE, int PAIR = 0>
__global__ void __launch_bounds__(kGemmThreads, 1)
i8_gemm_requant_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ GemmParams p) {
  using S = GemmSmem<BLOCK_N, STAGES, PAIR>;
  constexpr int kTileM = PAIR ? 2 * kBlockM : kBlockM;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;                 // CTA of the pair
  const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;   // which tile sequence this CTA follows
  const int walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles must start on 1024-byte boundaries.
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  ColParams *cols = reinterpret_cast<ColParams *>(smem + S::kTileBytes);
  uint8_t *out_stage = smem + S::kTileBytes + S::kColBytes;
  int32_t *out_rows = reinterpret_cast<int32_t *>(out_stage + kBlockM * S::kOutPitch);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + S::kTileBytes + S::kColBytes + S::kOutBytes);
  uint64_t *empty = full + STAGES;
  uint64_t *acc_full = empty + STAGES;   // [2]
  uint64_t *acc_empty = acc_full + 2;    // [2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  GEMM_TRACE(0, threadIdx.x == 0);
  const int m_tiles = (p.M + kTileM - 1) / kTileM, n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int tiles = m_tiles * n_tiles;
  const int k_blocks = (p.K + kBlockK - 1) / kBlockK;
  // columns of one accumulator buffer: BLOCK_N rounded up to a power of two (240 -> 256)
  constexpr uint32_t kAccCols = BLOCK_N <= 32 ? 32 : BLOCK_N <= 64 ? 64 : BLOCK_N <= 128 ? 128 : 256;
  constexpr uint32_t kTmemCols = 2 * kAccCols;  // a power of two >= 64

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], (PAIR ? 2 : 1) * kEpilogueWarps);  // one arrival per epilogue warp (of both CTAs)
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();  // the partner's barriers exist before anything signals them
  tc_fence_after();
  // Everything above touched only this CTA's shared and tensor memory, so it may have run beside the
  // tail of the kernel before this one in the stream; the operands and the result are global memory.
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t tmem_base = *tmem_slot;
  GEMM_TRACE(1, threadIdx.x == 0);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;  // k-blocks issued so far, over all tiles of this CTA
      bool live = true;
      for (int t = walker; t < tiles && live; t += walkers) {
        const int m0 = (t % m_tiles) * kTileM + (int)rank * kBlockM, n0 = (t / m_tiles) * BLOCK_N;
        for (int kb = 0; kb < k_blocks; kb++, it++) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort_flag)) { live = false; break; }
          uint8_t *a_dst = smem + s * S::kStageBytes;
          uint8_t *b_dst = a_dst + S::kABytes;
          if constexpr (PAIR) {
            if (rank == 0) mbar_expect_tx(&full[s], 2 * S::kStageBytes);
            const uint32_t leader_full = map_to_cta(&full[s], 0);
            tma_load_2d_pair(a_dst, &map_a, kb * kBlockK, m0, leader_full);
            tma_load_2d_pair(b_dst, &map_b, kb * kBlockK, n0 + (int)rank * (BLOCK_N / 2), leader_full);
            continue;
          }
          mbar_expect_tx(&full[s], S::kStageBytes);
          if (p.conv_windows) {
            // four 128 x 32-byte sub-tiles: window a of plane kb of the 128 pixels, one per MMA k-step
            for (int a4 = 0; a4 < 4; a4++)
              tma_load_2d(a_dst + a4 * (kBlockM * 32), &map_a, 0, kb * p.conv_windows + m0 + a4 * p.conv_wp, &full[s]);
          } else if (p.conv_entries > 0) {
            const int e = kb / p.conv_cpb;
            tma_load_2d(a_dst, &map_a, (kb - e * p.conv_cpb) * kBlockK, m0 + p.conv_row_off[e], &full[s]);
          } else {
            tma_load_2d(a_dst, &map_a, kb * kBlockK, m0, &full[s]);
          }
          tma_load_2d(b_dst, &map_b, kb * kBlockK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_i8(kTileM, BLOCK_N);
      int it = 0, lt = 0;
      bool live = true;
      for (int t = walker; t < tiles && live; t += walkers, lt++) {
        const int buf = lt & 1;
        // wait until the epilogue has drained this buffer (passes at once on its first use)
        if (!mbar_wait(&acc_empty[buf], ((lt >> 1) & 1) ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * kAccCols;
        for (int kb = 0; kb < k_blocks; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag)) { live = false; break; }
          tc_fence_after();
          GEMM_TRACE(2, it == 0);
          const uint32_t a_addr = smem_u32(smem + s * S::kStageBytes);
          const uint32_t b_addr = a_addr + S::kABytes;
          const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(b_addr);
          if (!PAIR && p.conv_windows) {
            // the left operand of k-step k is its own 128 x 32-byte tile in the 32-byte swizzle
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; k++)
              umma_i8(d_tmem, smem_desc_sw32(a_addr + (uint32_t)k * (kBlockM * 32)), b_desc + (uint64_t)(k * (kUmmaK >> 4)), idesc,
                      (kb | k) != 0);
          } else
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; k++) {
            // advancing K inside the swizzle atom = advancing the start address by 32 bytes
            if constexpr (PAIR)
              umma_i8_pair(d_tmem, a_desc + (uint64_t)(k * (kUmmaK >> 4)), b_desc + (uint64_t)(k * (kUmmaK >> 4)), idesc,
                           (kb | k) != 0);
            else
              umma_i8(d_tmem, a_desc + (uint64_t)(k * (kUmmaK >> 4)), b_desc + (uint64_t)(k * (kUmmaK >> 4)), idesc,
                      (kb | k) != 0);
          }
          // the stage may be refilled once these MMAs have read it
          if constexpr (PAIR) umma_commit_pair(&empty[s]);
          else umma_commit(&empty[s]);
        }
        if (live) {  // this tile's accumulators are complete
          if constexpr (PAIR) umma_commit_pair(&acc_full[buf]);
          else umma_commit(&acc_full[buf]);
        }
        GEMM_TRACE(3, lt == 0);
      }
    }
  } else {
    // ---------------- epilogue: warps 2..17 ----------------
    // Warp w may read tensor-memory lanes 32*(w%4)..+31 only; the four warps that share a lane
    // quarter split the tile's columns between them.
    const int et = threadIdx.x - 64;          // 0..511
    const int quarter = warp & 3;
    const int col_group = (warp - 2) >> 2;     // 0..3
    // columns per warp, in whole 16-column drains: 64 (BLOCK_N 256 and 240, whose last group has 48) ... 16 (BLOCK_N 64)
    constexpr int kGroupCols = ((BLOCK_N / 16 + 3) / 4) * 16;
    // columns drained from tensor memory per step: 16 keeps the drain loop inside the 96 registers
    // a 576-thread CTA leaves
    constexpr int kChunk = 16;
    const bool vec_ok = ((p.N & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    int lt = 0;
    int cols_n0 = -1;  // column block the records in shared memory belong to
    const uint32_t leader_acc_empty[2] = {PAIR ? map_to_cta(&acc_empty[0], 0) : 0u, PAIR ? map_to_cta(&acc_empty[1], 0) : 0u};
    for (int t = walker; t < tiles; t += walkers, lt++) {
      const int m0 = (t % m_tiles) * kTileM + (int)rank * kBlockM, n0 = (t / m_tiles) * BLOCK_N;
      const int buf = lt & 1;
      // (1) per-column constants of this tile (the main loop of this or the next tile is running).
      // Tiles are numbered row-block fastest, so a CTA's consecutive tiles mostly share their
      // column block: the records are rebuilt only when it changes (all epilogue threads see the
      // same n0, so the barriers stay matched).
      if (n0 != cols_n0) {
        if (cols_n0 >= 0) asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");  // everyone is done with the old records
        cols_n0 = n0;
        static_assert(BLOCK_N <= kEpilogueThreads, "one column record per epilogue thread");
        const int j = n0 + et;
        ColParams cp = {0, 0, 0, 0};
        if (et < BLOCK_N && j < p.N) {
          if constexpr (MODE == 2) {  // {unused, column scale, float bias, weight offset}
            cp.scale = __float_as_int(p.col_scales ? p.col_scales[j] : p.u_col_scale);
            cp.shifts = __float_as_int(p.bias_f32[j]);
            cp.b_off = p.b_offsets ? p.b_offsets[j] : p.u_b_offset;
          } else {                    // {c, scale, pre | post << 8, weight offset}
            const ColQuant q = col_quant(p, j);
            int32_t term = 0;
            if (p.bias)
              term = scale32(load_bias(p, j) - (p.bias_offsets ? p.bias_offsets[j] : p.bias_offset), q.bias_pre, q.bias_post,
                             q.bias_scale, 0);
            const uint32_t corr = (uint32_t)term - (uint32_t)p.a_offset * (uint32_t)p.b_row_sums[j] +
                                  (uint32_t)p.k_corr * (uint32_t)p.a_offset * (uint32_t)q.b_off;
            cp.c = (int32_t)corr;
            cp.scale = q.out_scale;
            cp.shifts = q.out_pre | (q.out_post << 8);
            cp.b_off = q.b_off;
          }
        }
        if (et < BLOCK_N) cols[et] = cp;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");  // epilogue warps only
      }
      // (2) drain the accumulators of this tile
      const int row = m0 + quarter * 32 + lane;
      // All epilogue threads agree on the outcome of the (bounded) wait through a reducing
      // barrier, so either all of them drain the tile or all of them leave the loop.
      const uint32_t mine = mbar_wait(&acc_full[buf], (lt >> 1) & 1, abort_flag) ? 1u : 0u;
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\t"
          "setp.ne.u32 q, %1, 0;\n\t"
          "barrier.cta.red.and.pred p, 1, %2, q;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(mine), "n"(kEpilogueThreads)
          : "memory");
      tc_fence_after();
      if (!ok) break;
      GEMM_TRACE(4, lt == 0 && et == 0);
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * kAccCols;
      int out_index = row;  // row of the result this accumulator row becomes
      bool row_ok = row < p.M;
      if (p.conv_entries > 0 || p.conv_windows) {  // padded pixel -> (image, oh, ow); the halo rows are dropped
        const int img = row / p.conv_hpwp, rem = row - img * p.conv_hpwp;
        const int oh = rem / p.conv_wp, ow = rem - oh * p.conv_wp;
        row_ok = row_ok && oh < p.conv_oh && ow < p.conv_ow;
        out_index = (img * p.conv_oh + oh) * p.conv_ow + ow;
      }
      const int c_end = (col_group + 1) * kGroupCols < BLOCK_N ? (col_group + 1) * kGroupCols : BLOCK_N;
      if constexpr (MODE == 2) {
        // float(sum) * (row scale * column scale) + bias, each operation rounded on its own
        // (fwdDynRowwiseQuantizedFullyConnectedInstImpl, InterpreterNodes.cpp:4690-4702), then fp16.
        // One accumulator row per lane (the 32x32b shape), a 16-byte record per element.
        const int32_t a_sum = (p.a_row_sums && row < p.M) ? p.a_row_sums[row] : 0;
        const float row_scale = row < p.M ? p.row_scales[row] : 0.0f;
#pragma unroll 1
        for (int c0 = col_group * kGroupCols; c0 < c_end; c0 += kChunk) {
          uint32_t acc[kChunk];
          tmem_ld_32x32b_x16(lane_addr + (uint32_t)c0, acc);
          tmem_ld_wait();
          if (c0 + kChunk >= c_end) {
            // everything this warp needs from the buffer is in registers: hand it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) mbar_arrive_cluster(leader_acc_empty[buf]);
              else mbar_arrive(&acc_empty[buf]);
            }
          }
          uint32_t h2[kChunk / 2];
#pragma unroll
          for (int i2 = 0; i2 < kChunk / 2; i2++) {
            float f[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const int4 cp = *reinterpret_cast<const int4 *>(&cols[c0 + 2 * i2 + e]);
              const int32_t v = (int32_t)(acc[2 * i2 + e] - (uint32_t)cp.w * (uint32_t)a_sum);
              f[e] = __fadd_rn(__fmul_rn((float)v, __fmul_rn(row_scale, __int_as_float(cp.y))), __int_as_float(cp.z));
            }
            asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(h2[i2]) : "f"(f[1]), "f"(f[0]));
          }
          if (row_ok) {
            __half *orow = p.out_f16 + (size_t)row * p.N + n0 + c0;
            if (((p.N & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.out_f16) & 15) == 0) && n0 + c0 + kChunk <= p.N) {
#pragma unroll
              for (int v4 = 0; v4 < kChunk / 8; v4++)
                *reinterpret_cast<uint4 *>(orow + 8 * v4) = make_uint4(h2[4 * v4], h2[4 * v4 + 1], h2[4 * v4 + 2], h2[4 * v4 + 3]);
            } else {
              for (int i = 0; i < kChunk; i++)
                if (n0 + c0 + i < p.N) orow[i] = __ushort_as_half((unsigned short)((h2[i >> 1] >> (16 * (i & 1))) & 0xffffu));
            }
          }
        }
      } else {
        // The int8 result.  A column's record is 16 bytes, and shared memory delivers 128 bytes
        // per clock per SM whether the lanes of a load read one address or 32: with one accumulator
        // row per lane (the 32x32b shape) every element costs a 16-byte broadcast load, 4096 clocks
        // for a 128 x 256 tile and, measured, the whole duration of its drain.  The 16x256b shape
        // hands each lane two neighbouring columns of four rows per eight columns instead -- register
        // i of the load of rows 16h..16h+15 holds row 16h + lane/4 + 8*((i>>1)&1), column
        // 8*(i>>2) + 2*(lane%4) + (i&1) -- so a record is loaded once per four elements.
        // A lane then owns two bytes of a row, and a warp's stores would be scattered over 32
        // lines either way (16-byte stores by row took 6500 clocks per 128 x 256 tile): the tile
        // passes through shared memory, swizzled in 16-byte pieces so that neither the writes nor
        // the reads along rows meet in a bank, and leaves as whole rows.
        const int jq = lane & 3, r0 = lane >> 2;
        uint8_t *stage_q = out_stage + quarter * 32 * S::kOutPitch;
        int32_t a_sums[4] = {0, 0, 0, 0};
        if constexpr (MODE == 1) {
          if (p.a_row_sums) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const int rr = m0 + quarter * 32 + 8 * i + r0;
              a_sums[i] = rr < p.M ? p.a_row_sums[rr] : 0;
            }
          }
        }
        const int32_t relu_floor = p.act_type == 1 ? p.out_offset : INT32_MIN;
        asm volatile("bar.sync %0, 128;" ::"r"(2 + quarter) : "memory");  // the quarter has read the last tile back
#pragma unroll 1
        for (int c0 = col_group * kGroupCols; c0 < c_end; c0 += kChunk) {
          uint32_t acc[16];  // [row half h][column group g][row rr][column cc] -> 8h + 4g + 2rr + cc
          tmem_ld_16x256b_x2(lane_addr + (uint32_t)c0, &acc[0]);
          tmem_ld_16x256b_x2(lane_addr + (16u << 16) + (uint32_t)c0, &acc[8]);
          tmem_ld_wait();
          GEMM_TRACE(7, lt == 0 && et == 0 && c0 == 0);
          if (c0 + kChunk >= c_end) {
            // everything this warp needs from the buffer is in registers: hand it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) mbar_arrive_cluster(leader_acc_empty[buf]);
              else mbar_arrive(&acc_empty[buf]);
            }
          }
          // the requantisation: libjit_scale, ((v >> pre) * scale + rtn) >> post, then + offset, with
          // rtn = 1 << (post - 1) (0 for post 0); Relu is max(x, out_offset), no activation max(x, INT_MIN)
#pragma unroll
          for (int g = 0; g < 2; g++) {
            int32_t res[2][4];  // [cc][row 8*i + r0 of the quarter]
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
              const int4 cp = *reinterpret_cast<const int4 *>(&cols[c0 + 8 * g + 2 * jq + cc]);
              const int32_t pre = cp.z & 0xff, post = cp.z >> 8;
              const uint32_t rtn = (1u << post) >> 1;
#pragma unroll
              for (int i = 0; i < 4; i++) {  // i = 2h + rr
                uint32_t v = acc[8 * (i >> 1) + 4 * g + 2 * (i & 1) + cc] + (uint32_t)cp.x;
                if constexpr (MODE == 1) v -= (uint32_t)cp.w * (uint32_t)a_sums[i];  // 0 when no row sums take part
                const int32_t m = (int32_t)((uint32_t)((int32_t)v >> pre) * (uint32_t)cp.y + rtn);
                // max((m >> post) + offset, floor) in one instruction (a wrapping add, like the two it replaces)
                int32_t x = __viaddmax_s32(m >> post, p.out_offset, relu_floor);
                if constexpr (MODE == 1) {
                  if (p.act_type > 1) x = activation_i32(x, p);
                }
                res[cc][i] = x;
              }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
              uint32_t two;  // sat8(column cc = 1) << 8 | sat8(column cc = 0): libjit_clip_i8 and the packing in one
              asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(two) : "r"(res[1][i]), "r"(res[0][i]), "r"(0));
              const int col = c0 + 8 * g + 2 * jq;
              *reinterpret_cast<uint16_t *>(stage_q + stage_offset<S::kOutPitch>(8 * i + r0, col >> 4) + (col & 15)) = (uint16_t)two;
            }
          }
          GEMM_TRACE(9, lt == 0 && et == 0 && c0 == 0);
        }
        constexpr int kRowPieces = S::kOutPitch / 16;
        if (col_group == 0) out_rows[quarter * 32 + lane] = row_ok ? out_index : -1;
        asm volatile("bar.sync %0, 128;" ::"r"(2 + quarter) : "memory");  // the quarter's 32 rows are complete
        const bool whole = vec_ok && n0 + BLOCK_N <= p.N;
#pragma unroll
        for (int piece = col_group * 32 + lane; piece < 32 * kRowPieces; piece += 128) {
          const int r = piece / kRowPieces, q16 = piece % kRowPieces;
          const int dst = out_rows[quarter * 32 + r];
          if (q16 * 16 >= BLOCK_N || dst < 0) continue;
          const uint4 v = *reinterpret_cast<const uint4 *>(stage_q + stage_offset<S::kOutPitch>(r, q16));
          int8_t *o = p.out + (size_t)dst * p.N + n0 + q16 * 16;
          if (whole) {
            *reinterpret_cast<uint4 *>(o) = v;
          } else {
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int b = 0; b < 16; b++)
              if (n0 + q16 * 16 + b < p.N) o[b] = (int8_t)((w4[b >> 2] >> (8 * (b & 3))) & 0xff);
          }
        }
      }

      GEMM_TRACE(5, lt == 0 && et == 0);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up.  Report it, then give copies that may still be in flight towards this
    // CTA's shared memory a bounded time to land before the CTA retires.
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, GLOWB200_STATUS_WAIT_TIMEOUT);
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000ll) {
    }
    __syncthreads();
  }
  if constexpr (PAIR) cluster_sync();  // neither CTA leaves while its partner may still read its tiles or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
  GEMM_TRACE(6, threadIdx.x == 32);
}

// ---------------------------------------------------------------------------------------
// Row sums of an int8 matrix [rows, K] -> int32 [rows]   (one warp per row, dp4a)
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) i8_row_sums_kernel(const int8_t *__restrict__ x, int rows, int K, int32_t *__restrict__ out) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int8_t *r = x + (size_t)row * K;
  int32_t acc = 0;
  if ((K & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    for (int k = lane * 16; k < K; k += 512) {
      const int4 v = *reinterpret_cast<const int4 *>(r + k);
      acc = __dp4a(v.x, 0x01010101, acc);
      acc = __dp4a(v.y, 0x01010101, acc);
      acc = __dp4a(v.z, 0x01010101, acc);
      acc = __dp4a(v.w, 0x01010101, acc);
    }
  } else {
    for (int k = lane; k < K; k += 32) acc += r[k];
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) out[row] = acc;
}

// ---------------------------------------------------------------------------------------
// Any-shape contraction (K not a multiple of 16, unaligned pointers): one thread per output,
// the reference's loop as written.  Also the cross-check of the tensor-core kernel in tests.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) i8_gemm_requant_any_kernel(const int8_t *__restrict__ a, const int8_t *__restrict__ b,
                                                                   const __grid_constant__ GemmParams p) {
  const int j = blockIdx.x * 16 + (threadIdx.x & 15), i = blockIdx.y * 16 + (threadIdx.x >> 4);
  if (i >= p.M || j >= p.N) return;
  const ColQuant q = col_quant(p, j);
  uint32_t sum = 0;
  for (int k = 0; k < p.k_corr; k++)
    sum += (uint32_t)(((int32_t)b[(size_t)j * p.K + k] - q.b_off) * ((int32_t)a[(size_t)i * p.K + k] - p.a_offset));
  if (p.bias)
    sum += (uint32_t)scale32(load_bias(p, j) - (p.bias_offsets ? p.bias_offsets[j] : p.bias_offset), q.bias_pre, q.bias_post,
                             q.bias_scale, 0);
  p.out[(size_t)i * p.N + j] =
      (int8_t)clip_i8(activation_i32(scale32((int32_t)sum, q.out_pre, q.out_post, q.out_scale, p.out_offset), p));
}

// The floating-point result (GemmParams::float_out) for any shape: b element (j, k) sits at
// b[j * b_stride_j + k * b_stride_k], so both the [N, K] and the [K, N] form of the weights serve.
__global__ void __launch_bounds__(256) i8_gemm_float_any_kernel(const int8_t *__restrict__ a, const int8_t *__restrict__ b,
                                                                 int64_t b_stride_j, int64_t b_stride_k,
                                                                 const __grid_constant__ GemmParams p) {
  const int j = blockIdx.x * 16 + (threadIdx.x & 15), i = blockIdx.y * 16 + (threadIdx.x >> 4);
  if (i >= p.M || j >= p.N) return;
  const int32_t b_off = p.b_offsets ? p.b_offsets[j] : p.u_b_offset;
  uint32_t sum = 0;
  for (int k = 0; k < p.k_corr; k++)
    sum += (uint32_t)(((int32_t)b[j * b_stride_j + k * b_stride_k] - b_off) * (int32_t)a[(size_t)i * p.K + k]);
  const float mm = __fmul_rn(p.row_scales[i], p.col_scales ? p.col_scales[j] : p.u_col_scale);
  p.out_f16[(size_t)i * p.N + j] = __float2half_rn(__fadd_rn(__fmul_rn((float)(int32_t)sum, mm), p.bias_f32[j]));
}

// [R, C] int8 -> [C, R] int8 (32x32 tiles through shared memory)
__global__ void __launch_bounds__(256) i8_transpose_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int R, int C) {
  __shared__ int8_t tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int y = threadIdx.y; y < 32; y += 8) {
    const int r = r0 + y, c = c0 + threadIdx.x;
    tile[y][threadIdx.x] = (r < R && c < C) ? in[(size_t)r * C + c] : (int8_t)0;
  }
  __syncthreads();
  for (int y = threadIdx.y; y < 32; y += 8) {
    const int c = c0 + y, r = r0 + threadIdx.x;
    if (c < C && r < R) out[(size_t)c * R + r] = tile[threadIdx.x][y];
  }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// int8 [rows, K] row-major -> 2-D map with a {128 bytes of K, box_rows} box, 128-byte swizzle;
// out-of-range elements read as zero.
// [rows, extent] bytes with `pitch` bytes between rows (pitch < extent: rows overlap, a sliding window)
int make_map(CUtensorMap *map, const void *base, int rows, int extent, int box_rows, int pitch);
int make_map(CUtensorMap *map, const void *base, int rows, int K, int box_rows) { return make_map(map, base, rows, K, box_rows, K); }
int make_map(CUtensorMap *map, const void *base, int rows, int K, int box_rows, int pitch) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return set_error(GLOWB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch};
  cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(GLOWB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return GLOWB200_OK;
}

template <int BLOCK_N, int STAGES, int MODE>
int launch_tile_mode(const CUtensorMap &ma, const CUtensorMap &mb, const GemmParams &p, cudaStream_t s) {
  using S = GemmSmem<BLOCK_N, STAGES>;
  // per device and cheap: set on every launch rather than tracked
  GLOWB200_CUDA_OK(cudaFuncSetAttribute(i8_gemm_requant_kernel<BLOCK_N, STAGES, MODE>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
  const int tiles = ((p.N + BLOCK_N - 1) / BLOCK_N) * ((p.M + kBlockM - 1) / kBlockM);
  const int sms = sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles < sms ? tiles : sms));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see pdl_wait() in the kernel
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  GLOWB200_CUDA_OK(cudaLaunchKernelEx(&cfg, i8_gemm_requant_kernel<BLOCK_N, STAGES, MODE>, ma, mb, p));
  return GLOWB200_OK;
}

// CTA pairs of the int8 kernel that fit the device at once (0: not asked yet).  The kernels' shapes differ
// only in shared memory, of which every one takes more than half an SM: one number serves them all.
int &resident_pairs() {
  static int n = 0;
  return n;
}

// The same for clusters of two CTAs walking 256-row tiles (int8 results only).
template <int BLOCK_N, int STAGES>
int launch_pair_kernel(const CUtensorMap &ma, const CUtensorMap &mb, const GemmParams &p, cudaStream_t s) {
  using S = GemmSmem<BLOCK_N, STAGES, 1>;
  const bool plain = p.a_row_sums == nullptr && p.act_type <= 1;
  auto kernel = plain ? i8_gemm_requant_kernel<BLOCK_N, STAGES, 0, 1> : i8_gemm_requant_kernel<BLOCK_N, STAGES, 1, 1>;
  GLOWB200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
  const int tiles = ((p.N + BLOCK_N - 1) / BLOCK_N) * ((p.M + 2 * kBlockM - 1) / (2 * kBlockM));
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // Pairs that can be resident at once: the kernel is persistent, so a pair that had to wait for
  // another to retire would start its tiles a whole kernel late.
  int pairs = resident_pairs();
  if (pairs <= 0) {
    cfg.gridDim = dim3(2u * (unsigned)(sm_count() / 2));
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) n = sm_count() / 2;
    pairs = n < sm_count() / 2 ? n : sm_count() / 2;
    resident_pairs() = pairs;
  }
  cfg.gridDim = dim3(2u * (unsigned)(tiles < pairs ? tiles : pairs));
  GLOWB200_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, ma, mb, p));
  return GLOWB200_OK;
}

template <int BLOCK_N, int STAGES>
int launch_tile_kernel(const CUtensorMap &ma, const CUtensorMap &mb, const GemmParams &p, cudaStream_t s) {
  if (p.float_out) return launch_tile_mode<BLOCK_N, STAGES, 2>(ma, mb, p, s);
  if (p.a_row_sums == nullptr && p.act_type <= 1) return launch_tile_mode<BLOCK_N, STAGES, 0>(ma, mb, p, s);
  return launch_tile_mode<BLOCK_N, STAGES, 1>(ma, mb, p, s);
}

bool ptr16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

#ifndef GLOWB200_GEMM_TILE_240
#define GLOWB200_GEMM_TILE_240 1
#endif
// Columns of an output tile.  64 for narrow results; 128 when 256-column tiles would leave half
// a tile (or more) of padding; else 256 -- unless 240-column tiles finish in fewer, or as many
// but narrower, rounds over the SMs: 2048 x 4096 is 256 tiles of 256 columns (two rounds on 148
// SMs, the second 73 % full) but 288 tiles of 240 (two rounds, 6 % shorter each).
// A product with few rows (a batch-sharded layer: 512 x 1024 is 20 tiles of 240 columns on 148
// SMs) takes narrower tiles until at least half of the SMs have one: the k loop of a tile is a
// chain of load and MMA latencies that narrower tiles run side by side.
int pick_block_n(int M, int N) {
  if (N <= 64) return 64;
  const long sms = sm_count(), m_tiles = (M + kBlockM - 1) / kBlockM;
  auto tiles = [&](long bn) { return m_tiles * ((N + bn - 1) / bn); };
  int bn = 256;
  if (((N + 127) / 128) & 1) {
    bn = 128;
  } else {
#if GLOWB200_GEMM_TILE_240
    auto cost = [&](long b) { return ((tiles(b) + sms - 1) / sms) * (b + 16); };
    if (cost(240) * 100 < cost(256) * 97) bn = 240;
#endif
  }
  if (bn > 128 && tiles(bn) * 2 <= sms) bn = 128;
  if (bn == 128 && tiles(128) * 2 <= sms) bn = 64;
  return bn;
}

// Tile shape of a product: the columns pick_block_n chooses, walked by single CTAs.  CTA pairs are
// an option the environment switches on (GLOWB200_GEMM_PAIR = 1: 240-column tiles, 2: 256-column
// tiles; int8 results of 256 rows or more): measured on 2048 x 4096 x 4096 a pair kernel took
// 32.1 - 33.5 us against 31.5 us for single CTAs.  Both main loops ran near 600 clocks per k-block
// (480 is the MMAs' own time) at an SM clock of 1.65 - 1.69 GHz instead of 1.965: with random int8
// operands the GPU sits at its power limit, and the pair's smaller operand traffic bought nothing
// that its cross-SM signalling did not cost.
struct TilePick { int bn, pair; };
TilePick pick_tile(int M, int N, bool allow_pair) {
  TilePick t{pick_block_n(M, N), 0};
  if (!allow_pair || N < 240 || M < 2 * kBlockM || sm_count() < 2) return t;
  if (const char *e = getenv("GLOWB200_GEMM_PAIR")) {
    if (e[0] == '1') t = {240, 1};
    if (e[0] == '2') t = {256, 1};
  }
  return t;
}

// `windows` 32-byte windows as a plain [windows, 32] matrix; a box is the same window of 128
// consecutive pixels, in the 32-byte swizzle the MMA descriptor of such a tile names.
int make_window_map(CUtensorMap *map, const void *base, int64_t windows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return set_error(GLOWB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {32, (cuuint64_t)windows};
  cuuint64_t strides[1] = {32};
  cuuint32_t box[2] = {32, (cuuint32_t)kBlockM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(GLOWB200_ERR_CUDA, "cuTensorMapEncodeTiled (row windows) failed with CUresult %d", (int)r);
  return GLOWB200_OK;
}

int launch_for_block_n(TilePick tile, const void *a, int a_rows, int a_extent, int a_pitch, const void *b, const GemmParams &p,
                       cudaStream_t s, const CUtensorMap *a_map = nullptr) {
  const int bn = tile.bn;
  CUtensorMap ma, mb;
  if (a_map) ma = *a_map;
  else if (int rc = make_map(&ma, a, a_rows, a_extent, kBlockM, a_pitch)) return rc;
  if (int rc = make_map(&mb, b, p.N, p.K, tile.pair ? bn / 2 : bn)) return rc;
  if (tile.pair) {
    if (bn == 240) return launch_pair_kernel<240, 6>(ma, mb, p, s);
    return launch_pair_kernel<256, 5>(ma, mb, p, s);
  }
  switch (bn) {
    case 64: return launch_tile_kernel<64, 6>(ma, mb, p, s);
    case 128: return launch_tile_kernel<128, 6>(ma, mb, p, s);
    case 240: return launch_tile_kernel<240, 4>(ma, mb, p, s);
    default: return launch_tile_kernel<256, 3>(ma, mb, p, s);  // (a fourth stage would leave no room for the result's staging area)
  }
}

// Runs out = requant(A[M,K] x B[N,K]^T ...) choosing the tensor-core or the any-shape kernel.
// `ws` holds b_row_sums (when not supplied) and a_row_sums (when needed).
}  // namespace

int run_gemm_shifted_rows(GemmParams p, const int8_t *padded, int64_t rows, int C, const int8_t *b,
                          const int32_t *b_row_sums, cudaStream_t s, int64_t buffer_rows) {
  if (buffer_rows < rows) buffer_rows = rows;
  GLOWB200_REQUIRE(rows > 0 && buffer_rows < (1ll << 31) && (C == 64 || C % 128 == 0) && p.K % kBlockK == 0 && p.conv_entries > 0 &&
                       p.conv_entries <= 32 && ptr16(padded) && ptr16(b) && b_row_sums != nullptr,
                   "shifted-rows convolution: unsupported shape");
  p.M = (int)rows;
  p.b_row_sums = b_row_sums;
  p.a_row_sums = nullptr;
  if (p.k_corr == 0) p.k_corr = p.K;
  // C = 64: a 128-byte window over two neighbouring pixels, sliding by one pixel per row
  return launch_for_block_n(pick_tile(p.M, p.N, false), padded, (int)buffer_rows, C == 64 ? 128 : C, C, b, p, s);
}

int run_gemm_row_windows(GemmParams p, const int8_t *planes, int64_t rows, int ow, const int8_t *b, const int32_t *b_row_sums,
                         cudaStream_t s) {
  GLOWB200_REQUIRE(rows > 0 && 2 * rows + 3 * (int64_t)ow < (1ll << 31) && ow > 0 && p.K == 2 * kBlockK && ptr16(planes) &&
                       ptr16(b) && b_row_sums != nullptr,
                   "row-window convolution: unsupported shape");
  p.M = (int)rows;
  p.conv_windows = (int)rows;  // windows per plane: plane e starts at window e * rows
  p.conv_wp = ow;
  p.b_row_sums = b_row_sums;
  p.a_row_sums = nullptr;
  if (p.k_corr == 0) p.k_corr = p.K;
  CUtensorMap ma;
  if (int rc = make_window_map(&ma, planes, 2 * rows + 3 * (int64_t)ow + 1)) return rc;
  return launch_for_block_n(pick_tile(p.M, p.N, false), nullptr, 0, 0, 0, b, p, s, &ma);
}

int run_gemm(GemmParams p, const int8_t *a, const int8_t *b, const int32_t *b_row_sums_in, bool b_offsets_zero,
             int force_any, void *ws, size_t ws_bytes, cudaStream_t s) {
  if (p.M == 0 || p.N == 0) return GLOWB200_OK;
  if (p.k_corr == 0) p.k_corr = p.K;
  const bool tc = !force_any && p.K > 0 && (p.K % 16) == 0 && ptr16(a) && ptr16(b);
  if (!tc) {
    dim3 grid((p.N + 15) / 16, (p.M + 15) / 16);
    if (p.float_out) i8_gemm_float_any_kernel<<<grid, 256, 0, s>>>(a, b, p.K, 1, p);
    else i8_gemm_requant_any_kernel<<<grid, 256, 0, s>>>(a, b, p);
    GLOWB200_CUDA_OK(cudaGetLastError());
    return GLOWB200_OK;
  }
  const size_t need = align_up((size_t)p.N * 4, 256) + align_up((size_t)p.M * 4, 256);
  if (ws == nullptr || ws_bytes < need)
    return set_error(GLOWB200_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", ws_bytes, need);
  int32_t *bs = reinterpret_cast<int32_t *>(ws);
  int32_t *as = reinterpret_cast<int32_t *>(reinterpret_cast<uint8_t *>(ws) + align_up((size_t)p.N * 4, 256));
  if (b_row_sums_in || p.float_out) {  // (the float result has no input offset: the sums are never read)
    p.b_row_sums = b_row_sums_in;
  } else {
    i8_row_sums_kernel<<<(p.N + 7) / 8, 256, 0, s>>>(b, p.N, p.K, bs);
    GLOWB200_CUDA_OK(cudaGetLastError());
    p.b_row_sums = bs;
  }
  if (p.float_out) {
    if (b_offsets_zero) p.a_row_sums = nullptr;  // else the caller's, written while it quantized the rows
  } else if (!b_offsets_zero) {
    i8_row_sums_kernel<<<(p.M + 7) / 8, 256, 0, s>>>(a, p.M, p.K, as);
    GLOWB200_CUDA_OK(cudaGetLastError());
    p.a_row_sums = as;
  } else {
    p.a_row_sums = nullptr;
  }
  return launch_for_block_n(pick_tile(p.M, p.N, !p.float_out), a, p.M, p.K, p.K, b, p, s);
}

int run_gemm_float_any(const GemmParams &p, const int8_t *a, const int8_t *b_kn, cudaStream_t s) {
  if (p.M == 0 || p.N == 0) return GLOWB200_OK;
  dim3 grid((p.N + 15) / 16, (p.M + 15) / 16);
  i8_gemm_float_any_kernel<<<grid, 256, 0, s>>>(a, b_kn, 1, p.N, p);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

int transpose_i8(const int8_t *in_rc, int8_t *out_cr, int R, int C, cudaStream_t s) {
  if (R == 0 || C == 0) return GLOWB200_OK;
  dim3 grid((C + 31) / 32, (R + 31) / 32), block(32, 8);
  i8_transpose_kernel<<<grid, block, 0, s>>>(in_rc, out_cr, R, C);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

namespace {
int check_dims(int64_t M, int64_t K, int64_t N) {
  GLOWB200_REQUIRE(M >= 0 && N >= 0 && K >= 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 24),
                   "matrix dimensions out of range");
  return GLOWB200_OK;
}

}  // namespace
}  // namespace glowb200

using namespace glowb200;

#ifdef GLOWB200_GEMM_TRACE
extern "C" int glowb200_debug_gemm_trace(unsigned long long *host512) {
  return cudaMemcpyFromSymbol(host512, glowb200::g_gemm_trace, 512 * sizeof(unsigned long long)) == cudaSuccess ? 0 : 4;
}
#endif

extern "C" size_t glowb200_i8_gemm_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  if (M < 0 || N < 0 || K < 0) return 0;
  // row sums of both operands + room for a transposed copy of a [K, N] right-hand side
  return align_up((size_t)N * 4, 256) + align_up((size_t)M * 4, 256) + align_up((size_t)N * (size_t)K, 256);
}

extern "C" int glowb200_i8_mma_issue_probe(int64_t mmas_per_sm, int64_t *ops_per_launch, int32_t *status,
                                           glowb200_stream_t stream) {
  GLOWB200_REQUIRE(mmas_per_sm > 0 && mmas_per_sm <= (1 << 24), "mmas_per_sm must be in (0, 2^24]");
  const int sms = sm_count();
  const int smem = (kBlockM + 256) * kBlockK + 1024;
  GLOWB200_CUDA_OK(cudaFuncSetAttribute(i8_mma_issue_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  i8_mma_issue_probe_kernel<<<sms, 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>((int)mmas_per_sm, status);
  GLOWB200_CUDA_OK(cudaGetLastError());
  if (ops_per_launch) *ops_per_launch = (int64_t)sms * mmas_per_sm * 2 * kBlockM * 256 * kUmmaK;
  return GLOWB200_OK;
}

extern "C" int glowb200_wait_limit_selftest(int64_t limit_cycles, int32_t *status, int32_t *waiters_that_gave_up,
                                            glowb200_stream_t stream) {
  GLOWB200_REQUIRE(limit_cycles > 0 && limit_cycles <= 100000000ll, "limit_cycles must be in (0, 1e8]");
  GLOWB200_REQUIRE(waiters_that_gave_up != nullptr, "NULL pointer");
  wait_limit_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(limit_cycles, status, waiters_that_gave_up);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

extern "C" int glowb200_i8_row_sums(const int8_t *matrix, int64_t rows, int64_t K, int32_t *sums, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(rows >= 0 && K >= 0 && rows < (1ll << 31) && K < (1ll << 31), "bad dimensions");
  if (rows == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(matrix && sums, "NULL pointer");
  i8_row_sums_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(matrix, (int)rows, (int)K, sums);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

extern "C" int glowb200_rowwise_quantized_fc_i8_i32(
    int8_t *out, const int8_t *in, const int8_t *weights, const int32_t *bias, const int32_t *weights_offsets,
    const int32_t *bias_pre, const int32_t *bias_post, const int32_t *bias_scale, const int32_t *out_pre,
    const int32_t *out_post, const int32_t *out_scale, int64_t M, int64_t K, int64_t N, int32_t out_offset,
    int32_t in_offset, int32_t bias_offset, const int32_t *weights_row_sums, int flags, void *workspace,
    size_t workspace_bytes, int32_t *status, glowb200_stream_t stream) {
  if (int rc = check_dims(M, K, N)) return rc;
  if (M == 0 || N == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(out && in && weights && bias && weights_offsets && bias_pre && bias_post && bias_scale && out_pre &&
                       out_post && out_scale, "NULL tensor pointer");
  GemmParams p{};
  p.out = out;
  p.bias = bias;
  p.b_offsets = weights_offsets;
  p.bias_pre = bias_pre; p.bias_post = bias_post; p.bias_scale = bias_scale;
  p.out_pre = out_pre; p.out_post = out_post; p.out_scale = out_scale;
  p.status = status;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.uniform = 0;
  p.a_offset = in_offset; p.bias_offset = bias_offset; p.out_offset = out_offset;
  p.act_type = (flags & GLOWB200_FC_FUSE_RELU) ? 1 : 0;
  p.bias_is_i8 = (flags & GLOWB200_FC_BIAS_INT8) ? 1 : 0;
  return run_gemm(p, in, weights, weights_row_sums, (flags & GLOWB200_FC_WEIGHT_OFFSETS_ZERO) != 0,
                  (flags & GLOWB200_FC_FORCE_ANY_SHAPE_KERNEL) != 0, workspace, workspace_bytes,
                  reinterpret_cast<cudaStream_t>(stream));
}

namespace {
// Shared tail of the two per-tensor entry points, whose right-hand side is [K, N]: transposes it
// into the workspace (unless the caller already holds the [N, K] form) and runs the contraction
// with every per-column array read at stride 0.
int run_per_tensor(GemmParams p, const int8_t *lhs, const int8_t *rhs_kn, const int8_t *rhs_nk, int flags, void *workspace,
                   size_t workspace_bytes, cudaStream_t s) {
  const size_t sums = align_up((size_t)p.N * 4, 256) + align_up((size_t)p.M * 4, 256);
  const int8_t *b = rhs_nk;
  if (b == nullptr) {
    const size_t need = sums + align_up((size_t)p.N * (size_t)p.K, 256);
    if (workspace == nullptr || workspace_bytes < need)
      return set_error(GLOWB200_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
    int8_t *t = reinterpret_cast<int8_t *>(workspace) + sums;
    if (p.K > 0) {
      dim3 grid((p.N + 31) / 32, (p.K + 31) / 32), block(32, 8);
      i8_transpose_kernel<<<grid, block, 0, s>>>(rhs_kn, t, p.K, p.N);
      GLOWB200_CUDA_OK(cudaGetLastError());
    }
    b = t;
  }
  return run_gemm(p, lhs, b, nullptr, (flags & GLOWB200_FC_WEIGHT_OFFSETS_ZERO) != 0,
                  (flags & GLOWB200_FC_FORCE_ANY_SHAPE_KERNEL) != 0, workspace, workspace_bytes, s);
}
}  // namespace

extern "C" int glowb200_fc_i8_i32(int8_t *out, const int8_t *in, const int8_t *weights, const int32_t *bias, int64_t M,
                                  int64_t K, int64_t N, int32_t out_offset, int32_t in_offset, int32_t weights_offset,
                                  int32_t bias_offset, int32_t bias_pre, int32_t bias_post, int32_t bias_scale,
                                  int32_t out_pre, int32_t out_post, int32_t out_scale,
                                  const int8_t *weights_transposed, int flags, void *workspace,
                                  size_t workspace_bytes, int32_t *status, glowb200_stream_t stream) {
  if (int rc = check_dims(M, K, N)) return rc;
  if (M == 0 || N == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(out && in && (weights || weights_transposed) && bias, "NULL tensor pointer");
  GemmParams p{};
  p.out = out;
  p.bias = bias;
  p.status = status;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.a_offset = in_offset; p.bias_offset = bias_offset; p.out_offset = out_offset;
  p.uniform = 1;
  p.u_b_offset = weights_offset;
  p.u_bias_pre = bias_pre; p.u_bias_post = bias_post; p.u_bias_scale = bias_scale;
  p.u_out_pre = out_pre; p.u_out_post = out_post; p.u_out_scale = out_scale;
  p.bias_is_i8 = (flags & GLOWB200_FC_BIAS_INT8) ? 1 : 0;
  if (weights_offset == 0) flags |= GLOWB200_FC_WEIGHT_OFFSETS_ZERO;
  return run_per_tensor(p, in, weights, weights_transposed, flags, workspace, workspace_bytes,
                        reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int glowb200_matmul_i8(int8_t *out, const int8_t *lhs, const int8_t *rhs, int64_t M, int64_t K, int64_t N,
                                  int32_t out_offset, int32_t lhs_offset, int32_t rhs_offset, int32_t out_pre,
                                  int32_t out_post, int32_t out_scale, int flags, void *workspace,
                                  size_t workspace_bytes, int32_t *status, glowb200_stream_t stream) {
  if (int rc = check_dims(M, K, N)) return rc;
  if (M == 0 || N == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(out && lhs && rhs, "NULL tensor pointer");
  GemmParams p{};
  p.out = out;
  p.bias = nullptr;
  p.status = status;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.a_offset = lhs_offset; p.bias_offset = 0; p.out_offset = out_offset;
  p.uniform = 1;
  p.u_b_offset = rhs_offset;
  p.u_out_pre = out_pre; p.u_out_post = out_post; p.u_out_scale = out_scale;
  if (rhs_offset == 0) flags |= GLOWB200_FC_WEIGHT_OFFSETS_ZERO;
  return run_per_tensor(p, lhs, rhs, nullptr, flags, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}
