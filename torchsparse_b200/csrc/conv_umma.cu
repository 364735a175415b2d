// Implicit-GEMM sparse convolution forward on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   Y[m, :] = sum_k  X[map[m][k], :] . W[k]      (fp16 / bf16 operands, or fp32 operands multiplied
//                                                  as TF32; fp32 accumulation in every case)
//
// A work item is a tile of 128 consecutive map rows times an N tile of at most 256 output channels.
// Its reduction runs over "K blocks": one kernel offset k times a group of 128-byte channel chunks
// (64 16-bit or 32 32-bit channels per chunk).  Which offsets a tile needs is given by a per-tile
// bit mask (tile_mask, built once per kernel map): offsets without a neighbour in the whole tile are
// never touched, so the issued work follows the sparsity of the map.  With a row-sorted map the rows
// of a tile share their neighbour pattern, the masks get sparse, and the output rows are scattered
// through reorder_loc.
//
// Operands of a K block (one pipeline stage; every chunk is a 128B-swizzled K-major tile):
//   A  128 gathered feature-row slices of 128 bytes per chunk (zeros for a missing neighbour), copied
//      by all eight gather warps with 16-byte cp.async, four rows per thread.  The four map entries
//      of an offset are read from global memory into registers one offset ahead (the map may be
//      row-major [rows][kvol] or column-major [kvol][rows]: the entry of (row, k) is at
//      map[row * rs + k * cs]), so the copies go out back to back once the stage is released; each
//      thread's arrival on the stage's "full" barrier is attached to its copies
//      (cp.async.mbarrier.arrive.noinc), so no thread ever blocks on data.  The channels may come from
//      two feature matrices (a channel concatenation that is never materialised).
//   B  one TMA tile copy per chunk of N_tile rows of the K-major packed weights, counted in bytes on
//      the same barrier.
//
// Roles (480 threads, persistent CTAs, one or two per SM):
//   warps 0-7   gather (A operand)
//   warps 8-11  epilogue: tcgen05.ld of their TMEM lane quarter, optional fp32 partial sum in/out,
//               scale / bias / residual / ReLU, rounding and 16-byte stores
//   warp 12     weight loader: one elected thread issues the TMA copies
//   warp 13     allocates TMEM; one elected thread issues tcgen05.mma (M=128, N=N_tile, 32 bytes of K
//               per instruction) and releases stages / publishes accumulators with tcgen05.commit
//   warp 14     scheduler: takes the CTA's next work item from a global counter (tiles differ in how
//               many offsets they hold, so a fixed assignment would leave CTAs idle at the end) when the
//               gather warps reach the last offset of the current item, and publishes (item, offset
//               mask) through a small ring
//
// Pair-list mode (the GatherScatter / FetchOnDemand dataflows, conv_pairs.cu): the map is one column of
// input rows, every 128-row tile belongs to one kernel offset (tile_k[tile] picks its weight block),
// and the fp32 products are either stored as rows of a buffer or added to the output rows with
// 16-byte atomic adds.
//
// The number of output rows may live in device memory (n_out_dev): then the host-side n_out is only
// an upper bound that sizes the grid, and a launch sequence can be replayed as a CUDA graph for
// inputs of any size up to that bound.
//
// Every wait on an mbarrier is bounded: when it runs out the thread records an error code and the
// CTA stops issuing work, gives its copies in flight time to land, frees its TMEM and returns.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "conv_dispatch.h"

namespace tsb {
namespace {

constexpr int kTileM = 128;
constexpr int kRowBytes = 128;              // bytes of K per stage row = one swizzle span
constexpr int kABytes = kTileM * kRowBytes; // 16 KiB
constexpr int kGatherWarps = 8;
constexpr int kGatherThreads = kGatherWarps * 32;
constexpr int kRowsPerPass = kGatherThreads / 8;   // rows covered by one copy of every gather thread (32)
constexpr int kCopies = kTileM / kRowsPerPass;     // copies per gather thread per K block (4)
constexpr int kEpilogueWarps = 4;      // warps 8..11: warp % 4 = TMEM lane quarter
constexpr int kThreads = 480;
// The TMA-gather variant keeps the role order with a gather group of four warps (one producer, three spares):
constexpr int kGatherWarpsTma = 4;
constexpr int kThreadsTma = (kGatherWarpsTma + kEpilogueWarps + 3) * 32;   // 352
constexpr int kRing = 4;               // scheduler ring: (work item, offset mask) published ahead of the other roles
constexpr int kMaxStages = 8;
constexpr int kMaxKvolUmma = 32;
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr uint64_t kWaitLimitNs = 2000000000ull;   // 2 s

enum { kErrFullWait = 1, kErrEmptyWait = 2, kErrAccWait = 3, kErrSchedWait = 4, kErrSplitWait = 5 };
enum { kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2 };

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait with a suspend-time hint: the thread is parked in hardware until the phase completes (it resumes at
// once then) or the hint runs out.  Without the hint a failed try comes back after ~100 cycles, and the dozen
// waiting roles of a CTA spend more issue slots on polling than the working roles get for their instructions.
constexpr uint32_t kSuspendHintNs = 1000000u;   // 1 ms
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ long long clk() {
  long long t;
  asm volatile("mov.u64 %0, %clock64;" : "=l"(t));
  return t;
}
// Debugging aid, compiled in only with -DTSB_TRACE_BUILD: per-block timestamps of one CTA.
// trace layout: [block][8] = {producer: at the block, after the empty wait, after issue; spare;
//                             mma: at the block, after the full wait, after commit; spare}
// (producer = thread 0 of the gather warps)
#ifdef TSB_TRACE_BUILD
#define TSB_TRACE_HOT(slot, it_)                                                                     \
  do {                                                                                               \
    if (p.trace && (int)blockIdx.x == p.trace_cta && (it_) < 256) p.trace[(it_) * 8 + (slot)] = clk(); \
  } while (0)
#else
#define TSB_TRACE_HOT(slot, it_) do { } while (0)
#endif
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: try_wait parks the thread in hardware instead of spinning on shared memory.  The
// wall clock is read only after the first 64 failed tries (reading it costs hundreds of cycles);
// the wait gives up kWaitLimitNs after that.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_test(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) return false;
    }
  }
  return false;
}
// one lane waits for the warp; the others are released by the shuffle
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int lane) {
  uint32_t ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity) ? 1u : 0u;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// true in exactly one lane of a converged warp (the same lane every time)
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM101_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL)
#define TSB_TCGEN05 1
#endif

__device__ __forceinline__ void tc_fence_before() {
#ifdef TSB_TCGEN05
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
#endif
}
__device__ __forceinline__ void tc_fence_after() {
#ifdef TSB_TCGEN05
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#endif
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
#ifdef TSB_TCGEN05
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
#endif
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
#ifdef TSB_TCGEN05
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
#endif
}
// D[tmem] (+)= A[smem] . B[smem]; kind::f16 for fp16 / bf16 operands, kind::tf32 for fp32 operands
template <bool TF32>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                     uint32_t accumulate) {
#ifdef TSB_TCGEN05
  if constexpr (TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
#endif
}
// arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
#ifdef TSB_TCGEN05
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
#endif
}
// issues the load of 16 consecutive accumulator columns of this warp's 32 lanes; tmem_ld_wait16 completes it
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
#ifdef TSB_TCGEN05
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
#endif
}
// Waits for the tcgen05.ld issued before it.  The loaded registers pass through the statement as
// in/out operands so that no use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&v)[16]) {
#ifdef TSB_TCGEN05
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                 "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
               :
               : "memory");
#endif
}

// instruction descriptor: D fp32, A/B format (0 fp16, 1 bf16, 2 tf32), both K-major, M = 128, N = n
__host__ __device__ inline uint32_t make_idesc(int ab_format, int n) {
  return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kTileM >> 4) << 24);
}

struct UmmaParams {
  const void* x;        // [n_in, c1]   channels [0, c1) of the input features
  const void* x2;       // nullable, [n_in, cin - c1]: channels [c1, cin) (a concatenation that is not materialised)
  const int* map;       // entry (row, k) at map[row * map_rs + k * map_cs]; null: row m reads input row m (kvol = 1)
  const unsigned* tile_mask;   // nullable, [tiles]: bit k set when some row of the tile has a neighbour at offset k
  const int4* items;    // nullable work-item table {row tile, offset mask, part | parts << 8 | first slot << 16, 0}: tiles
                        // with many offsets appear as several parts whose fp32 accumulators meet in split_scratch
  const int* n_items_dev;      // number of entries of `items` (device memory); n_items is its upper bound
  float* split_scratch;        // fp32 [slots][128][cout]: one slot per part of a split tile
  int* split_flags;            // [row tiles * N tiles], zero between launches: parts of the tile finished so far
  int n_items;
  const int* reorder;   // nullable
  void* y;              // [n_out, cout]
  const float* scale;   // nullable, fp32 [cout]: y = acc * scale + bias (+ residual), then ReLU
  const float* bias;    // nullable
  const void* residual; // nullable, [n_out, cout]
  const float* acc_in;  // nullable, fp32 [dst_rows, cout]: partial sums of earlier launches, added to the accumulator
  float* acc_out;       // nullable, fp32 [dst_rows, cout]: the accumulator (+ acc_in) is stored here, no epilogue
  const int* n_out_dev; // nullable: the number of output rows, read on the device (n_out is then its upper bound)
  int* error;           // device error word (0 = fine)
  int* sched;           // {next work item, CTAs finished}: both zero at launch, reset by the last CTA
  const int* tile_k;    // nullable ("pair list" mode): weight offset of each 128-row tile; the map is one column
  long long map_rs, map_cs;
  int c1;               // channels taken from x (= cin without x2)
  int dst_rows;         // rows of y (bound of the reorder scatter)
  int out_fp32;         // 16-bit operands, fp32 output rows (no residual)
  int atomic_out;       // fp32 output accumulated with atomic adds (rows may repeat between tiles)
#ifdef TSB_TRACE_BUILD
  long long* trace;     // debugging aid: per-block timestamps of one CTA
  int trace_cta;
#endif
  int n_in, n_out, kvol, cin, cout;
  unsigned k_range;     // bits of the kernel offsets this launch covers
  int n_tile;           // UMMA N of a full tile (multiple of 16, <= 256)
  int acc_cols;         // TMEM columns of one accumulator buffer (power of two >= n_tile, >= 32)
  int stages;
  int cpb;              // 128-byte channel chunks per K block (pipeline stage)
  int relu;
  int ab_format;        // kFmtF16 / kFmtBF16 / kFmtTF32
};

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2*>(&v));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}

// TMA tile load of a weight chunk: box = 128 bytes of channels x n_tile rows of the packed
// weights, written 128B-swizzled; completion is counted in bytes on the mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// TMA gather of four rows of a 2-D tensor (box = 128 bytes of columns x 1 row): the rows land one after the other,
// 128B-swizzled by their shared-memory address; a row index outside the tensor (-1: no neighbour) is filled with
// zeros and still counted in bytes on the mbarrier.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void* tmap, uint32_t bar, int col, int4 rows) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      :
      : "r"(dst), "l"(tmap), "r"(bar), "r"(col), "r"(rows.x), "r"(rows.y), "r"(rows.z), "r"(rows.w)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// Map entries are fetched one offset ahead of their use; as plain loads the compiler would sink them to
// the use and expose their latency, as volatile asm they are issued where they stand.
__device__ __forceinline__ int ld_map_entry(const int* p) {
  int v;
  asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ int4 ld_map_entry4(const int* p) {
  int4 v;
  asm volatile("ld.global.nc.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// The next (work item, offset mask) of the scheduler ring, read by lane 0 and handed to the whole warp; the
// slot is released at once (its two words now live in registers).  false: a bounded wait ran out.
__device__ __forceinline__ bool ring_take(uint64_t* s_full, uint64_t* s_empty, const int* s_tile, const uint32_t* s_kmask,
                                          const int* s_aux, int it, int lane, int& w, uint32_t& kmask, int& aux) {
  const int slot = it % kRing;
  int ww = -1, aa = 0;
  uint32_t mm = 0, ok = 1;
  if (lane == 0) {
    ok = mbar_wait(smem_u32(&s_full[slot]), (uint32_t)(it / kRing) & 1u) ? 1u : 0u;
    if (ok) {
      ww = s_tile[slot];
      mm = s_kmask[slot];
      aa = s_aux[slot];
      mbar_arrive(smem_u32(&s_empty[slot]));
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  w = __shfl_sync(0xffffffffu, ww, 0);
  kmask = __shfl_sync(0xffffffffu, mm, 0);
  aux = __shfl_sync(0xffffffffu, aa, 0);
  return ok != 0;
}

// Persistent kernel: each CTA takes (row tile, N tile) work items from a shared counter until none is left.
// Three rings decouple the roles so that the copies of the next tile are in flight while the
// current tile is multiplied and the previous one is written out:
//   stage ring      (p.stages)  A+B operands of one K block      full[] / empty[]
//   scheduler ring  (kRing)     work item + offset mask           sched_full[] / sched_empty[]
//   accumulator     (2)         TMEM column ranges                acc_full[] / acc_empty[]
template <typename T, bool kTma>
__global__ void __launch_bounds__(kTma ? kThreadsTma : kThreads, 2)
igemm_umma_kernel(const UmmaParams p, const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                  const __grid_constant__ CUtensorMap x2_map) {
  constexpr bool kTF32 = sizeof(T) == 4;
  constexpr int kGW = kTma ? kGatherWarpsTma : kGatherWarps;     // warps of the gather group
  constexpr int kTmaWarp = kGW + kEpilogueWarps, kMmaWarp = kTmaWarp + 1, kSchedWarp = kTmaWarp + 2;
  constexpr int kChunk = kRowBytes / (int)sizeof(T);     // channels per 128-byte chunk
  constexpr int kStepK = 32 / (int)sizeof(T);            // channels per MMA instruction (32 bytes of K)
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t s_full[kMaxStages];
  __shared__ uint64_t s_empty[kMaxStages];
  __shared__ uint64_t s_sched_full[kRing];
  __shared__ uint64_t s_sched_empty[kRing];
  __shared__ uint64_t s_acc_full[2];
  __shared__ uint64_t s_acc_empty[2];
  __shared__ uint64_t s_req;             // the gather warps ask the scheduler for the next work item
  __shared__ uint64_t s_epi;             // the four epilogue warps meet here around the count of a split tile's parts
  __shared__ volatile int s_split_last;  // this CTA counted the last part of the split tile at hand
  __shared__ uint32_t s_kmask[kRing];
  __shared__ int s_tile[kRing];          // row tile * N tiles + N tile of the ring slot; -1 = no more work
  __shared__ int s_aux[kRing];           // part | parts << 8 of a tile that is split into parts (0: whole tile)
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef TSB_TRACE_BUILD
  if (tid == 0) TSB_TRACE_HOT(7, 0);     // CTA entry
  if (tid == 0 && p.trace && blockIdx.x < 1024) p.trace[2048 + 2 * blockIdx.x] = (long long)global_ns();   // every CTA: wall clock
#endif
  const int b_bytes = p.n_tile * kRowBytes;              // one weight chunk
  const int stage_bytes = p.cpb * (kABytes + b_bytes);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t acc_cols = p.acc_cols;            // TMEM columns of one accumulator (power of two)
  // Channel chunks of a kernel offset.  cp.async gather: the concatenated channels cut every 128 bytes.  TMA gather:
  // the chunks of the first feature matrix, then those of the second (a box never spans both), the last chunk
  // of each possibly narrower; the weight columns of a chunk start where its channels start in the concatenation.
  const int chunks1 = kTma ? (p.c1 + kChunk - 1) / kChunk : 0;
  const int chunks = kTma ? chunks1 + (p.cin - p.c1 + kChunk - 1) / kChunk : (p.cin + kChunk - 1) / kChunk;
  const int groups = (chunks + p.cpb - 1) / p.cpb;       // K blocks per kernel offset
  // chunk c: first column inside its feature matrix, first weight column, MMA instructions (32 bytes of K each)
  auto chunk_geometry = [&](int c, int& col_src, int& col_w, int& steps) {
    if constexpr (kTma) {
      const bool second = c >= chunks1;
      col_src = (second ? c - chunks1 : c) * kChunk;
      col_w = second ? p.c1 + col_src : col_src;
      const int width = min(kChunk, (second ? p.cin - p.c1 : p.c1) - col_src);
      steps = (width + kStepK - 1) / kStepK;
    } else {
      col_src = col_w = c * kChunk;
      steps = (min(kChunk, p.cin - col_src) + kStepK - 1) / kStepK;
    }
  };

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      // every gather thread (attached to its copies) + the weight loader's arrive.expect_tx
      // TMA gather: the producer's and the weight loader's arrive.expect_tx
      mbar_init(smem_u32(&s_full[s]), kTma ? 2 : kGatherThreads + 1);
      mbar_init(smem_u32(&s_empty[s]), 1);   // tcgen05.commit
    }
    for (int b = 0; b < kRing; ++b) {
      mbar_init(smem_u32(&s_sched_full[b]), 1);
      // readers of a ring slot: gather warps, weight loader, MMA warp, epilogue warps
      mbar_init(smem_u32(&s_sched_empty[b]), (kTma ? 1 : kGatherWarps) + 2 + kEpilogueWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_acc_full[b]), 1);
      mbar_init(smem_u32(&s_acc_empty[b]), kEpilogueWarps);
    }
    mbar_init(smem_u32(&s_epi), kEpilogueWarps);
    mbar_init(smem_u32(&s_req), 1);
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) tmem_alloc(smem_u32(&s_tmem), 2 * acc_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  // rows of this launch: a device-side count (bounded by the host-side one that sized the grid) or the host's
  int n_out = p.n_out;
  if (p.n_out_dev) n_out = max(0, min(__ldg(p.n_out_dev), p.n_out));
  const int tiles_n = (p.cout + p.n_tile - 1) / p.n_tile;
  const int tiles_m = (n_out + kTileM - 1) / kTileM;
  int n_work = tiles_m * tiles_n;
  if (p.items) n_work = max(0, min(__ldg(p.n_items_dev), p.n_items)) * tiles_n;

  if (kTma && warp < kGW) {
    // ------------------------------------------------------------ TMA producer (A operand), warp 0 of the group
    // Lane l owns rows 4 l .. 4 l + 3 of the tile: it reads their four map entries (one 16-byte load from a
    // column-major map) one offset ahead and issues one gather4 copy per channel chunk; the copy engine fetches
    // the 128-byte row slices and writes zeros for a missing neighbour.  One warp instruction moves a whole
    // 16 KiB chunk, so the A operand costs the SM a handful of issue slots per K block.
    if (warp == 0) {
      const uint32_t full0 = smem_u32(&s_full[0]), empty0 = smem_u32(&s_empty[0]);
      const bool vec_map = p.map && p.map_rs == 1 && (p.map_cs & 3) == 0 && (reinterpret_cast<uintptr_t>(p.map) & 15) == 0;
      uint32_t stage = 0, phase = 0;
      bool first_pass = true, ok = true;
      int it = 0;
      uint32_t km = 0;
      int row0 = 0;
#ifdef TSB_TRACE_BUILD
      int blk = 0;
#endif
      auto next_offset = [&](int4& src) -> bool {
        while (km == 0) {
          int w, aux;
          uint32_t m;
          if (!ring_take(s_sched_full, s_sched_empty, s_tile, s_kmask, s_aux, it, lane, w, m, aux)) {
            if (lane == 0) atomicExch(p.error, kErrSchedWait);
            s_abort = 1;
            ok = false;
            return false;
          }
          ++it;
          if (w < 0 || s_abort) return false;
          row0 = (w / tiles_n) * kTileM;
          km = m;
          if (km == 0 && lane == 0) mbar_arrive(smem_u32(&s_req));   // nothing to copy for this item: ask for the next
        }
        const int k = __ffs(km) - 1;
        km &= km - 1;
        // the item's last offset is being fetched: ask the scheduler for the next item (see the cp.async variant)
        if (km == 0 && lane == 0) mbar_arrive(smem_u32(&s_req));
        const int r = row0 + 4 * lane;
        if (!p.map) {
          src = make_int4(r < n_out ? r : -1, r + 1 < n_out ? r + 1 : -1, r + 2 < n_out ? r + 2 : -1, r + 3 < n_out ? r + 3 : -1);
        } else if (vec_map) {
          src = ld_map_entry4(p.map + (long long)k * p.map_cs + r);
        } else {
          const int* e = p.map + (long long)r * p.map_rs + (long long)k * p.map_cs;
          src = make_int4(ld_map_entry(e), ld_map_entry(e + p.map_rs), ld_map_entry(e + 2 * p.map_rs), ld_map_entry(e + 3 * p.map_rs));
        }
        return true;
      };
      int4 src, nxt = make_int4(-1, -1, -1, -1);
      bool have = next_offset(src);
      while (have && ok) {
        const bool have_next = next_offset(nxt);       // in flight while this offset is copied
        if (!ok) break;
        for (int g = 0; g < groups && ok; ++g) {
          if (lane == 0) TSB_TRACE_HOT(0, blk);
          if (!first_pass && !mbar_wait_warp(empty0 + stage * 8, phase ^ 1u, lane)) {
            if (lane == 0) atomicExch(p.error, kErrEmptyWait);
            s_abort = 1;
            ok = false;
            break;
          }
          if (lane == 0) TSB_TRACE_HOT(1, blk);
          const int c_lo = g * p.cpb, c_hi = min(c_lo + p.cpb, chunks);
          const uint32_t bar = full0 + stage * 8;
          if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)((c_hi - c_lo) * kABytes));
          __syncwarp();
          const uint32_t a_dst = smem_base + stage * (uint32_t)stage_bytes + (uint32_t)lane * (4u * kRowBytes);
          for (int c = c_lo; c < c_hi; ++c) {
            int col_src, col_w, steps;
            chunk_geometry(c, col_src, col_w, steps);
            tma_gather4(a_dst + (uint32_t)(c - c_lo) * kABytes, c >= chunks1 ? &x2_map : &x_map, bar, col_src, src);
          }
          if (lane == 0) TSB_TRACE_HOT(2, blk);
#ifdef TSB_TRACE_BUILD
          ++blk;
#endif
          if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; first_pass = false; }
        }
        src = nxt;
        have = have_next;
      }
    }
  } else if (!kTma && warp < kGW) {
    // ------------------------------------------------------------ gather warps (A operand)
    // Thread t copies the 16-byte granule (t & 7) of rows (t >> 3) + 32 j, j = 0..3, of every chunk:
    // a warp instruction covers four whole 128-byte row slices.  The four map entries of an offset
    // are read one offset ahead and serve all channel chunks of that offset.
    constexpr int kGran = 16 / (int)sizeof(T);                     // channels per 16-byte granule
    const T* x1 = reinterpret_cast<const T*>(p.x);
    const T* x2 = reinterpret_cast<const T*>(p.x2);
    const int c2w = p.cin - p.c1;                                   // channels of x2
    const int gran = tid & 7;
    const int rbase = tid >> 3;
    const uint32_t dst_off = (uint32_t)rbase * kRowBytes + (uint32_t)((gran ^ (rbase & 7)) << 4);
    const uint32_t full0 = smem_u32(&s_full[0]), empty0 = smem_u32(&s_empty[0]);
    const int cin_mma = (p.cin + kStepK - 1) / kStepK * kStepK;     // K extent the MMAs read
    uint32_t stage = 0, phase = 0;      // stage of the current block; phase = parity of its use count
    bool first_pass = true;              // the first use of a stage needs no release
    bool ok = true;
    int it = 0;                          // work items taken from the ring so far
    uint32_t km = 0;                     // offsets of the current item not yet fetched
    int row0 = 0;
#ifdef TSB_TRACE_BUILD
    int blk = 0;
#endif
    // fetches the map entries of this thread's four rows for the next offset of the item stream
    auto next_offset = [&](int (&src)[kCopies]) -> bool {
      while (km == 0) {
        int w, aux;
        uint32_t m;
        if (!ring_take(s_sched_full, s_sched_empty, s_tile, s_kmask, s_aux, it, lane, w, m, aux)) {
          atomicExch(p.error, kErrSchedWait);
          s_abort = 1;
          ok = false;
          return false;
        }
        ++it;
        if (w < 0 || s_abort) return false;
        row0 = (w / tiles_n) * kTileM;
        km = m;
        if (km == 0 && tid == 0) mbar_arrive(smem_u32(&s_req));   // nothing to copy for this item: ask for the next
      }
      const int k = __ffs(km) - 1;
      km &= km - 1;
      // The item's last offset is now being fetched: time to ask the scheduler for the next item, so that it
      // arrives while the remaining copies of this one are issued.  Asking any earlier would let every CTA hold
      // several items from the start, and with a few items per CTA the dynamic assignment would balance nothing.
      // (Measured: asking two offsets earlier, or fetching map entries two offsets ahead, changes nothing.)
      if (km == 0 && tid == 0) mbar_arrive(smem_u32(&s_req));
#pragma unroll
      for (int j = 0; j < kCopies; ++j) {
        const int r = row0 + rbase + j * kRowsPerPass;
        if (p.map) src[j] = ld_map_entry(p.map + (long long)r * p.map_rs + (long long)k * p.map_cs);
        else src[j] = r < n_out ? r : -1;
      }
      return true;
    };
    int src[kCopies], nxt[kCopies];
    const uint32_t a_stage0 = smem_base + dst_off;     // this thread's first destination in stage 0
    uint32_t a_stage = a_stage0;
    bool have = next_offset(src);
    while (have && ok) {
      const bool have_next = next_offset(nxt);       // in flight while this offset is copied
      if (!ok) break;
      for (int g = 0; g < groups && ok; ++g) {
#ifdef TSB_TRACE_BUILD
        if (tid == 0) TSB_TRACE_HOT(0, blk);
#endif
        if (!first_pass && !mbar_wait_warp(empty0 + stage * 8, phase ^ 1u, lane)) {
          atomicExch(p.error, kErrEmptyWait);
          s_abort = 1;
          ok = false;
          break;
        }
#ifdef TSB_TRACE_BUILD
        if (tid == 0) TSB_TRACE_HOT(1, blk);
#endif
        for (int cc = 0; cc < p.cpb; ++cc) {
          const int c = g * p.cpb + cc;
          const int col = c * kChunk + gran * kGran;
          // granules beyond the K extent of the chunk's last MMA (Cin rounded up to one instruction's K) are
          // never read: their threads copy nothing; granules between Cin and that bound are zero-filled (the
          // weights there are zero, but stale shared memory could hold NaN patterns)
          if (col >= cin_mma) break;
          const bool col_ok = col < p.cin;                  // rows are 16-byte multiples: all-in or all-out
          const bool from2 = col >= p.c1;
          const T* xc = from2 ? x2 + (col - p.c1) : x1 + col;
          const int rstride = from2 ? c2w : p.c1;
          const uint32_t a_dst = a_stage + (uint32_t)cc * kABytes;
#pragma unroll
          for (int j = 0; j < kCopies; ++j) {
            const bool live = col_ok && (unsigned)src[j] < (unsigned)p.n_in;
            cp_async16(a_dst + (uint32_t)(j * kRowsPerPass) * kRowBytes,
                       live ? (const void*)(xc + (int64_t)src[j] * rstride) : (const void*)x1, live ? 16u : 0u);
          }
        }
        cp_async_arrive_noinc(full0 + stage * 8);
#ifdef TSB_TRACE_BUILD
        if (tid == 0) TSB_TRACE_HOT(2, blk);
        ++blk;
#endif
        a_stage += (uint32_t)stage_bytes;
        if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; first_pass = false; a_stage = a_stage0; }
      }
#pragma unroll
      for (int j = 0; j < kCopies; ++j) src[j] = nxt[j];
      have = have_next;
    }
    cp_async_wait_all();   // nothing of this thread may still be writing shared memory at exit
  } else if (warp < kGW + kEpilogueWarps) {
    // ------------------------------------------------------------ epilogue warps
    // warp q reads TMEM lanes 32 q .. 32 q + 31 = its 32 output rows, all columns of the tile
    const int quarter = warp & 3;
    T* y = reinterpret_cast<T*>(p.y);
    const T* res = reinterpret_cast<const T*>(p.residual);
    int acc_count = 0;   // tiles that used an accumulator so far (tiles with an empty mask use none)
    uint32_t epi_uses = 0;
    // all four epilogue warps have reached this point (bounded, like every other wait)
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_epi));
      const bool met = mbar_wait_warp(smem_u32(&s_epi), epi_uses & 1u, lane);
      ++epi_uses;
      return met;
    };
    // eight fp32 sums of row dst_row, channels nh .. nh + 7  ->  partial sums in / out, scale, bias, residual,
    // ReLU, one rounding, one 16-byte (or two, fp32) store
    auto emit8 = [&](float (&f)[8], int nh, int64_t dst_row) {
      if (p.acc_in) {    // partial sums of the launches that covered the other kernel offsets
        const float* ap = p.acc_in + dst_row * p.cout + nh;
        const float4 a = __ldg(reinterpret_cast<const float4*>(ap));
        const float4 b = __ldg(reinterpret_cast<const float4*>(ap) + 1);
        f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
        f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
      }
      if (p.acc_out) {   // this launch is not the last of its group: keep the sum in fp32
        float* ao = p.acc_out + dst_row * p.cout + nh;
        reinterpret_cast<float4*>(ao)[0] = make_float4(f[0], f[1], f[2], f[3]);
        reinterpret_cast<float4*>(ao)[1] = make_float4(f[4], f[5], f[6], f[7]);
        return;
      }
      if (p.scale) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p.scale + nh));
        const float4 b = __ldg(reinterpret_cast<const float4*>(p.scale + nh) + 1);
        f[0] *= a.x; f[1] *= a.y; f[2] *= a.z; f[3] *= a.w;
        f[4] *= b.x; f[5] *= b.y; f[6] *= b.z; f[7] *= b.w;
      }
      if (p.bias) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p.bias + nh));
        const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + nh) + 1);
        f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
        f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
      }
      if (kTF32 || p.out_fp32) {
        float* yo = reinterpret_cast<float*>(p.y) + dst_row * p.cout + nh;
        if (kTF32 && res) {
          const float* rp = reinterpret_cast<const float*>(res) + dst_row * p.cout + nh;
          const float4 ra = __ldg(reinterpret_cast<const float4*>(rp));
          const float4 rb = __ldg(reinterpret_cast<const float4*>(rp) + 1);
          f[0] += ra.x; f[1] += ra.y; f[2] += ra.z; f[3] += ra.w;
          f[4] += rb.x; f[5] += rb.y; f[6] += rb.z; f[7] += rb.w;
        }
        if (p.relu) {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = fmaxf(f[e], 0.f);
        }
        if (p.atomic_out) {
          atomicAdd(reinterpret_cast<float4*>(yo), make_float4(f[0], f[1], f[2], f[3]));
          atomicAdd(reinterpret_cast<float4*>(yo) + 1, make_float4(f[4], f[5], f[6], f[7]));
        } else {
          reinterpret_cast<float4*>(yo)[0] = make_float4(f[0], f[1], f[2], f[3]);
          reinterpret_cast<float4*>(yo)[1] = make_float4(f[4], f[5], f[6], f[7]);
        }
      } else if constexpr (!kTF32) {
        if (res) {
          const uint4 rv = __ldg(reinterpret_cast<const uint4*>(res + dst_row * p.cout + nh));
          const uint32_t* rw = reinterpret_cast<const uint32_t*>(&rv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 t = unpack2<T>(rw[e]);
            f[2 * e] += t.x;
            f[2 * e + 1] += t.y;
          }
        }
        if (p.relu) {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = fmaxf(f[e], 0.f);
        }
        *reinterpret_cast<uint4*>(y + dst_row * p.cout + nh) =
            make_uint4(pack2<T>(f[0], f[1]), pack2<T>(f[2], f[3]), pack2<T>(f[4], f[5]), pack2<T>(f[6], f[7]));
      }
    };
    for (int it = 0;; ++it) {
      int w, aux;
      uint32_t kmask;
      if (!ring_take(s_sched_full, s_sched_empty, s_tile, s_kmask, s_aux, it, lane, w, kmask, aux)) {
        atomicExch(p.error, kErrSchedWait);
        s_abort = 1;
        break;
      }
      if (s_abort || w < 0) break;
      // A tile with many offsets is worked on by several items ("parts", possibly on other CTAs).  Every part
      // stores its fp32 accumulator in its own slot of split_scratch and counts itself in split_flags[tile];
      // the part that counts last adds the slots in part order (so the sum does not depend on the schedule),
      // runs the epilogue and puts the counter back to zero.  No part waits for another.
      const int part = aux & 0xff, parts = (aux >> 8) & 0xff, slot0 = aux >> 16;
      const bool split = parts > 1;
      const int row0 = (w / tiles_n) * kTileM;
      const int n0 = (w % tiles_n) * p.n_tile;
      const int n_valid = min(p.n_tile, p.cout - n0);
      const int n_mma = (n_valid + 15) & ~15;
      const bool have_acc = kmask != 0;
      const int ab = acc_count & 1;
      if (have_acc && !mbar_wait_warp(smem_u32(&s_acc_full[ab]), (acc_count >> 1) & 1, lane)) {
        atomicExch(p.error, kErrAccWait);
        s_abort = 1;
        break;
      }
      tc_fence_after();
#ifdef TSB_TRACE_BUILD
      if (warp == kGW && lane == 0 && p.trace && (int)blockIdx.x == p.trace_cta && it < 256) p.trace[5120 + it] = clk();
#endif
      const int r = quarter * 32 + lane;
      const int64_t grow = (int64_t)row0 + r;
      int64_t dst_row = -1;
      if (grow < n_out) {
        dst_row = p.reorder ? (int64_t)__ldg(&p.reorder[grow]) : grow;
        if (dst_row >= p.dst_rows) dst_row = -1;
      }
      const uint32_t acc_addr = tmem_base + (uint32_t)ab * acc_cols + ((uint32_t)(quarter * 32) << 16);
      const int64_t slot_elems = (int64_t)kTileM * p.cout;
      float* my_slot = split ? p.split_scratch + (int64_t)(slot0 + part) * slot_elems + (int64_t)r * p.cout : nullptr;
      for (int j = 0; j < n_mma; j += 16) {
        uint32_t v[16];
        if (have_acc) {
          tmem_ld16(acc_addr + (uint32_t)j, v);
          tmem_ld_wait16(v);
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = 0u;
        }
        const int n = n0 + j;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int nh = n + 8 * h;
          if (dst_row < 0 || nh >= p.cout) continue;      // cout % 8 == 0
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[8 * h + e]);
          if (split) {
            reinterpret_cast<float4*>(my_slot + nh)[0] = make_float4(f[0], f[1], f[2], f[3]);
            reinterpret_cast<float4*>(my_slot + nh)[1] = make_float4(f[4], f[5], f[6], f[7]);
          } else {
            emit8(f, nh, dst_row);
          }
        }
      }
      // this warp is done with the accumulator buffer
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && have_acc) mbar_arrive(smem_u32(&s_acc_empty[ab]));
      if (have_acc) ++acc_count;
      if (split) {
        __threadfence();                              // this thread's slot rows are visible before the count
        if (!epi_sync()) {
          atomicExch(p.error, kErrSplitWait);
          s_abort = 1;
          break;
        }
        if (warp == kGW && lane == 0) {
          int* flag = p.split_flags + w;
          const int before = atomicAdd(flag, 1);
          __threadfence();
          const int last = before == parts - 1;
          if (last) atomicExch(flag, 0);             // no other part of this tile is left to count
          s_split_last = last;
        }
        if (!epi_sync()) {
          atomicExch(p.error, kErrSplitWait);
          s_abort = 1;
          break;
        }
        if (s_split_last) {
          const float* slots = p.split_scratch + (int64_t)slot0 * slot_elems + (int64_t)r * p.cout;
          for (int nh = n0; nh < n0 + n_mma; nh += 8) {
            if (dst_row < 0 || nh >= p.cout) continue;
            float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int q = 0; q < parts; ++q) {
              const float4 a = __ldcg(reinterpret_cast<const float4*>(slots + q * slot_elems + nh));
              const float4 b = __ldcg(reinterpret_cast<const float4*>(slots + q * slot_elems + nh) + 1);
              f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
              f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
            }
            emit8(f, nh, dst_row);
          }
        }
      }
#ifdef TSB_TRACE_BUILD
      if (warp == kGW && lane == 0) TSB_TRACE_HOT(7, it + 1);   // item written out (first epilogue warp)
#endif
    }
  } else if (warp == kSchedWarp) {
    // ------------------------------------------------------------ scheduler warp
    // one lane: takes the next item from the global counter each time the gather warps ask for one (the
    // first without being asked), reads its table entry and publishes it through the ring
    if (lane == 0) {
      for (int i = 0;; ++i) {
        const int slot = i % kRing;
        if (i >= 1 && !mbar_wait(smem_u32(&s_req), (uint32_t)(i - 1) & 1u)) {
          atomicExch(p.error, kErrSchedWait);
          s_abort = 1;
          break;
        }
        if (i >= kRing && !mbar_wait(smem_u32(&s_sched_empty[slot]), ((uint32_t)(i / kRing) + 1u) & 1u)) {
          atomicExch(p.error, kErrSchedWait);
          s_abort = 1;
          break;
        }
#ifdef TSB_TRACE_BUILD
        if (p.trace && (int)blockIdx.x == p.trace_cta && i < 256) p.trace[4096 + i * 4] = clk();       // asked
#endif
        const int w = atomicAdd(p.sched, 1);
#ifdef TSB_TRACE_BUILD
        if (p.trace && (int)blockIdx.x == p.trace_cta && i < 256) p.trace[4096 + i * 4 + 1] = clk() + (w & 0);   // counted
#endif
        if (w >= n_work || s_abort) {
          s_tile[slot] = -1;                  // tells the other roles that the CTA is done
          mbar_arrive(smem_u32(&s_sched_full[slot]));
          break;
        }
        uint32_t mask = p.k_range;
        int item = w, aux = 0;
        if (p.items) {
          const int4 e = __ldg(&p.items[w / tiles_n]);
          item = e.x * tiles_n + (w % tiles_n);
          mask &= (uint32_t)e.y;
          aux = e.z;
        } else if (p.tile_mask) {
          mask &= __ldg(&p.tile_mask[w / tiles_n]);
        }
        s_kmask[slot] = mask;
        s_tile[slot] = item;
        s_aux[slot] = aux;
        mbar_arrive(smem_u32(&s_sched_full[slot]));
#ifdef TSB_TRACE_BUILD
        if (p.trace && blockIdx.x < 1024) {       // every CTA: items taken, offsets taken, wall clock of the last claim
          p.trace[6144 + 4 * blockIdx.x] += 1;
          p.trace[6144 + 4 * blockIdx.x + 1] += __popc(mask);
          p.trace[6144 + 4 * blockIdx.x + 2] = (long long)global_ns();
        }
#endif
#ifdef TSB_TRACE_BUILD
        if (p.trace && (int)blockIdx.x == p.trace_cta && i < 256) {
          p.trace[4096 + i * 4 + 2] = clk();       // published
          p.trace[4096 + i * 4 + 3] = (long long)mask;
        }
#endif
      }
    }
  } else if (warp == kTmaWarp) {
    // ------------------------------------------------------------ weight loader (B operand)
    // the whole warp walks the blocks converged; one elected lane posts the byte count and issues the copies
    const uint32_t full0 = smem_u32(&s_full[0]), empty0 = smem_u32(&s_empty[0]);
    uint32_t stage = 0, phase = 0;
    bool first_pass = true;
    bool ok = true;
    for (int it = 0; ok; ++it) {
      int w, aux;
      uint32_t kmask;
      if (!ring_take(s_sched_full, s_sched_empty, s_tile, s_kmask, s_aux, it, lane, w, kmask, aux)) {
        if (lane == 0) atomicExch(p.error, kErrSchedWait);
        s_abort = 1;
        break;
      }
      if (s_abort || w < 0) break;
      const int n0 = (w % tiles_n) * p.n_tile;
      for (uint32_t km = kmask; km && ok; km &= km - 1) {
        // pair-list mode: the tile's rows all belong to one kernel offset, named by tile_k
        const int k = p.tile_k ? __ldg(&p.tile_k[w / tiles_n]) : (__ffs(km) - 1);
        const int wrow = k * p.cout + n0;
        for (int g = 0; g < groups; ++g) {
          if (!first_pass && !mbar_wait(empty0 + stage * 8, phase ^ 1u)) {
            if (lane == 0) atomicExch(p.error, kErrEmptyWait);
            s_abort = 1;
            ok = false;
            break;
          }
          const uint32_t bar = full0 + stage * 8;
          const int c_lo = g * p.cpb, c_hi = min(c_lo + p.cpb, chunks);
          if (elect_one()) {
            mbar_arrive_expect_tx(bar, (uint32_t)((c_hi - c_lo) * b_bytes));
            const uint32_t b_dst = smem_base + stage * (uint32_t)stage_bytes + (uint32_t)p.cpb * kABytes;
            for (int c = c_lo; c < c_hi; ++c) {
              int col_src, col_w, steps;
              chunk_geometry(c, col_src, col_w, steps);
              tma_load_2d(b_dst + (uint32_t)((c - c_lo) * b_bytes), &w_map, bar, col_w, wrow);
            }
          }
          __syncwarp();
          if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; first_pass = false; }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    // The instruction stream of this warp is on the critical path of the whole CTA: the warp stays
    // converged so that stage index, barrier phase and descriptors are warp-uniform values.
    const uint32_t full0 = smem_u32(&s_full[0]), empty0 = smem_u32(&s_empty[0]);
    const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, SWIZZLE_128B
    const uint32_t lo_flag = 1u << 16;
    const uint32_t stage_units = (uint32_t)stage_bytes >> 4;
    const uint32_t a_units = (uint32_t)kABytes >> 4;
    const uint32_t b_units = (uint32_t)b_bytes >> 4;
    const uint32_t b_first = (uint32_t)p.cpb * a_units;                 // first weight chunk of a stage
    // stage index, barrier phase and descriptor words are carried incrementally: no multiplication per block
    // in the instruction stream that every other role of the CTA waits for
    const uint32_t a_lo0 = ((smem_base >> 4) & 0x3FFFu) | lo_flag;      // stage 0, first A chunk
    const int last_steps = ((p.cin - (chunks - 1) * kChunk) + kStepK - 1) / kStepK;   // cp.async variant
    uint32_t stage = 0, phase = 0, a_lo = a_lo0;
    int acc_count = 0;
    bool ok = true;
#ifdef TSB_TRACE_BUILD
    int blk = 0;
#endif
    for (int it = 0; ok; ++it) {
      int w, aux;
      uint32_t kmask;
      if (!ring_take(s_sched_full, s_sched_empty, s_tile, s_kmask, s_aux, it, lane, w, kmask, aux)) {
        if (lane == 0) atomicExch(p.error, kErrSchedWait);
        s_abort = 1;
        break;
      }
      if (s_abort || w < 0) break;
      const int n0 = (w % tiles_n) * p.n_tile;
      const int n_mma = (min(p.n_tile, p.cout - n0) + 15) & ~15;
      const uint32_t idesc = make_idesc(p.ab_format, n_mma);
      if (!kmask) continue;                                      // nothing to multiply: the epilogue writes zeros
      // the epilogue must have drained this accumulator buffer (its previous use)
      const int ab = acc_count & 1;
      if (acc_count >= 2 && !mbar_wait(smem_u32(&s_acc_empty[ab]), ((acc_count >> 1) + 1) & 1)) {
        if (lane == 0) atomicExch(p.error, kErrAccWait);
        s_abort = 1;
        break;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + (uint32_t)ab * acc_cols;
      uint32_t accumulate = 0;
      for (uint32_t km = kmask; km && ok; km &= km - 1) {       // one trip per offset present in the tile
        for (int c_lo = 0; c_lo < chunks; c_lo += p.cpb) {
#ifdef TSB_TRACE_BUILD
          if (lane == 0) TSB_TRACE_HOT(4, blk);
#endif
          if (!mbar_wait(full0 + stage * 8, phase)) {
            if (lane == 0) atomicExch(p.error, kErrFullWait);
            s_abort = 1;
            ok = false;
            break;
          }
          tc_fence_after();
#ifdef TSB_TRACE_BUILD
          if (lane == 0) TSB_TRACE_HOT(5, blk);
#endif
          const int c_hi = min(c_lo + p.cpb, chunks);
          if (elect_one()) {
            uint32_t a_c = a_lo, b_c = a_lo + b_first;          // shared memory stays below 2^18 bytes: no carry
            for (int c = c_lo; c < c_hi; ++c, a_c += a_units, b_c += b_units) {
              int steps;
              if constexpr (kTma) {
                int col_src, col_w;
                chunk_geometry(c, col_src, col_w, steps);
              } else {
                steps = (c == chunks - 1) ? last_steps : 4;
              }
              // +32 bytes along K inside the swizzle atom = +2 in the descriptor's 16-byte address units
#pragma unroll
              for (int st = 0; st < 4; ++st) {
                if (st < steps) {
                  const uint64_t a_desc = ((uint64_t)desc_hi << 32) | (a_c + 2u * st);
                  const uint64_t b_desc = ((uint64_t)desc_hi << 32) | (b_c + 2u * st);
                  umma<kTF32>(acc, a_desc, b_desc, idesc, accumulate);
                  accumulate = 1;
                }
              }
            }
            umma_commit(empty0 + stage * 8);
          }
          __syncwarp();
          accumulate = 1;
#ifdef TSB_TRACE_BUILD
          if (lane == 0) TSB_TRACE_HOT(6, blk);
          ++blk;
#endif
          a_lo += stage_units;
          if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; a_lo = a_lo0; }
        }
      }
      // also on the error path: ends the epilogue's bounded wait early
      if (elect_one()) umma_commit(smem_u32(&s_acc_full[ab]));
      __syncwarp();
      ++acc_count;
    }
    tc_fence_before();
  }
  // A CTA that gave up may still have copies in flight towards its shared memory: give them time
  // to land (bounded) before the CTA's resources are released.
  if (s_abort) {
    for (int t = 0; t < 1000; ++t) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * acc_cols);
  }
#ifdef TSB_TRACE_BUILD
  if (tid == 0) TSB_TRACE_HOT(3, 0);     // CTA exit
  if (tid == 0 && p.trace && blockIdx.x < 1024) p.trace[2048 + 2 * blockIdx.x + 1] = (long long)global_ns();
#endif
  // the last CTA to finish puts the scheduling words back to zero for a later launch
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
}

// Offset mask of every 128-row tile of a map: bit k = some row of the tile has an entry >= 0 in column k.
// One warp per tile; entry (row, k) at map[row * rs + k * cs]; rows >= n_rows (a device-side count
// when n_rows_dev is given) count as empty.
__global__ void tile_mask_kernel(const int* __restrict__ map, long long rs, long long cs, int kvol, int64_t n_rows,
                                 const int* __restrict__ n_rows_dev, int64_t tiles, unsigned* __restrict__ out) {
  if (n_rows_dev) n_rows = max((int64_t)0, min((int64_t)__ldg(n_rows_dev), n_rows));
  const int lane = threadIdx.x & 31;
  int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (; warp < tiles; warp += nwarps) {
    unsigned m = 0;
    const int64_t row0 = warp * kTileM;
    if (cs == 1 && rs == kvol) {
      // row-major: the valid rows of the tile are one contiguous run of ints; eight loads in flight per lane
      // (the pass is bound by load latency, not by bytes), the column of an element tracked incrementally
      const int64_t rows_here = min((int64_t)kTileM, n_rows - row0);
      const int total = rows_here > 0 ? (int)rows_here * kvol : 0;
      const int* base = map + row0 * rs;
      const int step = 32 % kvol;
      int c = lane % kvol;
      for (int e = lane; e < total; e += 32 * 8) {
        int v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = (e + 32 * u < total) ? __ldg(base + e + 32 * u) : -1;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (v[u] >= 0) m |= 1u << c;
          c += step;
          if (c >= kvol) c -= kvol;
        }
      }
    } else {
      for (int k = 0; k < kvol; ++k) {
        bool any = false;
#pragma unroll
        for (int j = 0; j < kTileM / 32; ++j) {
          const int64_t r = row0 + lane + 32 * j;
          any = any || (r < n_rows && __ldg(map + r * rs + (long long)k * cs) >= 0);
        }
        if (any) m |= 1u << k;
      }
    }
    for (int o = 16; o; o >>= 1) m |= __shfl_xor_sync(0xffffffffu, m, o);
    if (lane == 0) out[warp] = m;
  }
}

// Scheduling words, one slot per stream: launches on one stream run one after another, so they can share
// a slot (zero-initialised, and every launch zeroes it again when its last CTA leaves); launches on
// different streams may overlap and get different slots.
constexpr int kSchedSlots = 1024;
constexpr int kMaxDevices = 64;
__device__ int g_sched_slots[kSchedSlots * 2];

// W [kvol, cin, cout] -> Wt [kvol, cout, cin]
template <typename T>
__global__ void pack_weight_kernel(const T* __restrict__ w, T* __restrict__ wt, int cin, int cout) {
  __shared__ T tile[32][33];
  const int k = blockIdx.z;
  const int c0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  const T* src = w + (int64_t)k * cin * cout;
  T* dst = wt + (int64_t)k * cin * cout;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int c = c0 + i, n = n0 + threadIdx.x;
    if (c < cin && n < cout) tile[i][threadIdx.x] = src[(int64_t)c * cout + n];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int n = n0 + i, c = c0 + threadIdx.x;
    if (c < cin && n < cout) dst[(int64_t)n * cin + c] = tile[threadIdx.x][i];
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn tensor_map_encoder() {
  static EncodeFn fn = []() -> EncodeFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeFn>(ptr);
  }();
  return fn;
}

size_t smem_bytes_for(int n_tile, int stages, int cpb) {
  return 1024 + (size_t)stages * cpb * (kABytes + (size_t)n_tile * kRowBytes);
}

struct LaunchConfig {
  int n_tile, cpb, stages, ctas;
};

int acc_cols_for(int n_tile) {
  int c = 32;
  while (c < n_tile) c <<= 1;
  return c;
}

// Stages that fit `budget` bytes of dynamic shared memory (0: not even two).
int stages_that_fit(int n_tile, int cpb, size_t budget) {
  int best = 0;
  for (int s = 2; s <= kMaxStages; ++s)
    if (smem_bytes_for(n_tile, s, cpb) <= budget) best = s;
  return best;
}

// Two persistent CTAs per SM when two double-buffered accumulators fit TMEM (N tile <= 128 columns)
// and at least three stages fit half the shared memory: two MMA issuers per SM hide the per-block
// latency of the narrow layers.  Otherwise one CTA per SM with as many stages as fit.  Non-zero
// fields of `want` override the choice (tuning runs).
bool pick_config(int cout, int chunks, const LaunchConfig& want, LaunchConfig* out) {
  LaunchConfig c;
  c.n_tile = want.n_tile > 0 ? ((want.n_tile + 15) & ~15) : ((cout + 15) & ~15);
  if (c.n_tile > 256) c.n_tile = 256;
  if (c.n_tile > ((cout + 15) & ~15)) c.n_tile = (cout + 15) & ~15;
  c.cpb = want.cpb > 0 ? want.cpb : 1;
  if (c.cpb > chunks) c.cpb = chunks;
  const size_t half = 112 * 1024, whole = 226 * 1024;
  const int s2 = acc_cols_for(c.n_tile) <= 128 ? stages_that_fit(c.n_tile, c.cpb, half) : 0;
  const int s1 = stages_that_fit(c.n_tile, c.cpb, whole);
  c.ctas = want.ctas > 0 ? want.ctas : (s2 >= 3 ? 2 : 1);
  if (c.ctas == 2 && s2 < 2) c.ctas = 1;
  c.stages = c.ctas == 2 ? s2 : s1;
  if (want.stages > 0 && want.stages < c.stages) c.stages = want.stages;
  *out = c;
  return c.stages >= 2;
}

// scheduling words of `stream` on the current device (the array's address is looked up once per device,
// a stream gets the next free slot the first time it launches a convolution).  When every slot of a
// device has been handed out the call fails rather than letting two streams share a counter.
int* sched_slot_of(cudaStream_t stream, int dev) {
  static std::mutex mu;
  static int* addr[kMaxDevices] = {nullptr};
  static std::map<std::pair<int, cudaStream_t>, int> slot_of;
  static int next_slot[kMaxDevices] = {0};
  // the per-thread default stream is one handle value for a different stream in every host thread
  if (stream == cudaStreamPerThread) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_sched_slots) != cudaSuccess) return nullptr;
    addr[dev] = reinterpret_cast<int*>(ptr);
  }
  auto it = slot_of.find({dev, stream});
  if (it == slot_of.end()) {
    if (next_slot[dev] >= kSchedSlots) return nullptr;
    it = slot_of.emplace(std::make_pair(dev, stream), next_slot[dev]++).first;
  }
  return addr[dev] + 2 * it->second;
}

// per-device facts and one-time settings, looked up / applied on first use under a lock
struct DeviceState {
  int sms = 0;
  bool attr_set[2][3] = {{false, false, false}, {false, false, false}};
};
std::mutex g_dev_mu;
DeviceState g_dev[kMaxDevices];

template <typename T, bool kTma>
int prepare_device(int dev, int fmt, int* sms) {
  std::lock_guard<std::mutex> lock(g_dev_mu);
  DeviceState& d = g_dev[dev];
  if (!d.sms) {
    int v = kSmCount;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = kSmCount;
    d.sms = v;
  }
  if (!d.attr_set[kTma][fmt]) {
    TSB_CUDA_TRY(cudaFuncSetAttribute(igemm_umma_kernel<T, kTma>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    d.attr_set[kTma][fmt] = true;
  }
  *sms = d.sms;
  return TSB_OK;
}

int chunks_of(int cin, int dtype) { return (int)cdiv((int64_t)cin * (int64_t)dtype_size(dtype), kRowBytes); }

// The A operand is copied by the gather warps (cp.async) unless the caller asks for the copy engine
// (cfg_gather == 2, TMA gather4).  Measured on B200: the copy engine delivers one 128-byte row slice per ~9 cycles
// per SM whatever the number of issuing warps, CTAs per SM or chunks in flight (0.6 us per 16 KiB chunk), the
// gather warps one per ~2-3 cycles, and whole layers run 2.0-2.4x slower on the copy engine; it stays as an option.
bool use_tma_gather(const IgemmArgs& a) { return a.cfg_gather == 2 && a.n_in > 0; }
// channel chunks of a kernel offset: per feature matrix with the TMA gather (a box reads one matrix)
int chunks_for(const IgemmArgs& a) {
  if (use_tma_gather(a) && a.x2) return chunks_of(a.c1, a.dtype) + chunks_of(a.cin - a.c1, a.dtype);
  return chunks_of(a.cin, a.dtype);
}

// ---------------------------------------------------------------------------------------------
// Weight gradient on the tensor cores.
//
//   D[k][a][b] = sum over map rows m of  G[map[m][k]][a] * P[m][b]        (fp32 accumulation)
//
// G = the matrix addressed through the map ("gathered"), P = the matrix whose rows are the map's rows.  With the
// forward map, G = input features and P = output gradients gives dW[k][cin][cout]; with the transposed map,
// G = output gradients and P = input features gives the [kvol][cout][cin] form the reference returns
// (torchsparse/backend/convolution/convolution_backward_wgrad_implicit_gemm_cuda.cu:1614).
//
// The reduction runs over map rows, so both operands are read "MN-major": a stage holds 128 map rows, every
// row one 128-byte slice of 64 channels, 128B-swizzled by row - byte for byte the layout the forward kernel
// gathers its A operand into.  The shared-memory descriptors name it as canonical MN-major SWIZZLE_128B:
// 8-row groups 1024 bytes apart (stride byte offset), 64-channel blocks one chunk (16 KiB) apart (leading byte
// offset), and the instruction descriptor marks A and B as MN-major.  One tcgen05.mma covers 16 rows.
//
// A CTA owns (offset k, 128-channel tile of G, N tile of P, a share of the 128-row tiles) and keeps the 128 x N
// fp32 tile in TMEM over its whole share; tiles whose offset mask lacks k are skipped.  G rows are gathered by
// the eight gather warps (cp.async, zeros for a missing neighbour), P tiles are fetched by TMA.  At the end the
// four epilogue warps add the tile to the fp32 result with 16-byte atomic adds (the shares of the row range
// meet there).  Waits are bounded as in the forward kernel.
struct WgradParams {
  const void* g;         // [n_g, cg]
  const int* map;        // entry (row, k) at map[row * map_rs + k * map_cs]
  long long map_rs, map_cs;
  const unsigned* tile_mask;   // [tiles]
  float* out;            // [kvol, cg, cd], zero before the launch
  int* error;
  int n_g, n_rows, kvol, cg, cd;
  int m_tiles, n_tiles, splits, tiles;
  int n_tile;            // channels of P per CTA (multiple of 16, <= 256)
  int acc_cols, stages, ab_format;
};

constexpr int kWgradThreads = (kGatherWarps + kEpilogueWarps + 2) * 32;   // 448

template <typename T>
__global__ void __launch_bounds__(kWgradThreads, 1)
wgrad_umma_kernel(const WgradParams p, const __grid_constant__ CUtensorMap p_map) {
  constexpr int kChunk = kRowBytes / (int)sizeof(T);     // channels per 128-byte slice (64)
  constexpr int kGran = 16 / (int)sizeof(T);
  constexpr int kTmaW = kGatherWarps + kEpilogueWarps, kMmaW = kTmaW + 1;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t s_full[kMaxStages];
  __shared__ uint64_t s_empty[kMaxStages];
  __shared__ uint64_t s_acc_full;
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // work item of this CTA
  int w = blockIdx.x;
  const int split = w % p.splits; w /= p.splits;
  const int nt = w % p.n_tiles; w /= p.n_tiles;
  const int mt = w % p.m_tiles;
  const int k = w / p.m_tiles;
  const int t_lo = (int)((long long)p.tiles * split / p.splits), t_hi = (int)((long long)p.tiles * (split + 1) / p.splits);
  const int n0 = nt * p.n_tile;
  const int n_mma = (min(p.n_tile, p.cd - n0) + 15) & ~15;
  const int b_chunks = (n_mma + kChunk - 1) / kChunk;
  const int a_bytes = 2 * kABytes;                           // two 64-channel blocks of G (M = 128)
  const int stage_bytes = a_bytes + b_chunks * kABytes;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&s_full[s]), kGatherThreads + 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    mbar_init(smem_u32(&s_acc_full), 1);
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == kMmaW) tmem_alloc(smem_u32(&s_tmem), p.acc_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;
  auto tile_live = [&](int t) -> bool { return (__ldg(&p.tile_mask[t]) >> k) & 1u; };

  if (warp < kGatherWarps) {
    // ------------------------------------------------------------ gather warps: rows of G named by the map
    const T* g = reinterpret_cast<const T*>(p.g);
    const int gran = tid & 7, rbase = tid >> 3;
    const uint32_t dst_off = (uint32_t)rbase * kRowBytes + (uint32_t)((gran ^ (rbase & 7)) << 4);
    uint32_t stage = 0, phase = 0;
    bool first_pass = true;
    for (int t = t_lo; t < t_hi; ++t) {
      if (!tile_live(t)) continue;
      int src[kCopies];
#pragma unroll
      for (int j = 0; j < kCopies; ++j) {
        const long long r = (long long)t * kTileM + rbase + j * kRowsPerPass;
        src[j] = r < p.n_rows ? ld_map_entry(p.map + r * p.map_rs + (long long)k * p.map_cs) : -1;
      }
      if (!first_pass && !mbar_wait_warp(smem_u32(&s_empty[stage]), phase ^ 1u, lane)) {
        if (lane == 0) atomicExch(p.error, kErrEmptyWait);
        s_abort = 1;
        break;
      }
      const uint32_t a_stage = smem_base + stage * (uint32_t)stage_bytes + dst_off;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col = mt * 2 * kChunk + c * kChunk + gran * kGran;
        const bool col_ok = col < p.cg;
#pragma unroll
        for (int j = 0; j < kCopies; ++j) {
          const bool live = col_ok && (unsigned)src[j] < (unsigned)p.n_g;
          cp_async16(a_stage + (uint32_t)c * kABytes + (uint32_t)(j * kRowsPerPass) * kRowBytes,
                     live ? (const void*)(g + (int64_t)src[j] * p.cg + col) : (const void*)g, live ? 16u : 0u);
        }
      }
      cp_async_arrive_noinc(smem_u32(&s_full[stage]));
      if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; first_pass = false; }
    }
    cp_async_wait_all();
  } else if (warp < kGatherWarps + kEpilogueWarps) {
    // ------------------------------------------------------------ epilogue warps: D rows = channels of G
    bool any = false;
    for (int t = t_lo; t < t_hi && !any; ++t) any = tile_live(t);
    if (any) {
      if (!mbar_wait_warp(smem_u32(&s_acc_full), 0u, lane)) {
        if (lane == 0) atomicExch(p.error, kErrAccWait);
        s_abort = 1;
      } else {
        tc_fence_after();
        const int quarter = warp & 3;
        const int a = mt * 2 * kChunk + quarter * 32 + lane;      // channel of G
        const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float* orow = p.out + ((int64_t)k * p.cg + a) * p.cd + n0;
        for (int j = 0; j < n_mma; j += 16) {
          uint32_t v[16];
          tmem_ld16(acc_addr + (uint32_t)j, v);
          tmem_ld_wait16(v);
          if (a < p.cg) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (n0 + j + 4 * q < p.cd)
                atomicAdd(reinterpret_cast<float4*>(orow + j) + q,
                          make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                      __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])));
            }
          }
        }
        tc_fence_before();
      }
    }
  } else if (warp == kTmaW) {
    // ------------------------------------------------------------ P tiles by TMA (128 rows x 64 channels per chunk)
    uint32_t stage = 0, phase = 0;
    bool first_pass = true;
    for (int t = t_lo; t < t_hi; ++t) {
      if (!tile_live(t)) continue;
      if (!first_pass && !mbar_wait(smem_u32(&s_empty[stage]), phase ^ 1u)) {
        if (lane == 0) atomicExch(p.error, kErrEmptyWait);
        s_abort = 1;
        break;
      }
      if (elect_one()) {
        const uint32_t bar = smem_u32(&s_full[stage]);
        mbar_arrive_expect_tx(bar, (uint32_t)(b_chunks * kABytes));
        const uint32_t b_dst = smem_base + stage * (uint32_t)stage_bytes + (uint32_t)a_bytes;
        for (int c = 0; c < b_chunks; ++c) tma_load_2d(b_dst + (uint32_t)(c * kABytes), &p_map, bar, n0 + c * kChunk, t * kTileM);
      }
      __syncwarp();
      if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; first_pass = false; }
    }
  } else if (warp == kMmaW) {
    // ------------------------------------------------------------ MMA issuer
    // descriptors: SBO = 1024 (8-row groups), LBO = one chunk (the next 64 channels), version 1, SWIZZLE_128B
    const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    const uint32_t lbo = ((uint32_t)kABytes >> 4) << 16;
    const uint32_t idesc = make_idesc(p.ab_format, n_mma) | (1u << 15) | (1u << 16);    // A and B MN-major
    uint32_t stage = 0, phase = 0, accumulate = 0;
    bool ok = true, any = false;
    for (int t = t_lo; t < t_hi && ok; ++t) {
      if (!tile_live(t)) continue;
      any = true;
      if (!mbar_wait(smem_u32(&s_full[stage]), phase)) {
        if (lane == 0) atomicExch(p.error, kErrFullWait);
        s_abort = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_units = (smem_base + stage * (uint32_t)stage_bytes) >> 4;
        const uint32_t b_units = a_units + ((uint32_t)a_bytes >> 4);
#pragma unroll
        for (int ks = 0; ks < kTileM / 16; ++ks) {      // 16 map rows per instruction = 2048 bytes = 128 address units
          const uint64_t a_desc = ((uint64_t)desc_hi << 32) | (((a_units + 128u * ks) & 0x3FFFu) | lbo);
          const uint64_t b_desc = ((uint64_t)desc_hi << 32) | (((b_units + 128u * ks) & 0x3FFFu) | lbo);
          umma<false>(tmem_base, a_desc, b_desc, idesc, accumulate);
          accumulate = 1;
        }
        umma_commit(smem_u32(&s_empty[stage]));
      }
      __syncwarp();
      accumulate = 1;
      if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; }
    }
    if (any) {
      if (elect_one()) umma_commit(smem_u32(&s_acc_full));
      __syncwarp();
    }
    tc_fence_before();
  }
  if (s_abort) {
    for (int t = 0; t < 1000; ++t) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == kMmaW) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.acc_cols);
  }
}

}  // namespace

bool igemm_umma_supported(const IgemmArgs& a) {
  if (!tensor_map_encoder()) return false;
  if (a.dtype == TSB_F32) {
    if (a.math != TSB_MATH_TF32) return false;       // exact fp32 stays on the CUDA cores
  } else if (a.dtype != TSB_F16 && a.dtype != TSB_BF16) {
    return false;
  }
  // feature rows must be 16-byte multiples; outputs are written in 8-channel groups
  const int esz = (int)dtype_size(a.dtype);
  if ((a.cin * esz) % 16 || a.cout % 8) return false;
  if (a.x2 && (a.c1 <= 0 || a.c1 >= a.cin || (a.c1 * esz) % 16)) return false;
  if (a.n_in >= (int64_t)INT32_MAX || a.n_out >= (int64_t)INT32_MAX) return false;
  if (a.kvol > kMaxKvolUmma) return false;            // one bit per map column in a tile's offset mask
  if (a.tile_k && a.kvol != 1) return false;          // pair-list mode: one map column, weights chosen per tile
  if (!a.map && a.kvol != 1) return false;            // identity rows: a 1x1x1 kernel
  if (a.out_fp32 && a.residual) return false;
  if ((a.acc_in || a.acc_out) && (a.atomic_out || a.out_fp32)) return false;
  if (a.items && (!a.n_items_dev || !a.split_scratch || !a.split_flags || a.tile_k || a.n_items < 0 ||
                  ((uintptr_t)a.items & 15) || ((uintptr_t)a.split_scratch & 15)))
    return false;
  if (((uintptr_t)a.x | (uintptr_t)a.x2 | (uintptr_t)a.y | (uintptr_t)a.w | (uintptr_t)a.residual |
       (uintptr_t)a.packed_w | (uintptr_t)a.acc_in | (uintptr_t)a.acc_out) & 15)
    return false;
  LaunchConfig want{a.cfg_n_tile, a.cfg_cpb, a.cfg_stages, a.cfg_ctas}, got;
  return pick_config(a.cout, chunks_for(a), want, &got);
}

size_t packed_weight_bytes(int kvol, int cin, int cout, int dtype) {
  return align_up((size_t)kvol * cin * cout * dtype_size(dtype), 256);
}

size_t tile_mask_bytes(int64_t n_out) { return align_up((size_t)cdiv(n_out, kTileM) * sizeof(unsigned) + 4, 256); }

size_t igemm_umma_workspace_bytes(int kvol, int cin, int cout, int dtype, int64_t n_out) {
  // packed weights + error word + tile masks (each only used when the caller does not supply it)
  return packed_weight_bytes(kvol, cin, cout, dtype) + 256 + tile_mask_bytes(n_out);
}

int tile_masks(const int* map, long long rs, long long cs, int kvol, int64_t n_rows, const int* n_rows_dev,
               unsigned* out, cudaStream_t s) {
  const int64_t tiles = cdiv(n_rows, kTileM);
  if (tiles == 0) return TSB_OK;
  tile_mask_kernel<<<grid_for(tiles * 32, 256, 8), 256, 0, s>>>(map, rs, cs, kvol, n_rows, n_rows_dev, tiles, out);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

template <typename T>
static int pack_launch(const void* w, int kvol, int cin, int cout, void* packed, cudaStream_t s) {
  dim3 pgrid((unsigned)cdiv(cout, 32), (unsigned)cdiv(cin, 32), (unsigned)kvol);
  pack_weight_kernel<T><<<pgrid, dim3(32, 8), 0, s>>>((const T*)w, (T*)packed, cin, cout);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int pack_weight(const void* w, int kvol, int cin, int cout, int dtype, void* packed, cudaStream_t s) {
  if (dtype == TSB_F32) return pack_launch<float>(w, kvol, cin, cout, packed, s);
  if (dtype == TSB_F16) return pack_launch<__half>(w, kvol, cin, cout, packed, s);
  return pack_launch<__nv_bfloat16>(w, kvol, cin, cout, packed, s);
}

template <typename T>
static int umma_launch(const IgemmArgs& a, cudaStream_t s) {
  const int kvol_w = a.tile_k ? a.kvol_w : a.kvol;      // kernel offsets of the weight tensor
  const size_t w_bytes = packed_weight_bytes(kvol_w, a.cin, a.cout, a.dtype);
  const T* wt = reinterpret_cast<const T*>(a.packed_w);
  int* err = a.dev_status;
  const unsigned* tmask = a.tile_mask;
  const bool need_mask = !tmask && !a.items && a.map && !a.tile_k && a.kvol > 1;
  // workspace layout: [packed weights][error word, 256 bytes][tile masks]; only the parts the caller did
  // not supply are used, and the workspace has to reach the end of the last one used
  size_t need = 0;
  if (!wt) need = w_bytes;
  if (!err) need = w_bytes + 256;
  if (need_mask) need = w_bytes + 256 + tile_mask_bytes(a.n_out);
  char* ws = reinterpret_cast<char*>(a.workspace);
  if (need && (!ws || a.workspace_bytes < need)) return TSB_ERR_WORKSPACE;
  if (!err) {
    err = reinterpret_cast<int*>(ws + w_bytes);
    TSB_CUDA_TRY(cudaMemsetAsync(err, 0, sizeof(int), s));
  }
  if (!wt) {
    int rc = pack_launch<T>(a.w, kvol_w, a.cin, a.cout, ws, s);
    if (rc != TSB_OK) return rc;
    wt = reinterpret_cast<const T*>(ws);
  }
  const long long rs = a.map_rs ? a.map_rs : a.kvol, cs = a.map_cs ? a.map_cs : 1;
  if (need_mask) {
    unsigned* m = reinterpret_cast<unsigned*>(ws + w_bytes + 256);
    int rc = tile_masks(a.map, rs, cs, a.kvol, a.n_out, a.n_out_dev, m, s);
    if (rc != TSB_OK) return rc;
    tmask = m;
  }
  int dev = 0;
  TSB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return TSB_ERR_LIMIT;
  UmmaParams p;
  p.x = a.x; p.x2 = a.x2; p.c1 = a.x2 ? a.c1 : a.cin;
  p.map = a.map; p.map_rs = rs; p.map_cs = cs; p.tile_mask = tmask;
  p.reorder = a.reorder_loc; p.y = a.y; p.bias = a.bias; p.scale = a.scale;
  p.residual = a.residual; p.acc_in = a.acc_in; p.acc_out = a.acc_out; p.n_out_dev = a.n_out_dev; p.error = err;
  p.items = reinterpret_cast<const int4*>(a.items); p.n_items_dev = a.n_items_dev; p.n_items = (int)a.n_items;
  p.split_scratch = a.split_scratch; p.split_flags = a.split_flags;
  p.tile_k = a.tile_k; p.out_fp32 = a.out_fp32; p.atomic_out = a.atomic_out;
  p.dst_rows = (int)(a.dst_rows > 0 ? a.dst_rows : a.n_out);
  p.sched = sched_slot_of(s, dev);
  if (!p.sched) return TSB_ERR_LIMIT;   // more distinct streams than scheduling slots, or the per-thread default stream
#ifdef TSB_TRACE_BUILD
  p.trace = nullptr; p.trace_cta = 0;
  if (const char* tr = getenv("TSB_UMMA_TRACE")) {   // debugging aid: address of a 256x8 int64 device buffer
    p.trace = reinterpret_cast<long long*>(strtoull(tr, nullptr, 0));
    if (const char* tc = getenv("TSB_UMMA_TRACE_CTA")) p.trace_cta = atoi(tc);
  }
#endif
  p.n_in = (int)a.n_in; p.n_out = (int)a.n_out; p.kvol = a.kvol; p.cin = a.cin; p.cout = a.cout;
  const int k_lo = a.k_hi > a.k_lo ? a.k_lo : 0, k_hi = a.k_hi > a.k_lo ? a.k_hi : a.kvol;
  if (k_lo < 0 || k_hi > a.kvol) return TSB_ERR_BAD_ARG;
  p.k_range = (k_hi >= 32 ? 0xffffffffu : ((1u << k_hi) - 1u)) & ~((1u << k_lo) - 1u);
  LaunchConfig want{a.cfg_n_tile, a.cfg_cpb, a.cfg_stages, a.cfg_ctas}, cfg;
  if (!pick_config(a.cout, chunks_for(a), want, &cfg)) return TSB_ERR_UNSUPPORTED;
  const bool tma = use_tma_gather(a);
  p.n_tile = cfg.n_tile; p.cpb = cfg.cpb; p.stages = cfg.stages;
  p.acc_cols = acc_cols_for(cfg.n_tile);
  p.relu = a.relu;
  p.ab_format = (a.dtype == TSB_BF16) ? kFmtBF16 : (a.dtype == TSB_F32) ? kFmtTF32 : kFmtF16;
  const size_t smem = smem_bytes_for(cfg.n_tile, cfg.stages, cfg.cpb);
  int sms = kSmCount;
  {
    int rc = tma ? prepare_device<T, true>(dev, p.ab_format, &sms) : prepare_device<T, false>(dev, p.ab_format, &sms);
    if (rc != TSB_OK) return rc;
  }
  CUtensorMap w_map, x_map, x2_map;
  memset(&x_map, 0, sizeof(x_map));
  memset(&x2_map, 0, sizeof(x2_map));
  {
    auto encode = tensor_map_encoder();
    if (!encode) return TSB_ERR_UNSUPPORTED;
    const CUtensorMapDataType dt = a.dtype == TSB_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : a.dtype == TSB_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const cuuint32_t chunk = (cuuint32_t)(kRowBytes / sizeof(T));
    cuuint32_t estride[2] = {1, 1};
    // packed weights as a 2-D tensor [kvol * cout rows, cin columns]; box = 128 bytes of columns x n_tile rows
    cuuint64_t gdim[2] = {(cuuint64_t)a.cin, (cuuint64_t)kvol_w * (cuuint64_t)a.cout};
    cuuint64_t gstride[1] = {(cuuint64_t)a.cin * sizeof(T)};
    cuuint32_t box[2] = {chunk, (cuuint32_t)cfg.n_tile};
    CUresult r = encode(&w_map, dt, 2, const_cast<T*>(wt), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return TSB_ERR_BAD_ARG;
    if (tma) {
      // feature matrices as 2-D tensors [n_in rows, channels]; box = 128 bytes of channels x 1 row (gather4 takes
      // four row coordinates); columns past the matrix and rows outside it read as zeros
      cuuint32_t xbox[2] = {chunk, 1};
      const int c2 = a.cin - p.c1;
      cuuint64_t xdim[2] = {(cuuint64_t)p.c1, (cuuint64_t)a.n_in};
      cuuint64_t xstride[1] = {(cuuint64_t)p.c1 * sizeof(T)};
      r = encode(&x_map, dt, 2, const_cast<void*>(a.x), xdim, xstride, xbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return TSB_ERR_BAD_ARG;
      if (a.x2) {
        cuuint64_t x2dim[2] = {(cuuint64_t)c2, (cuuint64_t)a.n_in};
        cuuint64_t x2stride[1] = {(cuuint64_t)c2 * sizeof(T)};
        r = encode(&x2_map, dt, 2, const_cast<void*>(a.x2), x2dim, x2stride, xbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return TSB_ERR_BAD_ARG;
      }
    }
  }
  const int64_t n_work = (a.items ? a.n_items : cdiv(a.n_out, kTileM)) * cdiv(a.cout, cfg.n_tile);
  int64_t slots = (int64_t)cfg.ctas * sms;
  if (a.cfg_grid > 0 && a.cfg_grid < slots) slots = a.cfg_grid;
  const int grid = (int)(n_work < slots ? n_work : slots);
  if (tma) igemm_umma_kernel<T, true><<<grid, kThreadsTma, smem, s>>>(p, w_map, x_map, x2_map);
  else igemm_umma_kernel<T, false><<<grid, kThreads, smem, s>>>(p, w_map, x_map, x2_map);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int igemm_umma(const IgemmArgs& a, cudaStream_t s) {
  if (a.dtype == TSB_F16) return umma_launch<__half>(a, s);
  if (a.dtype == TSB_BF16) return umma_launch<__nv_bfloat16>(a, s);
  if (a.dtype == TSB_F32 && a.math == TSB_MATH_TF32) return umma_launch<float>(a, s);
  return TSB_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// Weight gradient (see wgrad_umma_kernel)
bool wgrad_umma_supported(const WgradArgs& a) {
  if (!tensor_map_encoder()) return false;
  if (a.dtype != TSB_F16 && a.dtype != TSB_BF16) return false;
  if (a.cg % 8 || a.cd % 16 || a.kvol < 1 || a.kvol > kMaxKvolUmma) return false;
  if (a.n_g <= 0 || a.n_rows <= 0 || a.n_g >= (int64_t)INT32_MAX || a.n_rows >= (int64_t)INT32_MAX) return false;
  if (((uintptr_t)a.g | (uintptr_t)a.p | (uintptr_t)a.out) & 15) return false;
  return true;
}

size_t wgrad_umma_workspace_bytes(int64_t n_rows) { return 256 + tile_mask_bytes(n_rows); }

template <typename T>
static int wgrad_launch(const WgradArgs& a, cudaStream_t s) {
  char* ws = reinterpret_cast<char*>(a.workspace);
  int* err = a.dev_status;
  const unsigned* tmask = a.tile_mask;
  const size_t need = (!tmask ? 256 + tile_mask_bytes(a.n_rows) : (!err ? 256 : 0));
  if (need && (!ws || a.workspace_bytes < need)) return TSB_ERR_WORKSPACE;
  if (!err) {
    err = reinterpret_cast<int*>(ws);
    TSB_CUDA_TRY(cudaMemsetAsync(err, 0, sizeof(int), s));
  }
  const long long rs = a.map_rs ? a.map_rs : a.kvol, cs = a.map_cs ? a.map_cs : 1;
  if (!tmask) {
    unsigned* m = reinterpret_cast<unsigned*>(ws + 256);
    int rc = tile_masks(a.map, rs, cs, a.kvol, a.n_rows, nullptr, m, s);
    if (rc != TSB_OK) return rc;
    tmask = m;
  }
  int dev = 0;
  TSB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return TSB_ERR_LIMIT;
  int sms = kSmCount;
  {
    static std::mutex mu;
    static bool attr_set[kMaxDevices][2] = {};
    std::lock_guard<std::mutex> lock(mu);
    const int f = a.dtype == TSB_BF16 ? 1 : 0;
    if (!attr_set[dev][f]) {
      TSB_CUDA_TRY(cudaFuncSetAttribute(wgrad_umma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
      attr_set[dev][f] = true;
    }
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms = v;
  }
  WgradParams p;
  p.g = a.g; p.map = a.map; p.map_rs = rs; p.map_cs = cs; p.tile_mask = tmask; p.out = a.out; p.error = err;
  p.n_g = (int)a.n_g; p.n_rows = (int)a.n_rows; p.kvol = a.kvol; p.cg = a.cg; p.cd = a.cd;
  p.n_tile = a.cd < 256 ? a.cd : 256;
  p.n_tiles = (a.cd + p.n_tile - 1) / p.n_tile;
  p.m_tiles = (a.cg + 127) / 128;
  p.tiles = (int)cdiv(a.n_rows, kTileM);
  // shares of the row range: enough CTAs for two per SM, never more shares than row tiles
  const int64_t base = (int64_t)a.kvol * p.m_tiles * p.n_tiles;
  int64_t splits = (2 * (int64_t)sms + base - 1) / base;
  if (splits < 1) splits = 1;
  if (splits > p.tiles) splits = p.tiles;
  p.splits = (int)splits;
  p.acc_cols = acc_cols_for(p.n_tile);
  p.ab_format = a.dtype == TSB_BF16 ? kFmtBF16 : kFmtF16;
  const int b_chunks = (p.n_tile + 63) / 64;
  const size_t stage_bytes = (size_t)(2 + b_chunks) * kABytes;
  int stages = (int)((225 * 1024) / stage_bytes);
  if (stages > 4) stages = 4;
  if (stages < 2) return TSB_ERR_UNSUPPORTED;
  p.stages = stages;
  const size_t smem = 1024 + (size_t)stages * stage_bytes;
  CUtensorMap p_map;
  {
    auto encode = tensor_map_encoder();
    if (!encode) return TSB_ERR_UNSUPPORTED;
    const CUtensorMapDataType dt = a.dtype == TSB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint32_t estride[2] = {1, 1};
    cuuint64_t gdim[2] = {(cuuint64_t)a.cd, (cuuint64_t)a.n_rows};
    cuuint64_t gstride[1] = {(cuuint64_t)a.cd * sizeof(T)};
    cuuint32_t box[2] = {(cuuint32_t)(kRowBytes / sizeof(T)), (cuuint32_t)kTileM};
    CUresult r = encode(&p_map, dt, 2, const_cast<void*>(a.p), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return TSB_ERR_BAD_ARG;
  }
  TSB_CUDA_TRY(cudaMemsetAsync(a.out, 0, (size_t)a.kvol * a.cg * a.cd * sizeof(float), s));
  const int64_t grid = base * p.splits;
  if (grid > INT32_MAX) return TSB_ERR_LIMIT;
  wgrad_umma_kernel<T><<<(unsigned)grid, kWgradThreads, smem, s>>>(p, p_map);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int wgrad_umma(const WgradArgs& a, cudaStream_t s) {
  if (a.dtype == TSB_F16) return wgrad_launch<__half>(a, s);
  if (a.dtype == TSB_BF16) return wgrad_launch<__nv_bfloat16>(a, s);
  return TSB_ERR_UNSUPPORTED;
}

}  // namespace tsb
