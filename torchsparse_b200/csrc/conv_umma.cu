// Implicit-GEMM sparse convolution forward on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   Y[m, :] = sum_k  X[map[m][k], :] . W[k]      (fp16 / bf16 operands, or fp32 operands multiplied
//                                                  as TF32; fp32 accumulation in every case)
//
// One CTA owns 128 consecutive output rows (the rows of one map tile) and an N-tile of at most
// 256 output channels.  The reduction runs over "K blocks": one kernel offset k x one 128-byte
// chunk of Cin (64 16-bit or 32 32-bit channels).  K blocks whose offset has no neighbour in the
// whole tile are skipped (the tile's 128 x Kvol map slice is staged in shared memory first and
// OR-reduced into an offset mask), so the issued MMA work follows the sparsity of the map; with a
// row-sorted map the skipping gets coarser-grained and the output rows are scattered through
// reorder_loc.
//
// Operands of a K block (one pipeline stage, both 128B-swizzled K-major tiles):
//   A  128 gathered feature-row slices of 128 bytes (zeros for a missing neighbour), copied by
//      all eight gather warps with 16-byte cp.async, four per thread; each thread's arrival on the
//      stage's "full" barrier is attached to its copies (cp.async.mbarrier.arrive.noinc), so no
//      thread ever blocks on data.  The map entries are read into registers before the wait for
//      the stage, so the copies go out back to back once it is released.
//   B  one TMA tile copy of N_tile rows of the K-major packed weights, counted in bytes on the
//      same barrier.
//
// Roles (480 threads, persistent CTAs, one or two per SM):
//   warps 0-7   gather (A operand)
//   warps 8-11  epilogue: tcgen05.ld of their TMEM lane quarter, scale / bias / residual / ReLU,
//               rounding and 16-byte stores
//   warp 12     weight loader: one elected thread issues the TMA copies
//   warp 13     allocates TMEM; one elected thread issues tcgen05.mma (M=128, N=N_tile, 32 bytes of K
//               per instruction, 4 per stage) and releases stages / publishes accumulators with
//               tcgen05.commit.  Warps 12 and 13 run their loops converged and elect the issuing
//               lane per instruction, so that descriptors and coordinates stay warp-uniform.
//   warp 14     scheduler: takes the CTA's next work item from a global counter (tiles differ in how
//               many offsets they hold, so a fixed assignment would leave CTAs idle at the end), stages
//               its map slice and offset mask for the other roles
//
// Pair-list mode (the GatherScatter / FetchOnDemand dataflows, conv_pairs.cu): the map is one column of
// input rows, every 128-row tile belongs to one kernel offset (tile_k[tile] picks its weight block),
// and the fp32 products are either stored as rows of a buffer or added to the output rows with
// 16-byte atomic adds.
//
// Every wait on an mbarrier is bounded: when it runs out the thread records an error code and the
// CTA stops issuing work, gives its copies in flight time to land, frees its TMEM and returns.
#include <cuda.h>

#include <cstdlib>
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
constexpr int kTmaWarp = 12;
constexpr int kMmaWarp = 13;
constexpr int kSchedWarp = 14;
constexpr int kThreads = 480;
constexpr int kMaxRing = 4;            // tile ring: map slices + offset masks staged ahead of the other roles
constexpr int kMaxStages = 8;
constexpr int kMaxKvolUmma = 32;
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr uint64_t kWaitLimitNs = 2000000000ull;   // 2 s

enum { kErrFullWait = 1, kErrEmptyWait = 2, kErrAccWait = 3, kErrSchedWait = 4 };
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
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
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
  const void* x;        // [n_in, cin]
  const int* map;       // [pad128(n_out), kvol]
  const int* reorder;   // nullable
  void* y;              // [n_out, cout]
  const float* scale;   // nullable, fp32 [cout]: y = acc * scale + bias (+ residual), then ReLU
  const float* bias;    // nullable
  const void* residual; // nullable, [n_out, cout]
  int* error;           // device error word (0 = fine)
  int* sched;           // {next work item, CTAs finished}: both zero at launch, reset by the last CTA
  const int* tile_k;    // nullable ("pair list" mode): weight offset of each 128-row tile; the map is one column
  int dst_rows;         // rows of y (bound of the reorder scatter)
  int out_fp32;         // 16-bit operands, fp32 output rows (no residual)
  int atomic_out;       // fp32 output accumulated with atomic adds (rows may repeat between tiles)
  long long* trace;     // debugging aid (trace builds only)
  int trace_cta;
  int n_in, n_out, kvol, cin, cout;
  int n_tile;           // UMMA N of a full tile (multiple of 16, <= 256)
  int acc_cols;         // TMEM columns of one accumulator buffer (power of two >= n_tile, >= 32)
  int ring;             // tile ring depth (2..kMaxRing)
  int stages;
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

// TMA tile load of the weight block: box = 128 bytes of channels x n_tile rows of the packed
// weights, written 128B-swizzled; completion is counted in bytes on the mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// Persistent kernel: each CTA takes (row tile, N tile) work items from a shared counter until none is left.
// Three rings decouple the roles so that the copies of the next tile are in flight while the
// current tile is multiplied and the previous one is written out:
//   stage ring   (p.stages)  A+B operands of one K block         full[] / empty[]
//   tile ring    (p.ring)    work item, map slice + offset mask  sched_full[] / sched_empty[]
//   accumulator  (2)         TMEM column ranges                   acc_full[] / acc_empty[]
template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
igemm_umma_kernel(const UmmaParams p, const __grid_constant__ CUtensorMap w_map) {
  constexpr bool kTF32 = sizeof(T) == 4;
  constexpr int kChunk = kRowBytes / (int)sizeof(T);     // channels per stage row
  constexpr int kStepK = 32 / (int)sizeof(T);            // channels per MMA instruction (32 bytes of K)
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t s_full[kMaxStages];
  __shared__ uint64_t s_empty[kMaxStages];
  __shared__ uint64_t s_sched_full[kMaxRing];
  __shared__ uint64_t s_sched_empty[kMaxRing];
  __shared__ uint64_t s_acc_full[2];
  __shared__ uint64_t s_acc_empty[2];
  __shared__ uint32_t s_kmask[kMaxRing];
  __shared__ int s_tile[kMaxRing];       // work item of the ring slot; -1 = no more work
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) TSB_TRACE_HOT(7, 0);     // CTA entry
  const int tiles_n = (p.cout + p.n_tile - 1) / p.n_tile;
  const int tiles_m = (p.n_out + kTileM - 1) / kTileM;
  const int n_work = tiles_m * tiles_n;
  const int b_bytes = p.n_tile * kRowBytes;
  const int stage_bytes = kABytes + b_bytes;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t map_smem = smem_base + (uint32_t)p.stages * stage_bytes;
  const int map_ints = kTileM * p.kvol;
  int* s_map0 = reinterpret_cast<int*>(smem_raw + (map_smem - smem_u32(smem_raw)));
  const uint32_t acc_cols = p.acc_cols;            // TMEM columns of one accumulator (power of two)
  const int chunks = (p.cin + kChunk - 1) / kChunk;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      // every gather thread (attached to its copies) + the weight loader's arrive.expect_tx
      mbar_init(smem_u32(&s_full[s]), kGatherThreads + 1);
      mbar_init(smem_u32(&s_empty[s]), 1);   // tcgen05.commit
    }
    for (int b = 0; b < p.ring; ++b) {
      mbar_init(smem_u32(&s_sched_full[b]), 1);
      // readers of a ring slot: gather warps, weight loader, MMA warp, epilogue warps
      mbar_init(smem_u32(&s_sched_empty[b]), kGatherWarps + 2 + kEpilogueWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_acc_full[b]), 1);
      mbar_init(smem_u32(&s_acc_empty[b]), kEpilogueWarps);
    }
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) tmem_alloc(smem_u32(&s_tmem), 2 * acc_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  if (warp < kGatherWarps) {
    // ------------------------------------------------------------ gather warps (A operand)
    // Thread t copies the 16-byte granule (t & 7) of rows (t >> 3) + 32 j, j = 0..3, of every K block:
    // a warp instruction covers four whole 128-byte row slices.  The four map entries of an offset
    // are read once, before the wait for the stage, and serve all channel chunks of that offset.
    constexpr int kGran = 16 / (int)sizeof(T);                     // channels per 16-byte granule
    const T* x = reinterpret_cast<const T*>(p.x);
    const int gran = tid & 7;
    const int rbase = tid >> 3;
    const uint32_t dst_off = (uint32_t)rbase * kRowBytes + (uint32_t)((gran ^ (rbase & 7)) << 4);
    const uint32_t full0 = smem_u32(&s_full[0]), empty0 = smem_u32(&s_empty[0]);
    const int mrow = kRowsPerPass * p.kvol;                        // map ints between a thread's rows
    const int cin_mma = (p.cin + kStepK - 1) / kStepK * kStepK;     // K extent the MMAs read
    uint32_t stage = 0, phase = 0;      // stage of the current block; phase = parity of its use count
    bool first_pass = true;              // the first use of a stage needs no release
    bool ok = true;
    int i = 0;
#ifdef TSB_TRACE_BUILD
    int blk = 0;
#endif
    for (;; ++i) {
      const int buf = i % p.ring;
      const uint32_t use_parity = (uint32_t)(i / p.ring) & 1u;
      const int* mp = s_map0 + buf * map_ints + rbase * p.kvol;
      if (!mbar_wait_warp(smem_u32(&s_sched_full[buf]), use_parity, lane)) {
        atomicExch(p.error, kErrSchedWait);
        s_abort = 1;
        break;
      }
      if (s_abort || s_tile[buf] < 0) break;
      const uint32_t kmask = s_kmask[buf];
      for (int k = 0; k < p.kvol && ok; ++k) {
        if (!((kmask >> k) & 1u)) continue;
        int src[kCopies];
#pragma unroll
        for (int j = 0; j < kCopies; ++j) src[j] = mp[j * mrow + k];
        for (int c = 0; c < chunks; ++c) {
          const int col = c * kChunk + gran * kGran;
          const bool col_ok = col < p.cin;                          // rows are 16-byte multiples: all-in or all-out
          const T* xc = x + col;
          if (tid == 0) TSB_TRACE_HOT(0, blk);
          if (!first_pass && !mbar_wait_warp(empty0 + stage * 8, phase ^ 1u, lane)) {
            atomicExch(p.error, kErrEmptyWait);
            s_abort = 1;
            ok = false;
            break;
          }
          if (tid == 0) TSB_TRACE_HOT(1, blk);
          const uint32_t a_dst = smem_base + stage * (uint32_t)stage_bytes + dst_off;
          // granules beyond the K extent of the chunk's last MMA (Cin rounded up to one instruction's K) are
          // never read: their threads copy nothing and only arrive; granules between Cin and that bound are
          // zero-filled (the weights there are zero, but stale shared memory could hold NaN patterns)
          if (col < cin_mma) {
#pragma unroll
            for (int j = 0; j < kCopies; ++j) {
              const bool live = col_ok && src[j] >= 0;
              cp_async16(a_dst + (uint32_t)(j * kRowsPerPass) * kRowBytes,
                         live ? (const void*)(xc + (int64_t)src[j] * p.cin) : (const void*)x, live ? 16u : 0u);
            }
          }
          cp_async_arrive_noinc(full0 + stage * 8);
          if (tid == 0) TSB_TRACE_HOT(2, blk);
#ifdef TSB_TRACE_BUILD
          ++blk;
#endif
          if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; first_pass = false; }
        }
      }
      if (!ok) break;
      __syncwarp();   // every lane has read its rows of the slice
      if (lane == 0) mbar_arrive(smem_u32(&s_sched_empty[buf]));
    }
    cp_async_wait_all();   // nothing of this thread may still be writing shared memory at exit
  } else if (warp < kGatherWarps + kEpilogueWarps) {
    // ------------------------------------------------------------ epilogue warps
    // warp q reads TMEM lanes 32 q .. 32 q + 31 = its 32 output rows, all columns of the tile
    const int quarter = warp & 3;
    T* y = reinterpret_cast<T*>(p.y);
    const T* res = reinterpret_cast<const T*>(p.residual);
    int i = 0;
    int acc_count = 0;   // tiles that used an accumulator so far (tiles with an empty mask use none)
    bool ok = true;
    for (;; ++i) {
      const int buf = i % p.ring;
      if (!mbar_wait_warp(smem_u32(&s_sched_full[buf]), (uint32_t)(i / p.ring) & 1u, lane)) {
        atomicExch(p.error, kErrSchedWait);
        s_abort = 1;
        break;
      }
      const int w = s_tile[buf];
      if (s_abort || w < 0) break;
      const uint32_t kmask = s_kmask[buf];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_sched_empty[buf]));
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
      const int r = quarter * 32 + lane;
      const int64_t grow = (int64_t)row0 + r;
      int64_t dst_row = -1;
      if (grow < p.n_out) {
        dst_row = p.reorder ? (int64_t)__ldg(&p.reorder[grow]) : grow;
        if (dst_row >= p.dst_rows) dst_row = -1;
      }
      const uint32_t acc_addr = tmem_base + (uint32_t)ab * acc_cols + ((uint32_t)(quarter * 32) << 16);
      for (int j = 0; j < n_mma; j += 16) {
        // the accumulator load is in flight while the per-channel constants and the residual are fetched
        uint32_t v[16];
        if (have_acc) {
          tmem_ld16(acc_addr + (uint32_t)j, v);
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = 0u;
        }
        const int n = n0 + j;
        const bool ok8[2] = {dst_row >= 0 && n < p.cout, dst_row >= 0 && n + 8 < p.cout};   // cout % 8 == 0
        // residual of the 16 channels, still packed (fp32: fetched per half below)
        uint4 rv[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
        if constexpr (!kTF32) {
          if (res) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
              if (ok8[h]) rv[h] = __ldg(reinterpret_cast<const uint4*>(res + dst_row * p.cout + n) + h);
          }
        }
        if (have_acc) tmem_ld_wait16(v);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!ok8[h]) continue;
          const int nh = n + 8 * h;
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[8 * h + e]);
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
              const uint32_t* rw = reinterpret_cast<const uint32_t*>(&rv[h]);
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
        }
      }
      if (warp == kGatherWarps && lane == 0) TSB_TRACE_HOT(7, i + 1);   // tile i written out (first epilogue warp)
      // this warp is done with the accumulator buffer
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && have_acc) mbar_arrive(smem_u32(&s_acc_empty[ab]));
      if (have_acc) ++acc_count;
    }
  } else if (warp == kSchedWarp) {
    // ------------------------------------------------------------ scheduler warp
    // stages the map slice of each tile (128 rows x kvol ints, contiguous, 16-byte loads) into the
    // tile ring and publishes its offset mask, up to `ring` tiles ahead of the other roles
    const int n4 = map_ints / 4;
    int i = 0;
    for (;; ++i) {
      const int buf = i % p.ring;
      if (i >= p.ring && !mbar_wait_warp(smem_u32(&s_sched_empty[buf]), ((uint32_t)(i / p.ring) + 1u) & 1u, lane)) {
        atomicExch(p.error, kErrSchedWait);
        s_abort = 1;
        break;
      }
      int w = 0;
      if (lane == 0) w = atomicAdd(p.sched, 1);
      w = __shfl_sync(0xffffffffu, w, 0);
      if (w >= n_work || s_abort) {
        // tell the other roles that the CTA is done
        if (lane == 0) {
          s_tile[buf] = -1;
          mbar_arrive(smem_u32(&s_sched_full[buf]));
        }
        break;
      }
      const int row0 = (w / tiles_n) * kTileM;
      // all 16-byte copies of the slice go out before any of them is waited for: the slice costs one
      // memory round trip, not one per few loads
      const int4* src = reinterpret_cast<const int4*>(p.map + (int64_t)row0 * p.kvol);
      int4* dst = reinterpret_cast<int4*>(s_map0 + buf * map_ints);
      const uint32_t dst_s = map_smem + (uint32_t)(buf * map_ints) * 4u;
      for (int e = lane; e < n4; e += 32) cp_async16(dst_s + (uint32_t)e * 16u, src + e, 16u);
      cp_async_wait_all();
      __syncwarp();
      uint32_t mine = 0;
      int kk = (lane * 4) % p.kvol;                 // kernel offset of the first int of this lane's int4
      const int kstep = 128 % p.kvol;               // advance of that offset per loop trip (32 lanes x 4 ints)
#pragma unroll 4
      for (int e = lane; e < n4; e += 32) {
        int4 v = dst[e];
        int* c = reinterpret_cast<int*>(&v);
        int k = kk;
        bool changed = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (c[j] >= p.n_in) { c[j] = -1; changed = true; }   // defensive: an index beyond the features reads nothing
          if (c[j] >= 0) mine |= 1u << k;
          k = (k + 1 == p.kvol) ? 0 : k + 1;
        }
        if (changed) dst[e] = v;
        kk += kstep;
        if (kk >= p.kvol) kk -= p.kvol;
      }
      for (int o = 16; o; o >>= 1) mine |= __shfl_xor_sync(0xffffffffu, mine, o);
      __syncwarp();
      if (lane == 0) {
        s_kmask[buf] = mine;
        s_tile[buf] = w;
        mbar_arrive(smem_u32(&s_sched_full[buf]));
      }
    }
  } else if (warp == kTmaWarp) {
    // ------------------------------------------------------------ weight loader (B operand)
    // the whole warp walks the blocks converged; one elected lane posts the byte count and issues the copy
    const uint32_t bytes = (uint32_t)b_bytes;
    const uint32_t full0 = smem_u32(&s_full[0]), empty0 = smem_u32(&s_empty[0]);
    uint32_t stage = 0, phase = 0;
    bool first_pass = true;
    int i = 0;
    bool ok = true;
    for (; ok; ++i) {
      const int buf = i % p.ring;
      if (!mbar_wait(smem_u32(&s_sched_full[buf]), (uint32_t)(i / p.ring) & 1u)) {
        if (lane == 0) atomicExch(p.error, kErrSchedWait);
        s_abort = 1;
        break;
      }
      const int w = s_tile[buf];
      if (s_abort || w < 0) break;
      const uint32_t kmask = s_kmask[buf];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_sched_empty[buf]));
      const int n0 = (w % tiles_n) * p.n_tile;
      for (int k = 0; k < p.kvol && ok; ++k) {
        if (!((kmask >> k) & 1u)) continue;
        // pair-list mode: the tile's rows all belong to one kernel offset, named by tile_k
        const int wrow = (p.tile_k ? __ldg(&p.tile_k[w / tiles_n]) : k) * p.cout + n0;
        for (int c = 0; c < chunks; ++c) {
          if (!first_pass && !mbar_wait(empty0 + stage * 8, phase ^ 1u)) {
            if (lane == 0) atomicExch(p.error, kErrEmptyWait);
            s_abort = 1;
            ok = false;
            break;
          }
          const uint32_t bar = full0 + stage * 8;
          if (elect_one()) {
            mbar_arrive_expect_tx(bar, bytes);
            tma_load_2d(smem_base + stage * (uint32_t)stage_bytes + kABytes, &w_map, bar, c * kChunk, wrow);
          }
          __syncwarp();
          if (++stage == (uint32_t)p.stages) { stage = 0; phase ^= 1u; first_pass = false; }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    // The instruction stream of this warp is on the critical path of the whole CTA: stage index,
    // barrier phase and descriptors are carried incrementally (no division, no 64-bit arithmetic per
    // block), and the warp stays converged so that they are warp-uniform values.
    const uint32_t full0 = smem_u32(&s_full[0]), empty0 = smem_u32(&s_empty[0]);
    const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, SWIZZLE_128B
    const uint32_t a_lo0 = ((smem_base >> 4) & 0x3FFFu) | (1u << 16);  // stage 0, A operand
    const uint32_t stage_units = (uint32_t)stage_bytes >> 4;
    const uint32_t b_units = (uint32_t)kABytes >> 4;
    const int last_steps = ((p.cin - (chunks - 1) * kChunk) + kStepK - 1) / kStepK;
    uint32_t stage = 0, phase = 0, a_lo = a_lo0;
    int i = 0, acc_count = 0;
    bool ok = true;
#ifdef TSB_TRACE_BUILD
    int blk = 0;
#endif
    for (; ok; ++i) {
      const int buf = i % p.ring;
      if (!mbar_wait(smem_u32(&s_sched_full[buf]), (uint32_t)(i / p.ring) & 1u)) {
        if (lane == 0) atomicExch(p.error, kErrSchedWait);
        s_abort = 1;
        break;
      }
      const int w = s_tile[buf];
      if (s_abort || w < 0) break;
      const uint32_t kmask = s_kmask[buf];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_sched_empty[buf]));
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
        for (int c = 0; c < chunks; ++c) {
          if (lane == 0) TSB_TRACE_HOT(4, blk);
          if (!mbar_wait(full0 + stage * 8, phase)) {
            if (lane == 0) atomicExch(p.error, kErrFullWait);
            s_abort = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) TSB_TRACE_HOT(5, blk);
          const int steps = (c == chunks - 1) ? last_steps : 4;
          if (elect_one()) {
            // +32 bytes along K inside the swizzle atom = +2 in the descriptor's 16-byte address units
#pragma unroll
            for (int st = 0; st < 4; ++st) {
              if (st < steps) {
                const uint64_t a_desc = ((uint64_t)desc_hi << 32) | (a_lo + 2u * st);
                const uint64_t b_desc = ((uint64_t)desc_hi << 32) | (a_lo + b_units + 2u * st);
                umma<kTF32>(acc, a_desc, b_desc, idesc, (st == 0) ? accumulate : 1u);
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
  if (tid == 0) TSB_TRACE_HOT(3, 0);     // CTA exit
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

// Scheduling words, one slot per stream: launches on one stream run one after another, so they can share
// a slot (zero-initialised, and every launch zeroes it again when its last CTA leaves); launches on
// different streams may overlap and get different slots.
constexpr int kSchedSlots = 1024;
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

size_t smem_bytes_for(int n_tile, int stages, int kvol, int ring) {
  return 1024 + (size_t)stages * (kABytes + (size_t)n_tile * kRowBytes) + (size_t)ring * kTileM * kvol * sizeof(int);
}

int usable_stages(int s) { return s > kMaxStages ? kMaxStages : s; }

// Two persistent CTAs per SM when two double-buffered accumulators fit TMEM (N tile <= 128 columns)
// and three stages fit half the shared memory: two MMA issuers per SM hide the per-block latency
// of the narrow layers.  Otherwise one CTA per SM with as many stages as fit.
void pick_config(int n_tile, int kvol, int* stages, int* ring, int* ctas) {
  int acc_cols = 32;
  while (acc_cols < n_tile) acc_cols <<= 1;
  if (acc_cols <= 128) {
    const size_t half = 112 * 1024;
    int best = 0;
    for (int s = 2; s <= kMaxStages; ++s)
      if (smem_bytes_for(n_tile, s, kvol, 2) <= half) best = s;
    if (best >= 3) { *stages = usable_stages(best); *ring = 2; *ctas = 2; return; }
  }
  const size_t budget = 226 * 1024;
  int best[2] = {0, 0};
  for (int r = 2; r <= 3; ++r)
    for (int s = 2; s <= kMaxStages; ++s)
      if (smem_bytes_for(n_tile, s, kvol, r) <= budget) best[r - 2] = usable_stages(s);
  *ctas = 1;
  if (best[0] > best[1]) { *stages = best[0]; *ring = 2; }
  else { *stages = best[1]; *ring = 3; }
}

// scheduling words of `stream` on the current device (the array's address is looked up once per device,
// a stream gets the next free slot the first time it launches a convolution)
int* sched_slot_of(cudaStream_t stream) {
  static std::mutex mu;
  static int* addr[64] = {nullptr};
  static std::map<std::pair<int, cudaStream_t>, int> slot_of;
  static int next_slot[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_sched_slots) != cudaSuccess) return nullptr;
    addr[dev] = reinterpret_cast<int*>(ptr);
  }
  auto it = slot_of.find({dev, stream});
  if (it == slot_of.end()) it = slot_of.emplace(std::make_pair(dev, stream), next_slot[dev]++ % kSchedSlots).first;
  return addr[dev] + 2 * it->second;
}

int num_sms() {
  static int n = []() {
    int dev = 0, v = kSmCount;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : kSmCount;
  }();
  return n;
}

int pick_n_tile(int cout) {
  int n = (cout + 15) & ~15;
  return n > 256 ? 256 : n;
}

}  // namespace

bool igemm_umma_supported(const IgemmArgs& a) {
  if (!tensor_map_encoder()) return false;
  if ((a.kvol * kTileM) % 4 || ((uintptr_t)a.map & 15)) return false;
  if (a.dtype == TSB_F32) {
    if (a.math != TSB_MATH_TF32) return false;       // exact fp32 stays on the CUDA cores
  } else if (a.dtype != TSB_F16 && a.dtype != TSB_BF16) {
    return false;
  }
  // feature rows must be 16-byte multiples (tensor-map stride); outputs are written in 8-channel groups
  if ((a.cin * (int)dtype_size(a.dtype)) % 16 || a.cout % 8) return false;
  if (a.n_in >= (int64_t)INT32_MAX || a.n_out >= (int64_t)INT32_MAX) return false;
  if (a.kvol > kMaxKvolUmma) return false;            // one bit per map column in a tile's offset mask
  if (a.tile_k && a.kvol != 1) return false;          // pair-list mode: one map column, weights chosen per tile
  if (a.out_fp32 && a.residual) return false;
  if (((uintptr_t)a.x | (uintptr_t)a.y | (uintptr_t)a.w | (uintptr_t)a.residual | (uintptr_t)a.packed_w) & 15)
    return false;
  int st = 0, rg = 0, ct = 0;
  pick_config(pick_n_tile(a.cout), a.kvol, &st, &rg, &ct);
  return st >= 2;
}

size_t packed_weight_bytes(int kvol, int cin, int cout, int dtype) {
  return align_up((size_t)kvol * cin * cout * dtype_size(dtype), 256);
}

size_t igemm_umma_workspace_bytes(int kvol, int cin, int cout, int dtype) {
  return packed_weight_bytes(kvol, cin, cout, dtype) + 256;   // packed weights + error word
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
  if (!wt || !err) {
    if (!a.workspace || a.workspace_bytes < w_bytes + 256) return TSB_ERR_WORKSPACE;
  }
  if (!err) {
    err = reinterpret_cast<int*>(reinterpret_cast<char*>(a.workspace) + w_bytes);
    TSB_CUDA_TRY(cudaMemsetAsync(err, 0, sizeof(int), s));
  }
  if (!wt) {
    int rc = pack_launch<T>(a.w, kvol_w, a.cin, a.cout, a.workspace, s);
    if (rc != TSB_OK) return rc;
    wt = reinterpret_cast<const T*>(a.workspace);
  }
  UmmaParams p;
  p.x = a.x; p.map = a.map; p.reorder = a.reorder_loc; p.y = a.y; p.bias = a.bias; p.scale = a.scale;
  p.residual = a.residual; p.error = err;
  p.tile_k = a.tile_k; p.out_fp32 = a.out_fp32; p.atomic_out = a.atomic_out;
  p.dst_rows = (int)(a.dst_rows > 0 ? a.dst_rows : a.n_out);
  p.sched = sched_slot_of(s);
  if (!p.sched) return TSB_ERR_CUDA;
  p.trace = nullptr; p.trace_cta = 0;
  if (const char* tr = getenv("TSB_UMMA_TRACE")) {   // debugging aid: address of a 256x8 int64 device buffer
    p.trace = reinterpret_cast<long long*>(strtoull(tr, nullptr, 0));
    if (const char* tc = getenv("TSB_UMMA_TRACE_CTA")) p.trace_cta = atoi(tc);
  }
  p.n_in = (int)a.n_in; p.n_out = (int)a.n_out; p.kvol = a.kvol; p.cin = a.cin; p.cout = a.cout;
  p.n_tile = pick_n_tile(a.cout);
  int ctas = 1;
  pick_config(p.n_tile, a.kvol, &p.stages, &p.ring, &ctas);
  p.relu = a.relu;
  p.ab_format = (a.dtype == TSB_BF16) ? kFmtBF16 : (a.dtype == TSB_F32) ? kFmtTF32 : kFmtF16;
  const size_t smem = smem_bytes_for(p.n_tile, p.stages, a.kvol, p.ring);
  static bool attr_set[3] = {false, false, false};
  const int ti = p.ab_format;
  if (!attr_set[ti]) {
    TSB_CUDA_TRY(cudaFuncSetAttribute(igemm_umma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    attr_set[ti] = true;
  }
  CUtensorMap w_map;
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
    cuuint32_t box[2] = {chunk, (cuuint32_t)p.n_tile};
    CUresult r = encode(&w_map, dt, 2, const_cast<T*>(wt), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return TSB_ERR_BAD_ARG;
  }
  p.acc_cols = 32;
  while (p.acc_cols < p.n_tile) p.acc_cols <<= 1;
  const int64_t n_work = cdiv(a.n_out, kTileM) * cdiv(a.cout, p.n_tile);
  const int64_t slots = (int64_t)ctas * num_sms();
  const int grid = (int)(n_work < slots ? n_work : slots);
  igemm_umma_kernel<T><<<grid, kThreads, smem, s>>>(p, w_map);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int igemm_umma(const IgemmArgs& a, cudaStream_t s) {
  if (a.dtype == TSB_F16) return umma_launch<__half>(a, s);
  if (a.dtype == TSB_BF16) return umma_launch<__nv_bfloat16>(a, s);
  if (a.dtype == TSB_F32 && a.math == TSB_MATH_TF32) return umma_launch<float>(a, s);
  return TSB_ERR_UNSUPPORTED;
}

}  // namespace tsb
