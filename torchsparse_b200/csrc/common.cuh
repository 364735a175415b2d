// Shared helpers of the tsb200 library: status plumbing, launch geometry, the
// ravel index and the bounded-probe hash table used by every kernel-map kernel.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tsb200.h"

namespace tsb {

void set_cuda_error(cudaError_t e);  // records the message returned by tsb_last_cuda_error()

inline cudaStream_t as_stream(tsb_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

#define TSB_CUDA_TRY(expr)                 \
  do {                                     \
    cudaError_t _e = (expr);               \
    if (_e != cudaSuccess) {               \
      ::tsb::set_cuda_error(_e);           \
      return TSB_ERR_CUDA;                 \
    }                                      \
  } while (0)

void count_launch(int n = 1);  // bumps the counter read by tsb_launch_count()

#define TSB_LAUNCH_CHECK()                  \
  do {                                      \
    ::tsb::count_launch();                  \
    TSB_CUDA_TRY(cudaPeekAtLastError());    \
  } while (0)

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t pad128(int64_t n) { return cdiv(n, 128) * 128; }

constexpr int kSmCount = 148;  // B200: grids of grid-stride kernels are sized in multiples of this

// grid for a grid-stride kernel: enough blocks to cover `work` items, capped at a
// few waves of the machine.
inline int grid_for(int64_t work, int block, int max_blocks_per_sm = 16) {
  int64_t g = cdiv(work, block);
  int64_t cap = (int64_t)kSmCount * max_blocks_per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

// ---------------------------------------------------------------------------
// Ravel index of (b,x,y,z) with inclusive bounds; radices = max - min + 1.
struct Bounds {
  int mn[4];
  int mx[4];
  int sz[4];
};

inline Bounds make_bounds(const int32_t* cmin, const int32_t* cmax) {
  Bounds b;
  for (int i = 0; i < 4; ++i) {
    b.mn[i] = cmin[i];
    b.mx[i] = cmax[i];
    b.sz[i] = cmax[i] - cmin[i] + 1;
  }
  return b;
}

__host__ __device__ inline int64_t ravel4(const Bounds& b, int c0, int c1, int c2, int c3) {
  int64_t cur = (int64_t)(c0 - b.mn[0]);
  cur = cur * b.sz[1] + (c1 - b.mn[1]);
  cur = cur * b.sz[2] + (c2 - b.mn[2]);
  cur = cur * b.sz[3] + (c3 - b.mn[3]);
  return cur;
}

__host__ __device__ inline bool in_bounds_xyz(const Bounds& b, int x, int y, int z) {
  return x >= b.mn[1] && x <= b.mx[1] && y >= b.mn[2] && y <= b.mx[2] && z >= b.mn[3] && z <= b.mx[3];
}

// ---------------------------------------------------------------------------
// Open-addressing table over caller-owned arrays, in one of two layouts:
//   64-bit keys   keys int64[cap] (0 = empty) + vals int32[cap]; a probe reads the key word and, on a hit, the value
//   32-bit keys   vals == nullptr: keys[] holds cap packed slots, value << 32 | key (0 = empty), for key spaces below
//                 2^32; insert is one compare-and-swap of the whole slot, a probe one 8-byte load
struct TableView {
  unsigned long long* keys;
  int* vals;
  unsigned long long cap;
  unsigned long long mask;  // cap-1 when cap is a power of two, else 0
};

inline TableView make_table(int64_t* keys, int32_t* vals, int64_t cap) {
  TableView t;
  t.keys = reinterpret_cast<unsigned long long*>(keys);
  t.vals = vals;
  t.cap = (unsigned long long)cap;
  t.mask = ((cap & (cap - 1)) == 0) ? (unsigned long long)(cap - 1) : 0ull;
  return t;
}

// largest key a table of packed slots can hold
constexpr unsigned long long kPackedKeyMax = 0xffffffffull;

__device__ __forceinline__ unsigned long long mix64(unsigned long long k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return k;
}

__device__ __forceinline__ unsigned long long table_slot(const TableView& t, unsigned long long key) {
  unsigned long long h = mix64(key);
  return t.mask ? (h & t.mask) : (h % t.cap);
}

__device__ __forceinline__ unsigned long long table_next(const TableView& t, unsigned long long slot) {
  ++slot;
  return slot == t.cap ? 0ull : slot;
}

// 0 = stored; TSB_DEV_TABLE_FULL when every slot was probed without finding room; TSB_DEV_LIMIT when the key does
// not fit a packed slot.  key > 0.
__device__ __forceinline__ int table_insert(const TableView& t, unsigned long long key, int val) {
  unsigned long long slot = table_slot(t, key);
  if (!t.vals) {
    if (key > kPackedKeyMax) return TSB_DEV_LIMIT;
    const unsigned long long word = ((unsigned long long)(unsigned)val << 32) | key;
    for (unsigned long long probe = 0; probe < t.cap; ++probe) {
      const unsigned long long prev = atomicCAS(&t.keys[slot], 0ull, word);
      if (prev == 0ull) return 0;
      if ((prev & kPackedKeyMax) == key) {     // the key is there already: the later value stays, as in the other layout
        t.keys[slot] = word;
        return 0;
      }
      slot = table_next(t, slot);
    }
    return TSB_DEV_TABLE_FULL;
  }
  for (unsigned long long probe = 0; probe < t.cap; ++probe) {
    unsigned long long prev = atomicCAS(&t.keys[slot], 0ull, key);
    if (prev == 0ull || prev == key) {
      t.vals[slot] = val;
      return 0;
    }
    slot = table_next(t, slot);
  }
  return TSB_DEV_TABLE_FULL;
}

// 0 = not found.
__device__ __forceinline__ int table_lookup(const TableView& t, unsigned long long key) {
  unsigned long long slot = table_slot(t, key);
  if (!t.vals) {
    if (key > kPackedKeyMax) return 0;
    for (unsigned long long probe = 0; probe < t.cap; ++probe) {
      const unsigned long long cur = __ldg(&t.keys[slot]);
      if ((cur & kPackedKeyMax) == key) return (int)(cur >> 32);
      if (cur == 0ull) return 0;
      slot = table_next(t, slot);
    }
    return 0;
  }
  for (unsigned long long probe = 0; probe < t.cap; ++probe) {
    unsigned long long cur = __ldg(&t.keys[slot]);
    if (cur == key) return __ldg(&t.vals[slot]);
    if (cur == 0ull) return 0;
    slot = table_next(t, slot);
  }
  return 0;
}

// The rest of a lookup whose first probe (slot = table_slot(t, key), cur = the word read there) the caller has
// already made, so that several lookups of one thread can have their first loads in flight together.
__device__ __forceinline__ int table_lookup_after(const TableView& t, unsigned long long key, unsigned long long slot,
                                                  unsigned long long cur) {
  if (!t.vals) {
    if (key > kPackedKeyMax) return 0;
    for (unsigned long long probe = 0; probe < t.cap; ++probe) {
      if ((cur & kPackedKeyMax) == key) return (int)(cur >> 32);
      if (cur == 0ull) return 0;
      slot = table_next(t, slot);
      cur = __ldg(&t.keys[slot]);
    }
    return 0;
  }
  for (unsigned long long probe = 0; probe < t.cap; ++probe) {
    if (cur == key) return __ldg(&t.vals[slot]);
    if (cur == 0ull) return 0;
    slot = table_next(t, slot);
    cur = __ldg(&t.keys[slot]);
  }
  return 0;
}

// Kernel geometry passed by value to the map kernels.
struct KernelGeom {
  int ks[3];
  int st[3];
  int pd[3];
  int kvol;
  int odd;  // kernel volume is odd -> x is the fastest digit
};

inline KernelGeom make_geom(const int32_t* ks, const int32_t* st, const int32_t* pd) {
  KernelGeom g;
  for (int i = 0; i < 3; ++i) {
    g.ks[i] = ks[i];
    g.st[i] = st ? st[i] : 1;
    g.pd[i] = pd ? pd[i] : 0;
  }
  g.kvol = ks[0] * ks[1] * ks[2];
  g.odd = g.kvol & 1;
  return g;
}

// digits (dx,dy,dz) of kernel index k
__device__ __forceinline__ void kernel_digits(const KernelGeom& g, int k, int& dx, int& dy, int& dz) {
  if (g.odd) {
    dx = k % g.ks[0];
    k /= g.ks[0];
    dy = k % g.ks[1];
    dz = k / g.ks[1];
  } else {
    dz = k % g.ks[2];
    k /= g.ks[2];
    dy = k % g.ks[1];
    dx = k / g.ks[1];
  }
}

template <typename T>
struct DTypeOf;
template <>
struct DTypeOf<float> { static constexpr int value = TSB_F32; };
template <>
struct DTypeOf<__half> { static constexpr int value = TSB_F16; };
template <>
struct DTypeOf<__nv_bfloat16> { static constexpr int value = TSB_BF16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

inline size_t dtype_size(int dtype) { return dtype == TSB_F32 ? 4 : 2; }

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace tsb
