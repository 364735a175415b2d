// Coordinate hashing, the GPU hash table and kernel-map construction
// (submanifold, strided, transposed) plus the sorted-map artefacts and the pair
// lists of the GatherScatter / FetchOnDemand dataflows.
//
// All of this is integer, HBM/L2-latency bound work: one pass over the coordinates
// and one write of the map, with random 8-byte probes into an L2-resident table.
#include <cub/cub.cuh>

#include <mutex>

#include "common.cuh"

namespace tsb {

namespace {

constexpr int kBlock = 256;

// ------------------------------------------------------------------ hashing
__device__ __forceinline__ uint64_t fnv1a4(int c0, int c1, int c2, int c3) {
  uint64_t h = 14695981039346656037ULL;
  h ^= (unsigned int)c0; h *= 1099511628211ULL;
  h ^= (unsigned int)c1; h *= 1099511628211ULL;
  h ^= (unsigned int)c2; h *= 1099511628211ULL;
  h ^= (unsigned int)c3; h *= 1099511628211ULL;
  return h;
}

__global__ void coord_hash_kernel(const int4* __restrict__ coords, int64_t n, int64_t* __restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int4 c = __ldg(&coords[i]);
    out[i] = (int64_t)fnv1a4(c.x, c.y, c.z, c.w);
  }
}

// one thread per coordinate; the k hashes of a coordinate are written with stride n so
// that each warp stores 256 contiguous bytes per offset.
__global__ void kernel_hash_kernel(const int4* __restrict__ coords, int64_t n, const int* __restrict__ offsets,
                                   int k, int64_t* __restrict__ out) {
  extern __shared__ int s_off[];
  for (int i = threadIdx.x; i < k * 3; i += blockDim.x) s_off[i] = offsets[i];
  __syncthreads();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int4 c = __ldg(&coords[i]);
    for (int j = 0; j < k; ++j) {
      out[(int64_t)j * n + i] = (int64_t)fnv1a4(c.x, c.y + s_off[j * 3], c.z + s_off[j * 3 + 1], c.w + s_off[j * 3 + 2]);
    }
  }
}

// ------------------------------------------------------------------ table
__global__ void table_insert_kernel(TableView t, const int64_t* __restrict__ keys, int64_t n, int* status) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    { const int e = table_insert(t, (unsigned long long)keys[i], (int)(i + 1)); if (e && status) atomicOr(status, e); }
  }
}

__global__ void table_lookup_kernel(TableView t, const int64_t* __restrict__ keys, int64_t n, int* __restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    out[i] = table_lookup(t, (unsigned long long)keys[i]);
  }
}

__global__ void table_query_kernel(TableView t, const int64_t* __restrict__ keys, int64_t n, int64_t* __restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    out[i] = (int64_t)table_lookup(t, (unsigned long long)keys[i]) - 1;
  }
}

// ------------------------------------------------------------------ submanifold map
// Insert every coordinate (key = ravel+1, value = row+1) and fill the map with -1.
// The fill is block-cooperative: a block owns kBlock consecutive rows, i.e. one
// contiguous range of kBlock*kvol ints.
__global__ void subm_insert_fill_kernel(TableView t, const int4* __restrict__ coords, int64_t n, int64_t rows_pad,
                                        Bounds b, int kvol, int to_insert, int* __restrict__ map, int* status) {
  int64_t row0 = (int64_t)blockIdx.x * kBlock;
  int64_t row = row0 + threadIdx.x;
  if (to_insert && row < n) {
    int4 c = __ldg(&coords[row]);
    int64_t key = ravel4(b, c.x, c.y, c.z, c.w);
    { const int e = table_insert(t, (unsigned long long)(key + 1), (int)(row + 1)); if (e && status) atomicOr(status, e); }
  }
  int64_t lo = row0 * kvol;
  int64_t hi = min(row0 + kBlock, rows_pad) * (int64_t)kvol;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kBlock) map[i] = -1;
}

// Odd kernel volume: thread per (row, k < kvol/2); hit -> write [row][k] and the mirrored
// [nbr][kvol-1-k].  Thread k == 0 of a row also writes the centre column.
__global__ void subm_query_odd_kernel(TableView t, const int4* __restrict__ coords, int64_t n, Bounds b,
                                      KernelGeom g, int* __restrict__ map) {
  const int half = g.kvol / 2;
  const int64_t total = n * (int64_t)max(half, 1);
  for (int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; tid < total;
       tid += (int64_t)gridDim.x * blockDim.x) {
    int64_t row = half ? tid / half : tid;
    int k = half ? (int)(tid - row * half) : 0;
    if (k == 0) map[row * g.kvol + half] = (int)row;
    if (!half) continue;
    int dx, dy, dz;
    kernel_digits(g, k, dx, dy, dz);
    int4 c = __ldg(&coords[row]);
    int x = c.y + dx - (g.ks[0] - 1) / 2;
    int y = c.z + dy - (g.ks[1] - 1) / 2;
    int z = c.w + dz - (g.ks[2] - 1) / 2;
    if (!in_bounds_xyz(b, x, y, z)) continue;
    int64_t key = ravel4(b, c.x, x, y, z);
    int nbr = table_lookup(t, (unsigned long long)(key + 1)) - 1;
    if (nbr >= 0) {
      map[row * g.kvol + k] = nbr;
      map[(int64_t)nbr * g.kvol + (g.kvol - 1 - k)] = (int)row;
    }
  }
}

// "hashmap" kernel-map mode: the table is keyed by the FNV-1a hash of (x, y, z, b); for output row i and
// kernel index k the neighbour is  out * stride + digit - (kernel - 1) / 2  (x the fastest digit for an
// odd kernel volume, z for an even one); out[i][k] = stored value (input row + 1) or 0.
__global__ void lookup_coords_kernel(TableView t, const int4* __restrict__ coords_xyzb, int64_t n, KernelGeom g,
                                     int* __restrict__ out) {
  const int64_t total = n * (int64_t)g.kvol;
  for (int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; tid < total;
       tid += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = tid / g.kvol;
    const int k = (int)(tid - row * g.kvol);
    int d[3];
    kernel_digits(g, k, d[0], d[1], d[2]);
    const int4 c = __ldg(&coords_xyzb[row]);
    const int x = c.x * g.st[0] + d[0] - (g.ks[0] - 1) / 2;
    const int y = c.y * g.st[1] + d[1] - (g.ks[1] - 1) / 2;
    const int z = c.z * g.st[2] + d[2] - (g.ks[2] - 1) / 2;
    const unsigned long long key = fnv1a4(x, y, z, c.w);
    out[tid] = key ? table_lookup(t, key) : 0;
  }
}

// Even kernel volume: thread per (row, k); offsets are the raw digits (not centred).
__global__ void subm_query_even_kernel(TableView t, const int4* __restrict__ coords, int64_t n, Bounds b,
                                       KernelGeom g, int* __restrict__ map) {
  const int64_t total = n * (int64_t)g.kvol;
  for (int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; tid < total;
       tid += (int64_t)gridDim.x * blockDim.x) {
    int64_t row = tid / g.kvol;
    int k = (int)(tid - row * g.kvol);
    int dx, dy, dz;
    kernel_digits(g, k, dx, dy, dz);
    int4 c = __ldg(&coords[row]);
    int x = c.y + dx, y = c.z + dy, z = c.w + dz;
    if (!in_bounds_xyz(b, x, y, z)) continue;
    int64_t key = ravel4(b, c.x, x, y, z);
    int nbr = table_lookup(t, (unsigned long long)(key + 1)) - 1;
    if (nbr >= 0) map[tid] = nbr;
  }
}

// ------------------------------------------------------------------ strided map
// Number of kernel digits d' in [0,k) with (c + p - (k-1) + d') divisible by s is at most
// ceil(k/s) per dim; `slots` is the product over dims.
struct SlotGeom {
  int per[3];
  int slots;
};

inline SlotGeom make_slots(const int32_t* ks, const int32_t* st) {
  SlotGeom s;
  s.slots = 1;
  for (int i = 0; i < 3; ++i) {
    s.per[i] = (ks[i] + st[i] - 1) / st[i];
    s.slots *= s.per[i];
  }
  return s;
}

__device__ __forceinline__ int pos_mod(int a, int m) {
  int r = a % m;
  return r < 0 ? r + m : r;
}

// thread per (input, slot): the slot-th admissible digit combination -> candidate key,
// or `sentinel` when that combination does not exist / falls outside the bounds.
__global__ void down_candidates_kernel(const int4* __restrict__ coords, int64_t n, Bounds b, KernelGeom g,
                                       SlotGeom sg, int64_t sentinel, int64_t* __restrict__ cand) {
  const int64_t total = n * (int64_t)sg.slots;
  for (int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; tid < total;
       tid += (int64_t)gridDim.x * blockDim.x) {
    int64_t row = tid / sg.slots;
    int j = (int)(tid - row * sg.slots);
    int4 c = __ldg(&coords[row]);
    int in[3] = {c.y, c.z, c.w};
    int o[3];
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      int t = j % sg.per[i];
      j /= sg.per[i];
      int base = in[i] + g.pd[i] - (g.ks[i] - 1);
      int d = pos_mod(-base, g.st[i]) + t * g.st[i];
      ok = ok && (d < g.ks[i]);
      o[i] = (base + d) / g.st[i];  // exact when ok
    }
    ok = ok && in_bounds_xyz(b, o[0], o[1], o[2]);
    cand[tid] = ok ? ravel4(b, c.x, o[0], o[1], o[2]) : sentinel;
  }
}

// result[0] = number of outputs (unique keys minus the sentinel); result[1..4] = 0 for the max pass.
__global__ void down_count_kernel(const int64_t* __restrict__ uniq, const int* __restrict__ n_selected,
                                  int64_t sentinel, int* __restrict__ result) {
  int ns = *n_selected;
  int m = ns;
  if (ns > 0 && uniq[ns - 1] == sentinel) m = ns - 1;
  result[0] = m;
  result[1] = result[2] = result[3] = result[4] = INT_MIN;
  result[5] = result[6] = result[7] = 0;
}

__device__ __forceinline__ void unravel4(const Bounds& b, int64_t key, int& c0, int& c1, int& c2, int& c3) {
  c3 = b.mn[3] + (int)(key % b.sz[3]); key /= b.sz[3];
  c2 = b.mn[2] + (int)(key % b.sz[2]); key /= b.sz[2];
  c1 = b.mn[1] + (int)(key % b.sz[1]); key /= b.sz[1];
  c0 = b.mn[0] + (int)(key % b.sz[0]);
}

__global__ void down_max_kernel(const int64_t* __restrict__ uniq, Bounds b, int* __restrict__ result) {
  const int m = result[0];
  int mx[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < m; i += (int64_t)gridDim.x * blockDim.x) {
    int c[4];
    unravel4(b, uniq[i], c[0], c[1], c[2], c[3]);
#pragma unroll
    for (int d = 0; d < 4; ++d) mx[d] = max(mx[d], c[d]);
  }
#pragma unroll
  for (int d = 0; d < 4; ++d) {
    int v = mx[d];
    for (int o = 16; o; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0 && v != INT_MIN) atomicMax(&result[1 + d], v);
  }
}

// unravel + insert the outputs, and fill the map with -1 (block owns kBlock rows)
__global__ void down_insert_fill_kernel(TableView t, const int64_t* __restrict__ uniq, int64_t m, int64_t rows_pad,
                                        Bounds b, int kvol, int4* __restrict__ out_coords, int* __restrict__ map,
                                        int* status) {
  int64_t row0 = (int64_t)blockIdx.x * kBlock;
  int64_t row = row0 + threadIdx.x;
  if (row < m) {
    int64_t key = uniq[row];
    int4 c;
    unravel4(b, key, c.x, c.y, c.z, c.w);
    out_coords[row] = c;
    { const int e = table_insert(t, (unsigned long long)(key + 1), (int)(row + 1)); if (e && status) atomicOr(status, e); }
  }
  int64_t lo = row0 * kvol;
  int64_t hi = min(row0 + kBlock, rows_pad) * (int64_t)kvol;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kBlock) map[i] = -1;
}

// thread per (input, k'): map[out][kvol-1-k'] = in
__global__ void down_stage3_kernel(TableView t, const int4* __restrict__ coords, int64_t n, int64_t m, Bounds b,
                                   KernelGeom g, int* __restrict__ map, int* status) {
  const int64_t total = n * (int64_t)g.kvol;
  for (int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; tid < total;
       tid += (int64_t)gridDim.x * blockDim.x) {
    int64_t row = tid / g.kvol;
    int k = (int)(tid - row * g.kvol);
    int d[3];
    kernel_digits(g, k, d[0], d[1], d[2]);
    int4 c = __ldg(&coords[row]);
    int in[3] = {c.y, c.z, c.w};
    int o[3];
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      int v = in[i] + g.pd[i] + d[i] - (g.ks[i] - 1);
      ok = ok && (v % g.st[i] == 0);
      o[i] = v / g.st[i];
    }
    if (!ok || !in_bounds_xyz(b, o[0], o[1], o[2])) continue;
    int64_t key = ravel4(b, c.x, o[0], o[1], o[2]);
    int orow = table_lookup(t, (unsigned long long)(key + 1)) - 1;
    if (orow >= 0 && orow < m) {
      map[(int64_t)orow * g.kvol + (g.kvol - 1 - k)] = (int)row;
    } else if (status) {
      atomicOr(status, TSB_DEV_BAD_INDEX);
    }
  }
}

// The same pass as a block of inputs x offset lanes (32 x 8 or 16 x 16) with the offset digits precomputed (no
// 64-bit division, no digit arithmetic per thread) and power-of-two strides taken with masks and shifts.
constexpr int kMaxStage3Offsets = 128;
struct DownOffsets {
  signed char d[3][kMaxStage3Offsets];   // digit - (kernel size - 1) + padding, per dimension
  int shift[3];                           // log2(stride) when the stride is a power of two, else -1
};

__global__ void __launch_bounds__(256)
down_stage3_rows_kernel(TableView t, const int4* __restrict__ coords, int64_t n, int64_t m, Bounds b, KernelGeom g,
                        DownOffsets off, int* __restrict__ map, int* status) {
  const int64_t row = blockIdx.x * (int64_t)blockDim.y + threadIdx.y;
  if (row >= n) return;
  const int4 c = __ldg(&coords[row]);
  const int in[3] = {c.y, c.z, c.w};
  for (int k = threadIdx.x; k < g.kvol; k += blockDim.x) {
    int o[3];
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int v = in[i] + off.d[i][k];
      if (off.shift[i] >= 0) {
        ok = ok && ((v & ((1 << off.shift[i]) - 1)) == 0);
        o[i] = v >> off.shift[i];           // exact for the multiples of the stride that pass the test
      } else {
        ok = ok && (v % g.st[i] == 0);
        o[i] = v / g.st[i];
      }
    }
    if (!ok || !in_bounds_xyz(b, o[0], o[1], o[2])) continue;
    const int64_t key = ravel4(b, c.x, o[0], o[1], o[2]);
    const int orow = table_lookup(t, (unsigned long long)(key + 1)) - 1;
    if (orow >= 0 && orow < m) {
      map[(int64_t)orow * g.kvol + (g.kvol - 1 - k)] = (int)row;
    } else if (status) {
      atomicOr(status, TSB_DEV_BAD_INDEX);
    }
  }
}

// ------------------------------------------------------------------ builds with device-side sizes
// A "level record" (int32[16], device memory) describes the coordinates of one tensor stride when the host
// does not know their number: [0] rows, [1..4] lower and [5..8] upper bound (b,x,y,z) of the key space of the
// level's hash table, [9..12] the largest coordinate present.  The kernels below read sizes and bounds from
// records, are launched for the largest size the caller allows, and never report a size to the host, so a
// whole sequence of map builds and convolutions can be replayed (e.g. as a CUDA graph) for any input.
enum { kRecRows = 0, kRecMin = 1, kRecMax = 5, kRecActMax = 9, kRecInts = 16 };

__device__ __forceinline__ Bounds rec_bounds(const int* __restrict__ rec) {
  Bounds b;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    b.mn[i] = rec[kRecMin + i];
    b.mx[i] = rec[kRecMax + i];
    b.sz[i] = b.mx[i] - b.mn[i] + 1;
  }
  return b;
}
__device__ __forceinline__ int64_t rec_rows(const int* __restrict__ rec, int64_t cap) {
  return max((int64_t)0, min((int64_t)rec[kRecRows], cap));
}
__device__ __forceinline__ int floor_div(int a, int b) {   // b > 0
  int q = a / b;
  return (a % b != 0 && a < 0) ? q - 1 : q;
}

__global__ void subm_insert_fill_dyn_kernel(TableView t, const int4* __restrict__ coords, int64_t n_max,
                                            const int* __restrict__ rec, int kvol, int to_insert,
                                            int* __restrict__ map, int* status) {
  const int64_t n = rec_rows(rec, n_max);
  const int64_t rows_pad = (n + 127) / 128 * 128;
  const int64_t row0 = (int64_t)blockIdx.x * kBlock;
  if (row0 >= rows_pad) return;
  const int64_t row = row0 + threadIdx.x;
  if (to_insert && row < n) {
    const Bounds b = rec_bounds(rec);
    const int4 c = __ldg(&coords[row]);
    const int64_t key = ravel4(b, c.x, c.y, c.z, c.w);
    { const int e = table_insert(t, (unsigned long long)(key + 1), (int)(row + 1)); if (e && status) atomicOr(status, e); }
  }
  const int64_t lo = row0 * kvol;
  const int64_t hi = min(row0 + kBlock, rows_pad) * (int64_t)kvol;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kBlock) map[i] = -1;
}

// rows x offset lanes (blockDim = (lanes, rows per block)); odd kernel volume: lanes cover k < kvol / 2 and
// write the mirrored entry as well; even: lanes cover every k.  Offset digits are precomputed on the host.
struct SubmOffsets {
  signed char d[3][32];
};
// Rows per thread of subm_query_dyn_kernel: the probes of a thread's rows are independent, so their first loads
// are issued together.  The kernel is bound by the latency of those loads: a quarter of the threads with four
// loads in flight each finish in the same time (44 us at 110 k rows, 15 instead of 17 us at 12 k) and occupy a
// quarter of the thread slots while kernels of other streams run beside them.
constexpr int kQueryRows = 4;
__global__ void __launch_bounds__(256)
subm_query_dyn_kernel(TableView t, const int4* __restrict__ coords, int64_t n_max, const int* __restrict__ rec,
                      int kvol, int odd, const __grid_constant__ SubmOffsets off, int* __restrict__ map) {
  const int64_t n = rec_rows(rec, n_max);
  const int64_t row0 = blockIdx.x * (int64_t)(blockDim.y * kQueryRows) + threadIdx.y;
  if (row0 >= n) return;
  const Bounds b = rec_bounds(rec);
  const int half = kvol / 2;
  const int k_end = odd ? half : kvol;
  int4 c[kQueryRows];
  int64_t row[kQueryRows];
#pragma unroll
  for (int j = 0; j < kQueryRows; ++j) {
    row[j] = row0 + (int64_t)j * blockDim.y;
    c[j] = row[j] < n ? __ldg(&coords[row[j]]) : make_int4(0, 0, 0, 0);
  }
  if (odd && threadIdx.x == 0) {
#pragma unroll
    for (int j = 0; j < kQueryRows; ++j)
      if (row[j] < n) map[row[j] * kvol + half] = (int)row[j];
  }
  for (int k = threadIdx.x; k < k_end; k += blockDim.x) {
    unsigned long long key[kQueryRows], slot[kQueryRows], cur[kQueryRows];
    bool ok[kQueryRows];
#pragma unroll
    for (int j = 0; j < kQueryRows; ++j) {
      const int x = c[j].y + off.d[0][k], y = c[j].z + off.d[1][k], z = c[j].w + off.d[2][k];
      ok[j] = row[j] < n && in_bounds_xyz(b, x, y, z);
      key[j] = ok[j] ? (unsigned long long)(ravel4(b, c[j].x, x, y, z) + 1) : 1ull;
      slot[j] = table_slot(t, key[j]);
    }
#pragma unroll
    for (int j = 0; j < kQueryRows; ++j) cur[j] = ok[j] ? __ldg(&t.keys[slot[j]]) : 0ull;
#pragma unroll
    for (int j = 0; j < kQueryRows; ++j) {
      if (!ok[j]) continue;
      const int nbr = table_lookup_after(t, key[j], slot[j], cur[j]) - 1;
      if (nbr >= 0) {
        map[row[j] * kvol + k] = nbr;
        if (odd) map[(int64_t)nbr * kvol + (kvol - 1 - k)] = (int)row[j];
      }
    }
  }
}

// Output record of a strided build from the input record: key space [0, (max + 2 pad - (k - 1)) // stride]
// per axis (the reference's bound, torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:33-37);
// rows and the largest output coordinate are filled in by the later kernels.  Extents beyond the caller's
// static bound (which fixed the number of key bits that get sorted) set TSB_DEV_LIMIT in *status.
__global__ void down_prepare_kernel(const int* __restrict__ rec_in, KernelGeom g, long long max_key_space,
                                    int* __restrict__ rec_out, int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  rec_out[kRecRows] = 0;
  rec_out[kRecMin] = rec_in[kRecMin];          // batch index: unchanged
  rec_out[kRecMax] = rec_in[kRecActMax];
  long long space = (long long)(rec_out[kRecMax] - rec_out[kRecMin] + 1);
  for (int i = 0; i < 3; ++i) {
    rec_out[kRecMin + 1 + i] = 0;
    const int mx = floor_div(rec_in[kRecActMax + 1 + i] + 2 * g.pd[i] - (g.ks[i] - 1), g.st[i]);
    rec_out[kRecMax + 1 + i] = mx;
    space *= (long long)max(mx + 1, 0);
  }
  for (int i = 0; i < 4; ++i) rec_out[kRecActMax + i] = INT_MIN;
  for (int i = 13; i < kRecInts; ++i) rec_out[i] = 0;
  if (space >= max_key_space && status) atomicOr(status, TSB_DEV_LIMIT);
}

__global__ void down_candidates_dyn_kernel(const int4* __restrict__ coords, int64_t n_max, const int* __restrict__ rec_in,
                                           const int* __restrict__ rec_out, KernelGeom g, SlotGeom sg, int64_t sentinel,
                                           int64_t* __restrict__ cand) {
  const int64_t n = rec_rows(rec_in, n_max);
  const Bounds b = rec_bounds(rec_out);
  const bool empty = b.sz[0] < 1 || b.sz[1] < 1 || b.sz[2] < 1 || b.sz[3] < 1;
  const int64_t total = n_max * (int64_t)sg.slots;
  for (int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; tid < total;
       tid += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = tid / sg.slots;
    int j = (int)(tid - row * sg.slots);
    int64_t key = sentinel;
    if (row < n && !empty) {
      const int4 c = __ldg(&coords[row]);
      const int in[3] = {c.y, c.z, c.w};
      int o[3];
      bool ok = true;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int t = j % sg.per[i];
        j /= sg.per[i];
        const int base = in[i] + g.pd[i] - (g.ks[i] - 1);
        const int d = pos_mod(-base, g.st[i]) + t * g.st[i];
        ok = ok && (d < g.ks[i]);
        o[i] = (base + d) / g.st[i];  // exact when ok
      }
      ok = ok && in_bounds_xyz(b, o[0], o[1], o[2]);
      if (ok) key = ravel4(b, c.x, o[0], o[1], o[2]);
    }
    cand[tid] = key;
  }
}

// rec_out[0] = number of outputs (unique keys minus the sentinel)
__global__ void down_count_dyn_kernel(const int64_t* __restrict__ uniq, const int* __restrict__ n_selected,
                                      int64_t sentinel, int64_t m_max, int* __restrict__ rec_out, int* status) {
  const int ns = *n_selected;
  int m = ns;
  if (ns > 0 && uniq[ns - 1] == sentinel) m = ns - 1;
  if (m > m_max) {
    m = (int)m_max;
    if (status) atomicOr(status, TSB_DEV_LIMIT);
  }
  rec_out[kRecRows] = m;
}

// unravel + insert the outputs, fill the map with -1 (block owns kBlock rows), and find the largest coordinate
__global__ void down_insert_fill_dyn_kernel(TableView t, const int64_t* __restrict__ uniq, int64_t m_max,
                                            int* __restrict__ rec_out, int kvol, int4* __restrict__ out_coords,
                                            int* __restrict__ map, int* status) {
  const int64_t m = rec_rows(rec_out, m_max);
  const int64_t rows_pad = (m + 127) / 128 * 128;
  const int64_t row0 = (int64_t)blockIdx.x * kBlock;
  if (row0 >= rows_pad) return;
  const int64_t row = row0 + threadIdx.x;
  int mx[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
  if (row < m) {
    const Bounds b = rec_bounds(rec_out);
    const int64_t key = uniq[row];
    int4 c;
    unravel4(b, key, c.x, c.y, c.z, c.w);
    out_coords[row] = c;
    mx[0] = c.x; mx[1] = c.y; mx[2] = c.z; mx[3] = c.w;
    { const int e = table_insert(t, (unsigned long long)(key + 1), (int)(row + 1)); if (e && status) atomicOr(status, e); }
  }
#pragma unroll
  for (int d = 0; d < 4; ++d) {
    int v = mx[d];
    for (int o = 16; o; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0 && v != INT_MIN) atomicMax(&rec_out[kRecActMax + d], v);
  }
  const int64_t lo = row0 * kvol;
  const int64_t hi = min(row0 + kBlock, rows_pad) * (int64_t)kvol;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kBlock) map[i] = -1;
}

// input rows x offset lanes: map[out][kvol-1-k] = in, and (optionally) the transposed map [in][kvol-1-k] = out
__global__ void __launch_bounds__(256)
down_stage3_dyn_kernel(TableView t, const int4* __restrict__ coords, int64_t n_max, const int* __restrict__ rec_in,
                       int64_t m_max, const int* __restrict__ rec_out, KernelGeom g,
                       const __grid_constant__ DownOffsets off, int* __restrict__ map, int* __restrict__ map_t,
                       int* status) {
  const int64_t n = rec_rows(rec_in, n_max);
  const int64_t row = blockIdx.x * (int64_t)blockDim.y + threadIdx.y;
  const int64_t rows_pad_t = (n + 127) / 128 * 128;
  if (row >= rows_pad_t) return;
  if (row >= n) {   // padding rows of the transposed map
    if (map_t) for (int k = threadIdx.x; k < g.kvol; k += blockDim.x) map_t[row * g.kvol + k] = -1;
    return;
  }
  const int64_t m = rec_rows(rec_out, m_max);
  const Bounds b = rec_bounds(rec_out);
  const int4 c = __ldg(&coords[row]);
  const int in[3] = {c.y, c.z, c.w};
  for (int k = threadIdx.x; k < g.kvol; k += blockDim.x) {
    int o[3];
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int v = in[i] + off.d[i][k];
      if (off.shift[i] >= 0) {
        ok = ok && ((v & ((1 << off.shift[i]) - 1)) == 0);
        o[i] = v >> off.shift[i];
      } else {
        ok = ok && (v % g.st[i] == 0);
        o[i] = v / g.st[i];
      }
    }
    int orow = -1;
    if (ok && in_bounds_xyz(b, o[0], o[1], o[2])) {
      const int64_t key = ravel4(b, c.x, o[0], o[1], o[2]);
      orow = table_lookup(t, (unsigned long long)(key + 1)) - 1;
      if (orow >= 0 && orow < m) {
        map[(int64_t)orow * g.kvol + (g.kvol - 1 - k)] = (int)row;
      } else {
        orow = -1;
        if (status) atomicOr(status, TSB_DEV_BAD_INDEX);
      }
    }
    if (map_t) map_t[row * g.kvol + (g.kvol - 1 - k)] = orow;
  }
}

// level record of the finest level from the result of tsb_quantize_unique
// ({voxels, min x,y,z, max x,y,z}), batch index `batch`; voxel coordinates must be >= 0
__global__ void level0_record_kernel(const int* __restrict__ qresult, int batch, int* __restrict__ rec, int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  rec[kRecRows] = qresult[0];
  rec[kRecMin] = 0; rec[kRecMax] = batch; rec[kRecActMax] = batch;
  for (int i = 0; i < 3; ++i) {
    rec[kRecMin + 1 + i] = 0;
    rec[kRecMax + 1 + i] = qresult[4 + i];
    rec[kRecActMax + 1 + i] = qresult[4 + i];
    if (qresult[0] > 0 && qresult[1 + i] < 0 && status) atomicOr(status, TSB_DEV_LIMIT);
  }
  for (int i = 13; i < kRecInts; ++i) rec[i] = 0;
}

// ------------------------------------------------------------------ transpose / bitmask / reorder
__global__ void fill_i32_kernel(int* __restrict__ p, int64_t n, int v) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

__global__ void transpose_map_kernel(const int* __restrict__ map, int64_t total, int kvol, int64_t rows_t,
                                     int* __restrict__ map_t) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int in = __ldg(&map[i]);
    if (in < 0 || in >= rows_t) continue;
    int64_t out = i / kvol;
    int k = (int)(i - out * kvol);
    map_t[(int64_t)in * kvol + k] = (int)out;
  }
}

__global__ void bitmask_kernel(const int* __restrict__ map, int64_t rows, int kvol, int split, int64_t valid_n,
                               int* __restrict__ bitmask) {
  const int split_len = (kvol + split - 1) / split;
  const int64_t total = rows * split;
  for (int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; tid < total;
       tid += (int64_t)gridDim.x * blockDim.x) {
    int64_t row = tid / split;
    int s = (int)(tid - row * split);
    int v = -1;
    if (row < valid_n) {
      int lo = s * split_len;
      int len = (s == split - 1) ? kvol - lo : split_len;
      const int* p = map + row * kvol + lo;
      unsigned m = 0;
      for (int i = 0; i < len; ++i) m |= (unsigned)(__ldg(&p[i]) >= 0) << i;
      v = (int)m;
    }
    bitmask[(int64_t)s * rows + row] = v;
  }
}

__global__ void iota_kernel(int* __restrict__ p, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = (int)i;
}

// warp per tile
__global__ void reduce_mask_kernel(const int* __restrict__ bitmask, int64_t rows, int split, int tile, int64_t n_red,
                                   int* __restrict__ reduced) {
  int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  int64_t total = n_red * split;
  int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (; warp < total; warp += nwarps) {
    int s = (int)(warp / n_red);
    int64_t t = warp - (int64_t)s * n_red;
    int64_t lo = t * tile, hi = min(lo + tile, rows);
    int v = 0;
    for (int64_t i = lo + lane; i < hi; i += 32) v |= __ldg(&bitmask[(int64_t)s * rows + i]);
    for (int o = 16; o; o >>= 1) v |= __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) reduced[(int64_t)s * n_red + t] = v;
  }
}

__global__ void reorder_map_kernel(const int* __restrict__ map, int64_t rows, int kvol, const int* __restrict__ loc,
                                   int split_len, int* __restrict__ out) {
  const int64_t total = rows * kvol;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / kvol;
    int c = (int)(i - r * kvol);
    int src = __ldg(&loc[(int64_t)(c / split_len) * rows + r]);
    out[i] = __ldg(&map[(int64_t)src * kvol + c]);
  }
}

// ------------------------------------------------------------------ conv-ready sorted map
// Sort key of a map row: its neighbour mask (bit k = offset k has a neighbour); padding rows get 0.  The sort is
// stable and padding rows have the largest row numbers, so in descending order they end up behind every
// valid row, including valid rows without any neighbour.  iota[i] = i.
__global__ void row_sort_key_kernel(const int* __restrict__ map, int64_t rows, int kvol, int64_t valid_n,
                                    const int* __restrict__ valid_n_dev, unsigned* __restrict__ keys,
                                    int* __restrict__ iota) {
  if (valid_n_dev) valid_n = max((int64_t)0, min((int64_t)__ldg(valid_n_dev), valid_n));
  for (int64_t row = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; row < rows; row += (int64_t)gridDim.x * blockDim.x) {
    unsigned m = 0;
    if (row < valid_n) {
      const int* p = map + row * kvol;
      for (int i = 0; i < kvol; ++i) m |= (unsigned)(__ldg(&p[i]) >= 0) << i;
    }
    keys[row] = m;
    iota[row] = (int)row;
  }
}

// One block per 128-row tile of the sorted order: row r of the tile is map row loc[tile * 128 + r]; its kvol
// entries are written column-major (map_cm[k][tile * 128 + r], coalesced over r) and the tile's offset
// mask is the OR over its rows.  Padding positions (sorted key 0 at or beyond the valid count) get -1.
__global__ void __launch_bounds__(128)
reorder_cm_kernel(const int* __restrict__ map, const int* __restrict__ loc, int64_t rows, int kvol, int64_t valid_n,
                  const int* __restrict__ valid_n_dev, int* __restrict__ map_cm, unsigned* __restrict__ tile_mask) {
  if (valid_n_dev) valid_n = max((int64_t)0, min((int64_t)__ldg(valid_n_dev), valid_n));
  __shared__ unsigned s_mask[4];
  const int64_t pos = (int64_t)blockIdx.x * 128 + threadIdx.x;
  const bool live = pos < valid_n;
  const int src = live ? __ldg(&loc[pos]) : -1;
  const int* p = map + (int64_t)(src < 0 ? 0 : src) * kvol;
  unsigned mine = 0;
  for (int k = 0; k < kvol; ++k) {
    const int v = (live && src >= 0) ? __ldg(&p[k]) : -1;
    map_cm[(int64_t)k * rows + pos] = v;
    const unsigned bal = __ballot_sync(0xffffffffu, v >= 0);
    if (bal) mine |= 1u << k;
  }
  if ((threadIdx.x & 31) == 0) s_mask[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) tile_mask[blockIdx.x] = s_mask[0] | s_mask[1] | s_mask[2] | s_mask[3];
}

// Weight classes of work items (offsets of the item): 0 = heaviest.  Four classes order the table closely enough to
// "longest first" and cost four block scans per 1024 tiles.
constexpr int kItemClasses = 4;
__device__ __forceinline__ int item_class(int offsets) { return offsets >= 14 ? 0 : offsets >= 7 ? 1 : offsets >= 3 ? 2 : 3; }


// Work-item table of a map's tiles: a tile with more than `max_offsets` offsets becomes several consecutive
// items ("parts") that each take an equal share of its offsets, so that no single item is much longer than
// the others; every part of a split tile owns one slot of the convolution's fp32 scratch, and tiles are split
// only while slots are left (at most max_slots, < 32768).  items[i] = {row tile, offset mask of the part,
// part | parts << 8 | first slot of the tile << 16 (0 for a whole tile), 0}; *n_items = their number.
// One block; tiles are taken in chunks of the block size with running prefixes.
__global__ void __launch_bounds__(1024)
build_items_kernel(const unsigned* __restrict__ tile_mask, int64_t valid_n, const int* __restrict__ valid_n_dev,
                   int max_offsets, int max_slots, int4* __restrict__ items, int* __restrict__ n_items) {
  typedef cub::BlockScan<int, 1024> Scan;
  __shared__ typename Scan::TempStorage tmp;
  __shared__ int s_slots;
  __shared__ int s_class_items[kItemClasses];   // pass 1: items of each weight class; pass 2: next free entry of the class
  if (valid_n_dev) valid_n = max((int64_t)0, min((int64_t)__ldg(valid_n_dev), valid_n));
  const int tiles = (int)((valid_n + 127) / 128);
  // Items are written heaviest class first (the persistent CTAs take them in table order, and a long item that
  // starts last leaves every other CTA idle while it runs); inside a class they keep the tile order, so the table
  // is the same on every run.  Pass 1 decides how every tile is split and counts the items of each class, pass 2
  // writes them.
  for (int pass = 0; pass < 2; ++pass) {
    if (threadIdx.x == 0) s_slots = 0;
    if (pass == 1 && threadIdx.x == 0) {
      int at = 0;
      for (int c = 0; c < kItemClasses; ++c) {   // class 0 = heaviest
        const int cnt = s_class_items[c];
        s_class_items[c] = at;
        at += cnt;
      }
      *n_items = at;
    }
    if (pass == 0 && threadIdx.x < kItemClasses) s_class_items[threadIdx.x] = 0;
    __syncthreads();
    for (int t0 = 0; t0 < tiles; t0 += 1024) {
      const int t = t0 + threadIdx.x;
      const unsigned m = t < tiles ? tile_mask[t] : 0u;
      const int pc = __popc(m);
      int parts = t < tiles ? max(1, (pc + max_offsets - 1) / max_offsets) : 0;
      // slots: a tile is split only if its slots fit below max_slots
      int slot_first, slot_total;
      Scan(tmp).ExclusiveSum(parts > 1 ? parts : 0, slot_first, slot_total);
      const int slot_base = s_slots;
      __syncthreads();
      const int slot0 = slot_base + slot_first;
      if (parts > 1 && slot0 + parts > max_slots) parts = 1;
      const int per = parts ? (pc + parts - 1) / parts : 0;      // offsets per part (the last part may hold fewer)
      const int cls = item_class(per);
      for (int c = 0; c < kItemClasses; ++c) {
        int first, total;
        Scan(tmp).ExclusiveSum(cls == c ? parts : 0, first, total);
        const int base = s_class_items[c];
        __syncthreads();
        if (pass == 1 && t < tiles && cls == c) {
          unsigned rest = m;
          for (int j = 0; j < parts; ++j) {
            unsigned mj = 0;
            for (int q = 0; q < per && rest; ++q) {
              const unsigned low = rest & (0u - rest);
              mj |= low;
              rest ^= low;
            }
            if (parts == 1) mj = m;
            items[base + first + j] = make_int4(t, (int)mj, parts > 1 ? (j | (parts << 8) | (slot0 << 16)) : 0, 0);
          }
        }
        if (threadIdx.x == 0) s_class_items[c] = base + total;
        __syncthreads();
      }
      if (threadIdx.x == 0) s_slots = slot_base + slot_total;
      __syncthreads();
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ pair lists
constexpr int kMaxKvolSmem = 512;

// per-block, per-column counts of valid entries; also accumulates the global nbsizes
__global__ void pairs_block_count_kernel(const int* __restrict__ map, int64_t rows, int kvol,
                                         int* __restrict__ block_counts, int* __restrict__ nbsizes) {
  extern __shared__ int s_cnt[];
  for (int i = threadIdx.x; i < kvol; i += blockDim.x) s_cnt[i] = 0;
  __syncthreads();
  int64_t lo = (int64_t)blockIdx.x * kBlock * kvol;
  int64_t hi = min(((int64_t)blockIdx.x + 1) * kBlock, rows) * (int64_t)kvol;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    if (__ldg(&map[i]) >= 0) atomicAdd(&s_cnt[(int)(i % kvol)], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kvol; i += blockDim.x) {
    int c = s_cnt[i];
    if (block_counts) block_counts[(int64_t)blockIdx.x * kvol + i] = c;
    if (nbsizes && c) atomicAdd(&nbsizes[i], c);
  }
}

__global__ void scan_quantified_kernel(int kvol, const int* __restrict__ nbsizes, int* __restrict__ nbaddrs,
                                       int* __restrict__ qnbaddrs) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int acc = 0, qacc = 0;
    for (int k = 0; k < kvol; ++k) {
      if (nbaddrs) nbaddrs[k] = acc;
      if (qnbaddrs) qnbaddrs[k] = qacc;
      int v = nbsizes[k];
      acc += v;
      qacc += (v + 127) / 128 * 128;
    }
    if (nbaddrs) nbaddrs[kvol] = acc;
    if (qnbaddrs) qnbaddrs[kvol] = qacc;
  }
}

// exclusive scan over blocks of each column (thread per column), in place
__global__ void pairs_block_scan_kernel(int* __restrict__ block_counts, int64_t nblocks, int kvol) {
  int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= kvol) return;
  int acc = 0;
  for (int64_t b = 0; b < nblocks; ++b) {
    int v = block_counts[b * kvol + k];
    block_counts[b * kvol + k] = acc;
    acc += v;
  }
}

// block = kBlock rows; for each column the rank of a valid row = block offset + warp offset + lane rank
__global__ void pairs_fill_kernel(const int* __restrict__ map, int64_t rows, int kvol,
                                  const int* __restrict__ block_offsets, const int* __restrict__ nbaddrs,
                                  int64_t n_pairs, int transposed, int* __restrict__ nbmaps) {
  __shared__ int s_warp[kBlock / 32];
  int64_t row = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int k = 0; k < kvol; ++k) {
    int in = (row < rows) ? __ldg(&map[row * kvol + k]) : -1;
    unsigned bal = __ballot_sync(0xffffffffu, in >= 0);
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncthreads();
    int woff = 0;
    for (int w = 0; w < warp; ++w) woff += s_warp[w];
    if (in >= 0) {
      int64_t pos = (int64_t)nbaddrs[k] + block_offsets[(int64_t)blockIdx.x * kvol + k] + woff +
                    __popc(bal & ((1u << lane) - 1u));
      if (pos < n_pairs) {
        if (transposed) {
          nbmaps[pos] = in;
          nbmaps[n_pairs + pos] = (int)row;
        } else {
          nbmaps[2 * pos] = in;
          nbmaps[2 * pos + 1] = (int)row;
        }
      }
    }
    __syncthreads();
  }
}

__global__ void build_masks_kernel(const int* __restrict__ nbmaps, const int* __restrict__ nbaddrs, int kvol,
                                   int64_t n_pairs, int64_t n_in, int64_t n_out, int skip_centre,
                                   int* __restrict__ input_mask, int* __restrict__ output_mask) {
  extern __shared__ int s_addr[];
  for (int i = threadIdx.x; i <= kvol; i += blockDim.x) s_addr[i] = nbaddrs[i];
  __syncthreads();
  for (int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; p < n_pairs; p += (int64_t)gridDim.x * blockDim.x) {
    int lo = 0, hi = kvol;  // largest k with s_addr[k] <= p
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (s_addr[mid] <= p) lo = mid; else hi = mid;
    }
    int k = lo;
    if (skip_centre && k == kvol / 2) continue;
    int pos = (int)(p - s_addr[k]);
    int in = nbmaps[2 * p], out = nbmaps[2 * p + 1];
    if (in >= 0 && in < n_in) input_mask[(int64_t)k * n_in + in] = pos;
    if (out >= 0 && out < n_out) output_mask[(int64_t)k * n_out + out] = pos;
  }
}

int bits_for(int64_t v) {  // number of bits needed to represent v (v >= 0)
  int b = 0;
  while (v > 0) { ++b; v >>= 1; }
  return b < 1 ? 1 : b;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

// ====================================================================== C ABI
extern "C" {

int tsb_coord_hash(const int32_t* coords, int64_t n, int64_t* out, tsb_stream_t stream) {
  if (n < 0 || (n && (!coords || !out))) return TSB_ERR_BAD_ARG;
  if (n == 0) return TSB_OK;
  coord_hash_kernel<<<grid_for(n, kBlock), kBlock, 0, as_stream(stream)>>>(reinterpret_cast<const int4*>(coords), n, out);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_kernel_hash(const int32_t* coords, int64_t n, const int32_t* offsets, int32_t k, int64_t* out,
                    tsb_stream_t stream) {
  if (n < 0 || k < 0 || ((n && k) && (!coords || !out || !offsets))) return TSB_ERR_BAD_ARG;
  if (n == 0 || k == 0) return TSB_OK;
  if ((size_t)k * 3 * sizeof(int) > 48 * 1024) return TSB_ERR_LIMIT;
  kernel_hash_kernel<<<grid_for(n, kBlock), kBlock, (size_t)k * 3 * sizeof(int), as_stream(stream)>>>(
      reinterpret_cast<const int4*>(coords), n, offsets, k, out);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_hash_insert(int64_t* table_keys, int32_t* table_vals, int64_t capacity, const int64_t* keys, int64_t n,
                    int32_t* dev_status, tsb_stream_t stream) {
  if (!table_keys || capacity <= 0 || n < 0 || (n && !keys)) return TSB_ERR_BAD_ARG;
  if (n == 0) return TSB_OK;
  table_insert_kernel<<<grid_for(n, kBlock), kBlock, 0, as_stream(stream)>>>(make_table(table_keys, table_vals, capacity),
                                                                             keys, n, dev_status);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_hash_lookup(const int64_t* table_keys, const int32_t* table_vals, int64_t capacity, const int64_t* keys,
                    int64_t n, int32_t* out_vals, tsb_stream_t stream) {
  if (!table_keys || capacity <= 0 || n < 0 || (n && (!keys || !out_vals))) return TSB_ERR_BAD_ARG;
  if (n == 0) return TSB_OK;
  table_lookup_kernel<<<grid_for(n, kBlock), kBlock, 0, as_stream(stream)>>>(
      make_table(const_cast<int64_t*>(table_keys), const_cast<int32_t*>(table_vals), capacity), keys, n, out_vals);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

static int64_t query_capacity(int64_t n_ref) {
  int64_t cap = 512;
  while (cap < 2 * n_ref) cap <<= 1;
  return cap;
}

size_t tsb_hash_query_workspace_bytes(int64_t n_ref) {
  if (n_ref < 0) return 0;
  return (size_t)query_capacity(n_ref) * (sizeof(int64_t) + sizeof(int32_t)) + 256;
}

int tsb_hash_query(const int64_t* queries, int64_t n_q, const int64_t* refs, int64_t n_ref, int64_t* out,
                   void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  if (n_q < 0 || n_ref < 0 || (n_q && (!queries || !out)) || (n_ref && !refs)) return TSB_ERR_BAD_ARG;
  if (n_q == 0) return TSB_OK;
  if (!workspace || workspace_bytes < tsb_hash_query_workspace_bytes(n_ref)) return TSB_ERR_WORKSPACE;
  int64_t cap = query_capacity(n_ref);
  int64_t* tk = reinterpret_cast<int64_t*>(workspace);
  int32_t* tv = reinterpret_cast<int32_t*>(tk + cap);
  cudaStream_t s = as_stream(stream);
  TSB_CUDA_TRY(cudaMemsetAsync(workspace, 0, (size_t)cap * 12, s));
  TableView t = make_table(tk, tv, cap);
  if (n_ref) {
    table_insert_kernel<<<grid_for(n_ref, kBlock), kBlock, 0, s>>>(t, refs, n_ref, nullptr);
    TSB_LAUNCH_CHECK();
  }
  table_query_kernel<<<grid_for(n_q, kBlock), kBlock, 0, s>>>(t, queries, n_q, out);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

// ---------------------------------------------------------------------------------------------
// tsb_hash_query_static: the same join as tsb_hash_query, for callers that may not allocate.
// The private table lives in a file-scope device array instead of a caller workspace.
namespace {
constexpr int64_t kStaticQueryMaxRefs = 262144;                    // documented limit of the entry point
constexpr int64_t kStaticQueryCap = 2 * kStaticQueryMaxRefs;       // power of two, load factor <= 0.5
constexpr size_t kStaticQueryBytes = (size_t)kStaticQueryCap * (sizeof(int64_t) + sizeof(int32_t));  // 6 MiB
// Resident on every GPU that loads this library, from load to exit.
static __device__ __align__(256) unsigned char g_static_query_table[kStaticQueryBytes];

constexpr int kMaxDevices = 64;
void* g_static_query_ptr[kMaxDevices] = {};   // device address of the array, per device ordinal
std::mutex g_static_query_mutex;

// In host code the array's name is only a handle; the device address has to be asked for, once
// per device, with that device current.
int static_query_table(void** out) {
  int dev = -1;
  TSB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return TSB_ERR_LIMIT;
  std::lock_guard<std::mutex> lock(g_static_query_mutex);
  if (!g_static_query_ptr[dev]) {
    void* p = nullptr;
    TSB_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_query_table));
    if (!p) return TSB_ERR_CUDA;
    g_static_query_ptr[dev] = p;
  }
  *out = g_static_query_ptr[dev];
  return TSB_OK;
}
}  // namespace

int64_t tsb_hash_query_static_max_refs(void) { return kStaticQueryMaxRefs; }

int tsb_hash_query_static(const int64_t* queries, int64_t n_q, const int64_t* refs, int64_t n_ref, int64_t* out,
                          tsb_stream_t stream) {
  if (n_q < 0 || n_ref < 0 || (n_q && (!queries || !out)) || (n_ref && !refs)) return TSB_ERR_BAD_ARG;
  if (n_ref > kStaticQueryMaxRefs) return TSB_ERR_LIMIT;   // the fixed table cannot hold more keys
  if (n_q == 0) return TSB_OK;
  void* base = nullptr;
  int rc = static_query_table(&base);
  if (rc != TSB_OK) return rc;
  int64_t* tk = reinterpret_cast<int64_t*>(base);
  int32_t* tv = reinterpret_cast<int32_t*>(tk + kStaticQueryCap);
  cudaStream_t s = as_stream(stream);
  // the array keeps whatever the previous call left: empty it first
  TSB_CUDA_TRY(cudaMemsetAsync(base, 0, kStaticQueryBytes, s));
  TableView t = make_table(tk, tv, kStaticQueryCap);
  if (n_ref) {
    table_insert_kernel<<<grid_for(n_ref, kBlock), kBlock, 0, s>>>(t, refs, n_ref, nullptr);
    TSB_LAUNCH_CHECK();
  }
  table_query_kernel<<<grid_for(n_q, kBlock), kBlock, 0, s>>>(t, queries, n_q, out);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_hash_lookup_coords(const int64_t* table_keys, const int32_t* table_vals, int64_t capacity,
                           const int32_t* coords_xyzb, int64_t n, const int32_t* kernel_size, const int32_t* stride,
                           int32_t* out, tsb_stream_t stream) {
  if (!table_keys || !table_vals || capacity <= 0 || n < 0 || !kernel_size || !stride) return TSB_ERR_BAD_ARG;
  if (n && (!coords_xyzb || !out)) return TSB_ERR_BAD_ARG;
  for (int i = 0; i < 3; ++i) if (kernel_size[i] < 1 || stride[i] < 1) return TSB_ERR_BAD_ARG;
  KernelGeom g = make_geom(kernel_size, stride, nullptr);
  cudaStream_t s = as_stream(stream);
  const int64_t rows_pad = pad128(n);
  if (rows_pad) TSB_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)rows_pad * g.kvol * sizeof(int32_t), s));
  if (n == 0) return TSB_OK;
  TableView t = make_table(const_cast<int64_t*>(table_keys), const_cast<int32_t*>(table_vals), capacity);
  lookup_coords_kernel<<<grid_for(n * (int64_t)g.kvol, kBlock, 32), kBlock, 0, s>>>(
      t, reinterpret_cast<const int4*>(coords_xyzb), n, g, out);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

// keys are ravel index + 1 over the bounds: do they all fit the 32-bit half of a packed slot?
static bool fits_packed_keys(const Bounds& b) {
  unsigned __int128 total = 1;
  for (int i = 0; i < 4; ++i) total *= (unsigned __int128)(uint64_t)b.sz[i];
  return total < (unsigned __int128)kPackedKeyMax;
}

int tsb_kmap_subm(int64_t* table_keys, int32_t* table_vals, int64_t capacity, const int32_t* coords, int64_t n,
                  const int32_t* cmin, const int32_t* cmax, const int32_t* kernel_size, int32_t to_insert,
                  int32_t* out_in_map, int32_t* dev_status, tsb_stream_t stream) {
  if (!table_keys || capacity <= 0 || n < 0 || !cmin || !cmax || !kernel_size) return TSB_ERR_BAD_ARG;
  if (n && (!coords || !out_in_map)) return TSB_ERR_BAD_ARG;
  if (n == 0) return TSB_OK;
  for (int i = 0; i < 3; ++i) if (kernel_size[i] < 1) return TSB_ERR_BAD_ARG;
  KernelGeom g = make_geom(kernel_size, nullptr, nullptr);
  Bounds b = make_bounds(cmin, cmax);
  for (int i = 0; i < 4; ++i) if (b.sz[i] < 1) return TSB_ERR_BAD_ARG;
  if (!table_vals && !fits_packed_keys(b)) return TSB_ERR_LIMIT;
  TableView t = make_table(table_keys, table_vals, capacity);
  cudaStream_t s = as_stream(stream);
  const int64_t rows_pad = pad128(n);
  const int4* c4 = reinterpret_cast<const int4*>(coords);
  subm_insert_fill_kernel<<<(int)cdiv(rows_pad, kBlock), kBlock, 0, s>>>(t, c4, n, rows_pad, b, g.kvol, to_insert,
                                                                        out_in_map, dev_status);
  TSB_LAUNCH_CHECK();
  if (g.odd) {
    int64_t work = n * (int64_t)(g.kvol / 2 > 0 ? g.kvol / 2 : 1);
    subm_query_odd_kernel<<<grid_for(work, kBlock, 32), kBlock, 0, s>>>(t, c4, n, b, g, out_in_map);
  } else {
    subm_query_even_kernel<<<grid_for(n * (int64_t)g.kvol, kBlock, 32), kBlock, 0, s>>>(t, c4, n, b, g, out_in_map);
  }
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int32_t tsb_kmap_down_slots(const int32_t* kernel_size, const int32_t* stride) {
  if (!kernel_size || !stride) return 0;
  for (int i = 0; i < 3; ++i) if (kernel_size[i] < 1 || stride[i] < 1) return 0;
  return make_slots(kernel_size, stride).slots;
}

namespace {
struct DownWs {
  size_t cand_off, sorted_off, nsel_off, cub_off, total;
  size_t cub_bytes;
};
DownWs down_ws_layout(int64_t n, int slots) {
  DownWs w;
  size_t items = (size_t)n * slots;
  size_t sort_b = 0, uniq_b = 0;
  cub::DeviceRadixSort::SortKeys(nullptr, sort_b, (const int64_t*)nullptr, (int64_t*)nullptr, (int64_t)items, 0, 64);
  cub::DeviceSelect::Unique(nullptr, uniq_b, (const int64_t*)nullptr, (int64_t*)nullptr, (int*)nullptr, (int64_t)items);
  w.cub_bytes = sort_b > uniq_b ? sort_b : uniq_b;
  size_t off = 0;
  w.cand_off = off; off = align_up(off + items * 8, 256);
  w.sorted_off = off; off = align_up(off + items * 8, 256);
  w.nsel_off = off; off = align_up(off + 16, 256);
  w.cub_off = off; off = align_up(off + w.cub_bytes, 256);
  w.total = off;
  return w;
}
}  // namespace

size_t tsb_kmap_down_workspace_bytes(int64_t n, const int32_t* kernel_size, const int32_t* stride) {
  int slots = tsb_kmap_down_slots(kernel_size, stride);
  if (n <= 0 || slots <= 0) return 256;
  return down_ws_layout(n, slots).total;
}

int tsb_kmap_down_unique(const int32_t* coords, int64_t n, const int32_t* cmin, const int32_t* cmax_out,
                         const int32_t* kernel_size, const int32_t* stride, const int32_t* padding,
                         int64_t* uniq_keys, int32_t* result, void* workspace, size_t workspace_bytes,
                         tsb_stream_t stream) {
  if (n < 0 || !cmin || !cmax_out || !kernel_size || !stride || !padding || !result) return TSB_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  if (n == 0) {
    TSB_CUDA_TRY(cudaMemsetAsync(result, 0, 8 * sizeof(int32_t), s));
    return TSB_OK;
  }
  if (!coords || !uniq_keys) return TSB_ERR_BAD_ARG;
  int slots = tsb_kmap_down_slots(kernel_size, stride);
  if (slots <= 0) return TSB_ERR_BAD_ARG;
  Bounds b = make_bounds(cmin, cmax_out);
  // an empty output range (cmax_out < cmin on some dim) means no outputs at all
  for (int i = 0; i < 4; ++i) {
    if (b.sz[i] < 1) {
      TSB_CUDA_TRY(cudaMemsetAsync(result, 0, 8 * sizeof(int32_t), s));
      return TSB_OK;
    }
  }
  if ((int64_t)n * slots > (int64_t)INT32_MAX) return TSB_ERR_LIMIT;
  DownWs w = down_ws_layout(n, slots);
  if (!workspace || workspace_bytes < w.total) return TSB_ERR_WORKSPACE;
  char* base = reinterpret_cast<char*>(workspace);
  int64_t* cand = reinterpret_cast<int64_t*>(base + w.cand_off);
  int64_t* sorted = reinterpret_cast<int64_t*>(base + w.sorted_off);
  int* nsel = reinterpret_cast<int*>(base + w.nsel_off);
  void* cub_ws = base + w.cub_off;
  KernelGeom g = make_geom(kernel_size, stride, padding);
  SlotGeom sg = make_slots(kernel_size, stride);
  int64_t sentinel = (int64_t)b.sz[0] * b.sz[1] * b.sz[2] * b.sz[3];  // one past the largest key
  int64_t items = n * (int64_t)slots;
  down_candidates_kernel<<<grid_for(items, kBlock, 32), kBlock, 0, s>>>(reinterpret_cast<const int4*>(coords), n, b, g,
                                                                        sg, sentinel, cand);
  TSB_LAUNCH_CHECK();
  size_t cb = w.cub_bytes;
  TSB_CUDA_TRY(cub::DeviceRadixSort::SortKeys(cub_ws, cb, cand, sorted, items, 0, bits_for(sentinel), s));
  count_launch();
  cb = w.cub_bytes;
  TSB_CUDA_TRY(cub::DeviceSelect::Unique(cub_ws, cb, sorted, uniq_keys, nsel, items, s));
  count_launch();
  down_count_kernel<<<1, 1, 0, s>>>(uniq_keys, nsel, sentinel, result);
  TSB_LAUNCH_CHECK();
  down_max_kernel<<<grid_for(items, kBlock, 4), kBlock, 0, s>>>(uniq_keys, b, result);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_kmap_down_finish(int64_t* table_keys, int32_t* table_vals, int64_t capacity, const int32_t* coords, int64_t n,
                         const int64_t* uniq_keys, int64_t m, const int32_t* cmin, const int32_t* cmax_out,
                         const int32_t* kernel_size, const int32_t* stride, const int32_t* padding,
                         int32_t* out_coords, int32_t* out_in_map, int32_t* dev_status, tsb_stream_t stream) {
  if (!table_keys || capacity <= 0 || n < 0 || m < 0 || !cmin || !cmax_out || !kernel_size || !stride || !padding)
    return TSB_ERR_BAD_ARG;
  if (m == 0) return TSB_OK;
  if (!coords || !uniq_keys || !out_coords || !out_in_map) return TSB_ERR_BAD_ARG;
  if (capacity < m) return TSB_ERR_LIMIT;
  Bounds b = make_bounds(cmin, cmax_out);
  if (!table_vals && !fits_packed_keys(b)) return TSB_ERR_LIMIT;
  KernelGeom g = make_geom(kernel_size, stride, padding);
  TableView t = make_table(table_keys, table_vals, capacity);
  cudaStream_t s = as_stream(stream);
  const int64_t rows_pad = pad128(m);
  down_insert_fill_kernel<<<(int)cdiv(rows_pad, kBlock), kBlock, 0, s>>>(
      t, uniq_keys, m, rows_pad, b, g.kvol, reinterpret_cast<int4*>(out_coords), out_in_map, dev_status);
  TSB_LAUNCH_CHECK();
  bool small = g.kvol <= kMaxStage3Offsets && cdiv(n, 16) <= INT32_MAX;
  for (int i = 0; i < 3; ++i) small = small && g.ks[i] <= 64 && g.pd[i] >= 0 && g.pd[i] <= 63;
  if (small) {
    DownOffsets off;
    for (int k = 0; k < g.kvol; ++k) {
      int d[3];
      if (g.odd) { d[0] = k % g.ks[0]; d[1] = (k / g.ks[0]) % g.ks[1]; d[2] = k / (g.ks[0] * g.ks[1]); }
      else { d[2] = k % g.ks[2]; d[1] = (k / g.ks[2]) % g.ks[1]; d[0] = k / (g.ks[2] * g.ks[1]); }
      for (int i = 0; i < 3; ++i) off.d[i][k] = (signed char)(g.pd[i] + d[i] - (g.ks[i] - 1));
    }
    for (int i = 0; i < 3; ++i) {
      off.shift[i] = -1;
      for (int sh = 0; sh < 16; ++sh) if (g.st[i] == (1 << sh)) off.shift[i] = sh;
    }
    const int lanes = g.kvol <= 8 ? 8 : 16, rows = 256 / lanes;
    down_stage3_rows_kernel<<<(unsigned)cdiv(n, rows), dim3(lanes, rows), 0, s>>>(
        t, reinterpret_cast<const int4*>(coords), n, m, b, g, off, out_in_map, dev_status);
  } else {
    down_stage3_kernel<<<grid_for(n * (int64_t)g.kvol, kBlock, 32), kBlock, 0, s>>>(
        t, reinterpret_cast<const int4*>(coords), n, m, b, g, out_in_map, dev_status);
  }
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_map_transpose(const int32_t* out_in_map, int64_t rows, int32_t kvol, int32_t* map_t, int64_t rows_t,
                      int32_t fill, tsb_stream_t stream) {
  if (rows < 0 || rows_t < 0 || kvol < 1 || (rows && !out_in_map) || (rows_t && !map_t)) return TSB_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  if (fill && rows_t) {
    fill_i32_kernel<<<grid_for(rows_t * kvol / 4 + 1, kBlock), kBlock, 0, s>>>(map_t, rows_t * kvol, -1);
    TSB_LAUNCH_CHECK();
  }
  if (rows == 0 || rows_t == 0) return TSB_OK;
  transpose_map_kernel<<<grid_for(rows * kvol, kBlock, 32), kBlock, 0, s>>>(out_in_map, rows * kvol, kvol, rows_t, map_t);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_bitmask_derive(const int32_t* out_in_map, int64_t rows, int32_t kvol, int32_t split, int64_t valid_n,
                       int32_t* bitmask, tsb_stream_t stream) {
  if (rows < 0 || kvol < 1 || split < 1 || valid_n < 0 || valid_n > rows || (rows && (!out_in_map || !bitmask)))
    return TSB_ERR_BAD_ARG;
  if ((kvol + split - 1) / split > 31) return TSB_ERR_LIMIT;  // one int32 of mask bits per split
  if (rows == 0) return TSB_OK;
  bitmask_kernel<<<grid_for(rows * split, kBlock, 32), kBlock, 0, as_stream(stream)>>>(out_in_map, rows, kvol, split,
                                                                                      valid_n, bitmask);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

namespace {
struct SortWs { size_t iota_off, cub_off, total, cub_bytes; };
SortWs sort_ws_layout(int64_t rows) {
  SortWs w;
  size_t cb = 0;
  cub::DeviceRadixSort::SortPairsDescending(nullptr, cb, (const int*)nullptr, (int*)nullptr, (const int*)nullptr,
                                            (int*)nullptr, rows, 0, 32);
  w.cub_bytes = cb;
  size_t off = 0;
  w.iota_off = off; off = align_up(off + (size_t)rows * 4, 256);
  w.cub_off = off; off = align_up(off + cb, 256);
  w.total = off;
  return w;
}
}  // namespace

size_t tsb_bitmask_sort_workspace_bytes(int64_t rows, int32_t split) {
  (void)split;
  if (rows <= 0) return 256;
  return sort_ws_layout(rows).total;
}

int tsb_bitmask_sort(const int32_t* bitmask, int64_t rows, int32_t split, int32_t kvol, int32_t* sorted_mask,
                     int32_t* reorder_loc, void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  (void)kvol;
  if (rows < 0 || split < 1 || (rows && (!bitmask || !sorted_mask || !reorder_loc))) return TSB_ERR_BAD_ARG;
  if (rows == 0) return TSB_OK;
  if (rows > INT32_MAX) return TSB_ERR_LIMIT;
  SortWs w = sort_ws_layout(rows);
  if (!workspace || workspace_bytes < w.total) return TSB_ERR_WORKSPACE;
  cudaStream_t s = as_stream(stream);
  char* base = reinterpret_cast<char*>(workspace);
  int* iota = reinterpret_cast<int*>(base + w.iota_off);
  iota_kernel<<<grid_for(rows, kBlock), kBlock, 0, s>>>(iota, rows);
  TSB_LAUNCH_CHECK();
  for (int sp = 0; sp < split; ++sp) {
    size_t cb = w.cub_bytes;
    // signed keys: the -1 of padded rows sorts last; radix sort is stable, so ties keep row order
    TSB_CUDA_TRY(cub::DeviceRadixSort::SortPairsDescending(base + w.cub_off, cb, bitmask + (int64_t)sp * rows,
                                                           sorted_mask + (int64_t)sp * rows, iota,
                                                           reorder_loc + (int64_t)sp * rows, rows, 0, 32, s));
    count_launch();
  }
  return TSB_OK;
}

int tsb_bitmask_reduce(const int32_t* bitmask, int64_t rows, int32_t split, int32_t tile, int32_t* reduced,
                       tsb_stream_t stream) {
  if (rows < 0 || split < 1 || tile < 1 || (rows && (!bitmask || !reduced))) return TSB_ERR_BAD_ARG;
  if (tile % 4 != 0) return TSB_ERR_BAD_ARG;  // same restriction as the reference entry point
  if (rows == 0) return TSB_OK;
  int64_t n_red = (rows - 1) / tile + 1;
  reduce_mask_kernel<<<grid_for(n_red * split * 32, kBlock), kBlock, 0, as_stream(stream)>>>(bitmask, rows, split, tile,
                                                                                            n_red, reduced);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_map_reorder(const int32_t* out_in_map, int64_t rows, int32_t kvol, const int32_t* reorder_loc, int32_t split,
                    int32_t* out, tsb_stream_t stream) {
  if (rows < 0 || kvol < 1 || split < 1 || (rows && (!out_in_map || !reorder_loc || !out))) return TSB_ERR_BAD_ARG;
  if (rows == 0) return TSB_OK;
  int split_len = (kvol + split - 1) / split;
  reorder_map_kernel<<<grid_for(rows * kvol, kBlock, 32), kBlock, 0, as_stream(stream)>>>(out_in_map, rows, kvol,
                                                                                         reorder_loc, split_len, out);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

size_t tsb_map_sorted_workspace_bytes(int64_t rows) {
  if (rows <= 0) return 256;
  return align_up((size_t)rows * 4, 256) + sort_ws_layout(rows).total;
}

int tsb_map_sorted_artefacts(const int32_t* out_in_map, int64_t rows, int32_t kvol, int64_t valid_n, int32_t tile,
                             int32_t* sorted_mask, int32_t* reorder_loc, int32_t* reordered_map, int32_t* reduced_mask,
                             void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  if (rows < 0 || kvol < 1 || valid_n < 0 || valid_n > rows) return TSB_ERR_BAD_ARG;
  if (rows == 0) return TSB_OK;
  if (!out_in_map || !sorted_mask || !reorder_loc || !reordered_map || !reduced_mask) return TSB_ERR_BAD_ARG;
  const size_t mask_bytes = align_up((size_t)rows * 4, 256);
  if (!workspace || workspace_bytes < mask_bytes + sort_ws_layout(rows).total) return TSB_ERR_WORKSPACE;
  int32_t* bitmask = reinterpret_cast<int32_t*>(workspace);
  char* sort_ws = reinterpret_cast<char*>(workspace) + mask_bytes;
  int rc = tsb_bitmask_derive(out_in_map, rows, kvol, 1, valid_n, bitmask, stream);
  if (rc != TSB_OK) return rc;
  rc = tsb_bitmask_sort(bitmask, rows, 1, kvol, sorted_mask, reorder_loc, sort_ws, workspace_bytes - mask_bytes, stream);
  if (rc != TSB_OK) return rc;
  rc = tsb_map_reorder(out_in_map, rows, kvol, reorder_loc, 1, reordered_map, stream);
  if (rc != TSB_OK) return rc;
  return tsb_bitmask_reduce(sorted_mask, rows, 1, tile, reduced_mask, stream);
}

namespace {
struct SortCmWs { size_t key_off, key2_off, iota_off, cub_off, total, cub_bytes; };
SortCmWs sort_cm_layout(int64_t rows) {
  SortCmWs w;
  size_t cb = 0;
  cub::DeviceRadixSort::SortPairsDescending(nullptr, cb, (const unsigned*)nullptr, (unsigned*)nullptr, (const int*)nullptr,
                                            (int*)nullptr, rows, 0, 32);
  w.cub_bytes = cb;
  size_t off = 0;
  w.key_off = off; off = align_up(off + (size_t)rows * 4, 256);
  w.key2_off = off; off = align_up(off + (size_t)rows * 4, 256);
  w.iota_off = off; off = align_up(off + (size_t)rows * 4, 256);
  w.cub_off = off; off = align_up(off + cb, 256);
  w.total = off;
  return w;
}
}  // namespace

size_t tsb_map_sorted_cm_workspace_bytes(int64_t rows) {
  if (rows <= 0) return 256;
  return sort_cm_layout(rows).total;
}

int64_t tsb_map_items_max(int64_t rows, int32_t kvol, int32_t max_offsets) {
  if (rows <= 0 || kvol < 1 || max_offsets < 1) return 0;
  return cdiv(rows, 128) * cdiv(kvol, max_offsets);
}

int tsb_map_sorted_cm(const int32_t* out_in_map, int64_t rows, int32_t kvol, int64_t valid_n,
                      const int32_t* valid_n_dev, int32_t* reorder_loc, int32_t* map_cm, uint32_t* tile_mask,
                      int32_t max_offsets, int32_t max_slots, int32_t* items, int32_t* n_items, void* workspace,
                      size_t workspace_bytes, tsb_stream_t stream) {
  if (rows < 0 || rows % 128 || kvol < 1 || kvol > 31 || valid_n < 0 || valid_n > rows) return TSB_ERR_BAD_ARG;
  if (items && (!n_items || max_offsets < 1 || max_slots < 0 || ((uintptr_t)items & 15))) return TSB_ERR_BAD_ARG;
  if (rows == 0) return TSB_OK;
  if (rows > INT32_MAX) return TSB_ERR_LIMIT;
  if (!out_in_map || !reorder_loc || !map_cm || !tile_mask) return TSB_ERR_BAD_ARG;
  SortCmWs w = sort_cm_layout(rows);
  if (!workspace || workspace_bytes < w.total) return TSB_ERR_WORKSPACE;
  cudaStream_t s = as_stream(stream);
  char* base = reinterpret_cast<char*>(workspace);
  unsigned* keys = reinterpret_cast<unsigned*>(base + w.key_off);
  unsigned* keys2 = reinterpret_cast<unsigned*>(base + w.key2_off);
  int* iota = reinterpret_cast<int*>(base + w.iota_off);
  row_sort_key_kernel<<<grid_for(rows, kBlock, 8), kBlock, 0, s>>>(out_in_map, rows, kvol, valid_n, valid_n_dev, keys, iota);
  TSB_LAUNCH_CHECK();
  size_t cb = w.cub_bytes;
  // Stable: rows with the same neighbour pattern keep their original order (neighbouring rows share inputs).
  // Every bit of the mask is sorted (four 8-bit passes for a 3x3x3 kernel).  Leaving the lowest three offsets
  // out of the order saves a pass but costs about a tenth more (tile, offset) blocks at the finest levels of a
  // LiDAR scan; with several scans in flight the extra pass is hidden and the blocks are not.
  const int begin_bit = 0;
  TSB_CUDA_TRY(cub::DeviceRadixSort::SortPairsDescending(base + w.cub_off, cb, keys, keys2, iota, reorder_loc, rows,
                                                         begin_bit, kvol, s));
  count_launch();
  reorder_cm_kernel<<<(unsigned)(rows / 128), 128, 0, s>>>(out_in_map, reorder_loc, rows, kvol, valid_n, valid_n_dev,
                                                          map_cm, tile_mask);
  TSB_LAUNCH_CHECK();
  if (items) {
    build_items_kernel<<<1, 1024, 0, s>>>(tile_mask, valid_n, valid_n_dev, max_offsets,
                                          max_slots > 32767 ? 32767 : max_slots, reinterpret_cast<int4*>(items), n_items);
    TSB_LAUNCH_CHECK();
  }
  return TSB_OK;
}

// ---------------------------------------------------------------------------------------------
// Kernel-map builds whose sizes live in device memory (level records, see the kernels above).
namespace {
int fill_down_offsets(const KernelGeom& g, DownOffsets* off) {
  if (g.kvol > kMaxStage3Offsets) return TSB_ERR_LIMIT;
  for (int i = 0; i < 3; ++i) if (g.ks[i] > 64 || g.pd[i] < 0 || g.pd[i] > 63) return TSB_ERR_LIMIT;
  for (int k = 0; k < g.kvol; ++k) {
    int d[3];
    if (g.odd) { d[0] = k % g.ks[0]; d[1] = (k / g.ks[0]) % g.ks[1]; d[2] = k / (g.ks[0] * g.ks[1]); }
    else { d[2] = k % g.ks[2]; d[1] = (k / g.ks[2]) % g.ks[1]; d[0] = k / (g.ks[2] * g.ks[1]); }
    for (int i = 0; i < 3; ++i) off->d[i][k] = (signed char)(g.pd[i] + d[i] - (g.ks[i] - 1));
  }
  for (int i = 0; i < 3; ++i) {
    off->shift[i] = -1;
    for (int sh = 0; sh < 16; ++sh) if (g.st[i] == (1 << sh)) off->shift[i] = sh;
  }
  return TSB_OK;
}
}  // namespace

int tsb_level_record_from_quantize(const int32_t* quantize_result, int32_t batch, int32_t* rec, int32_t* dev_status,
                                   tsb_stream_t stream) {
  if (!quantize_result || !rec || batch < 0) return TSB_ERR_BAD_ARG;
  level0_record_kernel<<<1, 32, 0, as_stream(stream)>>>(quantize_result, batch, rec, dev_status);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_kmap_subm_dyn(int64_t* table_keys, int32_t* table_vals, int64_t capacity, const int32_t* coords, int64_t n_max,
                      const int32_t* rec, const int32_t* kernel_size, int32_t to_insert, int32_t* out_in_map,
                      int32_t* dev_status, tsb_stream_t stream) {
  if (!table_keys || capacity <= 0 || n_max < 0 || !rec || !kernel_size) return TSB_ERR_BAD_ARG;
  if (n_max == 0) return TSB_OK;
  if (!coords || !out_in_map) return TSB_ERR_BAD_ARG;
  for (int i = 0; i < 3; ++i) if (kernel_size[i] < 1 || kernel_size[i] > 64) return TSB_ERR_BAD_ARG;
  KernelGeom g = make_geom(kernel_size, nullptr, nullptr);
  if (g.kvol > 32) return TSB_ERR_LIMIT;
  if (capacity < 2 * n_max) return TSB_ERR_LIMIT;
  TableView t = make_table(table_keys, table_vals, capacity);
  cudaStream_t s = as_stream(stream);
  const int64_t rows_pad = pad128(n_max);
  const int4* c4 = reinterpret_cast<const int4*>(coords);
  if (to_insert) TSB_CUDA_TRY(cudaMemsetAsync(table_keys, 0, (size_t)capacity * sizeof(int64_t), s));
  subm_insert_fill_dyn_kernel<<<(int)cdiv(rows_pad, kBlock), kBlock, 0, s>>>(t, c4, n_max, rec, g.kvol, to_insert,
                                                                            out_in_map, dev_status);
  TSB_LAUNCH_CHECK();
  SubmOffsets off;
  for (int k = 0; k < g.kvol; ++k) {
    int d[3];
    if (g.odd) { d[0] = k % g.ks[0]; d[1] = (k / g.ks[0]) % g.ks[1]; d[2] = k / (g.ks[0] * g.ks[1]); }
    else { d[2] = k % g.ks[2]; d[1] = (k / g.ks[2]) % g.ks[1]; d[0] = k / (g.ks[2] * g.ks[1]); }
    // odd volumes are centred, even ones take the raw digits
    for (int i = 0; i < 3; ++i) off.d[i][k] = (signed char)(g.odd ? d[i] - (g.ks[i] - 1) / 2 : d[i]);
  }
  const int k_end = g.odd ? g.kvol / 2 : g.kvol;
  const int lanes = k_end <= 1 ? 1 : (k_end <= 8 ? 8 : 16), rows = 256 / lanes;
  subm_query_dyn_kernel<<<(unsigned)cdiv(n_max, rows * kQueryRows), dim3(lanes, rows), 0, s>>>(t, c4, n_max, rec, g.kvol, g.odd, off,
                                                                                 out_in_map);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

size_t tsb_kmap_down_dyn_workspace_bytes(int64_t n_max, const int32_t* kernel_size, const int32_t* stride) {
  int slots = tsb_kmap_down_slots(kernel_size, stride);
  if (n_max <= 0 || slots <= 0) return 256;
  DownWs w = down_ws_layout(n_max, slots);
  return w.total + align_up((size_t)n_max * slots * 8, 256);   // + the unique keys
}

int tsb_kmap_down_dyn(int64_t* table_keys, int32_t* table_vals, int64_t capacity, const int32_t* coords, int64_t n_max,
                      const int32_t* rec_in, const int32_t* kernel_size, const int32_t* stride, const int32_t* padding,
                      int32_t key_bits, int64_t m_max, int32_t* out_coords, int32_t* out_in_map, int32_t* out_in_map_t,
                      int32_t* rec_out, int32_t* dev_status, void* workspace, size_t workspace_bytes,
                      tsb_stream_t stream) {
  if (!table_keys || capacity <= 0 || n_max < 0 || m_max < 0 || !rec_in || !rec_out || !kernel_size || !stride ||
      !padding || key_bits < 1 || key_bits > 62)
    return TSB_ERR_BAD_ARG;
  if (!table_vals && key_bits > 32) return TSB_ERR_LIMIT;     // keys + 1 must fit the 32-bit half of a packed slot
  if (n_max == 0) return TSB_OK;
  if (!coords || !out_coords || !out_in_map) return TSB_ERR_BAD_ARG;
  const int slots = tsb_kmap_down_slots(kernel_size, stride);
  if (slots <= 0) return TSB_ERR_BAD_ARG;
  const int64_t items = n_max * (int64_t)slots;
  if (items > (int64_t)INT32_MAX || m_max > items) return TSB_ERR_LIMIT;
  if (capacity < 2 * m_max) return TSB_ERR_LIMIT;
  DownWs w = down_ws_layout(n_max, slots);
  if (!workspace || workspace_bytes < tsb_kmap_down_dyn_workspace_bytes(n_max, kernel_size, stride)) return TSB_ERR_WORKSPACE;
  char* base = reinterpret_cast<char*>(workspace);
  int64_t* cand = reinterpret_cast<int64_t*>(base + w.cand_off);
  int64_t* sorted = reinterpret_cast<int64_t*>(base + w.sorted_off);
  int* nsel = reinterpret_cast<int*>(base + w.nsel_off);
  void* cub_ws = base + w.cub_off;
  int64_t* uniq = reinterpret_cast<int64_t*>(base + w.total);
  KernelGeom g = make_geom(kernel_size, stride, padding);
  SlotGeom sg = make_slots(kernel_size, stride);
  DownOffsets off;
  {
    int rc = fill_down_offsets(g, &off);
    if (rc != TSB_OK) return rc;
  }
  cudaStream_t s = as_stream(stream);
  // keys are sorted on key_bits bits: the key space must stay below 2^key_bits - 1, which is the sentinel
  const int64_t sentinel = ((int64_t)1 << key_bits) - 1;
  const int4* c4 = reinterpret_cast<const int4*>(coords);
  TableView t = make_table(table_keys, table_vals, capacity);
  TSB_CUDA_TRY(cudaMemsetAsync(table_keys, 0, (size_t)capacity * sizeof(int64_t), s));
  down_prepare_kernel<<<1, 32, 0, s>>>(rec_in, g, (long long)sentinel, rec_out, dev_status);
  TSB_LAUNCH_CHECK();
  down_candidates_dyn_kernel<<<grid_for(items, kBlock, 32), kBlock, 0, s>>>(c4, n_max, rec_in, rec_out, g, sg, sentinel,
                                                                           cand);
  TSB_LAUNCH_CHECK();
  size_t cb = w.cub_bytes;
  TSB_CUDA_TRY(cub::DeviceRadixSort::SortKeys(cub_ws, cb, cand, sorted, items, 0, key_bits, s));
  count_launch();
  cb = w.cub_bytes;
  TSB_CUDA_TRY(cub::DeviceSelect::Unique(cub_ws, cb, sorted, uniq, nsel, items, s));
  count_launch();
  down_count_dyn_kernel<<<1, 1, 0, s>>>(uniq, nsel, sentinel, m_max, rec_out, dev_status);
  TSB_LAUNCH_CHECK();
  down_insert_fill_dyn_kernel<<<(int)cdiv(pad128(m_max), kBlock), kBlock, 0, s>>>(
      t, uniq, m_max, rec_out, g.kvol, reinterpret_cast<int4*>(out_coords), out_in_map, dev_status);
  TSB_LAUNCH_CHECK();
  const int lanes = g.kvol <= 8 ? 8 : 16, rows = 256 / lanes;
  down_stage3_dyn_kernel<<<(unsigned)cdiv(pad128(n_max), rows), dim3(lanes, rows), 0, s>>>(
      t, c4, n_max, rec_in, m_max, rec_out, g, off, out_in_map, out_in_map_t, dev_status);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_scan_quantified(int32_t kvol, const int32_t* nbsizes, int32_t* nbaddrs, int32_t* qnbaddrs,
                        tsb_stream_t stream) {
  if (kvol < 1 || !nbsizes) return TSB_ERR_BAD_ARG;
  scan_quantified_kernel<<<1, 32, 0, as_stream(stream)>>>(kvol, nbsizes, nbaddrs, qnbaddrs);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_pairs_count(const int32_t* out_in_map, int64_t rows, int32_t kvol, int32_t* nbsizes, int32_t* nbaddrs,
                    int32_t* qnbaddrs, tsb_stream_t stream) {
  if (rows < 0 || kvol < 1 || !nbsizes || (rows && !out_in_map)) return TSB_ERR_BAD_ARG;
  if (kvol > kMaxKvolSmem) return TSB_ERR_LIMIT;
  cudaStream_t s = as_stream(stream);
  TSB_CUDA_TRY(cudaMemsetAsync(nbsizes, 0, (size_t)kvol * sizeof(int32_t), s));
  if (rows) {
    pairs_block_count_kernel<<<(int)cdiv(rows, kBlock), kBlock, (size_t)kvol * sizeof(int), s>>>(out_in_map, rows, kvol,
                                                                                                nullptr, nbsizes);
    TSB_LAUNCH_CHECK();
  }
  if (nbaddrs || qnbaddrs) {
    scan_quantified_kernel<<<1, 32, 0, s>>>(kvol, nbsizes, nbaddrs, qnbaddrs);
    TSB_LAUNCH_CHECK();
  }
  return TSB_OK;
}

size_t tsb_pairs_fill_workspace_bytes(int64_t rows, int32_t kvol) {
  if (rows <= 0 || kvol < 1) return 256;
  return align_up((size_t)cdiv(rows, kBlock) * kvol * sizeof(int), 256);
}

int tsb_pairs_fill(const int32_t* out_in_map, int64_t rows, int32_t kvol, const int32_t* nbaddrs, int64_t n_pairs,
                   int32_t transposed, int32_t* nbmaps, void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  if (rows < 0 || kvol < 1 || n_pairs < 0 || !nbaddrs || (rows && !out_in_map)) return TSB_ERR_BAD_ARG;
  if (kvol > kMaxKvolSmem) return TSB_ERR_LIMIT;
  if (rows == 0 || n_pairs == 0) return TSB_OK;
  if (!nbmaps) return TSB_ERR_BAD_ARG;
  if (!workspace || workspace_bytes < tsb_pairs_fill_workspace_bytes(rows, kvol)) return TSB_ERR_WORKSPACE;
  cudaStream_t s = as_stream(stream);
  int* block_counts = reinterpret_cast<int*>(workspace);
  int64_t nblocks = cdiv(rows, kBlock);
  pairs_block_count_kernel<<<(int)nblocks, kBlock, (size_t)kvol * sizeof(int), s>>>(out_in_map, rows, kvol, block_counts,
                                                                                   nullptr);
  TSB_LAUNCH_CHECK();
  pairs_block_scan_kernel<<<(int)cdiv(kvol, 32), 32, 0, s>>>(block_counts, nblocks, kvol);
  TSB_LAUNCH_CHECK();
  pairs_fill_kernel<<<(int)nblocks, kBlock, 0, s>>>(out_in_map, rows, kvol, block_counts, nbaddrs, n_pairs, transposed,
                                                    nbmaps);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_build_masks(int64_t n_in, int64_t n_out, const int32_t* nbmaps, const int32_t* nbaddrs, int32_t kvol,
                    int64_t n_pairs, int32_t* input_mask, int32_t* output_mask, tsb_stream_t stream) {
  if (n_in < 0 || n_out < 0 || kvol < 1 || n_pairs < 0 || !nbaddrs) return TSB_ERR_BAD_ARG;
  if ((n_in && !input_mask) || (n_out && !output_mask) || (n_pairs && !nbmaps)) return TSB_ERR_BAD_ARG;
  if (kvol > kMaxKvolSmem) return TSB_ERR_LIMIT;
  cudaStream_t s = as_stream(stream);
  if (n_in) {
    fill_i32_kernel<<<grid_for(n_in * kvol, kBlock), kBlock, 0, s>>>(input_mask, n_in * kvol, -1);
    TSB_LAUNCH_CHECK();
  }
  if (n_out) {
    fill_i32_kernel<<<grid_for(n_out * kvol, kBlock), kBlock, 0, s>>>(output_mask, n_out * kvol, -1);
    TSB_LAUNCH_CHECK();
  }
  if (n_pairs == 0) return TSB_OK;
  int skip_centre = (n_in == n_out && (kvol & 1)) ? 1 : 0;
  build_masks_kernel<<<grid_for(n_pairs, kBlock), kBlock, (size_t)(kvol + 1) * sizeof(int), s>>>(
      nbmaps, nbaddrs, kvol, n_pairs, n_in, n_out, skip_centre, input_mask, output_mask);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

}  // extern "C"
