// CUDA-core (FMA) sparse convolution forward for all three dataflows.
//
// This is the exact-fp32 path (rel-L2 <= 1e-5 against an fp64 oracle needs real fp32
// products, which TF32 tensor cores do not give) and the path for channel counts the
// tensor-core kernel does not take (rows that are not 16-byte multiples, e.g. Cin = 4 or 5).
// fp16/bf16 inputs are widened to fp32 in shared memory; accumulation is fp32 with one
// rounding at the end.
#include <vector>

#include "common.cuh"
#include "conv_dispatch.h"

namespace tsb {
namespace {

constexpr int BM = 64;   // rows per tile
constexpr int BN = 64;   // output channels per tile
constexpr int BK = 16;   // reduction slice
constexpr int kThreads = 256;

struct TileSmem {
  float A[BK][BM + 4];
  float B[BK][BN + 4];
};

// rows[r] = source row of tile row r (or -1 -> zeros); A[kk][r] = X[rows[r]][c0+kk]
template <typename T>
__device__ __forceinline__ void load_a(TileSmem& sm, const T* __restrict__ x, const int* rows, int c0, int cin) {
  const int r = threadIdx.x >> 2;         // 0..63
  const int kk0 = (threadIdx.x & 3) * 4;  // 0,4,8,12
  const int src = rows[r];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int c = c0 + kk0 + j;
    float v = 0.f;
    if (src >= 0 && c < cin) v = to_f32(__ldg(&x[(int64_t)src * cin + c]));
    sm.A[kk0 + j][r] = v;
  }
}

template <typename T>
__device__ __forceinline__ void load_b(TileSmem& sm, const T* __restrict__ wk, int c0, int cin, int n0, int cout) {
  const int kk = threadIdx.x >> 4;        // 0..15
  const int n4 = (threadIdx.x & 15) * 4;  // 0..60
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int c = c0 + kk, n = n0 + n4 + j;
    float v = 0.f;
    if (c < cin && n < cout) v = to_f32(__ldg(&wk[(int64_t)c * cout + n]));
    sm.B[kk][n4 + j] = v;
  }
}

__device__ __forceinline__ void mac(const TileSmem& sm, float (&acc)[4][4]) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int kk = 0; kk < BK; ++kk) {
    float a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = sm.A[kk][ty * 4 + i];
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = sm.B[kk][tx * 4 + j];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// ------------------------------------------------------------------ implicit GEMM
template <typename T>
__global__ void __launch_bounds__(kThreads)
igemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, const int* __restrict__ map,
                  const int* __restrict__ reorder_loc, T* __restrict__ y, int64_t n_in, int64_t n_out, int kvol,
                  int cin, int cout, const float* __restrict__ scale, const float* __restrict__ bias,
                  const T* __restrict__ residual, int relu) {
  __shared__ TileSmem sm;
  __shared__ int s_rows[BM];
  const int64_t row0 = (int64_t)blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;
  float acc[4][4] = {};
  for (int k = 0; k < kvol; ++k) {
    int any = 0;
    if (threadIdx.x < BM) {
      int64_t r = row0 + threadIdx.x;
      int v = -1;
      if (r < n_out) {
        v = __ldg(&map[r * kvol + k]);
        if (v >= n_in) v = -1;
      }
      s_rows[threadIdx.x] = v;
      any = v >= 0;
    }
    if (!__syncthreads_or(any)) continue;  // whole tile has no neighbour at this offset
    const T* wk = w + (int64_t)k * cin * cout;
    for (int c0 = 0; c0 < cin; c0 += BK) {
      load_a(sm, x, s_rows, c0, cin);
      load_b(sm, wk, c0, cin, n0, cout);
      __syncthreads();
      mac(sm, acc);
      __syncthreads();
    }
  }
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t r = row0 + ty * 4 + i;
    if (r >= n_out) continue;
    int64_t dst = reorder_loc ? (int64_t)__ldg(&reorder_loc[r]) : r;
    if (dst < 0 || dst >= n_out) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      if (n >= cout) continue;
      float v = acc[i][j];
      if (scale) v *= __ldg(&scale[n]);
      if (bias) v += __ldg(&bias[n]);
      if (residual) v += to_f32(__ldg(&residual[dst * cout + n]));
      if (relu) v = fmaxf(v, 0.f);
      y[dst * cout + n] = from_f32<T>(v);
    }
  }
}

// ------------------------------------------------------------------ weight gradient on the CUDA cores
// out[k][a][b] += sum over the block's share of the map rows m of g[map[m][k]][a] * p[m][b]  (fp32 accumulation).
// Grid: (row shares, 32 x 32 tiles of (a, b), kernel offsets); a block walks its rows 32 at a time: the 32 gathered
// rows of g and the 32 rows of p are staged in shared memory, every thread owns a 2 x 2 patch of the tile.  For the
// shapes the tensor-core kernel does not take (fp32 tensors, channel counts that are not multiples of 8 / 16).
constexpr int kWgTile = 32, kWgRows = 32;
template <typename T>
__global__ void __launch_bounds__(256)
wgrad_simt_kernel(const T* __restrict__ g, const T* __restrict__ pm, const int* __restrict__ map, float* __restrict__ out,
                  int64_t n_g, int64_t n_rows, int kvol, int cg, int cd, int64_t rows_per_block) {
  __shared__ float s_g[kWgRows][kWgTile + 1];
  __shared__ float s_p[kWgRows][kWgTile + 1];
  __shared__ int s_src[kWgRows];
  const int k = blockIdx.z;
  const int tiles_b = (cd + kWgTile - 1) / kWgTile;
  const int a0 = (blockIdx.y / tiles_b) * kWgTile, b0 = (blockIdx.y % tiles_b) * kWgTile;
  const int64_t r_lo = (int64_t)blockIdx.x * rows_per_block;
  const int64_t r_hi = min(r_lo + rows_per_block, n_rows);
  const int ta = (threadIdx.x >> 4) * 2, tb = (threadIdx.x & 15) * 2;      // this thread's patch
  float acc[2][2] = {};
  for (int64_t r0 = r_lo; r0 < r_hi; r0 += kWgRows) {
    int any = 0;
    if (threadIdx.x < kWgRows) {
      const int64_t r = r0 + threadIdx.x;
      int v = -1;
      if (r < r_hi) {
        v = __ldg(&map[r * kvol + k]);
        if (v >= n_g) v = -1;
      }
      s_src[threadIdx.x] = v;
      any = v >= 0;
    }
    if (!__syncthreads_or(any)) continue;            // no pair of this offset among these rows
    for (int e = threadIdx.x; e < kWgRows * kWgTile; e += 256) {
      const int rr = e / kWgTile, cc = e % kWgTile;
      const int src = s_src[rr];
      const int64_t r = r0 + rr;
      s_g[rr][cc] = (src >= 0 && a0 + cc < cg) ? to_f32(__ldg(&g[(int64_t)src * cg + a0 + cc])) : 0.f;
      s_p[rr][cc] = (src >= 0 && r < r_hi && b0 + cc < cd) ? to_f32(__ldg(&pm[r * cd + b0 + cc])) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int rr = 0; rr < kWgRows; ++rr) {
      const float g0 = s_g[rr][ta], g1 = s_g[rr][ta + 1], p0 = s_p[rr][tb], p1 = s_p[rr][tb + 1];
      acc[0][0] = fmaf(g0, p0, acc[0][0]); acc[0][1] = fmaf(g0, p1, acc[0][1]);
      acc[1][0] = fmaf(g1, p0, acc[1][0]); acc[1][1] = fmaf(g1, p1, acc[1][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int a = a0 + ta + i, b = b0 + tb + j;
      if (a < cg && b < cd && acc[i][j] != 0.f) atomicAdd(&out[((int64_t)k * cg + a) * cd + b], acc[i][j]);
    }
}

// ------------------------------------------------------------------ gather-scatter
// in_buffer[p] = X[src(p)], 16-byte chunks when rows allow it (vec = elements per chunk)
template <typename T, int VEC>
__global__ void gs_gather_kernel(const T* __restrict__ x, const int* __restrict__ nbmaps, int64_t n_pairs, int col,
                                 int64_t n_in, int cin, T* __restrict__ buf) {
  const int chunks = cin / VEC;
  const int64_t total = n_pairs * chunks;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t p = i / chunks;
    int c = (int)(i - p * chunks);
    int src = __ldg(&nbmaps[2 * p + col]);
    if (VEC * sizeof(T) == 16) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (src >= 0 && src < n_in) v = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)src * cin) + c);
      reinterpret_cast<uint4*>(buf + p * cin)[c] = v;
    } else {
      T v = from_f32<T>(0.f);
      if (src >= 0 && src < n_in) v = __ldg(&x[(int64_t)src * cin + c]);
      buf[p * cin + c] = v;
    }
  }
}

// tile table: tile t covers pairs [start[t], start[t]+len[t]) of offset tk[t]
struct GsTiles {
  const int* tile_k;
  const int* tile_start;
  const int* tile_len;
};

// out_buffer[p] = in_buffer[p] . W[k(p)]   (fp32 buffer)
template <typename T>
__global__ void __launch_bounds__(kThreads)
gs_gemm_kernel(const T* __restrict__ in_buf, const T* __restrict__ w, GsTiles tiles, int cin, int cout,
               float* __restrict__ out_buf) {
  __shared__ TileSmem sm;
  __shared__ int s_rows[BM];
  const int t = blockIdx.x;
  const int k = tiles.tile_k[t], start = tiles.tile_start[t], len = tiles.tile_len[t];
  const int n0 = blockIdx.y * BN;
  if (threadIdx.x < BM) s_rows[threadIdx.x] = threadIdx.x < len ? start + threadIdx.x : -1;
  __syncthreads();
  float acc[4][4] = {};
  const T* wk = w + (int64_t)k * cin * cout;
  for (int c0 = 0; c0 < cin; c0 += BK) {
    load_a(sm, in_buf, s_rows, c0, cin);
    load_b(sm, wk, c0, cin, n0, cout);
    __syncthreads();
    mac(sm, acc);
    __syncthreads();
  }
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int r = ty * 4 + i;
    if (r >= len) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      if (n < cout) out_buf[(int64_t)(start + r) * cout + n] = acc[i][j];
    }
  }
}

// y[o] = sum_k out_buffer[addr[k] + mask[k*M + o]]  (deterministic: fixed k order, fp32)
template <typename T>
__global__ void gs_scatter_kernel(const float* __restrict__ out_buf, const int* __restrict__ mask,
                                  const int* __restrict__ addrs, int kvol, int centre_k, int64_t n_out,
                                  int cout, T* __restrict__ y) {
  const int64_t total = n_out * cout;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t o = i / cout;
    int n = (int)(i - o * cout);
    float v = 0.f;
    for (int k = 0; k < kvol; ++k) {
      // the masks leave out the centre offset of an odd submanifold map: its pair list is the identity
      int pos = (k == centre_k) ? (int)o : __ldg(&mask[(int64_t)k * n_out + o]);
      if (pos >= 0) v += __ldg(&out_buf[(int64_t)(__ldg(&addrs[k]) + pos) * cout + n]);
    }
    y[i] = from_f32<T>(v);
  }
}

// ------------------------------------------------------------------ fetch on demand
// one block per 64-row slice of the 128-quantised pair list
template <typename T>
__global__ void __launch_bounds__(kThreads)
fod_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, const int* __restrict__ imap,
                const int* __restrict__ omap, const int* __restrict__ nbaddrs, const int* __restrict__ qnbaddrs,
                int kvol, int64_t n_in, int64_t n_out, int cin, int cout, float* __restrict__ acc_out) {
  __shared__ TileSmem sm;
  __shared__ int s_rows[BM];
  __shared__ int s_out[BM];
  __shared__ int s_k;
  const int q0 = blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;
  if (threadIdx.x == 0) {
    int lo = 0, hi = kvol;  // largest k with qnbaddrs[k] <= q0
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (__ldg(&qnbaddrs[mid]) <= q0) lo = mid; else hi = mid;
    }
    s_k = lo;
  }
  __syncthreads();
  const int k = s_k;
  const int local = q0 - __ldg(&qnbaddrs[k]);
  const int base = __ldg(&nbaddrs[k]);
  const int len = __ldg(&nbaddrs[k + 1]) - base;
  int any = 0;
  if (threadIdx.x < BM) {
    int l = local + threadIdx.x;
    int src = -1, dst = -1;
    if (l < len) {
      src = __ldg(&imap[base + l]);
      dst = __ldg(&omap[base + l]);
      if (src < 0 || src >= n_in || dst < 0 || dst >= n_out) src = dst = -1;
    }
    s_rows[threadIdx.x] = src;
    s_out[threadIdx.x] = dst;
    any = src >= 0;
  }
  if (!__syncthreads_or(any)) return;
  float acc[4][4] = {};
  const T* wk = w + (int64_t)k * cin * cout;
  for (int c0 = 0; c0 < cin; c0 += BK) {
    load_a(sm, x, s_rows, c0, cin);
    load_b(sm, wk, c0, cin, n0, cout);
    __syncthreads();
    mac(sm, acc);
    __syncthreads();
  }
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int dst = s_out[ty * 4 + i];
    if (dst < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      if (n < cout) atomicAdd(&acc_out[(int64_t)dst * cout + n], acc[i][j]);
    }
  }
}

template <typename T>
__global__ void round_kernel(const float* __restrict__ src, int64_t n, T* __restrict__ dst) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<T>(src[i]);
}

}  // namespace

// ====================================================================== host launchers
template <typename T>
int igemm_simt_launch(const IgemmArgs& a, cudaStream_t s) {
  dim3 grid((unsigned)cdiv(a.n_out, BM), (unsigned)cdiv(a.cout, BN));
  igemm_simt_kernel<T><<<grid, kThreads, 0, s>>>((const T*)a.x, (const T*)a.w, a.map, a.reorder_loc, (T*)a.y, a.n_in,
                                                 a.n_out, a.kvol, a.cin, a.cout, a.scale, a.bias, (const T*)a.residual, a.relu);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int igemm_simt(const IgemmArgs& a, cudaStream_t s) {
  switch (a.dtype) {
    case TSB_F32: return igemm_simt_launch<float>(a, s);
    case TSB_F16: return igemm_simt_launch<__half>(a, s);
    case TSB_BF16: return igemm_simt_launch<__nv_bfloat16>(a, s);
  }
  return TSB_ERR_UNSUPPORTED;
}

template <typename T>
static int wgrad_simt_launch(const WgradArgs& a, cudaStream_t s) {
  TSB_CUDA_TRY(cudaMemsetAsync(a.out, 0, (size_t)a.kvol * a.cg * a.cd * sizeof(float), s));
  const int tiles = (int)(cdiv(a.cg, kWgTile) * cdiv(a.cd, kWgTile));
  // shares of the row range: a block walks its rows 32 at a time with three dependent memory round trips per step,
  // so the row range is cut into many short shares (about 1024 rows) rather than a few long ones
  int64_t shares = cdiv(a.n_rows, 1024);
  if (shares > 8192) shares = 8192;
  if (shares < 1) shares = 1;
  const int64_t rows_per_block = cdiv(cdiv(a.n_rows, shares), kWgRows) * kWgRows;
  dim3 grid((unsigned)cdiv(a.n_rows, rows_per_block), (unsigned)tiles, (unsigned)a.kvol);
  wgrad_simt_kernel<T><<<grid, 256, 0, s>>>((const T*)a.g, (const T*)a.p, a.map, a.out, a.n_g, a.n_rows, a.kvol, a.cg, a.cd,
                                            rows_per_block);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int wgrad_simt(const WgradArgs& a, cudaStream_t s) {
  if (a.map_rs != 0 || a.map_cs != 0) {
    if (a.map_rs != a.kvol || a.map_cs != 1) return TSB_ERR_UNSUPPORTED;      // row-major maps only
  }
  switch (a.dtype) {
    case TSB_F32: return wgrad_simt_launch<float>(a, s);
    case TSB_F16: return wgrad_simt_launch<__half>(a, s);
    case TSB_BF16: return wgrad_simt_launch<__nv_bfloat16>(a, s);
  }
  return TSB_ERR_UNSUPPORTED;
}

// ---- gather-scatter workspace layout
struct GsWs {
  size_t in_off, out_off, tk_off, ts_off, tl_off, addr_off, total;
  int64_t max_tiles;
};
static GsWs gs_layout(int64_t n_pairs, int kvol, int cin, int cout, int dtype) {
  GsWs w;
  w.max_tiles = cdiv(n_pairs, BM) + kvol;
  size_t off = 0;
  w.in_off = off; off = align_up(off + (size_t)n_pairs * cin * dtype_size(dtype), 256);
  w.out_off = off; off = align_up(off + (size_t)n_pairs * cout * sizeof(float), 256);
  w.tk_off = off; off = align_up(off + (size_t)w.max_tiles * 4, 256);
  w.ts_off = off; off = align_up(off + (size_t)w.max_tiles * 4, 256);
  w.tl_off = off; off = align_up(off + (size_t)w.max_tiles * 4, 256);
  w.addr_off = off; off = align_up(off + (size_t)(kvol + 1) * 4, 256);
  w.total = off;
  return w;
}

size_t gs_workspace_bytes(int64_t n_pairs, int kvol, int cin, int cout, int dtype) {
  return gs_layout(n_pairs < 1 ? 1 : n_pairs, kvol, cin, cout, dtype).total;
}

template <typename T>
static int gs_launch(const GsArgs& a, cudaStream_t s) {
  GsWs w = gs_layout(a.n_pairs, a.kvol, a.cin, a.cout, a.dtype);
  if (!a.workspace || a.workspace_bytes < w.total) return TSB_ERR_WORKSPACE;
  char* base = reinterpret_cast<char*>(a.workspace);
  T* in_buf = reinterpret_cast<T*>(base + w.in_off);
  float* out_buf = reinterpret_cast<float*>(base + w.out_off);
  int* tk = reinterpret_cast<int*>(base + w.tk_off);
  int* ts = reinterpret_cast<int*>(base + w.ts_off);
  int* tl = reinterpret_cast<int*>(base + w.tl_off);
  int* addrs = reinterpret_cast<int*>(base + w.addr_off);
  // tile table from the host-side sizes (the reference API passes nbsizes on the host)
  std::vector<int> h_tk, h_ts, h_tl, h_addr(a.kvol + 1, 0);
  int64_t acc = 0;
  for (int k = 0; k < a.kvol; ++k) {
    h_addr[k] = (int)acc;
    int nk = a.nbsizes_host[k];
    for (int st = 0; st < nk; st += BM) {
      h_tk.push_back(k);
      h_ts.push_back((int)acc + st);
      h_tl.push_back(nk - st < BM ? nk - st : BM);
    }
    acc += nk;
  }
  h_addr[a.kvol] = (int)acc;
  if (acc != a.n_pairs) return TSB_ERR_BAD_ARG;
  const int n_tiles = (int)h_tk.size();
  if (n_tiles) {
    TSB_CUDA_TRY(cudaMemcpyAsync(tk, h_tk.data(), n_tiles * 4, cudaMemcpyHostToDevice, s));
    TSB_CUDA_TRY(cudaMemcpyAsync(ts, h_ts.data(), n_tiles * 4, cudaMemcpyHostToDevice, s));
    TSB_CUDA_TRY(cudaMemcpyAsync(tl, h_tl.data(), n_tiles * 4, cudaMemcpyHostToDevice, s));
  }
  TSB_CUDA_TRY(cudaMemcpyAsync(addrs, h_addr.data(), (a.kvol + 1) * 4, cudaMemcpyHostToDevice, s));
  // the copies above read pageable host memory: they complete before returning, so the vectors may go
  const int col_in = a.transpose ? 1 : 0;
  const int64_t n_src = a.n_in;
  if (a.n_pairs) {
    constexpr int VEC = 16 / sizeof(T);
    if (a.cin % VEC == 0) {
      gs_gather_kernel<T, VEC><<<grid_for(a.n_pairs * (a.cin / VEC), 256, 32), 256, 0, s>>>(
          (const T*)a.x, a.nbmaps, a.n_pairs, col_in, n_src, a.cin, in_buf);
    } else {
      gs_gather_kernel<T, 1><<<grid_for(a.n_pairs * a.cin, 256, 32), 256, 0, s>>>((const T*)a.x, a.nbmaps, a.n_pairs,
                                                                                col_in, n_src, a.cin, in_buf);
    }
    TSB_LAUNCH_CHECK();
    GsTiles tiles{tk, ts, tl};
    dim3 grid((unsigned)n_tiles, (unsigned)cdiv(a.cout, BN));
    gs_gemm_kernel<T><<<grid, kThreads, 0, s>>>(in_buf, (const T*)a.w, tiles, a.cin, a.cout, out_buf);
    TSB_LAUNCH_CHECK();
  }
  if (a.n_out) {
    gs_scatter_kernel<T><<<grid_for(a.n_out * a.cout, 256, 32), 256, 0, s>>>(
        out_buf, a.scatter_mask, addrs, a.kvol, (a.n_in == a.n_out && (a.kvol & 1)) ? a.kvol / 2 : -1, a.n_out, a.cout,
        (T*)a.y);
    TSB_LAUNCH_CHECK();
  }
  return TSB_OK;
}

int gs_simt(const GsArgs& a, cudaStream_t s) {
  switch (a.dtype) {
    case TSB_F32: return gs_launch<float>(a, s);
    case TSB_F16: return gs_launch<__half>(a, s);
    case TSB_BF16: return gs_launch<__nv_bfloat16>(a, s);
  }
  return TSB_ERR_UNSUPPORTED;
}

template <typename T>
static int fod_launch(const FodArgs& a, cudaStream_t s) {
  const int64_t elems = a.n_out * a.cout;
  float* accum;
  if (a.dtype == TSB_F32) {
    accum = reinterpret_cast<float*>(a.y);
  } else {
    if (!a.workspace || a.workspace_bytes < (size_t)elems * sizeof(float)) return TSB_ERR_WORKSPACE;
    accum = reinterpret_cast<float*>(a.workspace);
  }
  if (elems) TSB_CUDA_TRY(cudaMemsetAsync(accum, 0, (size_t)elems * sizeof(float), s));
  if (a.qmapsize > 0 && a.n_pairs > 0) {
    const int* imap = a.nbmaps + (a.transpose ? a.n_pairs : 0);
    const int* omap = a.nbmaps + (a.transpose ? 0 : a.n_pairs);
    dim3 grid((unsigned)cdiv(a.qmapsize, BM), (unsigned)cdiv(a.cout, BN));
    fod_simt_kernel<T><<<grid, kThreads, 0, s>>>((const T*)a.x, (const T*)a.w, imap, omap, a.nbaddrs, a.qnbaddrs,
                                                 a.kvol, a.n_in, a.n_out, a.cin, a.cout, accum);
    TSB_LAUNCH_CHECK();
  }
  if (a.dtype != TSB_F32 && elems) {
    round_kernel<T><<<grid_for(elems, 256), 256, 0, s>>>(accum, elems, (T*)a.y);
    TSB_LAUNCH_CHECK();
  }
  return TSB_OK;
}

int fod_simt(const FodArgs& a, cudaStream_t s) {
  switch (a.dtype) {
    case TSB_F32: return fod_launch<float>(a, s);
    case TSB_F16: return fod_launch<__half>(a, s);
    case TSB_BF16: return fod_launch<__nv_bfloat16>(a, s);
  }
  return TSB_ERR_UNSUPPORTED;
}

}  // namespace tsb
