// GatherScatter and FetchOnDemand on the tensor cores.
//
// Both dataflows multiply pair lists: for kernel offset k, the input rows in_k[0..P_k) with W[k],
// products added into the output rows out_k[0..P_k).  Here the pair lists are laid out with every
// offset's segment padded to a multiple of 128 rows ("quantised" addresses, the layout the
// fetch-on-demand dataflow of the reference uses), so that each 128-row tile belongs to one offset,
// and the implicit-GEMM kernel runs over that list in its pair-list mode: the map is the single
// column of input rows (fetched on demand by the kernel's gather warps, no gathered copy of the
// features is made), the weight block of a tile is chosen by tile_k[tile], one K block per 128 bytes
// of input channels, fp32 accumulation in TMEM.
//   GatherScatter   products written as rows of a [P_pad, Cout] buffer in the tensors' own type (what the
//                   reference's per-offset GEMMs produce), then summed in fp32 per output row in fixed
//                   offset order through the scatter mask (no atomics, deterministic)
//   FetchOnDemand   products added straight into an fp32 [M, Cout] accumulator with vector atomic
//                   adds from the kernel's epilogue, then rounded once
#include <vector>

#include "common.cuh"
#include "conv_dispatch.h"

namespace tsb {
namespace {

// slot s of the padded list -> (offset k, position inside the offset's segment); fills the padded
// input-row list (-1 in padding), optionally the padded output-row list, and the offset of every tile
__global__ void pairs_pad_kernel(const int* __restrict__ in_list, int in_stride, const int* __restrict__ out_list,
                                 int out_stride, const int* __restrict__ addrs, const int* __restrict__ qaddrs,
                                 int kvol, int64_t n_pairs, int64_t q_total, int* __restrict__ in_pad,
                                 int* __restrict__ out_pad, int* __restrict__ tile_k) {
  for (int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; s < q_total; s += (int64_t)gridDim.x * blockDim.x) {
    int lo = 0, hi = kvol;   // largest k with qaddrs[k] <= s
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((int64_t)__ldg(&qaddrs[mid]) <= s) lo = mid; else hi = mid;
    }
    const int k = lo;
    const int64_t local = s - __ldg(&qaddrs[k]);
    const int64_t first = __ldg(&addrs[k]);
    const int64_t count = (k + 1 < kvol ? (int64_t)__ldg(&addrs[k + 1]) : n_pairs) - first;
    const bool live = local < count;
    in_pad[s] = live ? __ldg(&in_list[(first + local) * in_stride]) : -1;
    if (out_pad) out_pad[s] = live ? __ldg(&out_list[(first + local) * out_stride]) : -1;
    if ((s & 127) == 0) tile_k[s >> 7] = k;
  }
}

__device__ __forceinline__ float4 load4_f32(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4_f32(const __half* p) {
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 load4_f32(const __nv_bfloat16* p) {
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

// y[o, n..n+3] = sum_k buf[qaddrs[k] + mask[k*M + o], n..n+3]   (fixed k order, fp32 sums; the product rows are
// fp32 for fp32 tensors and 16-bit for 16-bit tensors, as the reference's per-offset GEMM outputs are)
template <typename T, typename B>
__global__ void pairs_scatter_kernel(const B* __restrict__ buf, const int* __restrict__ mask,
                                     const int* __restrict__ qaddrs, int kvol, int centre_k, int64_t n_out, int cout,
                                     T* __restrict__ y) {
  const int vecs = cout >> 2;
  const int64_t total = n_out * vecs;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = i / vecs;
    const int n = (int)(i - o * vecs) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < kvol; ++k) {
      // the masks leave out the centre offset of an odd submanifold map: its pair list is the identity
      const int pos = (k == centre_k) ? (int)o : __ldg(&mask[(int64_t)k * n_out + o]);
      if (pos >= 0) {
        const float4 v = load4_f32(buf + ((int64_t)__ldg(&qaddrs[k]) + pos) * cout + n);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    T* dst = y + o * cout + n;
    dst[0] = from_f32<T>(acc.x); dst[1] = from_f32<T>(acc.y); dst[2] = from_f32<T>(acc.z); dst[3] = from_f32<T>(acc.w);
  }
}

template <typename T>
__global__ void round_rows_kernel(const float* __restrict__ src, int64_t n, T* __restrict__ dst) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<T>(src[i]);
}

struct PairsWs {
  size_t buf_off, in_off, out_off, tk_off, addr_off, qaddr_off, w_off, err_off, total;
};
// q_total = rows of the padded pair list; buf_rows = rows of the fp32 buffer held in the workspace
PairsWs pairs_layout(int64_t q_total, int64_t buf_rows, int kvol, int cin, int cout, int dtype) {
  PairsWs w;
  size_t off = 0;
  w.buf_off = off; off = align_up(off + (size_t)buf_rows * cout * sizeof(float), 256);
  w.in_off = off; off = align_up(off + (size_t)q_total * 4, 256);
  w.out_off = off; off = align_up(off + (size_t)q_total * 4, 256);
  w.tk_off = off; off = align_up(off + (size_t)(q_total / 128 + 1) * 4, 256);
  w.addr_off = off; off = align_up(off + (size_t)(kvol + 1) * 4, 256);
  w.qaddr_off = off; off = align_up(off + (size_t)(kvol + 1) * 4, 256);
  w.w_off = off; off = align_up(off + packed_weight_bytes(kvol, cin, cout, dtype), 256);
  w.err_off = off; off += 256;
  w.total = off;
  return w;
}

IgemmArgs pair_mode_args(const void* x, const void* w, int64_t n_in, int64_t q_total, int kvol, int cin, int cout,
                         int dtype, int math) {
  IgemmArgs ia{};
  ia.x = x; ia.w = w; ia.n_in = n_in; ia.n_out = q_total; ia.kvol = 1; ia.cin = cin; ia.cout = cout;
  ia.dtype = dtype; ia.math = math; ia.kvol_w = kvol; ia.out_fp32 = (dtype != TSB_F32);
  return ia;
}

}  // namespace

bool pairs_umma_usable(const void* x, const void* w, int64_t n_in, int kvol, int cin, int cout, int dtype, int math) {
  if (cout % 8) return false;
  IgemmArgs ia = pair_mode_args(x, w, n_in, 128, kvol, cin, cout, dtype, math);
  static const int dummy_tile = 0;
  ia.tile_k = &dummy_tile;                 // only tested for null
  ia.map = reinterpret_cast<const int*>(uintptr_t(256));   // alignment check only
  ia.y = const_cast<void*>(x);
  return igemm_umma_supported(ia);
}

size_t gs_umma_workspace_bytes(int64_t n_pairs, int kvol, int cin, int cout, int dtype) {
  const int64_t q_max = pad128(n_pairs + (int64_t)127 * kvol);
  return pairs_layout(q_max, q_max, kvol, cin, cout, dtype).total;
}

size_t fod_umma_workspace_bytes(int64_t n_out, int64_t qmapsize, int kvol, int cin, int cout, int dtype) {
  // the fp32 accumulator of the output lives in the buffer slot (fp32 tensors accumulate in place)
  return pairs_layout(pad128(qmapsize), dtype == TSB_F32 ? 0 : n_out, kvol, cin, cout, dtype).total;
}

template <typename T>
static int gs_umma_launch(const GsArgs& a, cudaStream_t s) {
  // quantised addresses from the host-side sizes (the reference API passes nbsizes on the host)
  std::vector<int> h_addr(a.kvol + 1, 0), h_qaddr(a.kvol + 1, 0);
  int64_t acc = 0, qacc = 0;
  for (int k = 0; k < a.kvol; ++k) {
    h_addr[k] = (int)acc; h_qaddr[k] = (int)qacc;
    acc += a.nbsizes_host[k];
    qacc += pad128(a.nbsizes_host[k]);
  }
  h_addr[a.kvol] = (int)acc; h_qaddr[a.kvol] = (int)qacc;
  if (acc != a.n_pairs || qacc > INT32_MAX) return TSB_ERR_BAD_ARG;
  const int64_t q_total = qacc;
  PairsWs w = pairs_layout(q_total, q_total, a.kvol, a.cin, a.cout, a.dtype);
  if (!a.workspace || a.workspace_bytes < w.total) return TSB_ERR_WORKSPACE;
  char* base = reinterpret_cast<char*>(a.workspace);
  float* buf = reinterpret_cast<float*>(base + w.buf_off);
  int* in_pad = reinterpret_cast<int*>(base + w.in_off);
  int* tile_k = reinterpret_cast<int*>(base + w.tk_off);
  int* addrs = reinterpret_cast<int*>(base + w.addr_off);
  int* qaddrs = reinterpret_cast<int*>(base + w.qaddr_off);
  int* err = reinterpret_cast<int*>(base + w.err_off);
  // pageable host memory: these copies complete before they return, so the vectors may go
  TSB_CUDA_TRY(cudaMemcpyAsync(addrs, h_addr.data(), (a.kvol + 1) * 4, cudaMemcpyHostToDevice, s));
  TSB_CUDA_TRY(cudaMemcpyAsync(qaddrs, h_qaddr.data(), (a.kvol + 1) * 4, cudaMemcpyHostToDevice, s));
  TSB_CUDA_TRY(cudaMemsetAsync(err, 0, sizeof(int), s));
  if (q_total) {
    const int col_in = a.transpose ? 1 : 0;
    pairs_pad_kernel<<<grid_for(q_total, 256, 8), 256, 0, s>>>(a.nbmaps + col_in, 2, nullptr, 0, addrs, qaddrs, a.kvol,
                                                              a.n_pairs, q_total, in_pad, nullptr, tile_k);
    TSB_LAUNCH_CHECK();
    IgemmArgs ia = pair_mode_args(a.x, a.w, a.n_in, q_total, a.kvol, a.cin, a.cout, a.dtype, a.math);
    ia.map = in_pad; ia.tile_k = tile_k; ia.y = buf; ia.dev_status = err;
    ia.workspace = base + w.w_off; ia.workspace_bytes = w.total - w.w_off;     // packed weights
    ia.out_fp32 = 0;           // product rows in the tensors' own type: half the bytes written and read again
    int rc = igemm_umma(ia, s);
    if (rc != TSB_OK) return rc;
  }
  if (a.n_out) {
    pairs_scatter_kernel<T, T><<<grid_for(a.n_out * (a.cout / 4), 256, 16), 256, 0, s>>>(
        reinterpret_cast<const T*>(buf), a.scatter_mask, qaddrs, a.kvol, (a.n_in == a.n_out && (a.kvol & 1)) ? a.kvol / 2 : -1, a.n_out, a.cout,
        (T*)a.y);
    TSB_LAUNCH_CHECK();
  }
  return TSB_OK;
}

int gs_umma(const GsArgs& a, cudaStream_t s) {
  switch (a.dtype) {
    case TSB_F32: return gs_umma_launch<float>(a, s);
    case TSB_F16: return gs_umma_launch<__half>(a, s);
    case TSB_BF16: return gs_umma_launch<__nv_bfloat16>(a, s);
  }
  return TSB_ERR_UNSUPPORTED;
}

template <typename T>
static int fod_umma_launch(const FodArgs& a, cudaStream_t s) {
  const int64_t q_total = pad128(a.qmapsize);
  PairsWs w = pairs_layout(q_total, a.dtype == TSB_F32 ? 0 : a.n_out, a.kvol, a.cin, a.cout, a.dtype);
  if (!a.workspace || a.workspace_bytes < w.total) return TSB_ERR_WORKSPACE;
  char* base = reinterpret_cast<char*>(a.workspace);
  float* accum = a.dtype == TSB_F32 ? reinterpret_cast<float*>(a.y) : reinterpret_cast<float*>(base + w.buf_off);
  int* in_pad = reinterpret_cast<int*>(base + w.in_off);
  int* out_pad = reinterpret_cast<int*>(base + w.out_off);
  int* tile_k = reinterpret_cast<int*>(base + w.tk_off);
  int* err = reinterpret_cast<int*>(base + w.err_off);
  const int64_t elems = a.n_out * a.cout;
  if (elems) TSB_CUDA_TRY(cudaMemsetAsync(accum, 0, (size_t)elems * sizeof(float), s));
  TSB_CUDA_TRY(cudaMemsetAsync(err, 0, sizeof(int), s));
  if (q_total > 0 && a.n_pairs > 0) {
    const int* imap = a.nbmaps + (a.transpose ? a.n_pairs : 0);
    const int* omap = a.nbmaps + (a.transpose ? 0 : a.n_pairs);
    pairs_pad_kernel<<<grid_for(q_total, 256, 8), 256, 0, s>>>(imap, 1, omap, 1, a.nbaddrs, a.qnbaddrs, a.kvol,
                                                              a.n_pairs, q_total, in_pad, out_pad, tile_k);
    TSB_LAUNCH_CHECK();
    IgemmArgs ia = pair_mode_args(a.x, a.w, a.n_in, q_total, a.kvol, a.cin, a.cout, a.dtype, a.math);
    ia.map = in_pad; ia.tile_k = tile_k; ia.reorder_loc = out_pad; ia.y = accum; ia.dev_status = err;
    ia.workspace = base + w.w_off; ia.workspace_bytes = w.total - w.w_off;
    ia.out_fp32 = 1; ia.atomic_out = 1; ia.dst_rows = a.n_out;
    int rc = igemm_umma(ia, s);
    if (rc != TSB_OK) return rc;
  }
  if (a.dtype != TSB_F32 && elems) {
    round_rows_kernel<T><<<grid_for(elems, 256), 256, 0, s>>>(accum, elems, (T*)a.y);
    TSB_LAUNCH_CHECK();
  }
  return TSB_OK;
}

int fod_umma(const FodArgs& a, cudaStream_t s) {
  switch (a.dtype) {
    case TSB_F32: return fod_umma_launch<float>(a, s);
    case TSB_F16: return fod_umma_launch<__half>(a, s);
    case TSB_BF16: return fod_umma_launch<__nv_bfloat16>(a, s);
  }
  return TSB_ERR_UNSUPPORTED;
}

}  // namespace tsb
