// GPU twin of sparse_quantize: floor-divide to voxel coordinates, unique by ravel key in
// ascending order, first-occurrence index and inverse map.  The division is evaluated in
// float64 so the voxel indices equal numpy's bit for bit.
#include <cub/cub.cuh>

#include "common.cuh"

namespace tsb {
namespace {

constexpr int kBlock = 256;

template <typename F>
__global__ void quantize_kernel(const F* __restrict__ xyz, int64_t n, double vx, double vy, double vz,
                                int* __restrict__ q_all, int* __restrict__ minmax) {
  int mn[3] = {INT_MAX, INT_MAX, INT_MAX}, mx[3] = {INT_MIN, INT_MIN, INT_MIN};
  const double v[3] = {vx, vy, vz};
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      int q = (int)floor((double)xyz[i * 3 + d] / v[d]);
      q_all[i * 3 + d] = q;
      mn[d] = min(mn[d], q);
      mx[d] = max(mx[d], q);
    }
  }
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    int a = mn[d], b = mx[d];
    for (int o = 16; o; o >>= 1) {
      a = min(a, __shfl_xor_sync(0xffffffffu, a, o));
      b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
    }
    if ((threadIdx.x & 31) == 0) {
      if (a != INT_MAX) atomicMin(&minmax[d], a);
      if (b != INT_MIN) atomicMax(&minmax[3 + d], b);
    }
  }
}

__global__ void init_minmax_kernel(int* minmax) {
  if (threadIdx.x < 3) minmax[threadIdx.x] = INT_MAX;
  else if (threadIdx.x < 6) minmax[threadIdx.x] = INT_MIN;
}

__global__ void ravel_kernel(const int* __restrict__ q_all, int64_t n, const int* __restrict__ minmax,
                             unsigned long long* __restrict__ keys, int* __restrict__ idx) {
  const int mnx = minmax[0], mny = minmax[1], mnz = minmax[2];
  const unsigned long long sy = (unsigned long long)((long long)minmax[4] - mny + 1);
  const unsigned long long sz = (unsigned long long)((long long)minmax[5] - mnz + 1);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    unsigned long long x = (unsigned long long)((long long)q_all[i * 3] - mnx);
    unsigned long long y = (unsigned long long)((long long)q_all[i * 3 + 1] - mny);
    unsigned long long z = (unsigned long long)((long long)q_all[i * 3 + 2] - mnz);
    keys[i] = (x * sy + y) * sz + z;
    idx[i] = (int)i;
  }
}

__global__ void head_flags_kernel(const unsigned long long* __restrict__ keys, int64_t n, int* __restrict__ flags) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    flags[i] = (i == 0 || keys[i] != keys[i - 1]) ? 1 : 0;
}

// scan[i] = inclusive sum of head flags = run id + 1
__global__ void emit_kernel(const unsigned long long* __restrict__ keys, const int* __restrict__ sorted_idx,
                            const int* __restrict__ scan, int64_t n, const int* __restrict__ q_all,
                            int* __restrict__ uniq_coords, int64_t* __restrict__ first_index,
                            int64_t* __restrict__ inverse, const int* __restrict__ minmax,
                            int* __restrict__ result) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int run = scan[i] - 1;
    int src = sorted_idx[i];
    if (inverse) inverse[src] = run;
    bool head = (i == 0) || (keys[i] != keys[i - 1]);
    if (head) {
      uniq_coords[run * 3 + 0] = q_all[(int64_t)src * 3 + 0];
      uniq_coords[run * 3 + 1] = q_all[(int64_t)src * 3 + 1];
      uniq_coords[run * 3 + 2] = q_all[(int64_t)src * 3 + 2];
      if (first_index) first_index[run] = src;
    }
    if (i == n - 1) {
      result[0] = run + 1;
#pragma unroll
      for (int d = 0; d < 6; ++d) result[1 + d] = minmax[d];   // min x,y,z then max x,y,z of the voxel coordinates
    }
  }
}

struct QWs {
  size_t keys_in, keys_out, idx_in, idx_out, scan, minmax, cub, total, cub_bytes;
};
QWs q_layout(int64_t n) {
  QWs w;
  size_t sort_b = 0, scan_b = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, sort_b, (const unsigned long long*)nullptr, (unsigned long long*)nullptr,
                                  (const int*)nullptr, (int*)nullptr, n, 0, 64);
  cub::DeviceScan::InclusiveSum(nullptr, scan_b, (const int*)nullptr, (int*)nullptr, n);
  w.cub_bytes = sort_b > scan_b ? sort_b : scan_b;
  size_t off = 0;
  w.keys_in = off; off = align_up(off + (size_t)n * 8, 256);
  w.keys_out = off; off = align_up(off + (size_t)n * 8, 256);
  w.idx_in = off; off = align_up(off + (size_t)n * 4, 256);
  w.idx_out = off; off = align_up(off + (size_t)n * 4, 256);
  w.scan = off; off = align_up(off + (size_t)n * 4, 256);
  w.minmax = off; off = align_up(off + 32, 256);
  w.cub = off; off = align_up(off + w.cub_bytes, 256);
  w.total = off;
  return w;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" {

size_t tsb_quantize_workspace_bytes(int64_t n) {
  if (n <= 0) return 256;
  return q_layout(n).total;
}

int tsb_quantize_unique(const void* xyz, int32_t xyz_is_f64, int64_t n, const double* voxel, int32_t* q_all,
                        int32_t* uniq_coords, int64_t* first_index, int64_t* inverse, int32_t* result,
                        void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  return tsb_quantize_unique_bits(xyz, xyz_is_f64, n, voxel, 64, q_all, uniq_coords, first_index, inverse, result,
                                  workspace, workspace_bytes, stream);
}

int tsb_quantize_unique_bits(const void* xyz, int32_t xyz_is_f64, int64_t n, const double* voxel, int32_t key_bits,
                             int32_t* q_all, int32_t* uniq_coords, int64_t* first_index, int64_t* inverse,
                             int32_t* result, void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  if (n < 0 || !voxel || !result || key_bits < 1 || key_bits > 64) return TSB_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  if (n == 0) {
    TSB_CUDA_TRY(cudaMemsetAsync(result, 0, 8 * sizeof(int32_t), s));
    return TSB_OK;
  }
  if (!xyz || !q_all || !uniq_coords) return TSB_ERR_BAD_ARG;
  if (n > INT32_MAX) return TSB_ERR_LIMIT;
  if (!(voxel[0] > 0) || !(voxel[1] > 0) || !(voxel[2] > 0)) return TSB_ERR_BAD_ARG;
  QWs w = q_layout(n);
  if (!workspace || workspace_bytes < w.total) return TSB_ERR_WORKSPACE;
  char* base = reinterpret_cast<char*>(workspace);
  auto* keys_in = reinterpret_cast<unsigned long long*>(base + w.keys_in);
  auto* keys_out = reinterpret_cast<unsigned long long*>(base + w.keys_out);
  int* idx_in = reinterpret_cast<int*>(base + w.idx_in);
  int* idx_out = reinterpret_cast<int*>(base + w.idx_out);
  int* scan = reinterpret_cast<int*>(base + w.scan);
  int* minmax = reinterpret_cast<int*>(base + w.minmax);
  init_minmax_kernel<<<1, 32, 0, s>>>(minmax);
  TSB_LAUNCH_CHECK();
  int grid = grid_for(n, kBlock);
  if (xyz_is_f64)
    quantize_kernel<double><<<grid, kBlock, 0, s>>>((const double*)xyz, n, voxel[0], voxel[1], voxel[2], q_all, minmax);
  else
    quantize_kernel<float><<<grid, kBlock, 0, s>>>((const float*)xyz, n, voxel[0], voxel[1], voxel[2], q_all, minmax);
  TSB_LAUNCH_CHECK();
  ravel_kernel<<<grid, kBlock, 0, s>>>(q_all, n, minmax, keys_in, idx_in);
  TSB_LAUNCH_CHECK();
  size_t cb = w.cub_bytes;
  // radix sort is stable: inside a run the original indices stay ascending, so the head of a
  // run is the first occurrence
  TSB_CUDA_TRY(cub::DeviceRadixSort::SortPairs(base + w.cub, cb, keys_in, keys_out, idx_in, idx_out, n, 0, key_bits, s));
  count_launch();
  int* flags = idx_in;  // idx_in is free after the sort
  head_flags_kernel<<<grid, kBlock, 0, s>>>(keys_out, n, flags);
  TSB_LAUNCH_CHECK();
  cb = w.cub_bytes;
  TSB_CUDA_TRY(cub::DeviceScan::InclusiveSum(base + w.cub, cb, flags, scan, n, s));
  count_launch();
  emit_kernel<<<grid, kBlock, 0, s>>>(keys_out, idx_out, scan, n, q_all, uniq_coords, first_index, inverse, minmax,
                                      result);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

}  // extern "C"
