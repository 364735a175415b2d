// Point <-> voxel operators: histogram, average-pool voxelization, trilinear
// devoxelization, dense scatter.  All are single-pass HBM-bound kernels: one thread per
// (point, 16-byte channel chunk) where the row length allows it, so each warp reads and
// writes whole 128-byte lines of a feature row.
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kBlock = 256;

__global__ void count_kernel(const int* __restrict__ idx, int64_t n, int64_t s, int* __restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int v = __ldg(&idx[i]);
    if (v >= 0 && v < s) atomicAdd(&out[v], 1);
  }
}

template <typename T>
__global__ void voxelize_kernel(const T* __restrict__ feats, const int* __restrict__ idx,
                                const int* __restrict__ counts, int64_t n, int64_t n_vox, int c,
                                float* __restrict__ out) {
  const int64_t total = n * c;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = t / c;
    int j = (int)(t - i * c);
    int pos = __ldg(&idx[i]);
    if (pos < 0 || pos >= n_vox) continue;
    int cnt = __ldg(&counts[pos]);
    if (cnt == 0) continue;
    atomicAdd(&out[(int64_t)pos * c + j], to_f32(__ldg(&feats[t])) / (float)cnt);
  }
}

// Four channels per thread: one 16-byte (fp32) or 8-byte (16-bit) load of the point's row and one 16-byte
// vector atomic add on the voxel's fp32 row, instead of four scalar atomics.
template <typename T>
__global__ void voxelize_vec4_kernel(const T* __restrict__ feats, const int* __restrict__ idx,
                                     const int* __restrict__ counts, int64_t n, int64_t n_vox, int c,
                                     float* __restrict__ out) {
  const int chunks = c >> 2;
  const int64_t total = n * chunks;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t / chunks;
    const int ch = (int)(t - i * chunks);
    const int pos = __ldg(&idx[i]);
    if (pos < 0 || pos >= n_vox) continue;
    const int cnt = __ldg(&counts[pos]);
    if (cnt == 0) continue;
    const float inv = (float)cnt;
    float4 v;
    if constexpr (sizeof(T) == 4) {
      v = __ldg(reinterpret_cast<const float4*>(feats + i * c) + ch);
    } else {
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(feats + i * c) + ch);
      const T* e = reinterpret_cast<const T*>(&raw);
      v = make_float4(to_f32(e[0]), to_f32(e[1]), to_f32(e[2]), to_f32(e[3]));
    }
    atomicAdd(reinterpret_cast<float4*>(out + (int64_t)pos * c) + ch, make_float4(v.x / inv, v.y / inv, v.z / inv, v.w / inv));
  }
}

template <typename T>
__global__ void devoxelize_kernel(const T* __restrict__ feats, const int* __restrict__ indices,
                                  const float* __restrict__ weights, int64_t n, int c, T* __restrict__ out) {
  const int64_t total = n * c;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = t / c;
    int j = (int)(t - i * c);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      int src = __ldg(&indices[i * 8 + k]);
      if (src >= 0) acc = fmaf(__ldg(&weights[i * 8 + k]), to_f32(__ldg(&feats[(int64_t)src * c + j])), acc);
    }
    out[t] = from_f32<T>(acc);
  }
}

// 8 channels of fp16/bf16 (or 4 of fp32) per thread: 16-byte loads of each of the 8 source rows
template <typename T>
__global__ void devoxelize_vec_kernel(const T* __restrict__ feats, const int* __restrict__ indices,
                                      const float* __restrict__ weights, int64_t n, int c, T* __restrict__ out) {
  constexpr int VEC = 16 / sizeof(T);
  const int chunks = c / VEC;
  const int64_t total = n * chunks;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = t / chunks;
    int ch = (int)(t - i * chunks);
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      int src = __ldg(&indices[i * 8 + k]);
      if (src < 0) continue;
      float w = __ldg(&weights[i * 8 + k]);
      uint4 raw = __ldg(reinterpret_cast<const uint4*>(feats + (int64_t)src * c) + ch);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = fmaf(w, to_f32(e[v]), acc[v]);
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int v = 0; v < VEC; ++v) oe[v] = from_f32<T>(acc[v]);
    reinterpret_cast<uint4*>(out + i * c)[ch] = o;
  }
}

template <typename T>
__global__ void to_dense_kernel(const T* __restrict__ feats, const int4* __restrict__ coords, int64_t n, int c,
                                int r0, int r1, int r2, int r3, T* __restrict__ out) {
  const int64_t total = n * c;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = t / c;
    int j = (int)(t - i * c);
    int4 p = __ldg(&coords[i]);
    if (p.x < 0 || p.x >= r0 || p.y < 0 || p.y >= r1 || p.z < 0 || p.z >= r2 || p.w < 0 || p.w >= r3) continue;
    int64_t pos = (((int64_t)p.x * r1 + p.y) * r2 + p.z) * r3 + p.w;
    out[pos * c + j] = feats[t];
  }
}

// Backward of to_dense: grad_feats[i] = grad_dense[cell of coords[i]] (zero for a row outside the range).
template <typename T>
__global__ void to_dense_bwd_kernel(const T* __restrict__ grad_dense, const int4* __restrict__ coords, int64_t n, int c,
                                    int r0, int r1, int r2, int r3, T* __restrict__ grad_feats) {
  const int64_t total = n * c;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = t / c;
    int j = (int)(t - i * c);
    int4 p = __ldg(&coords[i]);
    if (p.x < 0 || p.x >= r0 || p.y < 0 || p.y >= r1 || p.z < 0 || p.z >= r2 || p.w < 0 || p.w >= r3) {
      grad_feats[t] = T(0.f);
      continue;
    }
    int64_t pos = (((int64_t)p.x * r1 + p.y) * r2 + p.z) * r3 + p.w;
    grad_feats[t] = grad_dense[pos * c + j];
  }
}

// Backward of the average pooling: grad_feats[i] = grad_out[idx[i]] / counts[idx[i]] (a gather; fp32 gradients).
__global__ void voxelize_bwd_kernel(const float* __restrict__ grad_out, const int* __restrict__ idx,
                                    const int* __restrict__ counts, int64_t n, int64_t n_vox, int c,
                                    float* __restrict__ grad_feats) {
  const int64_t total = n * c;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t / c;
    const int j = (int)(t - i * c);
    const int pos = __ldg(&idx[i]);
    float g = 0.f;
    if (pos >= 0 && pos < n_vox) {
      const int cnt = __ldg(&counts[pos]);
      if (cnt > 0) g = __ldg(&grad_out[(int64_t)pos * c + j]) / (float)cnt;
    }
    grad_feats[t] = g;
  }
}

// Backward of the interpolation: grad_voxels[idx[i][k]] += w[i][k] * grad_out[i] (scatter by atomic adds, fp32).
__global__ void devoxelize_bwd_kernel(const float* __restrict__ grad_out, const int* __restrict__ indices,
                                      const float* __restrict__ weights, int64_t n, int64_t n_vox, int c,
                                      float* __restrict__ grad_voxels) {
  const int64_t total = n * c;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t / c;
    const int j = (int)(t - i * c);
    const float g = __ldg(&grad_out[t]);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int dst = __ldg(&indices[i * 8 + k]);
      if (dst >= 0 && dst < n_vox) atomicAdd(&grad_voxels[(int64_t)dst * c + j], __ldg(&weights[i * 8 + k]) * g);
    }
  }
}

// One thread per voxel: batch column + voxel coordinates, and the features of the voxel's first point cast
// to T and zero-padded to c_pad channels.  The voxel count is read from the quantisation result on the device.
template <typename T>
__global__ void voxel_inputs_kernel(const float* __restrict__ points, int c_in, const int64_t* __restrict__ first,
                                    const int* __restrict__ uniq, const int* __restrict__ qresult, int batch,
                                    int64_t n_max, int4* __restrict__ coords, T* __restrict__ feats, int c_pad) {
  const int64_t nv = max((int64_t)0, min((int64_t)qresult[0], n_max));
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nv; i += (int64_t)gridDim.x * blockDim.x) {
    coords[i] = make_int4(batch, uniq[i * 3], uniq[i * 3 + 1], uniq[i * 3 + 2]);
    const float* src = points + first[i] * c_in;
    T* dst = feats + i * c_pad;
    for (int c = 0; c < c_pad; ++c) dst[c] = from_f32<T>(c < c_in ? __ldg(&src[c]) : 0.f);
  }
}

}  // namespace
}  // namespace tsb

using namespace tsb;

template <typename T>
static int devox_launch(const void* feats, const int32_t* indices, const float* weights, int64_t n, int c, void* out,
                        cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  bool vec = (c % VEC == 0) && ((uintptr_t)feats % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (vec) {
    devoxelize_vec_kernel<T><<<grid_for(n * (int64_t)(c / VEC), kBlock, 32), kBlock, 0, st>>>(
        (const T*)feats, indices, weights, n, c, (T*)out);
  } else {
    devoxelize_kernel<T><<<grid_for(n * (int64_t)c, kBlock, 32), kBlock, 0, st>>>((const T*)feats, indices, weights, n,
                                                                                 c, (T*)out);
  }
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

extern "C" {

int tsb_count(const int32_t* idx, int64_t n, int32_t* out, int64_t s, tsb_stream_t stream) {
  if (n < 0 || s < 0 || (n && !idx) || (s && !out)) return TSB_ERR_BAD_ARG;
  cudaStream_t st = as_stream(stream);
  if (s) TSB_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)s * sizeof(int32_t), st));
  if (n == 0 || s == 0) return TSB_OK;
  count_kernel<<<grid_for(n, kBlock), kBlock, 0, st>>>(idx, n, s, out);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_voxelize_fwd(const void* feats, const int32_t* idx, const int32_t* counts, int64_t n, int64_t n_vox,
                     int32_t c, int32_t dtype, float* out, tsb_stream_t stream) {
  if (n < 0 || n_vox < 0 || c < 1 || (n && (!feats || !idx)) || (n_vox && (!counts || !out))) return TSB_ERR_BAD_ARG;
  cudaStream_t st = as_stream(stream);
  if (n_vox) TSB_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)n_vox * c * sizeof(float), st));
  if (n == 0 || n_vox == 0) return TSB_OK;
  if (c % 4 == 0 && ((uintptr_t)feats % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const int gridv = grid_for(n * (int64_t)(c / 4), kBlock, 32);
    switch (dtype) {
      case TSB_F32: voxelize_vec4_kernel<float><<<gridv, kBlock, 0, st>>>((const float*)feats, idx, counts, n, n_vox, c, out); break;
      case TSB_F16: voxelize_vec4_kernel<__half><<<gridv, kBlock, 0, st>>>((const __half*)feats, idx, counts, n, n_vox, c, out); break;
      case TSB_BF16: voxelize_vec4_kernel<__nv_bfloat16><<<gridv, kBlock, 0, st>>>((const __nv_bfloat16*)feats, idx, counts, n, n_vox, c, out); break;
      default: return TSB_ERR_UNSUPPORTED;
    }
    TSB_LAUNCH_CHECK();
    return TSB_OK;
  }
  int grid = grid_for(n * (int64_t)c, kBlock, 32);
  switch (dtype) {
    case TSB_F32: voxelize_kernel<float><<<grid, kBlock, 0, st>>>((const float*)feats, idx, counts, n, n_vox, c, out); break;
    case TSB_F16: voxelize_kernel<__half><<<grid, kBlock, 0, st>>>((const __half*)feats, idx, counts, n, n_vox, c, out); break;
    case TSB_BF16: voxelize_kernel<__nv_bfloat16><<<grid, kBlock, 0, st>>>((const __nv_bfloat16*)feats, idx, counts, n, n_vox, c, out); break;
    default: return TSB_ERR_UNSUPPORTED;
  }
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_devoxelize_fwd(const void* feats, const int32_t* indices, const float* weights, int64_t n, int32_t c,
                       int32_t dtype, void* out, tsb_stream_t stream) {
  if (n < 0 || c < 1 || (n && (!feats || !indices || !weights || !out))) return TSB_ERR_BAD_ARG;
  if (n == 0) return TSB_OK;
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case TSB_F32: return devox_launch<float>(feats, indices, weights, n, c, out, st);
    case TSB_F16: return devox_launch<__half>(feats, indices, weights, n, c, out, st);
    case TSB_BF16: return devox_launch<__nv_bfloat16>(feats, indices, weights, n, c, out, st);
  }
  return TSB_ERR_UNSUPPORTED;
}

int tsb_to_dense_fwd(const void* feats, const int32_t* coords, int64_t n, int32_t c, const int32_t* range,
                     int32_t dtype, void* out, tsb_stream_t stream) {
  if (n < 0 || c < 1 || !range || (n && (!feats || !coords || !out))) return TSB_ERR_BAD_ARG;
  if (n == 0) return TSB_OK;
  cudaStream_t st = as_stream(stream);
  int grid = grid_for(n * (int64_t)c, kBlock, 32);
  const int4* c4 = reinterpret_cast<const int4*>(coords);
  switch (dtype) {
    case TSB_F32: to_dense_kernel<float><<<grid, kBlock, 0, st>>>((const float*)feats, c4, n, c, range[0], range[1], range[2], range[3], (float*)out); break;
    case TSB_F16: to_dense_kernel<__half><<<grid, kBlock, 0, st>>>((const __half*)feats, c4, n, c, range[0], range[1], range[2], range[3], (__half*)out); break;
    case TSB_BF16: to_dense_kernel<__nv_bfloat16><<<grid, kBlock, 0, st>>>((const __nv_bfloat16*)feats, c4, n, c, range[0], range[1], range[2], range[3], (__nv_bfloat16*)out); break;
    default: return TSB_ERR_UNSUPPORTED;
  }
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_to_dense_bwd(const void* grad_dense, const int32_t* coords, int64_t n, int32_t c, const int32_t* range,
                     int32_t dtype, void* grad_feats, tsb_stream_t stream) {
  if (n < 0 || c < 1 || !range || (n && (!grad_dense || !coords || !grad_feats))) return TSB_ERR_BAD_ARG;
  if (n == 0) return TSB_OK;
  cudaStream_t st = as_stream(stream);
  int grid = grid_for(n * (int64_t)c, kBlock, 32);
  const int4* c4 = reinterpret_cast<const int4*>(coords);
  switch (dtype) {
    case TSB_F32: to_dense_bwd_kernel<float><<<grid, kBlock, 0, st>>>((const float*)grad_dense, c4, n, c, range[0], range[1], range[2], range[3], (float*)grad_feats); break;
    case TSB_F16: to_dense_bwd_kernel<__half><<<grid, kBlock, 0, st>>>((const __half*)grad_dense, c4, n, c, range[0], range[1], range[2], range[3], (__half*)grad_feats); break;
    case TSB_BF16: to_dense_bwd_kernel<__nv_bfloat16><<<grid, kBlock, 0, st>>>((const __nv_bfloat16*)grad_dense, c4, n, c, range[0], range[1], range[2], range[3], (__nv_bfloat16*)grad_feats); break;
    default: return TSB_ERR_UNSUPPORTED;
  }
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_voxel_inputs(const float* points, int32_t c_in, const int64_t* first_index, const int32_t* uniq_coords,
                     const int32_t* quantize_result, int32_t batch, int64_t n_max, int32_t* coords, void* feats,
                     int32_t c_pad, int32_t dtype, tsb_stream_t stream) {
  if (n_max < 0 || c_in < 1 || c_pad < c_in || batch < 0 || !quantize_result) return TSB_ERR_BAD_ARG;
  if (n_max == 0) return TSB_OK;
  if (!points || !first_index || !uniq_coords || !coords || !feats) return TSB_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(n_max, kBlock);
  int4* c4 = reinterpret_cast<int4*>(coords);
  switch (dtype) {
    case TSB_F32:
      voxel_inputs_kernel<float><<<grid, kBlock, 0, s>>>(points, c_in, first_index, uniq_coords, quantize_result, batch,
                                                         n_max, c4, (float*)feats, c_pad);
      break;
    case TSB_F16:
      voxel_inputs_kernel<__half><<<grid, kBlock, 0, s>>>(points, c_in, first_index, uniq_coords, quantize_result, batch,
                                                          n_max, c4, (__half*)feats, c_pad);
      break;
    case TSB_BF16:
      voxel_inputs_kernel<__nv_bfloat16><<<grid, kBlock, 0, s>>>(points, c_in, first_index, uniq_coords, quantize_result,
                                                                 batch, n_max, c4, (__nv_bfloat16*)feats, c_pad);
      break;
    default:
      return TSB_ERR_UNSUPPORTED;
  }
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_voxelize_bwd(const float* grad_out, const int32_t* idx, const int32_t* counts, int64_t n, int64_t n_vox,
                     int32_t c, float* grad_feats, tsb_stream_t stream) {
  if (n < 0 || n_vox < 0 || c < 1 || (n && (!idx || !grad_feats)) || (n && n_vox && (!grad_out || !counts)))
    return TSB_ERR_BAD_ARG;
  if (n == 0) return TSB_OK;
  voxelize_bwd_kernel<<<grid_for(n * (int64_t)c, kBlock, 32), kBlock, 0, as_stream(stream)>>>(grad_out, idx, counts, n,
                                                                                            n_vox, c, grad_feats);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

int tsb_devoxelize_bwd(const float* grad_out, const int32_t* indices, const float* weights, int64_t n, int64_t n_vox,
                       int32_t c, float* grad_voxels, tsb_stream_t stream) {
  if (n < 0 || n_vox < 0 || c < 1 || (n_vox && !grad_voxels) || (n && (!grad_out || !indices || !weights)))
    return TSB_ERR_BAD_ARG;
  cudaStream_t st = as_stream(stream);
  if (n_vox) TSB_CUDA_TRY(cudaMemsetAsync(grad_voxels, 0, (size_t)n_vox * c * sizeof(float), st));
  if (n == 0 || n_vox == 0) return TSB_OK;
  devoxelize_bwd_kernel<<<grid_for(n * (int64_t)c, kBlock, 32), kBlock, 0, st>>>(grad_out, indices, weights, n, n_vox, c,
                                                                                grad_voxels);
  TSB_LAUNCH_CHECK();
  return TSB_OK;
}

}  // extern "C"
