// Argument bundles and entry points shared by the convolution translation units.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace tsb {

struct IgemmArgs {
  const void* x;
  const void* w;
  const void* packed_w;  // nullable: weights already in [kvol, cout, cin] order
  const int* map;
  const int* reorder_loc;
  void* y;
  int64_t n_in, n_out;
  int kvol, cin, cout, dtype, math;
  const float* scale;  // nullable: y = acc * scale[n] + bias[n] (+ residual), then ReLU
  const float* bias;
  const void* residual;
  int relu;
  int* dev_status;  // nullable
  void* workspace;
  size_t workspace_bytes;
  // pair-list mode of the tensor-core kernel (zero / null otherwise): `map` is one column of input rows,
  // 128-row tile t multiplies with weight offset tile_k[t] of a [kvol_w, cin, cout] weight tensor
  const int* tile_k;
  int kvol_w;
  int out_fp32;     // 16-bit operands, fp32 output rows
  int atomic_out;   // fp32 output rows accumulated with atomic adds
  int64_t dst_rows; // rows of y when they are addressed through reorder_loc (0: n_out)
};

struct GsArgs {
  const void* x;
  const void* w;
  const int* nbmaps;        // [P,2]
  const int* nbsizes_host;  // [kvol]
  const int* scatter_mask;  // [kvol * n_out]
  void* y;
  int64_t n_in, n_out, n_pairs;
  int kvol, cin, cout, dtype, math, transpose;
  void* workspace;
  size_t workspace_bytes;
};

struct FodArgs {
  const void* x;
  const void* w;
  const int* nbmaps;  // [2,P]
  const int* nbaddrs;
  const int* qnbaddrs;
  void* y;
  int64_t n_in, n_out, n_pairs, qmapsize;
  int kvol, cin, cout, dtype, math, transpose;
  void* workspace;
  size_t workspace_bytes;
};

// CUDA-core kernels (conv_simt.cu)
int igemm_simt(const IgemmArgs& a, cudaStream_t s);
int gs_simt(const GsArgs& a, cudaStream_t s);
int fod_simt(const FodArgs& a, cudaStream_t s);
size_t gs_workspace_bytes(int64_t n_pairs, int kvol, int cin, int cout, int dtype);

// tcgen05 kernels (conv_umma.cu)
bool igemm_umma_supported(const IgemmArgs& a);
size_t igemm_umma_workspace_bytes(int kvol, int cin, int cout, int dtype);
int igemm_umma(const IgemmArgs& a, cudaStream_t s);
size_t packed_weight_bytes(int kvol, int cin, int cout, int dtype);
int pack_weight(const void* w, int kvol, int cin, int cout, int dtype, void* packed, cudaStream_t s);


// tensor-core pair-list paths of the other two dataflows (conv_pairs.cu)
bool pairs_umma_usable(const void* x, const void* w, int64_t n_in, int kvol, int cin, int cout, int dtype, int math);
size_t gs_umma_workspace_bytes(int64_t n_pairs, int kvol, int cin, int cout, int dtype);
size_t fod_umma_workspace_bytes(int64_t n_out, int64_t qmapsize, int kvol, int cin, int cout, int dtype);
int gs_umma(const GsArgs& a, cudaStream_t s);
int fod_umma(const FodArgs& a, cudaStream_t s);

}  // namespace tsb
