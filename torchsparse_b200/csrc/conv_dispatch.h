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
  // ---- optional extensions of the tensor-core kernel (zero / null: not used)
  const void* x2;            // second feature matrix [n_in, cin - c1]: input channels [c1, cin) come from it
  int c1;                    // channels held by x when x2 is given
  int64_t map_rs, map_cs;    // element strides of the map, entry (row, k) at map[row * map_rs + k * map_cs]
                             // (0, 0: row-major [rows][kvol]); a null map with kvol = 1 means row m reads input row m
  const unsigned* tile_mask; // [ceil(n_out / 128)] offsets present in each 128-row tile (null: derived in the workspace)
  const int* n_out_dev;      // number of output rows in device memory (n_out is then its upper bound)
  const float* acc_in;       // fp32 [dst_rows, cout] partial sums added to the accumulator before the epilogue
  float* acc_out;            // fp32 [dst_rows, cout]: store the accumulator (+ acc_in) here instead of y, no epilogue
  int k_lo, k_hi;            // kernel offsets [k_lo, k_hi) covered by this launch (0, 0: all)
  int cfg_n_tile, cfg_cpb, cfg_stages, cfg_ctas;   // tuning overrides of the launch configuration (0: automatic)
  int cfg_grid;         // upper bound of the persistent CTAs of a launch (0: every resident slot of the device)
  int cfg_gather;       // A operand: 0 / 1 = cp.async by the gather warps (default), 2 = TMA gather4 by the copy engine
  // work-item table of a map whose heavy tiles are split into parts (tsb_map_sorted_cm): int32 [n_items][4] =
  // {row tile, offset mask, part | parts << 8, 0}, its length in device memory, the fp32 running sums
  // [pad128(n_out), cout] and the per-(row tile, N tile) part counters (zero between launches)
  const int* items;
  const int* n_items_dev;
  int64_t n_items;           // upper bound of *n_items_dev (sizes the launch)
  float* split_scratch;
  int* split_flags;
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
size_t igemm_umma_workspace_bytes(int kvol, int cin, int cout, int dtype, int64_t n_out);
size_t tile_mask_bytes(int64_t n_out);
// offset mask of every 128-row tile of a map (entry (row, k) at map[row * rs + k * cs])
int tile_masks(const int* map, long long rs, long long cs, int kvol, int64_t n_rows, const int* n_rows_dev,
               unsigned* out, cudaStream_t s);
int igemm_umma(const IgemmArgs& a, cudaStream_t s);
// Weight gradient on the tensor cores: out[k][a][b] = sum over map rows m of g[map[m][k]][a] * p[m][b].
struct WgradArgs {
  const void* g;             // [n_g, cg]: the matrix addressed through the map
  const void* p;             // [n_rows, cd]: the matrix whose rows are the map's rows
  const int* map;            // entry (row, k) at map[row * map_rs + k * map_cs] (0, 0: row-major [rows][kvol])
  int64_t map_rs, map_cs;
  const unsigned* tile_mask; // nullable: offsets present in each 128-row tile (derived in the workspace when null)
  float* out;                // fp32 [kvol, cg, cd]; zeroed by the call
  int64_t n_g, n_rows;
  int kvol, cg, cd, dtype;
  int* dev_status;           // nullable
  void* workspace;
  size_t workspace_bytes;
};
bool wgrad_umma_supported(const WgradArgs& a);
size_t wgrad_umma_workspace_bytes(int64_t n_rows);
int wgrad_umma(const WgradArgs& a, cudaStream_t s);
int wgrad_simt(const WgradArgs& a, cudaStream_t s);   // CUDA cores: every dtype and channel count, row-major maps

size_t packed_weight_bytes(int kvol, int cin, int cout, int dtype);
int pack_weight(const void* w, int kvol, int cin, int cout, int dtype, void* packed, cudaStream_t s);


// tensor-core pair-list paths of the other two dataflows (conv_pairs.cu)
bool pairs_umma_usable(const void* x, const void* w, int64_t n_in, int kvol, int cin, int cout, int dtype, int math);
size_t gs_umma_workspace_bytes(int64_t n_pairs, int kvol, int cin, int cout, int dtype);
size_t fod_umma_workspace_bytes(int64_t n_out, int64_t qmapsize, int kvol, int cin, int cout, int dtype);
int gs_umma(const GsArgs& a, cudaStream_t s);
int fod_umma(const FodArgs& a, cudaStream_t s);

}  // namespace tsb
