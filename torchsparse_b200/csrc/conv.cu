// C ABI of the convolution forward entry points and the choice between the tcgen05
// (tensor-core) kernels and the CUDA-core kernels.
#include <cstdlib>

#include "common.cuh"
#include "conv_dispatch.h"

using namespace tsb;

namespace {
bool valid_dtype(int d) { return d == TSB_F32 || d == TSB_F16 || d == TSB_BF16; }
}  // namespace

extern "C" {

size_t tsb_conv_igemm_workspace_bytes(int32_t kvol, int32_t cin, int32_t cout, int32_t dtype) {
  if (kvol < 1 || cin < 1 || cout < 1 || !valid_dtype(dtype)) return 0;
  return igemm_umma_workspace_bytes(kvol, cin, cout, dtype, 0);
}

size_t tsb_map_tile_mask_bytes(int64_t n_rows) { return n_rows < 0 ? 0 : tile_mask_bytes(n_rows); }

int tsb_map_tile_mask(const int32_t* map, int64_t n_rows, int32_t kvol, int64_t row_stride, int64_t col_stride,
                      const int32_t* n_rows_dev, uint32_t* out, tsb_stream_t stream) {
  if (n_rows < 0 || kvol < 1 || kvol > 32 || row_stride < 1 || col_stride < 1) return TSB_ERR_BAD_ARG;
  if (n_rows == 0) return TSB_OK;
  if (!map || !out) return TSB_ERR_BAD_ARG;
  return tile_masks(map, row_stride, col_stride, kvol, n_rows, n_rows_dev, out, as_stream(stream));
}

size_t tsb_conv_packed_weight_bytes(int32_t kvol, int32_t cin, int32_t cout, int32_t dtype) {
  if (kvol < 1 || cin < 1 || cout < 1 || !valid_dtype(dtype)) return 0;
  return packed_weight_bytes(kvol, cin, cout, dtype);
}

int tsb_conv_pack_weight(const void* weight, int32_t kvol, int32_t cin, int32_t cout, int32_t dtype, void* packed,
                         tsb_stream_t stream) {
  if (kvol < 1 || cin < 1 || cout < 1 || !weight || !packed) return TSB_ERR_BAD_ARG;
  if (!valid_dtype(dtype)) return TSB_ERR_UNSUPPORTED;
  return pack_weight(weight, kvol, cin, cout, dtype, packed, as_stream(stream));
}

int tsb_conv_igemm_fwd(const void* in_feats, const void* weight, const void* packed_weight,
                       const int32_t* out_in_map, const int32_t* reorder_loc, const uint32_t* tile_mask,
                       void* out_feats, int64_t n_in, int64_t n_out, int32_t kvol, int32_t cin, int32_t cout,
                       int32_t dtype, int32_t math, const float* scale, const float* bias, const void* residual,
                       int32_t relu, int32_t* dev_status, void* workspace, size_t workspace_bytes,
                       tsb_stream_t stream) {
  if (n_in < 0 || n_out < 0 || kvol < 1 || cin < 1 || cout < 1) return TSB_ERR_BAD_ARG;
  if (!valid_dtype(dtype)) return TSB_ERR_UNSUPPORTED;
  if (n_out == 0) return TSB_OK;
  if (!weight || !out_in_map || !out_feats || (n_in && !in_feats)) return TSB_ERR_BAD_ARG;
  if (n_in > INT32_MAX || n_out > INT32_MAX) return TSB_ERR_LIMIT;
  IgemmArgs a{in_feats, weight, packed_weight, out_in_map, reorder_loc, out_feats, n_in, n_out, kvol, cin, cout,
              dtype, math, scale, bias, residual, relu, dev_status, workspace, workspace_bytes};
  a.tile_mask = tile_mask;
  if (igemm_umma_supported(a)) return igemm_umma(a, as_stream(stream));
  return igemm_simt(a, as_stream(stream));
}

int tsb_conv_igemm_run(const tsb_igemm_desc* d, tsb_stream_t stream) {
  if (!d || d->struct_bytes != sizeof(tsb_igemm_desc)) return TSB_ERR_BAD_ARG;
  if (d->n_in < 0 || d->n_out < 0 || d->kvol < 1 || d->cin < 1 || d->cout < 1) return TSB_ERR_BAD_ARG;
  if (!valid_dtype(d->dtype)) return TSB_ERR_UNSUPPORTED;
  if (d->n_out == 0) return TSB_OK;
  if (!d->weight || !d->in_feats || (!d->out_feats && !d->acc_out)) return TSB_ERR_BAD_ARG;
  if (!d->out_in_map && d->kvol != 1) return TSB_ERR_BAD_ARG;
  if (d->n_in > INT32_MAX || d->n_out > INT32_MAX || d->dst_rows > INT32_MAX) return TSB_ERR_LIMIT;
  if (d->in_feats2 && (d->c1 <= 0 || d->c1 >= d->cin)) return TSB_ERR_BAD_ARG;
  if ((d->map_row_stride == 0) != (d->map_col_stride == 0) || d->map_row_stride < 0 || d->map_col_stride < 0)
    return TSB_ERR_BAD_ARG;
  IgemmArgs a{d->in_feats, d->weight, d->packed_weight, d->out_in_map, d->reorder_loc, d->out_feats, d->n_in, d->n_out,
              d->kvol, d->cin, d->cout, d->dtype, d->math, d->scale, d->bias, d->residual, d->relu, d->dev_status,
              d->workspace, d->workspace_bytes};
  a.dst_rows = d->dst_rows;
  a.x2 = d->in_feats2; a.c1 = d->c1;
  a.map_rs = d->map_row_stride; a.map_cs = d->map_col_stride;
  a.tile_mask = d->tile_mask; a.n_out_dev = d->n_out_dev;
  a.acc_in = d->acc_in; a.acc_out = d->acc_out;
  a.k_lo = d->k_lo; a.k_hi = d->k_hi;
  a.cfg_n_tile = d->cfg_n_tile; a.cfg_cpb = d->cfg_cpb; a.cfg_stages = d->cfg_stages; a.cfg_ctas = d->cfg_ctas;
  a.cfg_gather = d->cfg_gather; a.cfg_grid = d->cfg_grid;
  a.items = d->items; a.n_items_dev = d->n_items_dev; a.n_items = d->n_items;
  a.split_scratch = d->split_scratch; a.split_flags = d->split_flags;
  if (a.items && a.n_items > INT32_MAX) return TSB_ERR_LIMIT;
  if (!igemm_umma_supported(a)) return TSB_ERR_UNSUPPORTED;
  return igemm_umma(a, as_stream(stream));
}

size_t tsb_conv_wgrad_igemm_workspace_bytes(int64_t n_rows) { return n_rows < 0 ? 0 : wgrad_umma_workspace_bytes(n_rows); }

int tsb_conv_wgrad_igemm(const void* gathered_feats, const void* row_feats, const int32_t* out_in_map,
                         const uint32_t* tile_mask, float* grad_weight, int64_t n_gathered, int64_t n_rows,
                         int64_t map_row_stride, int64_t map_col_stride, int32_t kvol, int32_t c_gathered, int32_t c_rows,
                         int32_t dtype, int32_t* dev_status, void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  if (n_gathered < 0 || n_rows < 0 || kvol < 1 || c_gathered < 1 || c_rows < 1) return TSB_ERR_BAD_ARG;
  if (!valid_dtype(dtype)) return TSB_ERR_UNSUPPORTED;
  if (!grad_weight) return TSB_ERR_BAD_ARG;
  if ((map_row_stride == 0) != (map_col_stride == 0) || map_row_stride < 0 || map_col_stride < 0) return TSB_ERR_BAD_ARG;
  if (n_gathered == 0 || n_rows == 0) {      // no pair: the gradient is zero
    TSB_CUDA_TRY(cudaMemsetAsync(grad_weight, 0, (size_t)kvol * c_gathered * c_rows * sizeof(float), as_stream(stream)));
    return TSB_OK;
  }
  if (!gathered_feats || !row_feats || !out_in_map) return TSB_ERR_BAD_ARG;
  WgradArgs a{gathered_feats, row_feats, out_in_map, map_row_stride, map_col_stride, tile_mask, grad_weight, n_gathered,
              n_rows, kvol, c_gathered, c_rows, dtype, dev_status, workspace, workspace_bytes};
  if (!wgrad_umma_supported(a)) return wgrad_simt(a, as_stream(stream));
  return wgrad_umma(a, as_stream(stream));
}

size_t tsb_conv_gs_workspace_bytes(int64_t n_pairs, int32_t kvol, int32_t cin, int32_t cout, int32_t dtype) {
  if (n_pairs < 0 || kvol < 1 || cin < 1 || cout < 1 || !valid_dtype(dtype)) return 0;
  const size_t simt = gs_workspace_bytes(n_pairs, kvol, cin, cout, dtype);
  const size_t umma = gs_umma_workspace_bytes(n_pairs, kvol, cin, cout, dtype);
  return simt > umma ? simt : umma;
}

int tsb_conv_gs_fwd(const void* in_feats, const void* weight, const int32_t* nbmaps, const int32_t* nbsizes_host,
                    const int32_t* scatter_mask, void* out_feats, int64_t n_in, int64_t n_out, int32_t kvol,
                    int32_t cin, int32_t cout, int32_t dtype, int32_t math, int32_t transpose, void* workspace,
                    size_t workspace_bytes, tsb_stream_t stream) {
  if (n_in < 0 || n_out < 0 || kvol < 1 || cin < 1 || cout < 1 || !nbsizes_host) return TSB_ERR_BAD_ARG;
  if (!valid_dtype(dtype)) return TSB_ERR_UNSUPPORTED;
  if (n_out == 0) return TSB_OK;
  int64_t n_pairs = 0;
  for (int k = 0; k < kvol; ++k) {
    if (nbsizes_host[k] < 0) return TSB_ERR_BAD_ARG;
    n_pairs += nbsizes_host[k];
  }
  if (!weight || !out_feats || !scatter_mask || (n_pairs && (!nbmaps || !in_feats))) return TSB_ERR_BAD_ARG;
  if (n_pairs > INT32_MAX) return TSB_ERR_LIMIT;
  GsArgs a{in_feats, weight, nbmaps, nbsizes_host, scatter_mask, out_feats, n_in, n_out, n_pairs, kvol, cin, cout,
           dtype, math, transpose, workspace, workspace_bytes};
  // tensor cores when the shape allows (16-bit tensors, or fp32 under TF32 math); else the CUDA cores
  if (pairs_umma_usable(in_feats, weight, n_in, kvol, cin, cout, dtype, math) &&
      workspace_bytes >= gs_umma_workspace_bytes(n_pairs, kvol, cin, cout, dtype))
    return gs_umma(a, as_stream(stream));
  return gs_simt(a, as_stream(stream));
}

size_t tsb_conv_fod_workspace_bytes(int64_t n_out, int64_t qmapsize, int32_t kvol, int32_t cin, int32_t cout,
                                    int32_t dtype) {
  if (n_out < 0 || qmapsize < 0 || kvol < 1 || cin < 1 || cout < 1 || !valid_dtype(dtype)) return 0;
  const size_t simt = dtype == TSB_F32 ? 256 : align_up((size_t)n_out * cout * sizeof(float), 256) + 256;
  const size_t umma = fod_umma_workspace_bytes(n_out, qmapsize, kvol, cin, cout, dtype);
  return simt > umma ? simt : umma;
}

int tsb_conv_fod_fwd(const void* in_feats, const void* weight, const int32_t* nbmaps, int64_t n_pairs,
                     const int32_t* nbaddrs, const int32_t* qnbaddrs, int64_t qmapsize, void* out_feats,
                     int64_t n_in, int64_t n_out, int32_t kvol, int32_t cin, int32_t cout, int32_t dtype,
                     int32_t math, int32_t transpose, void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  if (n_in < 0 || n_out < 0 || n_pairs < 0 || qmapsize < 0 || kvol < 1 || cin < 1 || cout < 1) return TSB_ERR_BAD_ARG;
  if (!valid_dtype(dtype)) return TSB_ERR_UNSUPPORTED;
  if (n_out == 0) return TSB_OK;
  if (!weight || !out_feats || !nbaddrs || !qnbaddrs || (n_pairs && (!nbmaps || !in_feats))) return TSB_ERR_BAD_ARG;
  if (qmapsize > INT32_MAX || n_pairs > INT32_MAX) return TSB_ERR_LIMIT;
  FodArgs a{in_feats, weight, nbmaps, nbaddrs, qnbaddrs, out_feats, n_in, n_out, n_pairs, qmapsize, kvol, cin, cout,
            dtype, math, transpose, workspace, workspace_bytes};
  // The tensor-core path adds its products to the output with vector atomics from the epilogue; below
  // 128 x 128 channels a launch is bound by those atomics and the CUDA-core kernel (whose lanes add to
  // consecutive floats of a row) is as fast or faster, so it keeps the narrow layers.
  if ((int64_t)cin * cout >= 128 * 128 && pairs_umma_usable(in_feats, weight, n_in, kvol, cin, cout, dtype, math) &&
      workspace_bytes >= fod_umma_workspace_bytes(n_out, qmapsize, kvol, cin, cout, dtype))
    return fod_umma(a, as_stream(stream));
  return fod_simt(a, as_stream(stream));
}

}  // extern "C"
