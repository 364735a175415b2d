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
  return igemm_umma_workspace_bytes(kvol, cin, cout, dtype);
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
                       const int32_t* out_in_map, const int32_t* reorder_loc, void* out_feats, int64_t n_in,
                       int64_t n_out, int32_t kvol, int32_t cin, int32_t cout, int32_t dtype, int32_t math,
                       const float* scale, const float* bias, const void* residual, int32_t relu,
                       int32_t* dev_status, void* workspace, size_t workspace_bytes, tsb_stream_t stream) {
  if (n_in < 0 || n_out < 0 || kvol < 1 || cin < 1 || cout < 1) return TSB_ERR_BAD_ARG;
  if (!valid_dtype(dtype)) return TSB_ERR_UNSUPPORTED;
  if (n_out == 0) return TSB_OK;
  if (!weight || !out_in_map || !out_feats || (n_in && !in_feats)) return TSB_ERR_BAD_ARG;
  if (n_in > INT32_MAX || n_out > INT32_MAX) return TSB_ERR_LIMIT;
  IgemmArgs a{in_feats, weight, packed_weight, out_in_map, reorder_loc, out_feats, n_in, n_out, kvol, cin, cout,
              dtype, math, scale, bias, residual, relu, dev_status, workspace, workspace_bytes};
  if (igemm_umma_supported(a)) return igemm_umma(a, as_stream(stream));
  return igemm_simt(a, as_stream(stream));
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
