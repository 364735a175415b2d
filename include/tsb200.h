/*
 * tsb200 - C ABI of the B200 (sm_100a) sparse-convolution hot path.
 *
 * Every entry point takes raw DEVICE pointers (unless a parameter says "host"),
 * explicit sizes and a CUDA stream, launches asynchronously on that stream and
 * returns a status code.  Except where a function says otherwise, nothing here
 * allocates, frees or synchronises: the caller owns every buffer, including
 * scratch (each op that needs scratch has a *_workspace_bytes query).
 *
 * Each declaration names the entry of the reference project's pybind module
 * (torchsparse/backend/pybind_cuda.cu) that it replaces, with file:line inside
 * the reference project.
 */
#ifndef TSB200_H_
#define TSB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* tsb_stream_t; /* a cudaStream_t */

/* status codes */
enum {
  TSB_OK = 0,
  TSB_ERR_BAD_ARG = 1,       /* null pointer, negative size, unsupported shape */
  TSB_ERR_UNSUPPORTED = 2,   /* dtype / configuration not implemented */
  TSB_ERR_WORKSPACE = 3,     /* workspace too small */
  TSB_ERR_CUDA = 4,          /* a CUDA runtime call failed (see tsb_last_cuda_error) */
  TSB_ERR_LIMIT = 5          /* size beyond a stated maximum */
};

/* element types of feature / weight tensors */
enum { TSB_F32 = 0, TSB_F16 = 1, TSB_BF16 = 2 };

/* arithmetic for TSB_F32 inputs: exact fp32 FMA, or TF32 tensor cores */
enum { TSB_MATH_FP32 = 0, TSB_MATH_TF32 = 1 };

/* bits of the device status word written by table kernels (0 = fine) */
enum { TSB_DEV_TABLE_FULL = 1, TSB_DEV_BAD_INDEX = 2,
       TSB_DEV_LIMIT = 4 /* a device-side size went beyond the bound the caller stated */ };

const char* tsb_version(void);
const char* tsb_status_string(int status);
/* cudaGetErrorString of the last failed runtime call inside this library (thread-local). */
const char* tsb_last_cuda_error(void);
/* Number of kernels this library has launched in this process so far (library sort / scan /
 * select passes count as one launch each).  No counterpart in the reference. */
long long tsb_launch_count(void);

/* ---------------------------------------------------------------- hashing */

/* FNV-1a-64 of each (b,x,y,z) int32 row -> int64 [n].
 * Replaces hash_cuda (torchsparse/backend/hash/hash_cuda.cu:66-72). */
int tsb_coord_hash(const int32_t* coords, int64_t n, int64_t* out, tsb_stream_t stream);

/* Hash of coords + offset for each of k offsets (int32 [k,3]) -> int64 [k,n].
 * Replaces kernel_hash_cuda (torchsparse/backend/hash/hash_cuda.cu:74-83). */
int tsb_kernel_hash(const int32_t* coords, int64_t n, const int32_t* offsets, int32_t k,
                    int64_t* out, tsb_stream_t stream);

/* ---------------------------------------------------------------- hash table
 * Open addressing over two caller-owned arrays: keys int64 [capacity] (0 = empty)
 * and vals int32 [capacity].  Stored value for the i-th inserted key is i+1; a
 * lookup miss returns 0.  Probes are bounded by the capacity: a full table sets
 * TSB_DEV_TABLE_FULL in *dev_status (int32, device, may be NULL) instead of
 * spinning.  Replaces class GPUHashTable
 * (torchsparse/backend/hashmap/hashmap_cuda.cuh:65-118) and its kernels
 * (hashmap_cuda.cuh:124-196, 316-347).
 *
 * 32-bit keys: table_vals == NULL selects the packed layout, in which table_keys holds `capacity`
 * 8-byte slots, value << 32 | key (0 = empty), for keys below 2^32.  Insert is one compare-and-swap
 * of the slot and a probe one 8-byte load.  tsb_hash_insert / tsb_hash_lookup, tsb_kmap_subm,
 * tsb_kmap_down_finish and the *_dyn builders take either layout and give the same maps; a key that
 * does not fit returns TSB_ERR_LIMIT where the host knows the key space (bounds, key_bits) and sets
 * TSB_DEV_LIMIT in *dev_status where only the device does.  Replaces the hashtable32 instantiation
 * behind build_kernel_map_subm_hashmap_int32 / build_kernel_map_downsample_hashmap_int32
 * (torchsparse/backend/others/sparsemapping_cuda.cu:259-300, 347-426;
 * torchsparse/backend/hashmap/hashmap_cuda.cuh). */
int tsb_hash_insert(int64_t* table_keys, int32_t* table_vals, int64_t capacity,
                    const int64_t* keys, int64_t n, int32_t* dev_status, tsb_stream_t stream);
int tsb_hash_lookup(const int64_t* table_keys, const int32_t* table_vals, int64_t capacity,
                    const int64_t* keys, int64_t n, int32_t* out_vals, tsb_stream_t stream);

/* Kernel-map lookup of the "hashmap" mode: the table holds FNV-1a hashes of (x, y, z, b) rows
 * (tsb_coord_hash + tsb_hash_insert); out int32 [pad128(n), kvol] (zero-filled by the call) gets, for
 * output row i and kernel index k, the value stored for  coords[i] * stride + digit_k - (kernel - 1) / 2,
 * i.e. input row + 1, or 0.  coords_xyzb: int32 [n,4] in (x, y, z, batch) order; kernel_size / stride:
 * host int32 [3].  Replaces GPUHashTable::lookup_coords
 * (torchsparse/backend/hashmap/hashmap_cuda.cuh:200-254, 307-314). */
int tsb_hash_lookup_coords(const int64_t* table_keys, const int32_t* table_vals, int64_t capacity,
                           const int32_t* coords_xyzb, int64_t n, const int32_t* kernel_size,
                           const int32_t* stride, int32_t* out, tsb_stream_t stream);

/* Join: out[i] = value stored for query[i] minus 1, i.e. row of the reference key or -1.
 * Builds a private table inside `workspace` (tsb_hash_query_workspace_bytes(n_ref)).
 * Replaces hash_query_cuda (torchsparse/backend/others/query_cuda.cu:33-47). */
size_t tsb_hash_query_workspace_bytes(int64_t n_ref);
int tsb_hash_query(const int64_t* queries, int64_t n_q, const int64_t* refs, int64_t n_ref,
                   int64_t* out, void* workspace, size_t workspace_bytes, tsb_stream_t stream);

/* The same join for callers that are not allowed to allocate device memory and have no scratch
 * buffer to lend: for example a plug-in that a host application calls with nothing but its input
 * and output buffers, or a real-time perception loop whose device memory is carved up once at
 * start-up and where a cudaMalloc in the loop (it synchronises the device and can fail) is ruled
 * out.  This entry point has no counterpart in the reference.
 *
 * The private table lives in a 6 MiB array compiled into the library (every GPU that loads the
 * library holds it until the process exits), so n_ref is limited to
 * tsb_hash_query_static_max_refs() = 262144 keys; a larger n_ref returns TSB_ERR_LIMIT and does
 * nothing.  The call allocates and frees nothing.  The first call on each device looks up the
 * array's device address (a host-side runtime query, not a launch): make that first call before
 * starting any stream capture.  All calls share the one array and each call clears it first, so
 * two calls whose work overlaps on the GPU (different streams, no dependency) race; calls issued
 * to one stream are safe.  Results equal tsb_hash_query's. */
int64_t tsb_hash_query_static_max_refs(void);
int tsb_hash_query_static(const int64_t* queries, int64_t n_q, const int64_t* refs, int64_t n_ref,
                          int64_t* out, tsb_stream_t stream);

/* ---------------------------------------------------------------- kernel maps
 * Coordinates are int32 rows (b,x,y,z).  cmin/cmax are HOST int32[4] arrays: the
 * inclusive bounds used for the ravel index and the x,y,z bounds check.
 * Kernel-index digit order: odd kernel volume -> x fastest, even -> z fastest.
 * Every map has rows padded to a multiple of 128 with -1. */

/* Submanifold map (all strides 1).  If to_insert != 0 the coordinates are first
 * inserted into the table (key = ravel+1, value = row+1).  out_in_map is int32
 * [pad128(n), kvol]; it is fully written (including the -1 fill).
 * Replaces build_kernel_map_subm_hashmap
 * (torchsparse/backend/others/sparsemapping_cuda.cu:303-345). */
int tsb_kmap_subm(int64_t* table_keys, int32_t* table_vals, int64_t capacity,
                  const int32_t* coords, int64_t n, const int32_t* cmin, const int32_t* cmax,
                  const int32_t* kernel_size, int32_t to_insert, int32_t* out_in_map,
                  int32_t* dev_status, tsb_stream_t stream);

/* Strided map, step 1 of 3: candidate output ravel keys of every input, sorted and
 * made unique.  Writes unique keys (ascending) to uniq_keys (int64, capacity
 * n*slots where slots = tsb_kmap_down_slots(...)), and to result (int32 [8],
 * device): result[0] = number of outputs M, result[1..4] = per-column maximum of
 * the output coordinates (b,x,y,z).  cmax_out is the bound in OUTPUT space.
 * Replaces stage 1 + torch::_unique of build_kernel_map_downsample_hashmap
 * (torchsparse/backend/others/sparsemapping_cuda.cu:60-107, 464-478). */
int32_t tsb_kmap_down_slots(const int32_t* kernel_size, const int32_t* stride);
size_t tsb_kmap_down_workspace_bytes(int64_t n, const int32_t* kernel_size, const int32_t* stride);
int tsb_kmap_down_unique(const int32_t* coords, int64_t n, const int32_t* cmin,
                         const int32_t* cmax_out, const int32_t* kernel_size,
                         const int32_t* stride, const int32_t* padding, int64_t* uniq_keys,
                         int32_t* result, void* workspace, size_t workspace_bytes,
                         tsb_stream_t stream);

/* Strided map, steps 2+3 (after the caller has read M from `result`): unravels the
 * unique keys into out_coords int32 [M,4], inserts them into the (empty) table
 * (key = ravel+1, value = row+1) and writes out_in_map int32 [pad128(M), kvol]
 * with map[out][kvol-1-k'] = in.
 * Replaces stages 2.1 and 3 (sparsemapping_cuda.cu:44-57, 110-126, 480-506). */
int tsb_kmap_down_finish(int64_t* table_keys, int32_t* table_vals, int64_t capacity,
                         const int32_t* coords, int64_t n, const int64_t* uniq_keys, int64_t m,
                         const int32_t* cmin, const int32_t* cmax_out, const int32_t* kernel_size,
                         const int32_t* stride, const int32_t* padding, int32_t* out_coords,
                         int32_t* out_in_map, int32_t* dev_status, tsb_stream_t stream);

/* map_t[in][k] = out for every map[out][k] = in.  map_t is int32 [rows_t, kvol]; when
 * fill != 0 it is first set to -1 by this call (the reference pre-fills it in Python).
 * Replaces convert_transposed_out_in_map (torchsparse/backend/others/query_cuda.cu:50-54). */
int tsb_map_transpose(const int32_t* out_in_map, int64_t rows, int32_t kvol, int32_t* map_t,
                      int64_t rows_t, int32_t fill, tsb_stream_t stream);

/* bitmask int32 [split, rows]: bit i of split s = (map[row][s*split_len+i] >= 0); rows >=
 * valid_n get -1.  Replaces derive_bitmask_from_out_in_map (query_cuda.cu:59-65). */
int tsb_bitmask_derive(const int32_t* out_in_map, int64_t rows, int32_t kvol, int32_t split,
                       int64_t valid_n, int32_t* bitmask, tsb_stream_t stream);

/* Descending stable sort of each split's bitmask row: sorted_mask int32 [split, rows],
 * reorder_loc int32 [split, rows] (original row of each sorted position).
 * Replaces the torch.sort call of the reference's Python side
 * (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:96). */
size_t tsb_bitmask_sort_workspace_bytes(int64_t rows, int32_t split);
int tsb_bitmask_sort(const int32_t* bitmask, int64_t rows, int32_t split, int32_t kvol,
                     int32_t* sorted_mask, int32_t* reorder_loc, void* workspace,
                     size_t workspace_bytes, tsb_stream_t stream);

/* reduced int32 [split, ceil(rows/tile)] = OR over each tile of rows.
 * Replaces reduce_bitmask_cuda (torchsparse/backend/others/reduce_bitmask_cuda.cu:60-87). */
int tsb_bitmask_reduce(const int32_t* bitmask, int64_t rows, int32_t split, int32_t tile,
                       int32_t* reduced, tsb_stream_t stream);

/* out[r][c] = map[loc[split(c)][r]][c].
 * Replaces reorder_out_in_map_cuda (torchsparse/backend/others/reorder_map_cuda.cu:25-47). */
int tsb_map_reorder(const int32_t* out_in_map, int64_t rows, int32_t kvol, const int32_t* reorder_loc,
                    int32_t split, int32_t* out, tsb_stream_t stream);

/* ---------------------------------------------------------------- kernel maps with sizes in device memory
 * The same maps as tsb_kmap_subm / tsb_kmap_down_*, for callers that must not read sizes back to the host
 * (a sequence of builds and convolutions recorded once and replayed, e.g. as a CUDA graph).  The number of
 * coordinates of a tensor stride and their bounds live in a "level record", int32[16] in device memory:
 * [0] rows, [1..4] lower and [5..8] upper bound (b,x,y,z) of the key space of the level's hash table,
 * [9..12] the largest coordinate present, rest reserved.  Launches are sized for n_max / m_max rows (the
 * caller's upper bounds; buffers have that many rows); rows beyond the device-side count are not written,
 * except that every map is -1 filled up to the next multiple of 128 rows.  Coordinates must be >= 0.
 * No counterpart in the reference, whose builders read two sizes back per strided map
 * (torchsparse/backend/others/sparsemapping_cuda.cu:435,477). */

/* Level record of the finest level from the result record of tsb_quantize_unique (voxel count, min, max);
 * all rows get batch index `batch`.  Negative voxel coordinates set TSB_DEV_LIMIT in *dev_status. */
int tsb_level_record_from_quantize(const int32_t* quantize_result, int32_t batch, int32_t* rec, int32_t* dev_status,
                                   tsb_stream_t stream);

/* tsb_kmap_subm with the row count and bounds read from `rec`.  capacity >= 2 * n_max; with to_insert != 0
 * the table keys are cleared first. */
int tsb_kmap_subm_dyn(int64_t* table_keys, int32_t* table_vals, int64_t capacity, const int32_t* coords, int64_t n_max,
                      const int32_t* rec, const int32_t* kernel_size, int32_t to_insert, int32_t* out_in_map,
                      int32_t* dev_status, tsb_stream_t stream);

/* The whole strided build in one call: candidates -> sort -> unique -> output coordinates + table insert ->
 * map, and (out_in_map_t != NULL) the transposed map int32 [pad128(n_max), kvol] of the matching transposed
 * convolution.  Writes the output level's record to rec_out (the table then holds the output coordinates,
 * as tsb_kmap_down_finish leaves it).  key_bits: the candidate keys are sorted on this many bits, so the
 * output key space (batch x X x Y x Z cells) must stay below 2^key_bits - 1: derive it from an upper bound
 * of the coordinates; a larger space sets TSB_DEV_LIMIT in *dev_status.  m_max <= n_max * slots: rows of
 * out_coords / out_in_map; capacity >= 2 * m_max. */
size_t tsb_kmap_down_dyn_workspace_bytes(int64_t n_max, const int32_t* kernel_size, const int32_t* stride);
int tsb_kmap_down_dyn(int64_t* table_keys, int32_t* table_vals, int64_t capacity, const int32_t* coords, int64_t n_max,
                      const int32_t* rec_in, const int32_t* kernel_size, const int32_t* stride, const int32_t* padding,
                      int32_t key_bits, int64_t m_max, int32_t* out_coords, int32_t* out_in_map, int32_t* out_in_map_t,
                      int32_t* rec_out, int32_t* dev_status, void* workspace, size_t workspace_bytes,
                      tsb_stream_t stream);

/* The four steps above for one split in one call: bitmask of every row, stable descending sort,
 * row-reordered map, per-tile OR of the sorted masks.  sorted_mask / reorder_loc int32 [rows],
 * reordered_map int32 [rows, kvol], reduced_mask int32 [ceil(rows / tile)].  At batch 1 the host cost
 * of four separate calls exceeds the device time of the steps.  No counterpart in the reference
 * (its Python side chains derive_bitmask_from_out_in_map, torch.sort, reorder_out_in_map_cuda and
 * reduce_bitmask_cuda, torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:86-111). */
size_t tsb_map_sorted_workspace_bytes(int64_t rows);
int tsb_map_sorted_artefacts(const int32_t* out_in_map, int64_t rows, int32_t kvol, int64_t valid_n, int32_t tile,
                             int32_t* sorted_mask, int32_t* reorder_loc, int32_t* reordered_map,
                             int32_t* reduced_mask, void* workspace, size_t workspace_bytes, tsb_stream_t stream);

/* The row order and map layout the tensor-core convolution is fastest on, for a map that is used by
 * several launches (every submanifold layer of a resolution level shares one map): rows sorted by their
 * neighbour mask (stable, descending, padding rows last) so that the 128 rows of a tile share their
 * offsets, the reordered map stored column-major (map_cm int32 [kvol][rows], entry of sorted row r and
 * offset k at map_cm[k * rows + r]), and the per-tile offset masks (tile_mask uint32 [rows / 128]).
 * reorder_loc int32 [rows]: sorted row r is map row reorder_loc[r] (the row its output is stored at).
 * rows = padded row count of out_in_map (a multiple of 128); valid_n rows are real; valid_n_dev (int32,
 * device, nullable) overrides valid_n with a count in device memory (valid_n is then its upper bound).
 * The same idea as the reference's derive_bitmask -> torch.sort -> reorder_out_in_map -> reduce_bitmask
 * chain (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:92-107); the layout and the
 * sort key are this library's own, so the results are not interchangeable with that chain's. */
size_t tsb_map_sorted_cm_workspace_bytes(int64_t rows);
/* Upper bound of the number of work items (below) of a map with `rows` padded rows. */
int64_t tsb_map_items_max(int64_t rows, int32_t kvol, int32_t max_offsets);
/* items (nullable) int32 [tsb_map_items_max(...)][4], 16-byte aligned, and n_items (int32, device): the
 * work-item table of the sorted map.  A tile with more than max_offsets offsets (in a sorted map these are
 * the first tiles, and they hold a large share of all the work) is listed as several consecutive items that
 * each take an equal share of its offsets: {row tile, offset mask of the part, part | parts << 8 | first
 * scratch slot << 16, 0} (third word 0 for a whole tile).  Each part of a split tile owns one slot (128 rows x
 * cout fp32) of the convolution's scratch; tiles are split only while slots remain (max_slots, at most 32767).
 * The table lists the items by weight class (offsets per item >= 14, >= 7, >= 3, fewer), heaviest class first and
 * in tile order inside a class: the convolution's CTAs take items in table order, so the long ones start first.
 * The convolution spreads the parts over its CTAs and adds their slots in part order (tsb_igemm_desc.items). */
int tsb_map_sorted_cm(const int32_t* out_in_map, int64_t rows, int32_t kvol, int64_t valid_n,
                      const int32_t* valid_n_dev, int32_t* reorder_loc, int32_t* map_cm, uint32_t* tile_mask,
                      int32_t max_offsets, int32_t max_slots, int32_t* items, int32_t* n_items, void* workspace,
                      size_t workspace_bytes, tsb_stream_t stream);

/* Pair lists for the GatherScatter / FetchOnDemand dataflows.
 * tsb_pairs_count: nbsizes int32 [kvol] = valid entries per column; also writes the
 * exclusive scans nbaddrs / qnbaddrs int32 [kvol+1] (q = 128 rounding).
 * tsb_pairs_fill: pairs grouped by k, ascending output row.  Layout: transposed == 0 ->
 * nbmaps int32 [P,2] = (in,out); transposed != 0 -> int32 [2,P].
 * Replace the torch nonzero/sum derivation
 * (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:138-141, 185-205) and
 * exclusive_scan_quantified_wrapper (torchsparse/backend/others/exclusive_scan_cuda.cu:31-44). */
int tsb_pairs_count(const int32_t* out_in_map, int64_t rows, int32_t kvol, int32_t* nbsizes,
                    int32_t* nbaddrs, int32_t* qnbaddrs, tsb_stream_t stream);
size_t tsb_pairs_fill_workspace_bytes(int64_t rows, int32_t kvol);
int tsb_pairs_fill(const int32_t* out_in_map, int64_t rows, int32_t kvol, const int32_t* nbaddrs,
                   int64_t n_pairs, int32_t transposed, int32_t* nbmaps, void* workspace,
                   size_t workspace_bytes, tsb_stream_t stream);
int tsb_scan_quantified(int32_t kvol, const int32_t* nbsizes, int32_t* nbaddrs, int32_t* qnbaddrs,
                        tsb_stream_t stream);

/* input_mask int32 [kvol*n_in], output_mask int32 [kvol*n_out]: position of each row inside
 * offset k's pair list, -1 elsewhere; the centre offset of an odd submanifold map is skipped.
 * Fully written by this call.
 * Replaces build_mask_from_kmap (torchsparse/backend/others/sparsemapping_cuda.cu:510-548). */
int tsb_build_masks(int64_t n_in, int64_t n_out, const int32_t* nbmaps, const int32_t* nbaddrs,
                    int32_t kvol, int64_t n_pairs, int32_t* input_mask, int32_t* output_mask,
                    tsb_stream_t stream);

/* ---------------------------------------------------------------- convolution forward
 * Y[m] = sum_k X[map[m][k]] . W[k], fp32 accumulation, one rounding to the output type.
 * X [n_in, cin], W [kvol, cin, cout], Y [n_out, cout] row-major, all of `dtype`. */

/* Implicit GEMM over an out_in_map [pad128(n_out), kvol].  If reorder_loc != NULL the map
 * is the row-sorted one and output row r is stored at reorder_loc[r] (sorted dataflow).
 * Empty (tile, offset) blocks are skipped in either case: tile_mask (uint32 [ceil(n_out / 128)], from
 * tsb_map_tile_mask) names the offsets present in each 128-row tile; with tile_mask == NULL the call
 * derives the masks into its workspace first (one more launch).  Optional fused epilogue, applied to the
 * fp32 accumulator before the single rounding: y = acc * scale[n] + bias[n] + residual[m][n], then
 * ReLU; scale / bias fp32 [cout], residual [n_out,cout] of `dtype`, each may be NULL (an
 * inference-mode BatchNorm folds into scale and bias).
 * fp16 / bf16 tensors, and fp32 tensors with math == TSB_MATH_TF32, run on the tensor cores when the
 * feature rows are 16-byte multiples, cout is a multiple of 8 and kvol <= 32; every other case
 * (exact fp32 arithmetic included) runs on the CUDA cores with the same results up to rounding.
 * Workspace: tsb_conv_igemm_workspace_bytes(...) bytes (packed weights + a status word), plus
 * tsb_map_tile_mask_bytes(n_out) when tile_mask == NULL; none is needed when packed_weight,
 * dev_status and tile_mask are all supplied.
 * Replaces conv_forward_implicit_gemm_cuda
 * (torchsparse/backend/convolution/convolution_forward_implicit_gemm_cuda.cu:1527-1987) and
 * conv_forward_implicit_gemm_sorted_cuda
 * (torchsparse/backend/convolution/convolution_forward_implicit_gemm_sorted_cuda.cu:1755-2230). */
size_t tsb_conv_igemm_workspace_bytes(int32_t kvol, int32_t cin, int32_t cout, int32_t dtype);
int tsb_conv_igemm_fwd(const void* in_feats, const void* weight, const void* packed_weight,
                       const int32_t* out_in_map, const int32_t* reorder_loc, const uint32_t* tile_mask,
                       void* out_feats, int64_t n_in, int64_t n_out, int32_t kvol, int32_t cin, int32_t cout,
                       int32_t dtype, int32_t math, const float* scale, const float* bias,
                       const void* residual, int32_t relu, int32_t* dev_status, void* workspace,
                       size_t workspace_bytes, tsb_stream_t stream);

/* Offsets present in each 128-row tile of a kernel map: out[t] has bit k set when some row of tile t has
 * an entry >= 0 in column k.  The entry of (row, k) is read at map[row * row_stride + k * col_stride]
 * (element strides: (kvol, 1) for the reference's row-major layout, (1, padded rows) for a
 * column-major copy).  n_rows_dev (int32, device, nullable) overrides n_rows with a count held in device
 * memory (n_rows is then its upper bound).  The reference computes the same word as the OR of the sorted
 * row masks, reduce_bitmask_cuda (torchsparse/backend/others/reduce_bitmask_cuda.cu:60-87), for sorted
 * maps only; here every implicit-GEMM launch uses it. */
size_t tsb_map_tile_mask_bytes(int64_t n_rows);
int tsb_map_tile_mask(const int32_t* map, int64_t n_rows, int32_t kvol, int64_t row_stride, int64_t col_stride,
                      const int32_t* n_rows_dev, uint32_t* out, tsb_stream_t stream);

/* The full form of the implicit-GEMM forward: every argument of tsb_conv_igemm_fwd plus the options
 * below, in one descriptor (zero / NULL = option not used).  A caller fills `struct_bytes` with
 * sizeof(tsb_igemm_desc); a library built against another layout refuses the call with TSB_ERR_BAD_ARG.
 *   in_feats2 / c1     the input channels are the concatenation of in_feats [n_in, c1] and in_feats2
 *                      [n_in, cin - c1]; the concatenated matrix is never written (replaces the
 *                      torchsparse.cat in front of a convolution, torchsparse/operators.py:12-16)
 *   map_row_stride / map_col_stride   element strides of the map (0, 0: row-major [rows][kvol]);
 *                      out_in_map == NULL with kvol == 1: output row m reads input row m (a 1x1x1
 *                      convolution, torchsparse/nn/functional/conv/conv.py:65-74, on the same kernel)
 *   n_out_dev          int32 in device memory holding the number of output rows; n_out is then only an
 *                      upper bound (it sizes the launch), so the same launch can be replayed for inputs of
 *                      other sizes, e.g. inside a CUDA graph
 *   k_lo, k_hi         only the kernel offsets [k_lo, k_hi) are multiplied (0, 0: all)
 *   acc_in / acc_out   fp32 [rows of out_feats, cout]: acc_in is added to the accumulator; with acc_out
 *                      the sum is stored there in fp32 and out_feats / the epilogue are skipped.  A group
 *                      of launches over disjoint offset ranges, chained through these buffers, is the
 *                      split-mask form of the sorted dataflow
 *                      (convolution_forward_implicit_gemm_sorted_cuda.cu:42-86, 2226-2229) with the
 *                      partial sums kept in fp32 instead of being rounded per split
 *   items / n_items_dev / n_items / split_scratch / split_flags
 *                      the work-item table of tsb_map_sorted_cm in place of tile_mask: int32 [n_items][4],
 *                      its length in device memory (n_items = upper bound, sizes the launch), fp32 scratch of
 *                      max_slots x 128 x cout elements for the parts of split tiles, and int32 [row tiles *
 *                      ceil(cout / N tile)] part counters that must be zero before the first launch (every
 *                      launch leaves them zero).  Launches that share scratch and counters must not overlap on
 *                      the GPU.  No part waits for another: each stores its accumulator in its slot and counts
 *                      itself; the part that counts last adds the slots in part order and runs the epilogue,
 *                      so results do not depend on the schedule
 *   cfg_*              launch-configuration overrides for tuning runs (N tile, 128-byte channel chunks
 *                      per pipeline stage, stages, CTAs per SM); 0 = chosen by the library.  cfg_gather picks
 *                      how the gathered operand reaches shared memory: 0 or 1 = by 16-byte cp.async of eight
 *                      gather warps (the default: faster on B200), 2 = by the copy engine (TMA gather4, four
 *                      feature rows per copy, zeros for a missing neighbour; same results up to the order of
 *                      the fp32 sums when a two-matrix input is not cut at a multiple of 128 bytes).  cfg_grid
 *                      bounds the persistent CTAs of the launch (0: every resident slot of the device); a caller
 *                      that keeps several streams busy gives each launch a share of the device, so that launches
 *                      of different streams run side by side instead of waiting for each other's last CTAs
 * Tensor-core shapes only (see above); other shapes return TSB_ERR_UNSUPPORTED. */
typedef struct tsb_igemm_desc {
  uint32_t struct_bytes;
  int32_t dtype, math, relu;
  const void* in_feats;
  const void* in_feats2;
  const void* weight;
  const void* packed_weight;
  const int32_t* out_in_map;
  const int32_t* reorder_loc;
  const uint32_t* tile_mask;
  void* out_feats;
  const float* scale;
  const float* bias;
  const void* residual;
  const float* acc_in;
  float* acc_out;
  const int32_t* n_out_dev;
  int32_t* dev_status;
  void* workspace;
  size_t workspace_bytes;
  int64_t n_in, n_out, dst_rows;
  int64_t map_row_stride, map_col_stride;
  int32_t kvol, cin, cout, c1;
  int32_t k_lo, k_hi;
  int32_t cfg_n_tile, cfg_cpb, cfg_stages, cfg_ctas;
  const int32_t* items;
  const int32_t* n_items_dev;
  int64_t n_items;
  float* split_scratch;
  int32_t* split_flags;
  int32_t cfg_gather;
  int32_t cfg_grid;
} tsb_igemm_desc;
int tsb_conv_igemm_run(const tsb_igemm_desc* desc, tsb_stream_t stream);

/* The tensor-core kernel reads the weights K-major ([kvol, cout, cin]).  A caller whose weights
 * do not change between calls (inference) packs them once and passes the result as
 * packed_weight above; with packed_weight == NULL every call packs into its workspace.
 * dev_status (int32, device, nullable) receives a non-zero code if a bounded wait inside the
 * kernel ran out (the output is then undefined).  No counterpart in the reference. */
size_t tsb_conv_packed_weight_bytes(int32_t kvol, int32_t cin, int32_t cout, int32_t dtype);
int tsb_conv_pack_weight(const void* weight, int32_t kvol, int32_t cin, int32_t cout, int32_t dtype,
                         void* packed, tsb_stream_t stream);

/* Weight gradient of the implicit-GEMM dataflow on the tensor cores (fp16 / bf16 operands, fp32 accumulation):
 *   grad_weight[k][a][b] = sum over map rows m of  gathered_feats[out_in_map[m][k]][a] * row_feats[m][b]
 * grad_weight is fp32 [kvol, c_gathered, c_rows]; the call zeroes it first.  With the forward map
 * (gathered = input features, rows = output gradients) this is dW [kvol, cin, cout]; with the transposed map
 * (gathered = output gradients, rows = input features) it is the [kvol, cout, cin] tensor that
 * conv_backward_wgrad_implicit_gemm_cuda returns
 * (torchsparse/backend/convolution/convolution_backward_wgrad_implicit_gemm_cuda.cu:1614-1700; its split_k_iters
 * argument has no counterpart: the row range is divided among CTAs by the library, and the shares meet in
 * grad_weight through fp32 atomic adds, so the last bits of a sum depend on the order in which CTAs finish).
 * tile_mask (nullable) = tsb_map_tile_mask of the map.  Tensor cores: fp16 / bf16, c_gathered % 8 == 0,
 * c_rows % 16 == 0, kvol <= 32; other shapes and fp32 tensors run a CUDA-core kernel (fp32 FMA, exact products) on
 * row-major maps. */
size_t tsb_conv_wgrad_igemm_workspace_bytes(int64_t n_rows);
int tsb_conv_wgrad_igemm(const void* gathered_feats, const void* row_feats, const int32_t* out_in_map,
                         const uint32_t* tile_mask, float* grad_weight, int64_t n_gathered, int64_t n_rows,
                         int64_t map_row_stride, int64_t map_col_stride, int32_t kvol, int32_t c_gathered, int32_t c_rows,
                         int32_t dtype, int32_t* dev_status, void* workspace, size_t workspace_bytes, tsb_stream_t stream);

/* Gather -> grouped GEMM -> scatter over pair lists (nbmaps [P,2], HOST nbsizes [kvol]).
 * 16-bit tensors (and fp32 under TSB_MATH_TF32) whose rows are 16-byte multiples run the GEMM on the
 * tensor cores over the 128-padded pair list, fetching the input rows straight from in_feats.
 * scatter_mask is the output_mask of tsb_build_masks (the input_mask when transpose != 0):
 * the scatter sums each output row's products in a fixed order, without atomics.
 * Replaces conv_forward_gather_scatter_cuda
 * (torchsparse/backend/convolution/convolution_gather_scatter_cuda.cu:279-311). */
size_t tsb_conv_gs_workspace_bytes(int64_t n_pairs, int32_t kvol, int32_t cin, int32_t cout,
                                   int32_t dtype);
int tsb_conv_gs_fwd(const void* in_feats, const void* weight, const int32_t* nbmaps,
                    const int32_t* nbsizes_host, const int32_t* scatter_mask, void* out_feats, int64_t n_in, int64_t n_out,
                    int32_t kvol, int32_t cin, int32_t cout, int32_t dtype, int32_t math,
                    int32_t transpose, void* workspace, size_t workspace_bytes,
                    tsb_stream_t stream);

/* Fetch-on-demand: one fused launch over the 128-quantised pair list (tensor cores where the shape
 * allows, as for tsb_conv_gs_fwd) (nbmaps [2,P],
 * nbaddrs/qnbaddrs int32 [kvol+1] on the device, qmapsize = qnbaddrs[kvol] on the host);
 * fp32 accumulation, scatter by atomic adds into an fp32 accumulator held in `workspace`,
 * rounded once into out_feats.
 * Replaces conv_forward_fetch_on_demand_cuda / _no_fusion_cuda
 * (torchsparse/backend/convolution/convolution_forward_fetch_on_demand_cuda.cu:1981-2260). */
size_t tsb_conv_fod_workspace_bytes(int64_t n_out, int64_t qmapsize, int32_t kvol, int32_t cin, int32_t cout,
                                    int32_t dtype);
int tsb_conv_fod_fwd(const void* in_feats, const void* weight, const int32_t* nbmaps,
                     int64_t n_pairs, const int32_t* nbaddrs, const int32_t* qnbaddrs,
                     int64_t qmapsize, void* out_feats, int64_t n_in, int64_t n_out, int32_t kvol,
                     int32_t cin, int32_t cout, int32_t dtype, int32_t math, int32_t transpose,
                     void* workspace, size_t workspace_bytes, tsb_stream_t stream);

/* ---------------------------------------------------------------- point / voxel ops */

/* out int32 [s] (zeroed by the call) += 1 at every idx[i] >= 0.
 * Replaces count_cuda (torchsparse/backend/others/count_cuda.cu:25-31). */
int tsb_count(const int32_t* idx, int64_t n, int32_t* out, int64_t s, tsb_stream_t stream);

/* out fp32 [n_vox, c] (zeroed by the call) += feats[i] / counts[idx[i]].  feats of `dtype`.
 * Replaces voxelize_forward_cuda (torchsparse/backend/voxelize/voxelize_cuda.cu:78-95). */
int tsb_voxelize_fwd(const void* feats, const int32_t* idx, const int32_t* counts, int64_t n,
                     int64_t n_vox, int32_t c, int32_t dtype, float* out, tsb_stream_t stream);

/* out[i] = sum_{k<8} w[i][k] * feats[idx[i][k]] (idx -1 contributes 0).  feats/out of `dtype`,
 * weights fp32 [n,8], indices int32 [n,8].
 * Replaces devoxelize_forward_cuda (torchsparse/backend/devoxelize/devoxelize_cuda.cu:61-78). */
int tsb_devoxelize_fwd(const void* feats, const int32_t* indices, const float* weights, int64_t n,
                       int32_t c, int32_t dtype, void* out, tsb_stream_t stream);

/* Backward of tsb_voxelize_fwd: grad_feats fp32 [n, c] (fully written) = grad_out[idx[i]] / counts[idx[i]],
 * 0 where idx[i] is out of range.  grad_out fp32 [n_vox, c].
 * Replaces voxelize_backward_cuda (torchsparse/backend/voxelize/voxelize_cuda.cu:58-76, 97-114). */
int tsb_voxelize_bwd(const float* grad_out, const int32_t* idx, const int32_t* counts, int64_t n, int64_t n_vox,
                     int32_t c, float* grad_feats, tsb_stream_t stream);

/* Backward of tsb_devoxelize_fwd with respect to the voxel features: grad_voxels fp32 [n_vox, c] (zeroed by the
 * call) += weights[i][k] * grad_out[i] at indices[i][k] >= 0.  grad_out fp32 [n, c].
 * Replaces devoxelize_backward_cuda (torchsparse/backend/devoxelize/devoxelize_cuda.cu:37-57, 80-98). */
int tsb_devoxelize_bwd(const float* grad_out, const int32_t* indices, const float* weights, int64_t n, int64_t n_vox,
                       int32_t c, float* grad_voxels, tsb_stream_t stream);

/* GPU twin of sparse_quantize: q = floor(xyz / voxel) (evaluated in float64, xyz float32 or
 * float64 [n,3], voxel HOST double[3]), unique by ravel key in ascending order.
 * Outputs: q_all int32 [n,3]; uniq_coords int32 [<=n,3]; first_index int64 [<=n] (smallest
 * original index of each voxel); inverse int64 [n]; result int32[8] (device): [0] = number of
 * voxels, [1..3] = minimum and [4..6] = maximum voxel coordinate per axis.
 * Replaces sparse_quantize / ravel_hash (torchsparse/utils/quantize.py:9-48), a numpy routine
 * in the reference. */
size_t tsb_quantize_workspace_bytes(int64_t n);
int tsb_quantize_unique(const void* xyz, int32_t xyz_is_f64, int64_t n, const double* voxel,
                        int32_t* q_all, int32_t* uniq_coords, int64_t* first_index,
                        int64_t* inverse, int32_t* result, void* workspace, size_t workspace_bytes,
                        tsb_stream_t stream);

/* tsb_quantize_unique for a caller that knows an upper bound of the voxel grid: the ravel keys of a grid of
 * X x Y x Z cells (extent of the voxel coordinates per axis) are below 2^key_bits, and only that many bits are
 * sorted (the general entry sorts 64).  A grid that does not fit gives a wrong result, not an error: state a
 * safe bound. */
int tsb_quantize_unique_bits(const void* xyz, int32_t xyz_is_f64, int64_t n, const double* voxel, int32_t key_bits,
                             int32_t* q_all, int32_t* uniq_coords, int64_t* first_index, int64_t* inverse,
                             int32_t* result, void* workspace, size_t workspace_bytes, tsb_stream_t stream);

/* The network input of one scan from the outputs of tsb_quantize_unique, without the host knowing the voxel
 * count: coords int32 [n_max,4] = (batch, x, y, z) and feats [n_max, c_pad] of `dtype` = the c_in fp32 values
 * of each voxel's first point, zero-padded to c_pad channels; rows at or beyond the voxel count (read from
 * quantize_result[0]) are not written.  Stands for the indexing and collating a caller of the reference does
 * in numpy / torch (torchsparse/utils/collate.py:11-33). */
int tsb_voxel_inputs(const float* points, int32_t c_in, const int64_t* first_index, const int32_t* uniq_coords,
                     const int32_t* quantize_result, int32_t batch, int64_t n_max, int32_t* coords, void* feats,
                     int32_t c_pad, int32_t dtype, tsb_stream_t stream);

/* Dense scatter: out [B,X,Y,Z,C] (zeroed by the CALLER) <- feats[i] at coords[i] = (b,x,y,z).
 * range is HOST int32[4] = (B,X,Y,Z).
 * Replaces to_dense_forward_cuda (torchsparse/backend/voxelize/voxelize_cuda.cu:116-127). */
int tsb_to_dense_fwd(const void* feats, const int32_t* coords, int64_t n, int32_t c,
                     const int32_t* range, int32_t dtype, void* out, tsb_stream_t stream);
/* grad_feats[i][:] = grad_dense[cell of coords[i]][:] (zeros for a row outside `range`).
 * Replaces to_dense_backward_cuda (torchsparse/backend/voxelize/voxelize_cuda.cu:26-37, 129-141). */
int tsb_to_dense_bwd(const void* grad_dense, const int32_t* coords, int64_t n, int32_t c,
                     const int32_t* range, int32_t dtype, void* grad_feats, tsb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TSB200_H_ */
