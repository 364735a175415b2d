"""ctypes binding of libtsb200.so (the C ABI declared in include/tsb200.h).

The library is the only compute path of this package: if it cannot be loaded the
import fails loudly, there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libtsb200.so")

P = C.c_void_p
I32 = C.c_int32
I64 = C.c_int64
SZ = C.c_size_t

# name -> (restype, argtypes); mirrors include/tsb200.h declaration by declaration
SIGNATURES = {
    "tsb_version": (C.c_char_p, []),
    "tsb_status_string": (C.c_char_p, [C.c_int]),
    "tsb_last_cuda_error": (C.c_char_p, []),
    "tsb_launch_count": (C.c_longlong, []),
    "tsb_coord_hash": (C.c_int, [P, I64, P, P]),
    "tsb_kernel_hash": (C.c_int, [P, I64, P, I32, P, P]),
    "tsb_hash_insert": (C.c_int, [P, P, I64, P, I64, P, P]),
    "tsb_hash_lookup": (C.c_int, [P, P, I64, P, I64, P, P]),
    "tsb_hash_lookup_coords": (C.c_int, [P, P, I64, P, I64, P, P, P, P]),
    "tsb_hash_query_workspace_bytes": (SZ, [I64]),
    "tsb_hash_query": (C.c_int, [P, I64, P, I64, P, P, SZ, P]),
    "tsb_hash_query_static_max_refs": (I64, []),
    "tsb_hash_query_static": (C.c_int, [P, I64, P, I64, P, P]),
    "tsb_kmap_subm": (C.c_int, [P, P, I64, P, I64, P, P, P, I32, P, P, P]),
    "tsb_kmap_down_slots": (I32, [P, P]),
    "tsb_kmap_down_workspace_bytes": (SZ, [I64, P, P]),
    "tsb_kmap_down_unique": (C.c_int, [P, I64, P, P, P, P, P, P, P, P, SZ, P]),
    "tsb_kmap_down_finish": (C.c_int, [P, P, I64, P, I64, P, I64, P, P, P, P, P, P, P, P, P]),
    "tsb_map_transpose": (C.c_int, [P, I64, I32, P, I64, I32, P]),
    "tsb_bitmask_derive": (C.c_int, [P, I64, I32, I32, I64, P, P]),
    "tsb_bitmask_sort_workspace_bytes": (SZ, [I64, I32]),
    "tsb_bitmask_sort": (C.c_int, [P, I64, I32, I32, P, P, P, SZ, P]),
    "tsb_bitmask_reduce": (C.c_int, [P, I64, I32, I32, P, P]),
    "tsb_map_reorder": (C.c_int, [P, I64, I32, P, I32, P, P]),
    "tsb_pairs_count": (C.c_int, [P, I64, I32, P, P, P, P]),
    "tsb_pairs_fill_workspace_bytes": (SZ, [I64, I32]),
    "tsb_pairs_fill": (C.c_int, [P, I64, I32, P, I64, I32, P, P, SZ, P]),
    "tsb_scan_quantified": (C.c_int, [I32, P, P, P, P]),
    "tsb_build_masks": (C.c_int, [I64, I64, P, P, I32, I64, P, P, P]),
    "tsb_conv_igemm_workspace_bytes": (SZ, [I32, I32, I32, I32]),
    "tsb_conv_igemm_fwd": (C.c_int, [P, P, P, P, P, P, P, I64, I64, I32, I32, I32, I32, I32, P, P, P, I32, P, P, SZ, P]),
    "tsb_map_tile_mask_bytes": (SZ, [I64]),
    "tsb_map_tile_mask": (C.c_int, [P, I64, I32, I64, I64, P, P, P]),
    "tsb_conv_igemm_run": (C.c_int, [P, P]),
    "tsb_map_sorted_cm_workspace_bytes": (SZ, [I64]),
    "tsb_map_items_max": (I64, [I64, I32, I32]),
    "tsb_map_sorted_cm": (C.c_int, [P, I64, I32, I64, P, P, P, P, I32, I32, P, P, P, SZ, P]),
    "tsb_conv_packed_weight_bytes": (SZ, [I32, I32, I32, I32]),
    "tsb_conv_pack_weight": (C.c_int, [P, I32, I32, I32, I32, P, P]),
    "tsb_conv_wgrad_igemm_workspace_bytes": (SZ, [I64]),
    "tsb_conv_wgrad_igemm": (I32, [P, P, P, P, P, I64, I64, I64, I64, I32, I32, I32, I32, P, P, SZ, P]),
    "tsb_conv_gs_workspace_bytes": (SZ, [I64, I32, I32, I32, I32]),
    "tsb_conv_gs_fwd": (C.c_int, [P, P, P, P, P, P, I64, I64, I32, I32, I32, I32, I32, I32, P, SZ, P]),
    "tsb_conv_fod_workspace_bytes": (SZ, [I64, I64, I32, I32, I32, I32]),
    "tsb_conv_fod_fwd": (C.c_int, [P, P, P, I64, P, P, I64, P, I64, I64, I32, I32, I32, I32, I32, I32, P, SZ, P]),
    "tsb_count": (C.c_int, [P, I64, P, I64, P]),
    "tsb_voxelize_fwd": (C.c_int, [P, P, P, I64, I64, I32, I32, P, P]),
    "tsb_devoxelize_fwd": (C.c_int, [P, P, P, I64, I32, I32, P, P]),
    "tsb_map_sorted_workspace_bytes": (SZ, [I64]),
    "tsb_map_sorted_artefacts": (C.c_int, [P, I64, I32, I64, I32, P, P, P, P, P, SZ, P]),
    "tsb_quantize_workspace_bytes": (SZ, [I64]),
    "tsb_quantize_unique": (C.c_int, [P, I32, I64, P, P, P, P, P, P, P, SZ, P]),
    "tsb_quantize_unique_bits": (C.c_int, [P, I32, I64, P, I32, P, P, P, P, P, P, SZ, P]),
    "tsb_voxel_inputs": (C.c_int, [P, I32, P, P, P, I32, I64, P, P, I32, I32, P]),
    "tsb_level_record_from_quantize": (C.c_int, [P, I32, P, P, P]),
    "tsb_kmap_subm_dyn": (C.c_int, [P, P, I64, P, I64, P, P, I32, P, P, P]),
    "tsb_kmap_down_dyn_workspace_bytes": (SZ, [I64, P, P]),
    "tsb_kmap_down_dyn": (C.c_int, [P, P, I64, P, I64, P, P, P, P, I32, I64, P, P, P, P, P, P, SZ, P]),
    "tsb_voxelize_bwd": (C.c_int, [P, P, P, I64, I64, I32, P, P]),
    "tsb_devoxelize_bwd": (C.c_int, [P, P, P, I64, I64, I32, P, P]),
    "tsb_to_dense_fwd": (C.c_int, [P, P, I64, I32, P, I32, P, P]),
    "tsb_to_dense_bwd": (C.c_int, [P, P, I64, I32, P, I32, P, P]),
}

class IgemmDesc(C.Structure):
    """tsb_igemm_desc of include/tsb200.h, field for field."""
    _fields_ = [
        ("struct_bytes", C.c_uint32), ("dtype", I32), ("math", I32), ("relu", I32),
        ("in_feats", P), ("in_feats2", P), ("weight", P), ("packed_weight", P), ("out_in_map", P),
        ("reorder_loc", P), ("tile_mask", P), ("out_feats", P), ("scale", P), ("bias", P), ("residual", P),
        ("acc_in", P), ("acc_out", P), ("n_out_dev", P), ("dev_status", P), ("workspace", P),
        ("workspace_bytes", SZ), ("n_in", I64), ("n_out", I64), ("dst_rows", I64),
        ("map_row_stride", I64), ("map_col_stride", I64),
        ("kvol", I32), ("cin", I32), ("cout", I32), ("c1", I32), ("k_lo", I32), ("k_hi", I32),
        ("cfg_n_tile", I32), ("cfg_cpb", I32), ("cfg_stages", I32), ("cfg_ctas", I32),
        ("items", P), ("n_items_dev", P), ("n_items", I64), ("split_scratch", P), ("split_flags", P),
        ("cfg_gather", I32), ("cfg_grid", I32),
    ]


def new_igemm_desc() -> "IgemmDesc":
    d = IgemmDesc()
    d.struct_bytes = C.sizeof(IgemmDesc)
    return d


TSB_OK = 0
TSB_F32, TSB_F16, TSB_BF16 = 0, 1, 2
TSB_MATH_FP32, TSB_MATH_TF32 = 0, 1
TSB_DEV_TABLE_FULL, TSB_DEV_BAD_INDEX, TSB_DEV_LIMIT = 1, 2, 4


class TsbError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python torchsparse_b200/csrc/build.py` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these operators.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status: int, what: str) -> None:
    """Turn a status code into the exception the reference's entry points raise
    (std::invalid_argument -> ValueError, std::runtime_error -> RuntimeError)."""
    if status == TSB_OK:
        return
    msg = lib.tsb_status_string(status).decode()
    if status == 4:
        msg += ": " + lib.tsb_last_cuda_error().decode()
    if status in (1, 5):
        raise ValueError(f"{what}: {msg}")
    raise TsbError(f"{what}: {msg}")


def i32x(vals):
    """Host int32 array argument."""
    return (I32 * len(vals))(*[int(v) for v in vals])
