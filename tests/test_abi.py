"""CPU suite, part 2: the C-ABI library loads and exports every symbol include/tsb200.h declares, the
ctypes table covers the same set, and argument checks that need no GPU answer with status codes."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tsb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tsb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    from torchsparse_b200 import _lib

    names = _declared()
    assert len(names) > 30
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in tsb200.h but not exported by libtsb200.so"
    assert sorted(_lib.SIGNATURES) == names


def test_ctypes_table_matches_the_header_prototypes():
    """Every prototype of include/tsb200.h has as many parameters as its entry in the ctypes table, pointer
    parameters are bound as pointers and 64-bit sizes as 64-bit integers: a drifted binding would pass garbage."""
    from torchsparse_b200 import _lib

    text = open(os.path.join(ROOT, "include", "tsb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = re.findall(r"\b(tsb_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S)
    assert sorted(n for n, _ in protos) == sorted(_lib.SIGNATURES)
    wide = (ctypes.c_int64, ctypes.c_uint64, ctypes.c_size_t, ctypes.c_longlong, ctypes.c_ulonglong)
    for name, args in protos:
        params = [] if args.strip() in ("", "void") else [a.strip() for a in args.split(",")]
        bound = _lib.SIGNATURES[name][1]
        assert len(params) == len(bound), f"{name}: {len(params)} parameters declared, {len(bound)} bound"
        for decl, ctype in zip(params, bound):
            if "*" in decl or decl.startswith("tsb_stream_t"):
                assert ctype in (ctypes.c_void_p, ctypes.c_char_p) or issubclass(ctype, ctypes._Pointer), (name, decl)
            elif decl.startswith(("int64_t", "size_t", "uint64_t")):
                assert ctype in wide, (name, decl, ctype)


def test_status_strings_and_argument_checks():
    from torchsparse_b200._lib import lib, i32x

    assert b"tsb200" in lib.tsb_version()
    assert lib.tsb_status_string(0) == b"ok"
    # null pointers / bad sizes are refused before any CUDA call
    assert lib.tsb_coord_hash(None, 5, None, None) == 1
    assert lib.tsb_coord_hash(None, 0, None, None) == 0
    assert lib.tsb_conv_igemm_fwd(None, None, None, None, None, None, None, 1, 1, 27, 0, 8, 0, 0, None, None, None, 0, None, None, 0, None) == 1
    assert lib.tsb_conv_igemm_fwd(None, None, None, None, None, None, None, 1, 1, 27, 8, 8, 9, 0, None, None, None, 0, None, None, 0, None) == 2
    assert lib.tsb_bitmask_reduce(None, 10, 1, 6, None, None) == 1
    assert lib.tsb_kmap_down_slots(i32x((2, 2, 2)), i32x((2, 2, 2))) == 1
    assert lib.tsb_kmap_down_slots(i32x((3, 3, 3)), i32x((2, 2, 2))) == 8
    assert lib.tsb_kmap_down_slots(i32x((1, 3, 1)), i32x((1, 2, 1))) == 2
    assert lib.tsb_kmap_down_slots(i32x((3, 3, 3)), i32x((0, 2, 2))) == 0
    assert lib.tsb_conv_fod_workspace_bytes(100, 256, 27, 32, 32, 1) >= 100 * 32 * 4


def test_product_has_no_oracle_or_cpu_fallback():
    """The package must not import the oracle, and its operators must refuse CPU tensors."""
    import torch
    import pytest
    import torchsparse_b200 as ts
    from torchsparse_b200 import backend

    pkg = os.path.join(ROOT, "torchsparse_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(".py"):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, f"{f} mentions the oracle"
    with pytest.raises(RuntimeError):
        backend.hash_cuda(torch.zeros(4, 4, dtype=torch.int32))
    assert ts.__version__
