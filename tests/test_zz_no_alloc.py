"""The allocation-free hash join (tsb_hash_query_static) against the workspace-based one.

Some users of the library cannot hand it scratch memory or let it allocate: a plug-in that is given
only input and output buffers, or a fixed-memory real-time loop.  For them the library carries one
entry point whose scratch (the private hash table) is a fixed array inside the library.  This test
calls it through the C ABI exactly as such a caller would: raw pointers, no workspace.

This file sorts last on purpose, so a run that stops at the first failure has already covered
everything else; it passes alone in a fresh process and after the rest of the suite.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(q: torch.Tensor, refs: torch.Tensor):
    from torchsparse_b200._lib import lib, check

    stream = torch.cuda.current_stream().cuda_stream
    out_ws = torch.empty(q.numel(), dtype=torch.int64, device="cuda")
    ws = torch.empty(lib.tsb_hash_query_workspace_bytes(refs.numel()), dtype=torch.uint8, device="cuda")
    check(lib.tsb_hash_query(q.data_ptr(), q.numel(), refs.data_ptr(), refs.numel(), out_ws.data_ptr(),
                             ws.data_ptr(), ws.numel(), stream), "tsb_hash_query")
    out_static = torch.full((q.numel(),), -7, dtype=torch.int64, device="cuda")
    check(lib.tsb_hash_query_static(q.data_ptr(), q.numel(), refs.data_ptr(), refs.numel(), out_static.data_ptr(),
                                    stream), "tsb_hash_query_static")
    torch.cuda.synchronize()
    return out_ws, out_static


def test_static_hash_query_matches_workspace_version_twice_in_a_row():
    from torchsparse_b200._lib import lib

    rng = np.random.default_rng(41)
    limit = lib.tsb_hash_query_static_max_refs()
    assert limit == 262144
    # two calls in a row with different key sets: anything the first call left in the shared table
    # would surface as false hits in the second
    for n_ref, n_q in ((200_000, 150_000), (30_000, 90_000)):
        universe = rng.choice(10**14, n_ref + n_q // 2, replace=False).astype(np.int64) + 1
        refs = torch.from_numpy(universe[:n_ref]).cuda()
        q_np = np.concatenate([universe[rng.integers(0, n_ref, n_q - n_q // 2)], universe[n_ref:]])
        q = torch.from_numpy(q_np).cuda()
        want, got = _both(q, refs)
        assert torch.equal(got, want)                      # integers: exact
        pos = torch.from_numpy(np.concatenate([np.ones(n_q - n_q // 2, bool), np.zeros(n_q // 2, bool)])).cuda()
        assert bool((got[pos] >= 0).all()) and bool((got[~pos] == -1).all())
        assert torch.equal(refs[got[pos]], q[pos])


def test_static_hash_query_at_its_limit_and_without_touching_device_memory():
    """The largest key set the fixed table takes (exactly the stated maximum), and the point of the entry: the
    amount of free device memory is the same before and after the call."""
    from torchsparse_b200._lib import lib, check

    n_ref = lib.tsb_hash_query_static_max_refs()
    rng = np.random.default_rng(43)
    universe = rng.choice(10**14, n_ref + 1000, replace=False).astype(np.int64) + 1
    refs = torch.from_numpy(universe[:n_ref]).cuda()
    q = torch.from_numpy(np.concatenate([universe[:5000], universe[n_ref:]])).cuda()
    want, _ = _both(q, refs)                       # also makes the entry's one-time address lookup happen
    out = torch.empty(q.numel(), dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    check(lib.tsb_hash_query_static(q.data_ptr(), q.numel(), refs.data_ptr(), n_ref, out.data_ptr(), stream),
          "tsb_hash_query_static")
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.equal(out, want)
    assert bool((out[:5000] == torch.arange(5000, device="cuda")).all()) and bool((out[5000:] == -1).all())


def test_static_hash_query_rejects_sizes_beyond_its_table():
    from torchsparse_b200._lib import lib

    n = lib.tsb_hash_query_static_max_refs() + 1
    refs = torch.arange(1, n + 1, dtype=torch.int64, device="cuda")
    q = refs[:10].clone()
    out = torch.full((10,), -7, dtype=torch.int64, device="cuda")
    rc = lib.tsb_hash_query_static(q.data_ptr(), 10, refs.data_ptr(), n, out.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 5                                          # TSB_ERR_LIMIT
    assert lib.tsb_status_string(rc) == b"size beyond a stated maximum"
    torch.cuda.synchronize()
    assert bool((out == -7).all())                          # nothing ran
    # empty inputs are fine
    assert lib.tsb_hash_query_static(None, 0, None, 0, None, None) == 0
