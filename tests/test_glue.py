"""Host-side pieces of the reference's Python surface that need no CUDA kernel of their own: global
pooling, crop, functional activations (torchsparse/nn/functional/{pooling,crop,activation}.py).
They run on CPU tensors, so these tests do too."""
import numpy as np
import torch


def _tensor():
    import torchsparse_b200 as ts

    rng = np.random.default_rng(3)
    coords = np.concatenate([rng.integers(0, 3, (200, 1)), rng.integers(0, 12, (200, 3))], 1).astype(np.int32)
    feats = rng.standard_normal((200, 6)).astype(np.float32)
    return ts.SparseTensor(torch.from_numpy(feats), torch.from_numpy(coords)), coords, feats


def test_global_pooling_matches_a_loop_over_the_batch():
    from torchsparse_b200 import nn as spnn
    from torchsparse_b200.nn import functional as F

    x, coords, feats = _tensor()
    avg, mx = F.global_avg_pool(x).numpy(), F.global_max_pool(x).numpy()
    for b in range(3):
        rows = feats[coords[:, 0] == b]
        assert np.allclose(avg[b], rows.mean(0), atol=1e-6)
        assert np.array_equal(mx[b], rows.max(0))
    assert torch.equal(spnn.GlobalAvgPool()(x), F.global_avg_pool(x))
    assert torch.equal(spnn.GlobalMaxPool()(x), F.global_max_pool(x))


def test_spcrop_keeps_the_half_open_box_over_the_first_three_columns():
    from torchsparse_b200 import nn as spnn
    from torchsparse_b200.nn import functional as F

    x, coords, feats = _tensor()
    lo, hi = (0, 2, 3), (2, 9, 10)
    keep = np.all((coords[:, :3] >= lo) & (coords[:, :3] < hi), axis=1)
    y = F.spcrop(x, lo, hi)
    assert np.array_equal(y.coords.numpy(), coords[keep]) and np.array_equal(y.feats.numpy(), feats[keep])
    assert y.stride == x.stride
    assert np.array_equal(spnn.SparseCrop(lo, hi)(x).coords.numpy(), coords[keep])
    assert F.spcrop(x).coords.shape == x.coords.shape          # no bounds: everything stays


def test_functional_activations_keep_coords_and_cache():
    from torchsparse_b200.nn import functional as F

    x, coords, feats = _tensor()
    for fn, ref in ((F.relu, np.maximum(feats, 0)), (F.leaky_relu, np.where(feats > 0, feats, 0.1 * feats))):
        x2, _, _ = _tensor()
        y = fn(x2, inplace=False)
        assert np.allclose(y.feats.numpy(), ref, atol=1e-6)
        assert y.coords is x2.coords and y._caches is x2._caches


def test_spdownsample_stride_equal_kernel_on_cpu():
    """The branch of spdownsample that is plain tensor arithmetic (every stride 1 or the kernel size)."""
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(4)
    coords = np.unique(np.concatenate([rng.integers(0, 2, (500, 1)), rng.integers(0, 30, (500, 3))], 1), axis=0)
    got = F.spdownsample(torch.from_numpy(coords.astype(np.int32)), (2, 2, 1), (2, 2, 1)).numpy()
    want = np.unique(np.concatenate([coords[:, :1], coords[:, 1:] // np.array([2, 2, 1])], 1), axis=0)
    assert np.array_equal(got, want) and got.dtype == np.int32


def test_sparse_collate_prepends_batch_index():
    import torchsparse_b200 as ts
    from torchsparse_b200.utils.collate import sparse_collate, sparse_collate_fn

    a = ts.SparseTensor(torch.ones(3, 2), torch.tensor([[0, 0, 0], [1, 1, 1], [2, 2, 2]], dtype=torch.int32))
    b = ts.SparseTensor(torch.zeros(2, 2), np.array([[5, 5, 5], [6, 6, 6]], dtype=np.int32))
    out = sparse_collate([a, b])
    assert out.coords.tolist() == [[0, 0, 0, 0], [0, 1, 1, 1], [0, 2, 2, 2], [1, 5, 5, 5], [1, 6, 6, 6]]
    assert out.feats.shape == (5, 2) and out.stride == (1, 1, 1)
    batch = sparse_collate_fn([{"x": a, "y": np.zeros(2), "meta": {"n": 1}}, {"x": b, "y": np.ones(2), "meta": {"n": 2}}])
    assert batch["x"].coords.shape == (5, 4) and batch["y"].shape == (2, 2) and batch["meta"]["n"] == [1, 2]


def test_32bit_key_tables_are_taken_only_where_every_ravel_key_fits():
    from torchsparse_b200 import backend

    assert backend.fits_32bit_keys((0, 0, 0, 0), (0, 2399, 2399, 159))            # a LiDAR grid at 5 cm: 9.2e8 cells
    assert backend.fits_32bit_keys((0, -100, -100, -10), (3, 1500, 1500, 100))    # 4 scans: 1.1e9 cells
    assert not backend.fits_32bit_keys((0, 0, 0, 0), (0, 70000, 70000, 8))        # 4.4e10 cells
    assert not backend.fits_32bit_keys((0, 0, 0, 0), (0, 65535, 65535, 0))        # exactly 2^32 cells
    assert backend.fits_32bit_keys((0, 0, 0, 0), (0, 65535, 65534, 0))
