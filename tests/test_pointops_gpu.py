"""GPU parity: hashing, hash query, count, voxelize, devoxelize, sparse_quantize, to_dense."""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from oracle import kmap_oracle as ko

pytestmark = pytest.mark.gpu


def test_hash_matches_reference(golden):
    from torchsparse_b200.nn import functional as F
    from torchsparse_b200.nn.utils import get_kernel_offsets

    hc = golden["hash/coords"]
    h = F.sphash(torch.from_numpy(hc).cuda()).cpu().numpy()
    assert np.array_equal(h, ko.fnv_hash(hc))                       # raw 64-bit, as the reference's CUDA build
    u = h.view(np.uint64)
    fold = ((u >> np.uint64(60)) ^ (u & np.uint64(0xFFFFFFFFFFFFFFF))).view(np.int64)
    assert np.array_equal(fold, golden["hash/ref_cpu_fold60"])      # folded = the reference's CPU build
    offs = get_kernel_offsets(3, device="cuda")
    assert np.array_equal(offs.cpu().numpy(), golden["k3s1/offsets"])
    hk = F.sphash(torch.from_numpy(hc).cuda(), offs).cpu().numpy()
    assert hk.shape == (27, 500)
    assert np.array_equal(hk, ko.kernel_fnv_hash(hc, offs.cpu().numpy()))


def test_hash_query():
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(1)
    refs = rng.choice(10**15, 30000, replace=False).astype(np.int64)
    q = np.concatenate([refs[rng.integers(0, 30000, 5000)], rng.integers(10**15, 2 * 10**15, 500)]).reshape(50, 110)
    got = F.sphashquery(torch.from_numpy(q).cuda(), torch.from_numpy(refs).cuda()).cpu().numpy()
    assert got.shape == q.shape
    assert np.array_equal(got.reshape(-1), ko.hash_query(q.reshape(-1), refs))
    empty = F.sphashquery(torch.zeros(0, dtype=torch.int64, device="cuda"), torch.from_numpy(refs).cuda())
    assert empty.numel() == 0


def test_count_voxelize_devoxelize_golden(golden):
    from torchsparse_b200.nn import functional as F

    idx = torch.from_numpy(golden["pts/idx"]).cuda()
    cnt = F.spcount(idx, 90)
    assert np.array_equal(cnt.cpu().numpy(), golden["pts/counts"])
    feats = torch.from_numpy(golden["pts/feats"]).cuda()
    vox = F.spvoxelize(feats, torch.from_numpy(golden["pts/idx_nonneg"]).cuda(), cnt)
    assert rel_l2(vox.cpu().numpy(), golden["pts/voxelized"]) < 1e-5
    dv = F.spdevoxelize(torch.from_numpy(golden["devox/vox_feats"]).cuda(),
                        torch.from_numpy(golden["devox/indices"]).cuda(),
                        torch.from_numpy(golden["devox/weights"]).cuda())
    assert rel_l2(dv.cpu().numpy(), golden["devox/out"]) < 1e-5


@pytest.mark.parametrize("dtype,c,tol", [(torch.float32, 32, 1e-5), (torch.float16, 64, 2e-3), (torch.float16, 19, 2e-3)])
def test_voxelize_devoxelize_sizes(dtype, c, tol):
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(c)
    n, nv = 120_000, 90_000
    idx = rng.integers(0, nv, n).astype(np.int32)
    feats = rng.standard_normal((n, c)).astype(np.float32)
    f_r = torch.from_numpy(feats).to(dtype).float().numpy()
    cnt = ko.count(idx, nv)
    got = F.spvoxelize(torch.from_numpy(feats).cuda().to(dtype), torch.from_numpy(idx).cuda(),
                       torch.from_numpy(cnt).cuda())
    assert rel_l2(got.float().cpu().numpy(), ko.voxelize(f_r, idx, cnt)) < tol
    di = rng.integers(-1, nv, (n, 8)).astype(np.int32)
    dw = rng.uniform(0, 1, (n, 8)).astype(np.float32)
    vf = rng.standard_normal((nv, c)).astype(np.float32)
    v_r = torch.from_numpy(vf).to(dtype).float().numpy()
    got = F.spdevoxelize(torch.from_numpy(vf).cuda().to(dtype), torch.from_numpy(di).cuda(),
                         torch.from_numpy(dw).cuda())
    assert rel_l2(got.float().cpu().numpy(), ko.devoxelize(v_r, di, dw)) < tol


def test_calc_ti_weights_sum_to_one():
    from torchsparse_b200.nn import functional as F

    g = torch.Generator(device="cuda").manual_seed(0)
    p = torch.rand(1000, 3, device="cuda", generator=g) * 10
    idx = torch.randint(-1, 50, (1000, 8), device="cuda", generator=g)
    w = F.calc_ti_weights(p, idx)
    assert w.shape == (1000, 8) and bool((w[idx == -1] == 0).all())
    s = w.sum(1)
    ok = (idx >= 0).any(1)
    assert torch.allclose(s[ok], torch.ones_like(s[ok]), atol=1e-4)


def test_sparse_quantize_matches_reference_numpy(golden):
    from torchsparse_b200.utils import sparse_quantize

    for tag, vs in (("q05", 0.05), ("q37", (0.3, 0.7, 0.25)), ("q64", 0.1)):
        pts = golden[f"{tag}/points"]
        c, i, inv = sparse_quantize(pts, vs, return_index=True, return_inverse=True)
        assert isinstance(c, np.ndarray) and c.dtype == np.int32
        assert np.array_equal(c, golden[f"{tag}/coords"])
        assert np.array_equal(i, golden[f"{tag}/index"])
        assert np.array_equal(inv, golden[f"{tag}/inverse"])
        only = sparse_quantize(torch.from_numpy(pts).cuda(), vs)
        assert only.is_cuda and np.array_equal(only.cpu().numpy(), golden[f"{tag}/coords"])


def test_sparse_quantize_lidar_size_and_idempotence():
    from torchsparse_b200.utils import sparse_quantize

    rng = np.random.default_rng(3)
    pts = np.concatenate([rng.uniform(-80, 80, (144_000, 2)), rng.uniform(-3, 3, (144_000, 1))], 1).astype(np.float32)
    c, i, inv = sparse_quantize(pts, 0.05, return_index=True, return_inverse=True)
    cw, iw, invw = ko.sparse_quantize(pts, 0.05, return_index=True, return_inverse=True)
    assert np.array_equal(c, cw) and np.array_equal(i, iw) and np.array_equal(inv, invw)
    # quantising the voxel centres again changes nothing
    c2 = sparse_quantize(c.astype(np.float64) + 0.5, 1.0)
    assert np.array_equal(c2, c)


def test_to_dense():
    import torchsparse_b200 as ts

    rng = np.random.default_rng(5)
    lin = rng.choice(2 * 6 * 7 * 8, 200, replace=False)
    coords = np.stack(np.unravel_index(lin, (2, 6, 7, 8)), 1).astype(np.int32)
    feats = rng.standard_normal((200, 5)).astype(np.float32)
    t = ts.SparseTensor(torch.from_numpy(feats).cuda(), torch.from_numpy(coords).cuda(), spatial_range=(2, 6, 7, 8))
    d = t.dense().cpu().numpy()
    want = np.zeros((2, 6, 7, 8, 5), np.float32)
    want[coords[:, 0], coords[:, 1], coords[:, 2], coords[:, 3]] = feats
    assert np.array_equal(d, want)
